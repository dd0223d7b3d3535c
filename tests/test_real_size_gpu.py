"""The engine at the layer sizes of real models of the family, with seeded random weights, against the plain
implementation. The tiny configurations exercise every option; these exercise the kernels and the rules that choose
between them at the sizes the benchmark times: SmolLM2-135M whole (30 layers, hidden 576, 9 heads over 3 key/value
heads of 64, feed-forward 1,536, vocabulary 49,152, tied head) at batch 2, at batch 64 through the decode graph, with
a prompt of 2,048 tokens and with eight contexts of about 2,000 tokens; and two layers each at the layer sizes of
SmolLM2-1.7B (24 layers in the full model) and Llama-3.1-8B (32 layers: heads of 128, llama3 rotary scaling, an
untied head over 128,256 tokens)."""
import numpy as np
import pytest

import plain_llama as P
from helpers import TOL, PlainLogits, host, make_engine, prompts_for, rel_error

pytestmark = pytest.mark.gpu

SMOLLM2_135M_SHAPE = {
    "model_type": "llama", "vocab_size": 49152, "hidden_size": 576, "intermediate_size": 1536,
    "num_hidden_layers": 30, "num_attention_heads": 9, "num_key_value_heads": 3, "head_dim": 64,
    "rope_theta": 100000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192,
    "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
SMOLLM2_1P7B_LAYERS = dict(SMOLLM2_135M_SHAPE, num_hidden_layers=2, hidden_size=2048, num_attention_heads=32,
                           num_key_value_heads=32, intermediate_size=8192, rope_theta=130000.0)
LLAMA_8B_LAYERS = dict(
    SMOLLM2_135M_SHAPE, num_hidden_layers=2, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
    head_dim=128, intermediate_size=14336, vocab_size=128256, rope_theta=500000.0, tie_word_embeddings=False,
    rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                  "original_max_position_embeddings": 8192})


@pytest.fixture(scope="module")
def real_size():
    weights = P.random_weights(SMOLLM2_135M_SHAPE, seed=5)
    return weights, PlainLogits(SMOLLM2_135M_SHAPE, weights)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompts_then_single_tokens_at_real_size(real_size, dtype):
    weights, plain = real_size
    engine = make_engine(SMOLLM2_135M_SHAPE, weights, dtype, max_tokens=64 * 8, max_length=256)
    long_prompt, short_prompt = prompts_for(SMOLLM2_135M_SHAPE, (70, 9), seed=6)
    slots = engine.open(2)
    rows = [0, 31, 63, 64, 69]
    got = host(engine.step(slots, [long_prompt, short_prompt], [rows, [8]]))
    assert rel_error(got[:5], plain(long_prompt)[rows]) <= TOL[dtype]
    assert rel_error(got[5], plain(short_prompt)[8]) <= TOL[dtype]
    contexts = [long_prompt, short_prompt]
    for step in range(3):
        tokens = [[1000 + 17 * step], [40000 - 9 * step]]
        got = host(engine.step(slots, tokens))
        for i in range(2):
            contexts[i] = contexts[i] + tokens[i]
            want = plain(contexts[i])[-1]
            assert rel_error(got[i], want) <= TOL[dtype], (step, i)
            if dtype == "float32":
                assert int(np.argmax(got[i])) == int(np.argmax(want))
    engine.close(slots)
    engine.cache.check()


def test_greedy_generation_at_real_size_in_float32(real_size):
    """Tokens through the entry point against the plain implementation's greedy loop (float32: the logits agree to
    5e-5, far below the gap between the two largest of 49,152 logits of a random model at these steps)."""
    weights, plain = real_size
    engine = make_engine(SMOLLM2_135M_SHAPE, weights, "float32", max_tokens=64 * 4, max_length=128)
    prompt = prompts_for(SMOLLM2_135M_SHAPE, (12,), seed=8)[0]
    result = engine.generate([prompt], max_new_tokens=6, ignore_eos=True)[0]
    context = list(prompt)
    for token in result.tokens:
        logits = plain(context)[-1]
        best = int(np.argmax(logits))
        runner_up = float(np.partition(logits, -2)[-2])
        assert float(logits[best]) - runner_up > 1e-3 * float(np.abs(logits).max()), "a tie too close to call"
        assert token == best
        context.append(token)


def _decode_and_compare(engine, config, weights, dtype, prompts, slots, first_logits, steps):
    """Decodes `steps` tokens for every sequence through `Engine.decode` (the captured graph), one step a call so
    that each step's logits can be read from the graph's buffer, then compares the prompt step's last rows and every
    decode step's rows with ONE plain forward per sequence over prompt + chosen tokens (a position's logits do not
    depend on what follows it)."""
    chosen = [np.argmax(first_logits, axis=1).tolist()]
    per_step = [first_logits]
    for _ in range(steps):
        out = engine.decode(slots, chosen[-1], 1)
        logits = host(engine.last_decode_graph.logits)
        assert out[0] == np.argmax(logits, axis=1).tolist()  # the graph's choice is the first largest of its logits
        per_step.append(logits)
        chosen.append(out[0])
    sequences = [list(p) + [chosen[s][i] for s in range(steps)] for i, p in enumerate(prompts)]
    rows = [list(range(len(p) - 1, len(p) + steps)) for p in prompts]
    wanted = P.forward_many(config, weights, sequences, rows)
    worst = 0.0
    for i, want in enumerate(wanted):
        got = np.stack([per_step[s][i] for s in range(steps + 1)])
        error = rel_error(got, want)
        worst = max(worst, error)
        assert error <= TOL[dtype], (i, len(prompts[i]), error)
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_batch_of_64_through_the_decode_graph_at_real_size(real_size, dtype):
    """What the benchmark's batch-64 point runs: products with 64 rows of activations (sixteen warps a block, the
    head product the other way round on tcgen05), decode attention with one or two blocks a pair. Prompts of 8 to
    80 tokens enter in two steps of 32 sequences; then three decode steps of all 64 through the graph."""
    weights, _ = real_size
    config = SMOLLM2_135M_SHAPE
    rng = np.random.default_rng(64)
    lengths = rng.integers(8, 81, 64).tolist()
    prompts = prompts_for(config, lengths, seed=65)
    engine = make_engine(config, weights, dtype, max_tokens=64 * 2 * 64, max_length=192, decode_logits=True)
    slots = engine.open(64)
    first = np.concatenate([host(engine.step(slots[:32], prompts[:32])), host(engine.step(slots[32:], prompts[32:]))])
    _decode_and_compare(engine, config, weights, dtype, prompts, slots, first, steps=3)
    engine.check()
    engine.close(slots)
    engine.cache.check()


def test_a_batch_of_12_through_the_decode_graph_at_real_size(real_size):
    """Twelve rows of activations: the products whose weights are above a megabyte split their reduction over a
    cluster (four blocks at most with so few rows), the output product (smaller) keeps a block per 16 rows of W."""
    weights, _ = real_size
    config = SMOLLM2_135M_SHAPE
    lengths = np.random.default_rng(12).integers(8, 60, 12).tolist()
    prompts = prompts_for(config, lengths, seed=13)
    engine = make_engine(config, weights, "bfloat16", max_tokens=64 * 2 * 12, max_length=192, decode_logits=True)
    slots = engine.open(12)
    first = host(engine.step(slots, prompts))
    _decode_and_compare(engine, config, weights, "bfloat16", prompts, slots, first, steps=3)
    engine.check()
    engine.close(slots)
    engine.cache.check()


@pytest.fixture(scope="module")
def long_prompt_case(real_size):
    weights, _ = real_size
    prompt = prompts_for(SMOLLM2_135M_SHAPE, (2048,), seed=66)[0]
    rows = [0, 63, 64, 1023, 1024, 1500, 2046, 2047]
    return prompt, rows, P.forward_many(SMOLLM2_135M_SHAPE, weights, [prompt], [rows])[0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_prompt_of_2048_tokens_at_real_size(real_size, long_prompt_case, dtype):
    """The benchmark's prefill: in bfloat16 the tcgen05 attention (thousands of keys against the plain attention)
    and the wide q/k/v tile; in float32 the blockwise kernel of the 32-bit path."""
    weights, _ = real_size
    prompt, rows, want = long_prompt_case
    engine = make_engine(SMOLLM2_135M_SHAPE, weights, dtype, max_tokens=2048 + 64, max_length=2048 + 64)
    slot = engine.open(1)
    got = host(engine.step(slot, [prompt], [rows]))
    engine.check()
    assert rel_error(got, want) <= TOL[dtype]
    for i in range(len(rows)):
        assert rel_error(got[i], want[i]) <= 2 * TOL[dtype], rows[i]
    engine.close(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_eight_long_contexts_through_the_decode_graph(dtype):
    """The benchmark's headline point: batch 8 with about 2,000 cached tokens each (decode attention in clusters of
    eight blocks over 32 pages). Four of the model's thirty layers, at full layer sizes, keep the plain forwards of
    16,000 tokens short; what is tested is the choice and the indexing of the kernels, which layers do not change."""
    config = dict(SMOLLM2_135M_SHAPE, num_hidden_layers=4)
    weights = P.random_weights(config, seed=9)
    lengths = [1900, 2048, 1987, 2001, 1923, 2040, 1961, 2017]
    prompts = prompts_for(config, lengths, seed=67)
    engine = make_engine(config, weights, dtype, max_tokens=8 * 2112, max_length=2112, decode_logits=True)
    slots = engine.open(8)
    first = np.concatenate([host(engine.step(slots[i:i + 2], prompts[i:i + 2])) for i in range(0, 8, 2)])
    _decode_and_compare(engine, config, weights, dtype, prompts, slots, first, steps=2)
    engine.check()
    engine.close(slots)
    engine.cache.check()


def _large_random_weights(config, seed, std=0.02):
    """`plain_llama.random_weights` for models of a billion weights: the same distributions and the same rounding to
    bfloat16-exact values, drawn and rounded with torch on the device (a second instead of minutes for NumPy's
    double draws; the values for a seed differ from `random_weights`, which no test here depends on)."""
    import torch

    generator = torch.Generator(device="cuda:0").manual_seed(seed)
    out = {}
    for name, shape in P.tensor_shapes(config).items():
        norm = name.endswith("norm.weight")
        values = torch.randn(shape, generator=generator, dtype=torch.float32, device="cuda:0")
        values = values * (0.01 if norm else std) + (1.0 if norm else 0.0)
        out[name] = values.to(torch.bfloat16).to(torch.float32).cpu().numpy()
    return out


@pytest.fixture(scope="module", params=["smollm2-1.7b", "llama-3.1-8b"])
def larger_layers(request):
    """Two layers at the layer sizes of a larger model of the family, a prompt of 40 tokens followed by three single
    tokens, and 33 short sequences that take one more token together; the plain logits of all of it in one call."""
    config = SMOLLM2_1P7B_LAYERS if request.param == "smollm2-1.7b" else LLAMA_8B_LAYERS
    weights = _large_random_weights(config, seed=10)
    prompt = prompts_for(config, (43,), seed=68)[0]
    short = prompts_for(config, np.random.default_rng(69).integers(2, 13, 33).tolist(), seed=70)
    rows = [[0, 20, 39, 40, 41, 42]] + [[len(s) - 2, len(s) - 1] for s in short]
    plain = P.forward_many(config, weights, [prompt] + short, rows)
    return config, weights, prompt, short, plain


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_layers_at_the_sizes_of_larger_models(larger_layers, dtype):
    """Reaches, through the engine's own rules: products that stream W through shared memory (one or two rows, long
    rows of W), the tile product with W as the 128-row operand (33 rows against the head and the gate/up matrix), the
    same with the reduction cut (33 rows against the output and down projections), the cluster kernel on large W,
    256-wide tiles, heads of 128 in every attention kernel, llama3 rotary scaling and an untied head."""
    config, weights, prompt, short, plain = larger_layers
    engine = make_engine(config, weights, dtype, max_tokens=64 * 40, max_length=128, decode_logits=True)
    slot = engine.open(1)
    got = [host(engine.step(slot, [prompt[:40]], [[0, 20, 39]]))]
    for token in prompt[40:]:
        got.append(host(engine.step(slot, [[token]])))
    assert rel_error(np.concatenate(got), plain[0]) <= TOL[dtype]
    many = engine.open(33)
    before = host(engine.step(many, [s[:-1] for s in short]))
    after = host(engine.step(many, [[s[-1]] for s in short]))
    engine.check()
    for i in range(33):
        assert rel_error(np.stack([before[i], after[i]]), plain[1 + i]) <= TOL[dtype], i
    # the same single tokens through the decode graph: the graph's logits for the last token of every sequence
    engine.close(many)
    many = engine.open(33)
    engine.step(many, [s[:-1] for s in short], [[] for _ in short])
    engine.decode(many, [s[-1] for s in short], 1)
    graph_logits = host(engine.last_decode_graph.logits)
    engine.check()
    for i in range(33):
        assert rel_error(graph_logits[i], plain[1 + i][1]) <= TOL[dtype], i
    engine.close(many + slot)
    # six and twelve of them as batches of their own: with 3 to 16 rows the rules send wide matrices to the tile
    # product with W as the 128-row operand and very long rows of W through shared memory
    for count in (6, 12):
        few = engine.open(count)
        engine.step(few, [s[:-1] for s in short[:count]], [[] for _ in range(count)])
        last = host(engine.step(few, [[s[-1]] for s in short[:count]]))
        engine.check()
        for i in range(count):
            assert rel_error(last[i], plain[1 + i][1]) <= TOL[dtype], (count, i)
        engine.close(few)
    engine.cache.check()
