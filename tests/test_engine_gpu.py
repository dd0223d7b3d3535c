"""The engine against the plain implementation, in float32 and in bfloat16, for two tiny configurations that differ
in every size and option: whole prompts, token-by-token decoding, unequal batches with slot reuse, long decoding,
first tokens, generation through the entry point."""
import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import TOL, PlainLogits, host, make_engine, model_case, prompts_for, rel_error

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
TAGS = ["a", "b"]


@pytest.fixture(scope="module", params=[(t, d) for t in TAGS for d in DTYPES], ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request):
    tag, dtype = request.param
    config, weights = model_case(tag)
    engine = make_engine(config, weights, dtype, max_tokens=64 * 24)
    return tag, dtype, config, weights, engine, PlainLogits(config, weights)


def test_each_request_alone_and_whole(setup):
    _, dtype, config, _, engine, plain = setup
    for prompt in prompts_for(config, (1, 2, 7, 23, 40, 64, 65, 100)):
        slot = engine.open(1)
        logits = host(engine.step(slot, [prompt], [list(range(len(prompt)))]))
        engine.close(slot)
        assert logits.shape == (len(prompt), config["vocab_size"])
        assert rel_error(logits, plain(prompt)) <= TOL[dtype], len(prompt)
    engine.cache.check()


def test_last_32_tokens_one_by_one(setup):
    _, dtype, config, _, engine, plain = setup
    for prompt in prompts_for(config, (33, 70, 120), seed=3):
        slot = engine.open(1)
        head = len(prompt) - 32
        rows = [host(engine.step(slot, [prompt[:head]]))[0]]
        for token in prompt[head:]:
            rows.append(host(engine.step(slot, [[token]]))[0])
        engine.close(slot)
        want = plain(prompt)[head - 1:]
        for index, (got, ref) in enumerate(zip(rows, want)):
            assert rel_error(got, ref) <= TOL[dtype], (len(prompt), index)


def test_unequal_batches_one_after_another(setup):
    """Batches of unequal lengths; shorter requests end earlier; the next batch reuses their slots and pages."""
    _, dtype, config, _, engine, plain = setup
    rng = np.random.default_rng(9)
    held_before = engine.cache.pages_held()
    for round_index, lengths in enumerate(((5, 11, 17), (1, 7, 23, 40), (66, 3, 64))):
        prompts = prompts_for(config, lengths, seed=20 + round_index)
        decode = [int(rng.integers(2, 9)) for _ in prompts]  # how many tokens each sequence goes on for
        tails = [rng.integers(0, config["vocab_size"], n).tolist() for n in decode]
        slots = engine.open(len(prompts))
        logits = host(engine.step(slots, prompts, [list(range(len(p))) for p in prompts]))
        offset = 0
        for prompt in prompts:
            assert rel_error(logits[offset:offset + len(prompt)], plain(prompt)) <= TOL[dtype]
            offset += len(prompt)
        live = list(range(len(prompts)))
        for step in range(max(decode)):
            live = [i for i in live if step < decode[i]]
            got = host(engine.step([slots[i] for i in live], [[tails[i][step]] for i in live]))
            for row, i in enumerate(live):
                context = prompts[i] + tails[i][:step + 1]
                assert rel_error(got[row], plain(context)[-1]) <= TOL[dtype], (round_index, i, step)
            ended = [i for i in live if step + 1 == decode[i]]
            engine.close([slots[i] for i in ended])
        engine.cache.check()
        assert engine.cache.pages_held() == held_before and engine.cache.slots.held == 0


def test_long_decoding(setup):
    _, dtype, config, _, engine, plain = setup
    tokens = prompts_for(config, (100,), seed=5)[0]
    slot = engine.open(1)
    engine.step(slot, [tokens[:3]], [[]])
    reference = plain(tokens)
    for index in range(3, len(tokens)):
        got = host(engine.step(slot, [[tokens[index]]]))[0]
        if index % 8 == 0 or index >= 60:
            assert rel_error(got, reference[index]) <= TOL[dtype], index
    engine.close(slot)


def test_first_tokens_of_a_sequence(setup):
    _, dtype, config, _, engine, plain = setup
    tokens = prompts_for(config, (6,), seed=6)[0]
    slot = engine.open(1)
    for index, token in enumerate(tokens):
        got = host(engine.step(slot, [[token]]))[0]
        assert rel_error(got, plain(tokens[:index + 1])[-1]) <= TOL[dtype], index
    engine.close(slot)


def test_chunked_prompt_equals_whole(setup):
    _, dtype, config, _, engine, plain = setup
    prompt = prompts_for(config, (90,), seed=8)[0]
    slot = engine.open(1)
    parts = [prompt[:10], prompt[10:64], prompt[64:65], prompt[65:]]
    rows = []
    for part in parts:
        rows.append(host(engine.step(slot, [part], [list(range(len(part)))])))
    engine.close(slot)
    assert rel_error(np.concatenate(rows), plain(prompt)) <= TOL[dtype]


def test_float32_logits_do_not_depend_on_the_cut(setup):
    """In 32-bit a position's logits are the same bits alone, in a batch, decoded one by one, in a reused slot."""
    _, dtype, config, _, engine, _ = setup
    if dtype != "float32":
        pytest.skip("bit equality is the float32 path's property")
    prompts = prompts_for(config, (9, 30, 70), seed=12)
    alone = []
    for prompt in prompts:
        slot = engine.open(1)
        alone.append(engine.step(slot, [prompt], [list(range(len(prompt)))]).clone())
        engine.close(slot)
    slots = engine.open(3)
    together = engine.step(slots[::-1], prompts[::-1], [list(range(len(p))) for p in prompts[::-1]]).clone()
    engine.close(slots)
    assert torch.equal(together, torch.cat(alone[::-1]))
    slot = engine.open(1)
    engine.step(slot, [prompts[2][:40]], [[]])
    rows = [engine.step(slot, [[t]]).clone() for t in prompts[2][40:]]
    engine.close(slot)
    assert torch.equal(torch.cat(rows), alone[2][40:])


def test_greedy_generation_through_the_entry_point(setup):
    from etalii.dllm_b200 import SamplingOptions

    tag, dtype, config, weights, engine, plain = setup
    prompts = prompts_for(config, (5, 11, 17, 3, 40), seed=30)
    results = engine.generate(prompts, 8, SamplingOptions(), ignore_eos=True, max_batch=3)
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "length" and result.prompt_tokens == len(prompt) and len(result.tokens) == 8
        if dtype == "float32":
            assert list(result.tokens) == P.generate(config, weights, prompt, 8)[0]
        else:  # each chosen token must be (nearly) the best token of the plain logits for the same context
            context = list(prompt)
            for token in result.tokens:
                ref = plain(context)[-1]
                assert ref[token] >= ref.max() - 2 * TOL[dtype] * np.abs(ref).max()
                context.append(token)
    assert engine.cache.slots.held == 0
    engine.cache.check()


def test_sampled_generation_and_stop_tokens(setup):
    from etalii.dllm_b200 import SamplingOptions

    tag, dtype, config, weights, engine, _ = setup
    if dtype != "float32":
        pytest.skip("seeded draws are compared token for token in float32")
    prompts = prompts_for(config, (1, 7, 23, 40), seed=31)
    options = SamplingOptions(temperature=0.8, seed=5)
    results = engine.generate(prompts, 12, options, ignore_eos=True)
    for index, (prompt, result) in enumerate(zip(prompts, results)):
        want, _ = P.generate(config, weights, prompt, 12, temperature=0.8, seed=5 + index)
        assert list(result.tokens) == want
    # a stop token ends its sequence early and is not part of the output; the others go on
    stop = results[1].tokens[3]
    stopped = engine.generate(prompts, 12, options, ignore_eos=True, stop_token_ids=[stop])
    for index, (prompt, result) in enumerate(zip(prompts, stopped)):
        want, reason = P.generate(config, weights, prompt, 12, temperature=0.8, seed=5 + index, stop_tokens=[stop])
        assert list(result.tokens) == want and result.finish_reason == reason
    assert stopped[1].finish_reason == "stop" and len(stopped[1].tokens) <= 3
    alone = engine.generate([prompts[2]], 12, SamplingOptions(temperature=0.8, seed=7))
    assert alone[0].tokens == engine.generate(prompts, 12, SamplingOptions(temperature=0.8, seed=5))[2].tokens


SIZES = [
    # heads, kv_heads, head_dim, hidden, intermediate, vocab, window-less Llama layers
    dict(num_attention_heads=8, num_key_value_heads=1, head_dim=32, hidden_size=72, intermediate_size=200, vocab_size=130),
    dict(num_attention_heads=4, num_key_value_heads=2, head_dim=128, hidden_size=96, intermediate_size=136, vocab_size=514),
    dict(num_attention_heads=3, num_key_value_heads=3, head_dim=80, hidden_size=120, intermediate_size=96, vocab_size=90),
    dict(num_attention_heads=34, num_key_value_heads=2, head_dim=16, hidden_size=64, intermediate_size=72, vocab_size=258),
    dict(num_attention_heads=2, num_key_value_heads=1, head_dim=256, hidden_size=40, intermediate_size=48, vocab_size=66),
    dict(num_attention_heads=5, num_key_value_heads=5, head_dim=144, hidden_size=56, intermediate_size=64, vocab_size=100),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("sizes", SIZES, ids=lambda s: f"h{s['num_attention_heads']}k{s['num_key_value_heads']}d{s['head_dim']}")
def test_other_sizes(sizes, dtype):
    """Head sizes in steps of 16 (and one that is not), any number of heads and groups, widths and vocabularies that
    are no power of two: whole prompts in a batch, then single tokens, against the plain implementation."""
    config = dict(P.TINY_A, num_hidden_layers=1, tie_word_embeddings=False, max_position_embeddings=512, **sizes)
    weights = P.random_weights(config, seed=7, std=0.08)
    engine = make_engine(config, weights, dtype, max_tokens=64 * 12)
    plain = PlainLogits(config, weights)
    prompts = prompts_for(config, (70, 3, 129), seed=13)
    slots = engine.open(3)
    logits = host(engine.step(slots, prompts, [list(range(len(p))) for p in prompts]))
    offset = 0
    for prompt in prompts:
        assert rel_error(logits[offset:offset + len(prompt)], plain(prompt)) <= TOL[dtype]
        offset += len(prompt)
    tails = prompts_for(config, (3, 3, 3), seed=14)
    for step in range(3):
        got = host(engine.step(slots, [[t[step]] for t in tails]))
        for row, (prompt, tail) in enumerate(zip(prompts, tails)):
            assert rel_error(got[row], plain(prompt + tail[:step + 1])[-1]) <= TOL[dtype], (row, step)
    engine.close(slots)
    chosen = engine.generate(prompts[:2], 4, ignore_eos=True)  # the CUDA-graph decode path at these sizes
    assert all(len(r.tokens) == 4 for r in chosen)


def test_sizes_the_kernels_refuse_are_refused_when_the_engine_is_built():
    """config.json allows widths and head sizes the kernels cannot run (rows are read in 16-byte pieces). Every
    part is asked before weights go to the device, and the error names the part and the rule; the kernels keep
    their own refusal for a caller that comes another way."""
    from etalii.dllm_b200.engine.model import UnsupportedConfiguration
    from etalii.dllm_b200.kernels.ops import KernelError
    from etalii.dllm_b200.kernels import ops

    config = dict(P.TINY_A, num_hidden_layers=1, intermediate_size=100)  # rows of 100 bfloat16 are not 16-byte pieces
    weights = P.random_weights(config, seed=1)
    before = torch.cuda.memory_allocated()
    with pytest.raises(UnsupportedConfiguration, match=r"layers\.0\.feed_forward: intermediate_size 100.*multiple of 8"):
        make_engine(config, weights, "bfloat16", max_tokens=128)
    assert torch.cuda.memory_allocated() == before  # nothing was uploaded
    make_engine(config, weights, "float32", max_tokens=128)  # 100 is a multiple of 4: the 32-bit path takes it
    odd = dict(P.TINY_A, num_hidden_layers=1, head_dim=20, num_attention_heads=4, num_key_value_heads=2)
    with pytest.raises(UnsupportedConfiguration, match="head_dim 20"):
        make_engine(odd, P.random_weights(odd, seed=1), "float32", max_tokens=128)
    c = torch.zeros((3, 16), dtype=torch.float32, device="cuda:0")
    a = torch.zeros((3, 100), dtype=torch.bfloat16, device="cuda:0")
    w = torch.zeros((16, 100), dtype=torch.bfloat16, device="cuda:0")
    with pytest.raises(KernelError, match="multiple of 8"):
        ops.gemm(c, a, w, ops.EPI_STORE_F32)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_step_shape_that_comes_again_with_other_tokens_slots_and_pages(dtype, name):
    """The same step shape (two prompts of unequal lengths, the same wanted rows) with other tokens each time, in
    other slots and pages, and a different shape in between: every time the logits are those of the plain
    implementation for THAT time's tokens (anything kept from an earlier step of the same shape, a buffer view, a
    tensor map or a table, would show if it were stale)."""
    config = P.TINY_A if name == "A" else P.TINY_B
    weights = P.random_weights(config, seed=31)
    engine = make_engine(config, weights, dtype, max_tokens=64 * 12)
    plain = PlainLogits(config, weights)
    want = [[0, 17, 69], [4]]
    held = engine.open(1)  # a slot that stays taken, so the prompts' slots change between rounds
    engine.step(held, [[1, 2, 3]])
    for turn in range(5):
        a, b = prompts_for(config, (70, 5), seed=40 + turn)
        extra = engine.open(turn % 2)  # shifts which slots and pages the prompts get
        slots = engine.open(2)
        got = host(engine.step(slots, [a, b], want))
        assert rel_error(got[:3], plain(a)[[0, 17, 69]]) <= TOL[dtype], turn
        assert rel_error(got[3], plain(b)[4]) <= TOL[dtype], turn
        if turn == 2:  # another shape in between
            other = prompts_for(config, (33,), seed=50)[0]
            slot = engine.open(1)
            assert rel_error(host(engine.step(slot, [other]))[0], plain(other)[-1]) <= TOL[dtype]
            engine.close(slot)
        # the prompts go on by a token each: a step from the cache that the replayed step wrote
        nxt = [[7], [9]]
        got = host(engine.step(slots, nxt))
        assert rel_error(got[0], plain(a + nxt[0])[-1]) <= TOL[dtype], turn
        assert rel_error(got[1], plain(b + nxt[1])[-1]) <= TOL[dtype], turn
        engine.close(slots + extra)
    engine.close(held)
    engine.cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_a_neighbour_in_decode_changes_no_bit_in_float32_and_a_repetition_none_in_bfloat16(name):
    """Two sequences decoded side by side in 32-bit give the bits each gives as a whole prompt alone (the
    reference's character, README.md:9-15: bits independent of batch and of how a sequence is split). In bfloat16
    the kernels differ with the number of rows, so only the repetition of a run gives the same bits there: no
    kernel sums in an order that depends on which block arrives first."""
    config = P.TINY_A if name == "A" else P.TINY_B
    weights = P.random_weights(config, seed=3, std=0.08)
    engine = make_engine(config, weights, "float32", max_tokens=64 * 16)
    a, b = prompts_for(config, (90, 33), seed=4)
    alone = []
    for prompt in (a, b):
        slot = engine.open(1)
        alone.append(host(engine.step(slot, [prompt], [list(range(len(prompt)))])))
        engine.close(slot)
    slots = engine.open(2)
    engine.step(slots, [a[:70], b[:13]], [[], []])
    for i in range(20):
        got = host(engine.step(slots, [[a[70 + i]], [b[13 + i]]]))
        assert np.array_equal(got[0], alone[0][70 + i]) and np.array_equal(got[1], alone[1][13 + i]), i
    engine.close(slots)
    engine.cache.check()
    bf16 = make_engine(config, weights, "bfloat16", max_tokens=64 * 16)
    runs = []
    for _ in range(2):
        slots = bf16.open(2)
        rows = [host(bf16.step(slots, [a, b], [[0, 89], [32]]))]
        rows += [host(bf16.step(slots, [[5 + i], [6 + i]])) for i in range(3)]
        bf16.close(slots)
        runs.append(np.concatenate(rows))
    assert np.array_equal(runs[0], runs[1])


def test_no_stop_token_before_min_tokens(setup):
    """`min_tokens`: the stop tokens are taken out of the choice until an output is that long (greedy: the runner-up
    is chosen where a stop token leads; sampled: the draw is made among the other tokens), in the prompt step, inside
    a run of decode steps and across runs; after that a stop token ends the sequence as ever."""
    from etalii.dllm_b200 import SamplingOptions

    tag, dtype, config, weights, engine, _ = setup
    if dtype != "float32":
        pytest.skip("tokens are compared one for one in float32")
    prompts = prompts_for(config, (6, 19, 2), seed=33)
    for options, kwargs in ((SamplingOptions(), {}), (SamplingOptions(temperature=0.9, seed=3), {"temperature": 0.9})):
        free = engine.generate(prompts, 24, options, ignore_eos=True)
        # stop tokens that each sequence would choose early: its first token and one a few steps in
        stops = sorted({free[0].tokens[0], free[1].tokens[2], free[2].tokens[5], free[0].tokens[9]})
        for min_tokens in (0, 1, 4, 7, 30):
            results = engine.generate(prompts, 24, options, ignore_eos=True, stop_token_ids=stops,
                                      min_tokens=min_tokens)
            for index, (prompt, result) in enumerate(zip(prompts, results)):
                want, reason = P.generate(config, weights, prompt, 24, seed=options.seed + index, stop_tokens=stops,
                                          min_tokens=min_tokens, **kwargs)
                assert list(result.tokens) == want and result.finish_reason == reason, (min_tokens, index)
                assert reason == "length" or len(want) >= min_tokens
    with pytest.raises(ValueError, match="min_tokens"):
        engine.generate(prompts, 4, min_tokens=-1)
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_an_odd_vocabulary(dtype):
    config = dict(P.TINY_A, num_hidden_layers=2, vocab_size=131, tie_word_embeddings=False)
    weights = P.random_weights(config, seed=1)
    engine = make_engine(config, weights, dtype, max_tokens=256)
    prompt = [5, 130, 17, 0, 99, 64, 3]
    want = P.forward(config, weights, prompt)
    slot = engine.open(1)
    got = host(engine.step(slot, [prompt[:5]], [list(range(5))]))
    assert rel_error(got, want[:5]) <= TOL[dtype]
    for index in (5, 6):  # decode-sized products with an odd number of outputs
        assert rel_error(host(engine.step(slot, [[prompt[index]]]))[0], want[index]) <= TOL[dtype]
    engine.close(slot)
    if dtype == "float32":  # the sampler over 131 logits
        tokens = list(prompt)
        for _ in range(4):
            tokens.append(P.argmax(P.forward(config, weights, tokens)[-1]))
        assert list(engine.generate([prompt], 4, ignore_eos=True)[0].tokens) == tokens[len(prompt):]


def test_long_generation_through_the_graph_path(setup):
    """Well over a hundred tokens through `generate` (CUDA-graph decode in runs of 16 steps, new cache pages on
    the way, sequences of unequal length) against the plain implementation."""
    from etalii.dllm_b200 import SamplingOptions

    tag, dtype, config, weights, engine, plain = setup
    if tag != "a":
        pytest.skip("Tiny A's context of 128 is the one that a long generation fills")
    prompts = prompts_for(config, (3, 60, 20), seed=40)
    results = engine.generate(prompts, 200, SamplingOptions(), ignore_eos=True)
    for prompt, result in zip(prompts, results):
        # the context window (128) ends the generation: prompt + output == window
        assert result.finish_reason == "length" and len(prompt) + len(result.tokens) == 128
        if dtype == "float32":
            assert list(result.tokens) == P.generate(config, weights, prompt, 200)[0]
        else:
            context = list(prompt) + list(result.tokens)
            for index in (len(prompt), len(prompt) + 40, 126):  # spot checks along the way
                ref = plain(context[:index])[-1]
                assert ref[context[index]] >= ref.max() - 2 * TOL[dtype] * np.abs(ref).max(), index
    assert engine.cache.slots.held == 0
    engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim", [64, 128])
def test_head_dims_of_the_tcgen05_attention_with_long_and_short_prompts(dtype, head_dim):
    """The head sizes of the tcgen05 attention at engine level: in bfloat16 a prompt of 700 tokens takes it and
    the tile product that ends in rotation and cache write, short prompts the mma.sync attention (a batch of 300 and
    40 tokens lies on either side of the change, by head size), single tokens the cluster kernel; a prompt that goes
    on from a cached prefix crosses tile and page edges."""
    config = dict(P.TINY_A, num_hidden_layers=2, tie_word_embeddings=False, max_position_embeddings=1024,
                  num_attention_heads=3, num_key_value_heads=1, head_dim=head_dim, hidden_size=72,
                  intermediate_size=120, vocab_size=203)
    weights = P.random_weights(config, seed=21, std=0.08)
    engine = make_engine(config, weights, dtype, max_tokens=64 * 40, max_length=1024)
    plain = PlainLogits(config, weights)
    long_prompt, short_a, short_b = prompts_for(config, (700, 130, 5), seed=22)
    slots = engine.open(3)
    rows = [0, 63, 64, 127, 128, 511, 512, 640, 699]
    got = host(engine.step([slots[0]], [long_prompt], [rows]))
    assert rel_error(got, plain(long_prompt)[rows]) <= TOL[dtype]
    got = host(engine.step(slots[1:], [short_a, short_b], [[129], [4]]))
    assert rel_error(got[0], plain(short_a)[-1]) <= TOL[dtype] and rel_error(got[1], plain(short_b)[-1]) <= TOL[dtype]
    more = prompts_for(config, (190,), seed=23)[0]  # goes on from position 700: a long context again
    got = host(engine.step([slots[0]], [more], [[0, 100, 189]]))
    assert rel_error(got, plain(long_prompt + more)[[700, 800, 889]]) <= TOL[dtype]
    contexts = [long_prompt + more, short_a, short_b]
    for step in range(3):
        tokens = [[(7 * step + i) % config["vocab_size"]] for i in range(3)]
        got = host(engine.step(slots, tokens))
        for i in range(3):
            contexts[i] = contexts[i] + tokens[i]
            assert rel_error(got[i], plain(contexts[i])[-1]) <= TOL[dtype], (step, i)
    engine.close(slots)
    middle, little = prompts_for(config, (300, 40), seed=24)
    slots = engine.open(2)
    got = host(engine.step(slots, [middle, little], [[0, 191, 192, 299], [39]]))
    assert rel_error(got[:4], plain(middle)[[0, 191, 192, 299]]) <= TOL[dtype]
    assert rel_error(got[4], plain(little)[-1]) <= TOL[dtype]
    engine.close(slots)
    engine.cache.check()


@pytest.fixture(scope="module")
def long_case():
    config = dict(P.TINY_B, num_hidden_layers=1, max_position_embeddings=8192, vocab_size=128, num_attention_heads=4,
                  num_key_value_heads=2, head_dim=16, hidden_size=64, intermediate_size=96)
    config["rope_scaling"] = dict(config["rope_scaling"], original_max_position_embeddings=2048)
    weights = P.random_weights(config, seed=3, std=0.08)
    tokens = prompts_for(config, (5010,), seed=50)[0]
    return config, weights, tokens, P.forward(config, weights, tokens)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_context(long_case, dtype):
    """Five thousand positions: many pages per sequence, rotary angles far out, several rounds of the decode
    attention's key split; a whole prompt, a prompt that goes on from a cached prefix, then single tokens."""
    config, weights, tokens, reference = long_case
    engine = make_engine(config, weights, dtype, max_tokens=64 * 170, max_length=8192)
    slots = engine.open(2)
    rows = list(range(0, 5000, 97)) + [4999]
    whole = host(engine.step([slots[0]], [tokens[:5000]], [rows]))
    assert rel_error(whole, reference[rows]) <= TOL[dtype]
    engine.step([slots[1]], [tokens[:3000]], [[]])
    rest = host(engine.step([slots[1]], [tokens[3000:5000]], [[0, 1000, 1999]]))
    assert rel_error(rest, reference[[3000, 4000, 4999]]) <= TOL[dtype]
    for index in range(5000, 5010):
        got = host(engine.step(slots, [[tokens[index]], [tokens[index]]]))
        assert rel_error(got[0], reference[index]) <= TOL[dtype], index
        assert rel_error(got[1], reference[index]) <= TOL[dtype], index
    engine.close(slots)
    engine.cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_sampled_batches_that_grow_and_shrink_keep_their_graphs_valid(name):
    """A captured decode graph holds the addresses of work buffers, the sampler's scratch among them. Batches of 8,
    3, 8, 3 and 4, 5, 6, 5 sequences on one engine make those buffers grow after graphs of smaller batches were
    captured; every run must still give the plain implementation's tokens (float32, seeded draws)."""
    from etalii.dllm_b200 import SamplingOptions

    config, weights = model_case(name.lower())
    engine = make_engine(config, weights, "float32", max_tokens=64 * 24)
    lengths = (5, 11, 17, 3, 9, 2, 14, 7)
    prompts = prompts_for(config, lengths, seed=44)

    memo = {}

    def run(count, options, seed_of):
        results = engine.generate(prompts[:count], 20, options, ignore_eos=True)
        for index, (prompt, result) in enumerate(zip(prompts, results)):
            key = (index, options.temperature, seed_of(index))
            if key not in memo:
                memo[key] = P.generate(config, weights, prompt, 20, temperature=options.temperature,
                                       seed=seed_of(index))[0]
            assert list(result.tokens) == memo[key], (count, index)

    run(8, SamplingOptions(), lambda i: 0)
    sampled = SamplingOptions(temperature=0.8, seed=5)
    for count in (3, 8, 3, 4, 5, 6, 5, 3):
        run(count, sampled, lambda i: 5 + i)
    assert engine.cache.slots.held == 0
    engine.cache.check()


@pytest.mark.parametrize("name", ["A", "B"])
def test_the_one_kernel_feed_forward_as_an_engine_option(name):
    """`ops.FUSED_FEED_FORWARD` (off by default: it measured slower than the two kernels it replaces) switches decode
    steps to the fused feed-forward kernel; the engine's logits then still agree with the plain implementation."""
    from etalii.dllm_b200.kernels import ops

    config, weights = model_case(name.lower())
    plain = PlainLogits(config, weights)
    prompts = prompts_for(config, (9, 20, 3), seed=51)
    launches = {}
    for fused in (True, False):
        ops.FUSED_FEED_FORWARD = fused
        try:
            engine = make_engine(config, weights, "bfloat16", max_tokens=64 * 6)
            slots = engine.open(3)
            engine.step(slots, [p[:-2] for p in prompts], [[], [], []])
            before = ops.launches
            for back in (2, 1):
                got = host(engine.step(slots, [[p[-back]] for p in prompts]))
                for i, p in enumerate(prompts):
                    assert rel_error(got[i], plain(p)[len(p) - back]) <= TOL["bfloat16"]
            launches[fused] = (ops.launches - before) // 2
            engine.close(slots)
        finally:
            ops.FUSED_FEED_FORWARD = False
    assert launches[False] - launches[True] == config["num_hidden_layers"]  # one launch fewer a layer


@pytest.mark.parametrize("head_dim", [32, 64, 128])
def test_the_native_launcher_of_prefill_steps_issues_what_the_parts_issue(head_dim):
    """Steps of more than 64 tokens of a model made of the library's own parts are launched from C++ in one call,
    with the norms folded around the products (five launches a layer); the same step driven part by part from
    Python runs the norms as kernels (seven a layer). Both agree with the plain implementation, and with each
    other far inside its tolerance. Models with other parts or head sizes have no native table."""
    from etalii.dllm_b200.kernels import launcher, ops

    config = dict(P.TINY_B, num_hidden_layers=2, head_dim=head_dim, num_attention_heads=4, num_key_value_heads=2,
                  hidden_size=128, intermediate_size=320, max_position_embeddings=1024)
    weights = P.random_weights(config, seed=3, std=0.05)
    plain = PlainLogits(config, weights)
    engine = make_engine(config, weights, "bfloat16", max_tokens=64 * 24, max_length=1024)
    assert engine.model.native_layers is not None
    prompts = prompts_for(config, (300, 70, 5), seed=21)
    results = {}
    for native in (True, False):
        launcher.ENABLED = native
        try:
            slots = engine.open(3)
            before = ops.launches
            logits = engine.step(slots, prompts, [[0, 299], [69], [4]]).clone()
            results[native] = (logits, ops.launches - before)
            got = host(engine.step(slots, [p[-1:] for p in prompts]))  # single tokens: the Python path either way
            engine.close(slots)
        finally:
            launcher.ENABLED = True
    assert engine.model.native_layers.norms_folded
    assert results[False][1] - results[True][1] == 2 * 2 - 1  # two norms a layer less, one pass over the first rows
    want = np.stack([plain(prompts[0])[0], plain(prompts[0])[299], plain(prompts[1])[69], plain(prompts[2])[4]])
    assert rel_error(host(results[True][0]), want) <= TOL["bfloat16"]
    assert rel_error(host(results[False][0]), want) <= TOL["bfloat16"]
    assert rel_error(host(results[True][0]), host(results[False][0])) <= TOL["bfloat16"] / 3
    engine.check()
    tiny, tiny_weights = model_case("a")
    assert make_engine(tiny, tiny_weights, "bfloat16", max_tokens=128).model.native_layers is None  # head_dim 16
    assert make_engine(config, weights, "float32", max_tokens=128).model.native_layers is None


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_decoding_without_logits_chooses_the_same_tokens(name):
    """By default a greedy decode run makes its choice inside the head product and stores no logits; an engine
    built with decode_logits=True stores them and chooses from them. Same kernels up to the epilogue: same tokens."""
    config, weights = model_case(name.lower())
    prompts = prompts_for(config, (9, 20, 3, 33), seed=61)
    outputs = {}
    for keep in (False, True):
        engine = make_engine(config, weights, "bfloat16", max_tokens=64 * 8, decode_logits=keep)
        outputs[keep] = [r.tokens for r in engine.generate(prompts, 24, ignore_eos=True)]
        assert (engine.last_decode_graph.logits is not None) == keep
    assert outputs[False] == outputs[True]


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("sequences", [9, 17, 40, 64])
def test_steps_of_nine_to_sixty_four_rows(name, sequences):
    """Steps whose products split their reduction over a cluster (17 rows and more at these sizes): a prompt step
    of at most 64 tokens, then single tokens for all sequences, every row against the plain implementation; and the
    same through the decode graph."""
    config, weights = model_case(name.lower())
    plain = PlainLogits(config, weights)
    rng = np.random.default_rng(sequences)
    lengths = [1] * sequences
    for _ in range(64 - sequences):  # prompts of unequal lengths, 64 tokens in all
        lengths[int(rng.integers(0, sequences))] += 1
    prompts = prompts_for(config, lengths, seed=sequences)
    engine = make_engine(config, weights, "bfloat16", max_tokens=64 * sequences, decode_logits=True)
    slots = engine.open(sequences)
    logits = host(engine.step(slots, prompts))
    contexts = [list(p) for p in prompts]
    for step in range(3):
        for i, context in enumerate(contexts):
            assert rel_error(logits[i], plain(context)[-1]) <= TOL["bfloat16"], (step, i)
        chosen = np.argmax(logits, axis=1).tolist()
        for context, token in zip(contexts, chosen):
            context.append(int(token))
        if step < 2:
            logits = host(engine.step(slots, [[t] for t in chosen]))
        else:
            out = engine.decode(slots, chosen, 1)
            logits = host(engine.last_decode_graph.logits)
            assert out[0] == np.argmax(logits, axis=1).tolist()
    for i, context in enumerate(contexts):
        assert rel_error(logits[i], plain(context)[-1]) <= TOL["bfloat16"], ("graph", i)
    engine.close(slots)
    engine.cache.check()
