"""The engine at the layer sizes of SmolLM2-135M (30 layers, hidden 576, 9 heads over 3 key/value heads of 64,
feed-forward 1,536, vocabulary 49,152, tied head) with seeded random weights: the tiny configurations exercise every
option, this one the kernels at the sizes the benchmark times (products streamed with the norm fused in front,
cluster decode attention, the head product over the whole vocabulary) and thirty layers of accumulated rounding."""
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
