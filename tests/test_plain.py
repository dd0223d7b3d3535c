"""The plain implementation against the reference project's own outputs (tests/golden/*.npz)."""
import os

import numpy as np
import pytest

import plain_llama as P

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = {"a": (P.TINY_A, 0, 0.02), "b": (P.TINY_B, 1, 0.08)}


def _load(tag):
    config, seed, std = CASES[tag]
    return config, seed, P.random_weights(config, seed, std=std), np.load(os.path.join(GOLDEN, f"tiny_{tag}.npz"))


@pytest.mark.parametrize("tag", ["a", "b"])
def test_logits_match_reference(tag):
    config, _, weights, golden = _load(tag)
    index = 0
    while f"prompt{index}" in golden:
        prompt = golden[f"prompt{index}"].tolist()
        want = golden[f"logits{index}"]
        got = P.forward(config, weights, prompt)
        # the reference's own bound against float64 (tests/test_transformer.py:158)
        assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()
        index += 1
    assert index >= 3


@pytest.mark.parametrize("tag", ["a", "b"])
def test_inv_freq_matches_reference(tag):
    config, _, _, golden = _load(tag)
    got = P.rope_inv_freq(config["head_dim"], config["rope_theta"], config.get("rope_scaling"))
    np.testing.assert_allclose(got, golden["inv_freq"], rtol=1e-14)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_generation_matches_reference(tag):
    config, seed, weights, golden = _load(tag)
    index = 0
    while f"prompt{index}" in golden:
        prompt = golden[f"prompt{index}"].tolist()
        greedy, _ = P.generate(config, weights, prompt, 8)
        assert greedy == golden[f"greedy{index}"].tolist()
        sampled, _ = P.generate(config, weights, prompt, 12, temperature=0.8, seed=seed + index)
        assert sampled == golden[f"sampled{index}"].tolist()
        nucleus, _ = P.generate(config, weights, prompt, 12, temperature=1.3, top_k=20, top_p=0.9, min_p=0.02,
                                seed=7 + index)
        assert nucleus == golden[f"nucleus{index}"].tolist()
        index += 1


def test_random_matches_reference_stream():
    # first outputs of xoshiro256** seeded by SplitMix64(0): the published test vector of the generator
    r = P.Random(0)
    assert r.next_u64() == 0x99EC5F36CB75F2B4
    assert 0.0 <= P.Random(2**64 + 5).next_double() < 1.0
    assert P.Random(2**64 + 5).next_u64() == P.Random(5).next_u64()


def test_window_attention_edges():
    rng = np.random.default_rng(0)
    q = rng.standard_normal((9, 4, 8)).astype(np.float32)
    k = rng.standard_normal((9, 2, 8)).astype(np.float32)
    v = rng.standard_normal((9, 2, 8)).astype(np.float32)
    full = P.attention(q, k, v, 0.35)
    windowed = P.attention(q, k, v, 0.35, window=3)
    assert np.array_equal(full[:3], windowed[:3])  # the window does not bind for the first 3 queries
    assert not np.allclose(full[5], windowed[5])
    alone = P.attention(q[6:7], k[4:7], v[4:7], 0.35)  # query 6 sees keys 4, 5, 6 only... as a 1-query sequence
    # a lone query at offset 0 sees only its first key, so compare through a 3-key causal run instead
    run = P.attention(np.repeat(q[6:7], 3, 0), k[4:7], v[4:7], 0.35)
    np.testing.assert_allclose(run[2], windowed[6], rtol=1e-6)
    assert alone.shape == (1, 4, 8)


def test_choosing_among_allowed_tokens_is_choosing_with_the_others_at_minus_infinity():
    """What the engine does for `min_tokens` (stop tokens' logits set to -inf before the choice) gives the token that
    the reference's rule gives (the same choice made on the logits of the allowed tokens alone,
    src/etalii_dllm/sampling.py:400-409): a probability of exactly zero is never the largest and never drawn."""
    rng = np.random.default_rng(3)
    for trial in range(40):
        logits = (rng.standard_normal(50) * 3).astype(np.float32)
        held_back = sorted(set(int(t) for t in rng.integers(0, 50, 3)) | {int(np.argmax(logits))})
        allowed = [t for t in range(50) if t not in held_back]
        masked = logits.copy()
        masked[held_back] = -np.inf
        for options in (dict(temperature=0.0), dict(temperature=0.8), dict(temperature=1.3, top_k=5),
                        dict(temperature=0.7, top_p=0.6), dict(temperature=1.0, min_p=0.2),
                        dict(temperature=0.9, top_k=48, top_p=0.99, min_p=0.01)):
            a = P.sample(logits, P.Random(trial), allowed=allowed, **options)
            b = P.sample(masked, P.Random(trial), **options)
            assert a == b and a not in held_back, (trial, options)


def test_attention_by_matrices_is_the_same_function_as_attention_by_queries():
    """The head-at-a-time form used at real sizes against the query-at-a-time form that restates the reference."""
    rng = np.random.default_rng(3)
    for heads, kv_heads, dim, length, window in ((6, 3, 24, 70, None), (4, 1, 16, 33, 9), (5, 5, 40, 130, 64)):
        q = rng.standard_normal((length, heads, dim)).astype(np.float32)
        k = rng.standard_normal((length, kv_heads, dim)).astype(np.float32)
        v = rng.standard_normal((length, kv_heads, dim)).astype(np.float32)
        a = P.attention(q, k, v, 0.3, window)
        b = P.attention_by_matrices(q, k, v, 0.3, window)
        assert np.abs(a.astype(np.float64) - b).max() <= 1e-6 * np.abs(a).max()


def test_forward_many_gives_each_sequence_the_logits_of_forward():
    weights = P.random_weights(P.TINY_B, 1, std=0.08)
    rng = np.random.default_rng(4)
    sequences = [rng.integers(0, P.TINY_B["vocab_size"], n).tolist() for n in (40, 1, 17)]
    rows = [[0, 39], [0], [3, 4, 16]]
    many = P.forward_many(P.TINY_B, weights, sequences, rows)
    for tokens, wanted, got in zip(sequences, rows, many):
        want = P.forward(P.TINY_B, weights, tokens)[wanted]
        assert got.shape == want.shape and np.abs(got.astype(np.float64) - want).max() <= 2e-6 * np.abs(want).max()
    block, P.LINEAR_BLOCK = P.LINEAR_BLOCK, 1000  # the product in row blocks of the weight: the same sums
    try:
        assert all(np.array_equal(a, b) for a, b in zip(many, P.forward_many(P.TINY_B, weights, sequences, rows)))
    finally:
        P.LINEAR_BLOCK = block
