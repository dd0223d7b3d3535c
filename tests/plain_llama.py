"""A plain, slow Llama decoder for the tests: whole sequences, no cache, one function per part.

It is written from the formulas of the reference project (vrenken/etalii.dllm); each function cites the file and
lines it restates. It shares no code with the product path: NumPy only, float64 arithmetic, every operation's result
rounded once to float32 exactly where the reference rounds. `tests/golden/` holds outputs of the reference's own
`etalii_dllm.reference.ReferenceTransformer` for two tiny models; `tests/test_plain.py` compares this file with them.

Weights are a dict of Hugging Face tensor names to float32 arrays (`model.embed_tokens.weight`, ...).
"""
from __future__ import annotations

import math
from typing import Mapping, Sequence

import numpy as np

F32 = np.float32
F64 = np.float64


def _round(x) -> np.ndarray:
    """float64 -> float32, round to nearest even (src/etalii_dllm/reference.py:44-46)."""
    return np.asarray(x, dtype=F64).astype(F32)


# ---- parts ----------------------------------------------------------------------------------------------------------

def embedding(table: np.ndarray, tokens: Sequence[int]) -> np.ndarray:
    """Row gather, no scaling for Llama (src/etalii_dllm/transformer.py:659-663); ids out of range are an error
    (transformer.py:668-669)."""
    ids = np.asarray(tokens, dtype=np.int64)
    if ids.size and (ids.min() < 0 or ids.max() >= table.shape[0]):
        raise ValueError("token id out of range")
    return np.asarray(table, dtype=F32)[ids]


LINEAR_BLOCK = 1 << 25
"""`linear` widens at most this many weights to double at a time (a head of 128,256 x 4,096 would otherwise need
4 GB for its double copy); the blocks are whole rows of the weight, so every output is the same sum either way."""


def linear(x: np.ndarray, weight: np.ndarray) -> np.ndarray:
    """out[r, n] = sum_k x[r, k] w[n, k] in double, rounded once (src/etalii_dllm/reference.py:322-335,
    cpp/include/dllm/nn.hpp:28-50)."""
    xd = np.asarray(x, F32).astype(F64)
    weight = np.asarray(weight, F32)
    if weight.size <= LINEAR_BLOCK:
        return _round(xd @ weight.astype(F64).T)
    rows = max(1, LINEAR_BLOCK // weight.shape[1])
    out = np.empty((xd.shape[0], weight.shape[0]), dtype=F32)
    for begin in range(0, weight.shape[0], rows):
        out[:, begin:begin + rows] = _round(xd @ weight[begin:begin + rows].astype(F64).T)
    return out


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """inv = 1/sqrt(sum x^2 / dim + eps); out = x * inv * w, rounded once (src/etalii_dllm/reference.py:389-402,
    cpp/include/dllm/nn.hpp:391-408)."""
    xd = np.asarray(x, F32).astype(F64)
    total = (xd * xd).sum(axis=-1, keepdims=True)
    inverse = 1.0 / np.sqrt(total / float(xd.shape[-1]) + eps)
    return _round(xd * inverse * np.asarray(weight, F32).astype(F64))


def rope_inv_freq(head_dim: int, theta: float, scaling: Mapping | None = None) -> np.ndarray:
    """exp(-(2i/d) log theta) in double, then the llama3 rule (src/etalii_dllm/reference.py:449-476,
    src/etalii_dllm/numerics.py:267-311)."""
    log_theta = math.log(float(theta))
    freqs = [math.exp(-(2 * i / head_dim) * log_theta) for i in range(head_dim // 2)]
    kind = "default" if not scaling else str(scaling.get("rope_type", scaling.get("type", "default")))
    if kind == "llama3":
        factor = float(scaling["factor"])
        low = float(scaling.get("low_freq_factor", 1.0))
        high = float(scaling.get("high_freq_factor", 4.0))
        original = float(scaling.get("original_max_position_embeddings", 8192))
        scaled = []
        for f in freqs:
            wavelen = 2 * math.pi / f
            if wavelen < original / high:
                scaled.append(f)
            elif wavelen > original / low:
                scaled.append(f / factor)
            else:
                smooth = (original / wavelen - low) / (high - low)
                scaled.append((1 - smooth) * f / factor + smooth * f)
        freqs = scaled
    elif kind == "linear":
        freqs = [f / float(scaling["factor"]) for f in freqs]
    elif kind != "default":
        raise ValueError(f"unsupported rope scaling {kind!r}")
    return np.array(freqs, dtype=F64)


def rope(x: np.ndarray, positions: np.ndarray, inv_freq: np.ndarray) -> np.ndarray:
    """Rotate pairs (i, i + d/2) of x[tokens, heads, d] by position * inv_freq[i]; a cos - b sin and a sin + b cos in
    double, rounded once (src/etalii_dllm/reference.py:500-515, cpp/include/dllm/nn.hpp:501-530)."""
    values = np.asarray(x, F32)
    half = inv_freq.shape[0]
    angles = np.asarray(positions, np.int64).astype(F64)[:, None] * inv_freq[None, :]
    c, s = np.cos(angles)[:, None, :], np.sin(angles)[:, None, :]
    a = values[:, :, :half].astype(F64)
    b = values[:, :, half : 2 * half].astype(F64)
    out = values.copy()
    out[:, :, :half] = _round(a * c - b * s)
    out[:, :, half : 2 * half] = _round(a * s + b * c)
    return out


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window: int | None = None) -> np.ndarray:
    """Causal grouped-query attention of a whole sequence: query t, head h reads kv head h // (heads/kv_heads) and
    keys 0..t (the last `window` of them when a window is set); scores (q.k)*scale, p = exp(s - max), out =
    (sum p v) * (1 / sum p), rounded once (src/etalii_dllm/reference.py:518-569,
    cpp/include/dllm/nn.hpp:535-569, 733-796)."""
    qv, kv, vv = (np.asarray(a, F32).astype(F64) for a in (q, k, v))
    q_len, q_heads, _ = qv.shape
    group = q_heads // kv.shape[1]
    out = np.zeros((q_len, q_heads, vv.shape[2]), dtype=F32)
    for t in range(q_len):
        end = t + 1
        first = end - window if window and end > window else 0
        for h in range(q_heads):
            g = h // group
            scores = (kv[first:end, g, :] @ qv[t, h]) * scale
            p = np.exp(scores - scores.max())
            out[t, h] = _round((p @ vv[first:end, g, :]) * (1.0 / p.sum()))
    return out


def attention_by_matrices(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float,
                          window: int | None = None) -> np.ndarray:
    """The same function as `attention`, a head at a time instead of a query at a time: all scores of a head as one
    matrix in double, keys outside [t - window + 1, t] masked, row-wise exp(s - max), (p v) * (1 / sum p), rounded
    once. For the tests at real sizes, where the loop over queries would take minutes; `tests/test_plain.py` holds
    it to `attention` (same formulas: src/etalii_dllm/reference.py:518-569)."""
    qv, kv, vv = (np.asarray(a, F32).astype(F64) for a in (q, k, v))
    q_len, q_heads, _ = qv.shape
    group = q_heads // kv.shape[1]
    out = np.zeros((q_len, q_heads, vv.shape[2]), dtype=F32)
    t = np.arange(q_len)
    visible = t[None, :] <= t[:, None]
    if window:
        visible &= t[None, :] > t[:, None] - window
    for h in range(q_heads):
        g = h // group
        scores = (qv[:, h, :] @ kv[:, g, :].T) * scale
        scores[~visible] = -np.inf
        p = np.exp(scores - scores.max(axis=1, keepdims=True))
        out[:, h, :] = _round((p @ vv[:, g, :]) * (1.0 / p.sum(axis=1, keepdims=True)))
    return out


def sigmoid(x: np.ndarray) -> np.ndarray:
    """1/(1+e^-x) for x >= 0, else e^x/(1+e^x) (src/etalii_dllm/reference.py:218-225)."""
    x = np.asarray(x, F64)
    with np.errstate(all="ignore"):
        positive = 1.0 / (1.0 + np.exp(-x))
        e = np.exp(x)
        negative = e / (1.0 + e)
    return np.where(x >= 0, positive, negative)


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """silu(gate) rounded to float32, then times up in float32 (src/etalii_dllm/reference.py:426-442,
    cpp/include/dllm/nn.hpp:467-470, 489-492)."""
    g = np.asarray(gate, F32).astype(F64)
    return _round(g * sigmoid(g)) * np.asarray(up, F32)


def feed_forward(h: np.ndarray, gate_w: np.ndarray, up_w: np.ndarray, down_w: np.ndarray) -> np.ndarray:
    """down(swiglu(gate(h), up(h))) (src/etalii_dllm/transformer.py:548-553)."""
    return linear(swiglu(linear(h, gate_w), linear(h, up_w)), down_w)


# ---- whole model ----------------------------------------------------------------------------------------------------

def forward(config: Mapping, weights: Mapping[str, np.ndarray], tokens: Sequence[int],
            rows: Sequence[int] | None = None) -> np.ndarray:
    """Logits [len(tokens), vocab] of one whole sequence from position 0: embedding, then per layer RMSNorm, q/k/v,
    RoPE, attention, o, float32 residual add, RMSNorm, SwiGLU feed-forward, float32 residual add; final RMSNorm and
    the (tied or own) head (src/etalii_dllm/reference.py:1231-1290, src/etalii_dllm/transformer.py:493-562).
    With `rows`, only the logits at those positions, [len(rows), vocab].

    `config` is the model's config.json as a dict (Hugging Face keys)."""
    return forward_many(config, weights, [tokens], None if rows is None else [rows], attention)[0]


def forward_many(config: Mapping, weights: Mapping[str, np.ndarray], sequences: Sequence[Sequence[int]],
                 rows: Sequence[Sequence[int]] | None = None, attend=attention_by_matrices) -> list[np.ndarray]:
    """`forward` for several whole sequences at once, for the tests at real sizes: the tokens of all sequences are
    stacked for everything that works on a token alone (embedding, norms, products, rotation by each token's own
    position, SwiGLU, residual adds: a row's result does not depend on the other rows), attention runs sequence by
    sequence. Every weight is widened to double once per call instead of once per sequence. Returns each
    sequence's logits at its `rows` (default: all positions)."""
    heads = int(config["num_attention_heads"])
    kv_heads = int(config.get("num_key_value_heads") or heads)
    hidden = int(config["hidden_size"])
    head_dim = int(config.get("head_dim") or hidden // heads)
    eps = float(config.get("rms_norm_eps", 1e-6))
    inv_freq = rope_inv_freq(head_dim, float(config.get("rope_theta", 10000.0)), config.get("rope_scaling"))
    scale = 1.0 / math.sqrt(head_dim)  # src/etalii_dllm/architecture.py:310-312
    counts = [len(tokens) for tokens in sequences]
    bounds = np.concatenate([[0], np.cumsum(counts)])
    count = int(bounds[-1])
    positions = np.concatenate([np.arange(n) for n in counts])
    x = embedding(weights["model.embed_tokens.weight"], [t for tokens in sequences for t in tokens])
    for layer in range(int(config["num_hidden_layers"])):
        p = f"model.layers.{layer}."
        h = rms_norm(x, weights[p + "input_layernorm.weight"], eps)
        q = linear(h, weights[p + "self_attn.q_proj.weight"]).reshape(count, heads, head_dim)
        k = linear(h, weights[p + "self_attn.k_proj.weight"]).reshape(count, kv_heads, head_dim)
        v = linear(h, weights[p + "self_attn.v_proj.weight"]).reshape(count, kv_heads, head_dim)
        q, k = rope(q, positions, inv_freq), rope(k, positions, inv_freq)
        attended = np.concatenate([attend(q[a:b], k[a:b], v[a:b], scale) for a, b in zip(bounds[:-1], bounds[1:])])
        x = x + linear(attended.reshape(count, heads * head_dim), weights[p + "self_attn.o_proj.weight"])
        h = rms_norm(x, weights[p + "post_attention_layernorm.weight"], eps)
        x = x + feed_forward(
            h, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"], weights[p + "mlp.down_proj.weight"]
        )
    if rows is not None:
        x = x[np.concatenate([bounds[i] + np.asarray(r, dtype=np.int64) for i, r in enumerate(rows)]).astype(np.int64)]
        counts = [len(r) for r in rows]
        bounds = np.concatenate([[0], np.cumsum(counts)])
    hidden_rows = rms_norm(x, weights["model.norm.weight"], eps)
    tied = bool(config.get("tie_word_embeddings", False))
    head = weights["model.embed_tokens.weight"] if tied else weights["lm_head.weight"]
    logits = linear(hidden_rows, head)
    return [logits[a:b] for a, b in zip(bounds[:-1], bounds[1:])]


# ---- sampling -------------------------------------------------------------------------------------------------------

_MASK = (1 << 64) - 1


class Random:
    """xoshiro256** seeded through SplitMix64 (cpp/include/dllm/random.hpp:11-55,
    src/etalii_dllm/reference.py:660-694)."""

    def __init__(self, seed: int) -> None:
        state = seed & _MASK
        self.s = []
        for _ in range(4):
            state = (state + 0x9E3779B97F4A7C15) & _MASK
            z = state
            z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
            z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
            self.s.append(z ^ (z >> 31))

    @staticmethod
    def _rotl(x: int, k: int) -> int:
        return ((x << k) | (x >> (64 - k))) & _MASK

    def next_u64(self) -> int:
        s0, s1, s2, s3 = self.s
        result = (self._rotl((s1 * 5) & _MASK, 7) * 9) & _MASK
        t = (s1 << 17) & _MASK
        s2 ^= s0
        s3 ^= s1
        s1 ^= s2
        s0 ^= s3
        s2 ^= t
        s3 = self._rotl(s3, 45)
        self.s = [s0, s1, s2, s3]
        return result

    def next_double(self) -> float:
        """The top 53 bits times 2^-53."""
        return float(self.next_u64() >> 11) * (1.0 / 9007199254740992.0)


def argmax(values: np.ndarray) -> int:
    """The first index of the largest value (src/etalii_dllm/reference.py:272-279)."""
    return int(np.argmax(np.asarray(values)))  # numpy returns the first maximum


def softmax(logits: np.ndarray) -> np.ndarray:
    """exp(l - max) * (1 / total), rounded to float32 (src/etalii_dllm/reference.py:282-286)."""
    values = np.asarray(logits, F32).astype(F64)
    e = np.exp(values - values.max())
    return _round(e * (1.0 / e.sum()))


def sample(logits: np.ndarray, random: Random, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
           min_p: float = 0.0, allowed: Sequence[int] | None = None) -> int:
    """Greedy at temperature 0; else float32 logits / float32 temperature, softmax, candidates ordered by
    (probability descending, id ascending), top-k, top-p (shortest prefix reaching it), min-p, then one
    next_double() scaled by the kept mass picks the first candidate whose running sum exceeds it
    (src/etalii_dllm/reference.py:909-982, src/etalii_dllm/sampling.py:441-500). With `allowed` (ascending ids) the
    choice is made among those tokens only: the same rule on the logits of the subset
    (src/etalii_dllm/sampling.py:400-409)."""
    if allowed is not None:
        ids = [int(i) for i in allowed]
        subset = np.asarray(logits, F32)[ids]
        return ids[sample(subset, random, temperature, top_k, top_p, min_p)]
    if temperature == 0:
        return argmax(logits)
    scaled = np.asarray(logits, F32) / F32(temperature)
    probabilities = softmax(scaled).astype(F64)
    order = sorted(range(len(probabilities)), key=lambda i: (-probabilities[i], i))
    candidates = order[:top_k] if top_k > 0 else order
    if top_p < 1:
        cumulative = 0.0
        for n, i in enumerate(candidates):
            cumulative += probabilities[i]
            if cumulative >= top_p:
                candidates = candidates[: n + 1]
                break
    if min_p > 0:
        floor = min_p * probabilities[candidates[0]]
        keep = len(candidates)
        for n in range(1, len(candidates)):
            if probabilities[candidates[n]] < floor:
                keep = n
                break
        candidates = candidates[:keep]
    total = 0.0
    for i in candidates:
        total += probabilities[i]
    target = random.next_double() * total
    running = 0.0
    for i in candidates:
        running += probabilities[i]
        if target < running:
            return int(i)
    return int(candidates[-1])


def generate(config: Mapping, weights: Mapping[str, np.ndarray], prompt: Sequence[int], max_tokens: int,
             temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, seed: int = 0,
             stop_tokens: Sequence[int] = (), min_tokens: int = 0) -> tuple[list[int], str]:
    """One sequence: forward over the whole context each time (no cache), choose, stop on a stop token (which is not
    part of the output), else append; ends at max_tokens or a full context window
    (src/etalii_dllm/generation.py:277-330, src/etalii_dllm/reference.py:1372-1396). While the output is shorter
    than `min_tokens` the stop tokens are taken out of the choice (src/etalii_dllm/generation.py:316, 373-381)."""
    window = int(config.get("max_position_embeddings", 2048))
    if len(prompt) >= window:
        raise ValueError(f"the prompt has {len(prompt)} tokens; the context window holds {window}")
    random = Random(seed)
    context = list(prompt)
    out: list[int] = []
    finish = "length"
    while len(out) < max_tokens:
        if len(context) >= window:
            break
        logits = forward(config, weights, context)[-1]
        allowed = None
        if len(out) < min_tokens and stop_tokens:
            allowed = [t for t in range(len(logits)) if t not in stop_tokens]
        token = sample(logits, random, temperature, top_k, top_p, min_p, allowed)
        if token in stop_tokens:
            finish = "stop"
            break
        out.append(token)
        context.append(token)
    return out, finish


# ---- helpers for the tests ------------------------------------------------------------------------------------------

TINY_A = {
    "model_type": "llama", "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 2, "hidden_size": 64,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 160, "vocab_size": 256,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 128,
    "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
TINY_B = {
    "model_type": "llama", "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 3, "hidden_size": 144,
    "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 24, "intermediate_size": 384, "vocab_size": 384,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256, "hidden_act": "silu",
    "bos_token_id": 0, "eos_token_id": [3, 5],
}


def tensor_shapes(config: Mapping) -> dict[str, tuple[int, ...]]:
    """Hugging Face tensor names and shapes of a Llama checkpoint (src/etalii_dllm/importing/importer.py:74-113,
    src/etalii_dllm/architecture.py:418-468)."""
    heads = int(config["num_attention_heads"])
    kv_heads = int(config.get("num_key_value_heads") or heads)
    hidden = int(config["hidden_size"])
    head_dim = int(config.get("head_dim") or hidden // heads)
    inter = int(config["intermediate_size"])
    vocab = int(config["vocab_size"])
    shapes: dict[str, tuple[int, ...]] = {"model.embed_tokens.weight": (vocab, hidden)}
    for layer in range(int(config["num_hidden_layers"])):
        p = f"model.layers.{layer}."
        shapes[p + "input_layernorm.weight"] = (hidden,)
        shapes[p + "self_attn.q_proj.weight"] = (heads * head_dim, hidden)
        shapes[p + "self_attn.k_proj.weight"] = (kv_heads * head_dim, hidden)
        shapes[p + "self_attn.v_proj.weight"] = (kv_heads * head_dim, hidden)
        shapes[p + "self_attn.o_proj.weight"] = (hidden, heads * head_dim)
        shapes[p + "post_attention_layernorm.weight"] = (hidden,)
        shapes[p + "mlp.gate_proj.weight"] = (inter, hidden)
        shapes[p + "mlp.up_proj.weight"] = (inter, hidden)
        shapes[p + "mlp.down_proj.weight"] = (hidden, inter)
    shapes["model.norm.weight"] = (hidden,)
    if not config.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (vocab, hidden)
    return shapes


def random_weights(config: Mapping, seed: int, std: float = 0.02, bf16_exact: bool = True) -> dict[str, np.ndarray]:
    """Seeded float32 weights for the tests: N(0, std) matrices, 1 + N(0, 0.01) norm weights. With `bf16_exact` the
    values are rounded to what bfloat16 holds, so that a bfloat16 engine and this float32 model read the same
    numbers (the reference's fixtures do the same, tests/model_fixtures.py:303-308)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        norm = name.endswith("norm.weight")
        values = (rng.standard_normal(shape) * (0.01 if norm else std) + (1.0 if norm else 0.0)).astype(F32)
        if bf16_exact:
            bits = values.view(np.uint32)  # (finite values: the additions below cannot carry out of 32 bits)
            bits = ((bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)) << np.uint32(16)
            values = bits.view(F32).reshape(shape)  # rounded to nearest even on the top 16 bits
        out[name] = values
    return out
