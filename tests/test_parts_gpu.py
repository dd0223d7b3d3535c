"""Each part of a layer alone against the plain implementation's function for it, and a toy mixer with state of its
own that is registered, built and stepped without a change to the library's files."""
import math

import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import host, rel_error

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _runtime(dtype, max_length=256):
    from etalii.dllm_b200.engine.runtime import Runtime

    return Runtime(DEV, dtype, max_length)


def _batch(cache, lengths):
    from etalii.dllm_b200.engine.batch import BatchBuffers

    slots = cache.acquire(len(lengths))
    for slot, n in zip(slots, lengths):
        cache.reserve(slot, n)
    cache.sync_tables()
    return BatchBuffers(DEV).fill(slots, [[0] * n for n in lengths], [0] * len(lengths), [[] for _ in lengths])


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 8e-3)])
def test_rmsnorm_part(dtype, tol):
    from etalii.dllm_b200.parts import PartSpec, build_part

    rt = _runtime(dtype)
    norm = build_part("norm", PartSpec("rmsnorm", {"hidden_size": 72, "eps": 3e-4}))
    w = torch.randn(72) * 0.1 + 1
    norm.bind({"weight": w}, rt)
    x = torch.randn(11, 72, device=DEV) * 2
    got = host(norm.forward(x, rt))
    assert rel_error(got, P.rms_norm(x.cpu().numpy(), w.numpy(), 3e-4)) <= tol


def test_rotary_part_matches_plain_frequencies():
    from etalii.dllm_b200.parts import PartSpec, build_part

    rt = _runtime(torch.float32, max_length=300)
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 64}
    rotary = build_part("position", PartSpec("rotary", {"head_dim": 24, "theta": 5e5, "scaling": scaling}))
    rotary.bind({}, rt)
    table = rotary.table().cpu().double().numpy()
    angles = np.arange(300)[:, None] * P.rope_inv_freq(24, 5e5, scaling)[None, :]
    assert table.shape == (300, 12, 2)
    assert np.abs(table[..., 0] - np.cos(angles)).max() < 1e-7 and np.abs(table[..., 1] - np.sin(angles)).max() < 1e-7


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("heads,kv_heads,head_dim,hidden", [(4, 2, 16, 72), (6, 3, 24, 40)])
def test_attention_part(dtype, tol, heads, kv_heads, head_dim, hidden):
    """Whole sequences through the attention part (projection, rotation, cache, attention, output projection)."""
    from etalii.dllm_b200.cache.paged import PagedCache
    from etalii.dllm_b200.parts import PartSpec, build_part

    rt = _runtime(dtype)
    spec = PartSpec("attention", {
        "hidden_size": hidden, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": head_dim,
        "scale": 1 / math.sqrt(head_dim), "window": None,
        "position": PartSpec("rotary", {"head_dim": head_dim, "theta": 1e4, "scaling": None})})
    part = build_part("mixer", spec)
    g = torch.Generator().manual_seed(1)
    weights = {n: (torch.randn(s, generator=g) * 0.2).to(torch.bfloat16) for n, s in
               {"q": (heads * head_dim, hidden), "k": (kv_heads * head_dim, hidden),
                "v": (kv_heads * head_dim, hidden), "o": (hidden, heads * head_dim)}.items()}
    part.bind(weights, rt)
    cache = PagedCache([part.cache_need()], 64 * 8, 256, dtype=dtype, device=DEV)
    lengths = [70, 3, 17]
    batch = _batch(cache, lengths)
    h = (torch.randn(sum(lengths), hidden, generator=g)).to(dtype).to(DEV)
    residual = torch.zeros(sum(lengths), hidden, device=DEV)
    part.forward(h, residual, batch, cache.kv_view(0), rt)
    w = {k: v.float().numpy() for k, v in weights.items()}
    inv_freq = P.rope_inv_freq(head_dim, 1e4)
    offset = 0
    for n in lengths:
        x = h[offset:offset + n].float().cpu().numpy()
        q = P.rope(P.linear(x, w["q"]).reshape(n, heads, head_dim), np.arange(n), inv_freq)
        k = P.rope(P.linear(x, w["k"]).reshape(n, kv_heads, head_dim), np.arange(n), inv_freq)
        v = P.linear(x, w["v"]).reshape(n, kv_heads, head_dim)
        want = P.linear(P.attention(q, k, v, 1 / math.sqrt(head_dim)).reshape(n, -1), w["o"])
        assert rel_error(host(residual[offset:offset + n]), want) <= tol
        offset += n


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("rows", [3, 40])
def test_swiglu_part(dtype, tol, rows):
    from etalii.dllm_b200.parts import PartSpec, build_part

    rt = _runtime(dtype)
    part = build_part("feed_forward", PartSpec("swiglu", {"hidden_size": 72, "intermediate_size": 200}))
    g = torch.Generator().manual_seed(2)
    weights = {"gate": torch.randn(200, 72, generator=g) * 0.3, "up": torch.randn(200, 72, generator=g) * 0.3,
               "down": torch.randn(72, 200, generator=g) * 0.3}
    weights = {k: v.to(torch.bfloat16) for k, v in weights.items()}
    part.bind(weights, rt)
    h = torch.randn(rows, 72, generator=g).to(dtype).to(DEV)
    residual = torch.ones(rows, 72, device=DEV)
    part.forward(h, residual, None, rt)
    want = 1 + P.feed_forward(h.float().cpu().numpy(), *(weights[k].float().numpy() for k in ("gate", "up", "down")))
    assert rel_error(host(residual), want) <= tol


# ---- a toy architecture defined here: a mixer with fixed-size state of its own ------------------------------------

class DecayMixer:
    """state <- decay * state + h (per sequence, token by token); output = state @ w^T. State: [hidden] per slot."""

    CAPTURABLE = False  # written with allocating torch ops: the engine then decodes without CUDA graphs

    def __init__(self, hidden_size, decay):
        self.hidden_size, self.decay = hidden_size, decay

    @staticmethod
    def parameters(hidden_size, decay):
        from etalii.dllm_b200.parts import ParamSpec

        return {"w": ParamSpec((hidden_size, hidden_size))}

    def cache_need(self):
        from etalii.dllm_b200.cache.paged import CacheNeed

        return CacheNeed("state", state_shape=(self.hidden_size,))

    def bind(self, tensors, rt):
        self.w = rt.to_device(tensors["w"], torch.float32)

    def forward(self, h, residual, batch, state, rt, write_cache=True):
        from etalii.dllm_b200.kernels import ops

        out = torch.empty((batch.n_tokens, self.hidden_size), dtype=torch.float32, device=h.device)
        offset = 0
        for slot, n in zip(batch.h_slots, batch.h_new):
            s = state[slot]
            for t in range(offset, offset + n):
                s = self.decay * s + h[t].float()
                out[t] = s
            if write_cache:
                state[slot] = s
            offset += n
        ops.add_residual(residual, (out @ self.w.T).contiguous())


def _toy_spec(config):
    from etalii.dllm_b200.parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    hidden, vocab = config.hidden, config.vocab
    norm = lambda name: PartSpec("rmsnorm", {"hidden_size": hidden, "eps": 1e-5}, {"weight": name})  # noqa: E731
    attention = PartSpec("attention", {
        "hidden_size": hidden, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16, "scale": 0.25, "window": 5,
        "position": None}, {k: f"l1.{k}" for k in "qkvo"})
    ffn = lambda i: PartSpec("swiglu", {"hidden_size": hidden, "intermediate_size": 48},  # noqa: E731
                             {k: f"l{i}.{k}" for k in ("gate", "up", "down")})
    layers = (
        LayerSpec(PartSpec("decay", {"hidden_size": hidden, "decay": 0.5}, {"w": "l0.w"}), ffn(0), norm("l0.n1"),
                  norm("l0.n2")),
        LayerSpec(attention, ffn(1), norm("l1.n1"), norm("l1.n2")),
    )
    # layer 0 runs twice (a second state of its own); layer 1 runs twice, the second time reading the first's cache
    schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(0, 2), ScheduleEntry(1, 1, writes_cache=False))
    return ModelSpec(vocab, hidden, 128, PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": hidden},
                                                   {"weight": "emb"}),
                     layers, norm("final"), PartSpec("linear", {"vocab_size": vocab, "hidden_size": hidden},
                                                     {"weight": "emb"}), schedule=schedule)


class ToyConfig:
    model_type = "toy_decay"
    hidden, vocab = 32, 50

    @classmethod
    def from_hf(cls, config, generation=None):
        return cls()


def _toy_plain(w, tokens):
    """The toy architecture as a plain whole-sequence computation: the decay layer is the recurrence
    state_t = 0.5 state_(t-1) + h_t from a zero state, output state_t w^T; the schedule runs layer 0, layer 1,
    layer 0 again (a second state) and layer 1 again with the keys and values of its first run."""
    import plain_llama as P

    n = len(tokens)
    x = P.embedding(w["emb"], tokens)
    kept = {}
    for layer, reads_cache in ((0, False), (1, False), (0, False), (1, True)):
        h = P.rms_norm(x, w[f"l{layer}.n1"], 1e-5)
        if layer == 0:
            state, rows = np.zeros(h.shape[1]), []
            for t in range(n):
                state = 0.5 * state + h[t].astype(np.float64)
                rows.append(state.copy())
            x = x + P.linear(np.asarray(rows, dtype=np.float32), w["l0.w"])
        else:
            q = P.linear(h, w["l1.q"]).reshape(n, 2, 16)
            if not reads_cache:
                kept["k"] = P.linear(h, w["l1.k"]).reshape(n, 1, 16)
                kept["v"] = P.linear(h, w["l1.v"]).reshape(n, 1, 16)
            x = x + P.linear(P.attention(q, kept["k"], kept["v"], 0.25, window=5).reshape(n, -1), w["l1.o"])
        h = P.rms_norm(x, w[f"l{layer}.n2"], 1e-5)
        x = x + P.feed_forward(h, w[f"l{layer}.gate"], w[f"l{layer}.up"], w[f"l{layer}.down"])
    return P.linear(P.rms_norm(x, w["final"], 1e-5), w["emb"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_with_a_stateful_mixer(dtype):
    from etalii.dllm_b200.config.registry import register_architecture, unregister_architecture
    from etalii.dllm_b200.engine.engine import Engine
    from etalii.dllm_b200.parts import register_part, unregister_part
    from etalii.dllm_b200.weights.loader import expected_tensors

    register_part("mixer", "decay", DecayMixer)
    register_architecture("toy_decay", ToyConfig, _toy_spec)
    try:
        spec = _toy_spec(ToyConfig())
        g = torch.Generator().manual_seed(3)
        tensors = {name: ((torch.randn(p.shape, generator=g) * 0.2 + (1 if p.init == "ones" else 0))
                          .to(torch.bfloat16)) for name, p in expected_tensors(spec).items()}
        engine = Engine(ToyConfig(), tensors, dtype=dtype, max_tokens=64 * 8)
        assert engine.cuda_graphs is False  # the mixer said so
        groups = engine.cache.groups()
        assert len(groups) == 1 and groups[0][1] == [1] and groups[0][0].window == 5  # one kv entry, shared
        assert engine.cache.state(0).shape == (engine.cache.n_slots, 32) and engine.cache.state(2) is not None
        tokens = [[1, 2, 3, 4, 5, 6, 7, 8, 9], [10, 11, 12]]
        slots = engine.open(2)
        whole = host(engine.step(slots, tokens, [list(range(9)), list(range(3))]))
        engine.close(slots)
        # against the plain recurrence, not only against itself
        w = {k: v.float().numpy() for k, v in tensors.items()}
        plain_tol = 5e-5 if dtype == "float32" else 3e-2
        assert rel_error(whole[:9], _toy_plain(w, tokens[0])) <= plain_tol
        assert rel_error(whole[9:], _toy_plain(w, tokens[1])) <= plain_tol
        slots = engine.open(2)  # the same slots again: the state must start from zero
        first = host(engine.step(slots, [tokens[0][:4], tokens[1][:1]], [list(range(4)), [0]]))
        rest = []
        for index in range(4, 9):
            live = [0, 1] if index - 3 < 3 else [0]
            got = host(engine.step([slots[i] for i in live],
                                   [[tokens[0][index]]] + ([[tokens[1][index - 3]]] if 1 in live else [])))
            rest.append(got)
        engine.close(slots)
        tol = 1e-5 if dtype == "float32" else 3e-2
        assert rel_error(first[:4], whole[:4]) <= tol and rel_error(first[4], whole[9]) <= tol
        for index, got in zip(range(4, 9), rest):
            assert rel_error(got[0], whole[index]) <= tol, index
            if got.shape[0] > 1:
                assert rel_error(got[1], whole[9 + index - 3]) <= tol, index
        results = engine.generate([[1, 2, 3], [4]], 5)
        assert all(len(r.tokens) == 5 for r in results)
    finally:
        unregister_part("mixer", "decay")
        unregister_architecture("toy_decay")
