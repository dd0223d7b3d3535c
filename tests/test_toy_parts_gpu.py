"""Parts that no shipped architecture has, defined here and registered from outside the library: a feed-forward that
routes every token to two of its experts, and a position encoding with frequencies and a rotated width of its own.
A toy architecture mixes them with the library's own parts layer by layer; its logits are compared with a plain
whole-sequence computation written here from `plain_llama`'s functions, whole and cut into steps. These toys only
show that the interfaces carry other parts: they are nobody's model."""
import numpy as np
import pytest
import torch

import plain_llama as P
from helpers import host, rel_error

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HIDDEN, VOCAB, EXPERTS, INNER, HEADS, KV_HEADS, HEAD_DIM, ROTATED = 40, 61, 3, 24, 4, 2, 16, 8
EPS = 2e-5


class RoutedExperts:
    """Feed-forward with routing: router logits in float32, the two largest choose the experts, their softmax (over
    the two) weighs the experts' SwiGLU outputs."""

    CAPTURABLE = False  # written with allocating torch ops: the engine then decodes without CUDA graphs

    def __init__(self, hidden_size, intermediate_size, experts):
        self.hidden_size, self.intermediate_size, self.experts = hidden_size, intermediate_size, experts

    @staticmethod
    def parameters(hidden_size, intermediate_size, experts):
        from etalii.dllm_b200.parts import ParamSpec

        return {"router": ParamSpec((experts, hidden_size)),
                "gate": ParamSpec((experts, intermediate_size, hidden_size)),
                "up": ParamSpec((experts, intermediate_size, hidden_size)),
                "down": ParamSpec((experts, hidden_size, intermediate_size))}

    def bind(self, tensors, rt):
        self.w = {k: rt.to_device(v, torch.float32) for k, v in tensors.items()}

    def forward(self, h, residual, batch, rt):
        from etalii.dllm_b200.kernels import ops

        x = h.float()
        logits = x @ self.w["router"].T
        top, chosen = logits.topk(2, dim=-1)
        weight = torch.softmax(top, dim=-1)
        out = torch.zeros_like(x)
        for e in range(self.experts):
            for k in range(2):
                rows = (chosen[:, k] == e).nonzero().flatten()
                if rows.numel():
                    xe = x[rows]
                    act = torch.nn.functional.silu(xe @ self.w["gate"][e].T) * (xe @ self.w["up"][e].T)
                    out[rows] += weight[rows, k, None] * (act @ self.w["down"][e].T)
        ops.add_residual(residual, out.contiguous())


def toy_frequencies():
    return np.array([0.9 / (1 + i * i) for i in range(ROTATED // 2)])  # neither geometric nor the whole head


class QuadraticRotary:
    """Another position encoding of the same role: it gives the mixer a table [positions, rotated / 2, (cos, sin)]
    and the number of rotated dimensions, here with frequencies 0.9 / (1 + i^2) over the first 8 of 16 dimensions."""

    def __init__(self, rotary_dim):
        self.rotary_dim = rotary_dim
        self._table = None

    @staticmethod
    def parameters(**_):
        return {}

    def bind(self, tensors, rt):
        angles = torch.arange(rt.max_length, dtype=torch.float64)[:, None] * torch.tensor(toy_frequencies())[None, :]
        self._table = torch.stack([angles.cos(), angles.sin()], dim=-1).float().contiguous().to(rt.device)

    def table(self):
        return self._table


class ToyConfig:
    model_type = "toy_routed"

    @classmethod
    def from_hf(cls, config, generation=None):
        return cls()


def toy_spec(config):
    from etalii.dllm_b200.parts import LayerSpec, ModelSpec, PartSpec

    norm = lambda name: PartSpec("rmsnorm", {"hidden_size": HIDDEN, "eps": EPS}, {"weight": name})  # noqa: E731

    def attention(i, position, window):
        return PartSpec("attention", {"hidden_size": HIDDEN, "num_heads": HEADS, "num_kv_heads": KV_HEADS,
                                      "head_dim": HEAD_DIM, "scale": 0.3, "window": window, "position": position},
                        {k: f"l{i}.{k}" for k in "qkvo"})

    routed = PartSpec("routed_experts", {"hidden_size": HIDDEN, "intermediate_size": INNER, "experts": EXPERTS},
                      {k: f"l0.{k}" for k in ("router", "gate", "up", "down")})
    dense = PartSpec("swiglu", {"hidden_size": HIDDEN, "intermediate_size": 56},
                     {k: f"l1.{k}" for k in ("gate", "up", "down")})
    layers = (
        LayerSpec(attention(0, PartSpec("quadratic_rotary", {"rotary_dim": ROTATED}), None), routed, norm("l0.n1"),
                  norm("l0.n2")),
        LayerSpec(attention(1, PartSpec("rotary", {"head_dim": HEAD_DIM, "theta": 300.0, "scaling": None}), 7), dense,
                  norm("l1.n1"), norm("l1.n2")),
    )
    return ModelSpec(VOCAB, HIDDEN, 128,
                     PartSpec("token_embedding", {"vocab_size": VOCAB, "hidden_size": HIDDEN}, {"weight": "emb"}),
                     layers, norm("final"),
                     PartSpec("linear", {"vocab_size": VOCAB, "hidden_size": HIDDEN}, {"weight": "head"}))


def plain_forward(w, tokens):
    """Whole sequence, no cache, from the plain implementation's functions; also the smallest gap between the second
    and third router logit (a routing decision closer than rounding would make the comparison meaningless)."""
    n = len(tokens)
    x = P.embedding(w["emb"], tokens)
    margin = np.inf
    for i, (freqs, window) in enumerate(((toy_frequencies(), None), (P.rope_inv_freq(HEAD_DIM, 300.0), 7))):
        h = P.rms_norm(x, w[f"l{i}.n1"], EPS)
        q = P.rope(P.linear(h, w[f"l{i}.q"]).reshape(n, HEADS, HEAD_DIM), np.arange(n), freqs)
        k = P.rope(P.linear(h, w[f"l{i}.k"]).reshape(n, KV_HEADS, HEAD_DIM), np.arange(n), freqs)
        v = P.linear(h, w[f"l{i}.v"]).reshape(n, KV_HEADS, HEAD_DIM)
        x = x + P.linear(P.attention(q, k, v, 0.3, window).reshape(n, -1), w[f"l{i}.o"])
        h = P.rms_norm(x, w[f"l{i}.n2"], EPS)
        if i == 1:
            x = x + P.feed_forward(h, w["l1.gate"], w["l1.up"], w["l1.down"])
            continue
        logits = h.astype(np.float64) @ w["l0.router"].astype(np.float64).T
        out = np.zeros((n, HIDDEN))
        for t in range(n):
            order = np.argsort(-logits[t])
            margin = min(margin, logits[t, order[1]] - logits[t, order[2]])
            top = logits[t, order[:2]]
            weight = np.exp(top - top.max()) / np.exp(top - top.max()).sum()
            for e, we in zip(order[:2], weight):
                out[t] += we * P.feed_forward(h[t:t + 1], w["l0.gate"][e], w["l0.up"][e], w["l0.down"][e])[0]
        x = x + out.astype(np.float32)
    return P.linear(P.rms_norm(x, w["final"], EPS), w["head"]), margin


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 3e-2)])
def test_routed_feed_forward_and_another_position_encoding(dtype, tol):
    from etalii.dllm_b200.config.registry import register_architecture, unregister_architecture
    from etalii.dllm_b200.engine.engine import Engine
    from etalii.dllm_b200.parts import register_part, unregister_part
    from etalii.dllm_b200.weights.loader import expected_tensors

    register_part("feed_forward", "routed_experts", RoutedExperts)
    register_part("position", "quadratic_rotary", QuadraticRotary)
    register_architecture("toy_routed", ToyConfig, toy_spec)
    try:
        g = torch.Generator().manual_seed(11)
        tensors = {}
        for name, p in expected_tensors(toy_spec(ToyConfig())).items():
            scale = 1.5 if name == "l0.router" else 0.1  # clear routing decisions, moderate activations
            tensors[name] = (torch.randn(p.shape, generator=g) * scale + (1 if p.init == "ones" else 0)).to(torch.bfloat16)
        w = {k: v.float().numpy() for k, v in tensors.items()}
        engine = Engine(ToyConfig(), tensors, dtype=dtype, max_tokens=64 * 8)
        assert engine.cuda_graphs is False  # the feed-forward said so
        prompts = [[int(t) for t in torch.randint(0, VOCAB, (n,), generator=g)] for n in (23, 9)]
        want = []
        for prompt in prompts:
            logits, margin = plain_forward(w, prompt)
            assert margin > 0.05, "the seed gives a routing decision too close to call; choose another"
            want.append(logits)
        scale = max(float(np.abs(x).max()) for x in want)
        # whole, both requests in one batch
        slots = engine.open(2)
        whole = host(engine.step(slots, prompts, [list(range(len(p))) for p in prompts]))
        engine.close(slots)
        assert np.abs(whole[:23] - want[0]).max() <= tol * scale and np.abs(whole[23:] - want[1]).max() <= tol * scale
        # cut: the first tokens in one step, the others one by one (the shorter request ends earlier)
        slots = engine.open(2)
        head = host(engine.step(slots, [prompts[0][:5], prompts[1][:5]], [[4], [4]]))
        assert np.abs(head[0] - want[0][4]).max() <= tol * scale and np.abs(head[1] - want[1][4]).max() <= tol * scale
        for index in range(5, 23):
            live = [0, 1] if index < 9 else [0]
            got = host(engine.step([slots[i] for i in live], [[prompts[i][index]] for i in live]))
            for row, i in enumerate(live):
                assert np.abs(got[row] - want[i][index]).max() <= tol * scale, (index, i)
            if index == 8:
                engine.close([slots[1]])
        engine.close([slots[0]])
        assert rel_error(whole[:23], want[0]) <= tol
    finally:
        unregister_part("feed_forward", "routed_experts")
        unregister_part("position", "quadratic_rotary")
        unregister_architecture("toy_routed")


class SandwichBlock:
    """Another arrangement, defined here: a third norm behind the mixer. x += post_norm(mixer(norm(x)));
    x += feed_forward(norm(x)). It names the parts it takes (and their roles) itself; the layer's spec gives them by
    those names, and no file of the library knows this arrangement."""

    PARTS = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "mixer_post_norm": "norm",
             "feed_forward_norm": "norm"}

    def __init__(self, mixer, feed_forward, mixer_norm, mixer_post_norm, feed_forward_norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.mixer_post_norm, self.feed_forward_norm = mixer_norm, mixer_post_norm, feed_forward_norm
        self.parts = dict(mixer=mixer, feed_forward=feed_forward, mixer_norm=mixer_norm,
                          mixer_post_norm=mixer_post_norm, feed_forward_norm=feed_forward_norm)

    def forward(self, x, batch, cache, rt, write_cache=True):
        from etalii.dllm_b200.kernels import ops

        mixed = torch.zeros_like(x)  # the mixer adds its output into what it is given as the residual
        self.mixer.forward(self.mixer_norm.forward(x, rt), mixed, batch, cache, rt, write_cache)
        ops.add_residual(x, self.mixer_post_norm.forward(mixed, rt, name="post_normed"))
        self.feed_forward.forward(self.feed_forward_norm.forward(x, rt), x, batch, rt)


class SandwichConfig:
    model_type = "toy_sandwich"

    @classmethod
    def from_hf(cls, config, generation=None):
        return cls()


def sandwich_spec(config):
    from etalii.dllm_b200.parts import LayerSpec, ModelSpec, PartSpec

    norm = lambda name, eps=EPS: PartSpec("rmsnorm", {"hidden_size": HIDDEN, "eps": eps}, {"weight": name})  # noqa: E731
    layers = []
    for i in range(2):
        parts = {
            "mixer": PartSpec("attention", {"hidden_size": HIDDEN, "num_heads": HEADS, "num_kv_heads": KV_HEADS,
                                            "head_dim": HEAD_DIM, "scale": 0.3, "window": None,
                                            "position": PartSpec("rotary", {"head_dim": HEAD_DIM, "theta": 300.0,
                                                                            "scaling": None})},
                              {k: f"l{i}.{k}" for k in "qkvo"}),
            "feed_forward": PartSpec("swiglu", {"hidden_size": HIDDEN, "intermediate_size": 56},
                                     {k: f"l{i}.{k}" for k in ("gate", "up", "down")}),
            "mixer_norm": norm(f"l{i}.n1"), "mixer_post_norm": norm(f"l{i}.n_post", 1e-3),
            "feed_forward_norm": norm(f"l{i}.n2"),
        }
        # layer 1 is the library's own arrangement: the two kinds of block stand side by side in one model
        if i == 1:
            del parts["mixer_post_norm"]
        layers.append(LayerSpec(block="sandwich" if i == 0 else "pre_norm", parts=parts))
    return ModelSpec(VOCAB, HIDDEN, 128,
                     PartSpec("token_embedding", {"vocab_size": VOCAB, "hidden_size": HIDDEN}, {"weight": "emb"}),
                     tuple(layers), norm("final"),
                     PartSpec("linear", {"vocab_size": VOCAB, "hidden_size": HIDDEN}, {"weight": "head"}))


def sandwich_plain(w, tokens):
    n = len(tokens)
    freqs = P.rope_inv_freq(HEAD_DIM, 300.0)
    x = P.embedding(w["emb"], tokens)
    for i in range(2):
        h = P.rms_norm(x, w[f"l{i}.n1"], EPS)
        q = P.rope(P.linear(h, w[f"l{i}.q"]).reshape(n, HEADS, HEAD_DIM), np.arange(n), freqs)
        k = P.rope(P.linear(h, w[f"l{i}.k"]).reshape(n, KV_HEADS, HEAD_DIM), np.arange(n), freqs)
        v = P.linear(h, w[f"l{i}.v"]).reshape(n, KV_HEADS, HEAD_DIM)
        mixed = P.linear(P.attention(q, k, v, 0.3).reshape(n, -1), w[f"l{i}.o"])
        x = x + (P.rms_norm(mixed, w["l0.n_post"], 1e-3) if i == 0 else mixed)
        x = x + P.feed_forward(P.rms_norm(x, w[f"l{i}.n2"], EPS), w[f"l{i}.gate"], w[f"l{i}.up"], w[f"l{i}.down"])
    return P.linear(P.rms_norm(x, w["final"], EPS), w["head"])


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 3e-2)])
def test_a_block_arrangement_with_a_third_norm_registered_from_outside(dtype, tol):
    from etalii.dllm_b200.config.registry import register_architecture, unregister_architecture
    from etalii.dllm_b200.engine.engine import Engine
    from etalii.dllm_b200.parts import LayerSpec, register_part, unregister_part
    from etalii.dllm_b200.weights.loader import expected_tensors

    register_part("block", "sandwich", SandwichBlock)
    register_architecture("toy_sandwich", SandwichConfig, sandwich_spec)
    try:
        spec = sandwich_spec(SandwichConfig())
        assert [path for path, role, _ in spec.part_specs() if role == "norm" and path.startswith("layers.0")] == \
            ["layers.0.mixer_norm", "layers.0.mixer_post_norm", "layers.0.feed_forward_norm"]
        with pytest.raises(ValueError, match="takes the parts"):  # a layer must give exactly what its block names
            LayerSpec(block="pre_norm", parts=spec.layers[0].parts).roles()
        g = torch.Generator().manual_seed(17)
        tensors = {name: (torch.randn(p.shape, generator=g) * 0.1 + (1 if p.init == "ones" else 0)).to(torch.bfloat16)
                   for name, p in expected_tensors(spec).items()}
        assert "l0.n_post" in tensors and "l1.n_post" not in tensors
        w = {k: v.float().numpy() for k, v in tensors.items()}
        engine = Engine(SandwichConfig(), tensors, dtype=dtype, max_tokens=64 * 4, cuda_graphs=False)
        prompts = [[int(t) for t in torch.randint(0, VOCAB, (n,), generator=g)] for n in (19, 6)]
        want = [sandwich_plain(w, p) for p in prompts]
        slots = engine.open(2)
        whole = host(engine.step(slots, prompts, [list(range(len(p))) for p in prompts]))
        engine.close(slots)
        assert rel_error(whole[:19], want[0]) <= tol and rel_error(whole[19:], want[1]) <= tol
        slots = engine.open(2)  # cut: a few tokens, then one by one
        engine.step(slots, [prompts[0][:4], prompts[1][:4]], [[], []])
        for index in range(4, 6):
            got = host(engine.step(slots, [[prompts[0][index]], [prompts[1][index]]]))
            assert rel_error(got[0], want[0][index]) <= tol and rel_error(got[1], want[1][index]) <= tol
        engine.close(slots)
    finally:
        unregister_part("block", "sandwich")
        unregister_architecture("toy_sandwich")
