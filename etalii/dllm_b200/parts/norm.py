"""RMSNorm: out = x / sqrt(mean(x^2) + eps) * weight, computed in float32 from the float32 residual stream
(reference: cpp/include/dllm/nn.hpp:391-408; plain weight, no 1 + w)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .registry import register_part
from .spec import ParamSpec


class NormedInput:
    """A norm's output that has not been computed yet: the float32 rows and the norm's weight and eps. A consumer
    whose kernel can apply the norm on the way in (the decode-sized products) takes it as it is; anyone else calls
    `tensor()` and gets the normed activations, computed once."""

    def __init__(self, norm: "RMSNorm", x: torch.Tensor, rt) -> None:
        self.norm, self.x, self.rt = norm, x, rt
        self.weight, self.eps = norm.weight, norm.eps
        self.shape = x.shape
        self._tensor = None

    def tensor(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = self.norm.forward(self.x, self.rt)
        return self._tensor


class RMSNorm:
    def __init__(self, hidden_size: int, eps: float) -> None:
        self.hidden_size, self.eps = int(hidden_size), float(eps)
        self.weight = None

    @staticmethod
    def parameters(hidden_size: int, eps: float) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((int(hidden_size),), "ones")}

    def bind(self, tensors, rt) -> None:
        self.weight = rt.to_device(tensors["weight"], torch.float32)
        self.folded = False

    def give_weight_to(self, consumer) -> bool:
        """Offers the norm's weight to the part that reads the normed rows: norm(x) W^T = (x / rms(x)) (W diag(w))^T,
        so a consumer whose first operation is a product may take w into the columns of its weight
        (`absorb_input_scale(w) -> bool`). The norm then keeps a weight of ones: every kernel that applies it still
        gives the right result, and kernels that fold the norm around the product need no weight at all."""
        absorb = getattr(consumer, "absorb_input_scale", None)
        if self.folded or absorb is None or not absorb(self.weight):
            return False
        self.weight = torch.ones_like(self.weight)
        self.folded = True
        return True

    def forward(self, x: torch.Tensor, rt, rows: torch.Tensor | None = None, n_rows: int | None = None,
                name: str = "normed") -> torch.Tensor:
        """x: float32 [tokens, hidden]. Returns the normed rows in the activation dtype; with `rows`, only those
        rows of x (gathered)."""
        n = x.shape[0] if rows is None else int(n_rows)
        out = rt.ws.buffer(name, (n, self.hidden_size), rt.dtype)
        ops.rmsnorm(out, x, self.weight, self.eps, rows)
        return out


    def lazy(self, x: torch.Tensor, rt) -> NormedInput:
        return NormedInput(self, x, rt)


FUSE_NORM_LIMIT = 16 << 20
"""Weights up to this many bytes take the norm inside their decode-sized product (one kernel less); with larger
weights every block of the product would redo the norm of all rows, and a separate norm kernel is cheaper."""


def fuses_norm(w: torch.Tensor) -> bool:
    return w.numel() * w.element_size() <= FUSE_NORM_LIMIT


def row_rule(rt, **widths: int) -> str | None:
    """The rule every product kernel has: rows are read in 16-byte pieces, so the reduced width of a product must be
    a multiple of 8 values in bfloat16 and of 4 in float32. Returns the reason if one of `widths` breaks it."""
    step = 4 if rt.dtype == torch.float32 else 8
    bad = [f"{name} {value}" for name, value in widths.items() if int(value) % step]
    if bad:
        return (f"{', '.join(bad)}: the products read rows in 16-byte pieces, so this width must be a multiple of "
                f"{step} in {'float32' if step == 4 else 'bfloat16'}")
    return None


def project(out: torch.Tensor, h, w: torch.Tensor, epilogue: int) -> None:
    """out = epilogue(h @ w^T). `h` is a tensor of activations or a `NormedInput`; a decode-sized bfloat16 product
    applies the pending norm inside the kernel, anything else computes the normed activations first."""
    if isinstance(h, NormedInput):
        if w.dtype == torch.bfloat16 and ops.streams(h.shape[0], w.shape[0], w.shape[1]) and fuses_norm(w):
            ops.gemm(out, h.x, w, epilogue, norm_weight=h.weight, eps=h.eps)
            return
        h = h.tensor()
    ops.gemm(out, h, w, epilogue)


register_part("norm", "rmsnorm", RMSNorm)
