"""RMSNorm: out = x / sqrt(mean(x^2) + eps) * weight, computed in float32 from the float32 residual stream
(reference: cpp/include/dllm/nn.hpp:391-408; plain weight, no 1 + w)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .registry import register_part
from .spec import ParamSpec


class RMSNorm:
    def __init__(self, hidden_size: int, eps: float) -> None:
        self.hidden_size, self.eps = int(hidden_size), float(eps)
        self.weight = None

    @staticmethod
    def parameters(hidden_size: int, eps: float) -> dict[str, ParamSpec]:
        return {"weight": ParamSpec((int(hidden_size),), "ones")}

    def bind(self, tensors, rt) -> None:
        self.weight = rt.to_device(tensors["weight"], torch.float32)

    def forward(self, x: torch.Tensor, rt, rows: torch.Tensor | None = None, n_rows: int | None = None,
                name: str = "normed") -> torch.Tensor:
        """x: float32 [tokens, hidden]. Returns the normed rows in the activation dtype; with `rows`, only those
        rows of x (gathered)."""
        n = x.shape[0] if rows is None else int(n_rows)
        out = rt.ws.buffer(name, (n, self.hidden_size), rt.dtype)
        ops.rmsnorm(out, x, self.weight, self.eps, rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)
