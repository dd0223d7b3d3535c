"""The SwiGLU feed-forward: down(silu(gate(h)) * up(h)). Gate and up are one matrix product whose rows interleave
(row 2i = gate_i, row 2i + 1 = up_i) so the product's epilogue applies silu(gate) * up on the accumulators; the down
projection adds into the residual in its epilogue (reference: src/etalii_dllm/transformer.py:548-558,
cpp/include/dllm/nn.hpp:467-492)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .norm import NormedInput, project, row_rule
from .registry import register_part
from .spec import ParamSpec


class SwiGLU:
    accepts_pending_norm = True

    def __init__(self, hidden_size: int, intermediate_size: int) -> None:
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.w_gate_up = self.w_down = None

    @staticmethod
    def parameters(hidden_size, intermediate_size) -> dict[str, ParamSpec]:
        return {"gate": ParamSpec((intermediate_size, hidden_size)), "up": ParamSpec((intermediate_size, hidden_size)),
                "down": ParamSpec((hidden_size, intermediate_size))}

    def supports(self, rt) -> str | None:
        return row_rule(rt, hidden_size=self.hidden_size, intermediate_size=self.intermediate_size)

    def bind(self, tensors, rt) -> None:
        gate, up = tensors["gate"].to(rt.dtype), tensors["up"].to(rt.dtype)
        fused = torch.stack([gate, up], dim=1).reshape(2 * self.intermediate_size, self.hidden_size)
        self.w_gate_up = fused.contiguous().to(rt.device)
        self.w_down = rt.to_device(tensors["down"], rt.dtype)

    def absorb_input_scale(self, scale: torch.Tensor) -> bool:
        """Takes a per-input-feature scale (the weight of the norm in front) into the columns of the gate/up
        matrix (bfloat16 only)."""
        if self.w_gate_up is None or self.w_gate_up.dtype != torch.bfloat16:
            return False
        self.w_gate_up = (self.w_gate_up.float() * scale.to(self.w_gate_up.device).float()[None, :]) \
            .to(torch.bfloat16).contiguous()
        return True

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, rt) -> None:
        rows = h.shape[0]
        if ops.FUSED_FEED_FORWARD and isinstance(h, NormedInput) and h.x is residual and \
                rt.dtype == torch.bfloat16 and ops.mlp_decode_supported(rows, self.hidden_size, self.intermediate_size):
            # (an option, off by default: norm, gate/up, SwiGLU, down and the residual sum in one kernel)
            scratch = rt.ws.buffer("mlp_partial", (ops.mlp_decode_scratch(rows, self.hidden_size,
                                                                          self.intermediate_size),), torch.float32)
            ops.mlp_decode(residual, h.weight, h.eps, self.w_gate_up, self.w_down, scratch,
                           rt.ws.zeros("mlp_tickets", 8, torch.int32))
            return
        act = rt.ws.buffer("ffn_act", (h.shape[0], self.intermediate_size), rt.dtype)
        project(act, h, self.w_gate_up, ops.EPI_SWIGLU)
        ops.gemm(residual, act, self.w_down, ops.EPI_RESIDUAL)


    def kernel_libraries(self, rt) -> set[str]:
        if rt.dtype != torch.bfloat16:
            return {"gemm_simt"}
        names = {"gemv", "gemm_tcgen05"}
        if any(ops.splits_over_clusters(64, w.shape[0], w.shape[1]) for w in (self.w_gate_up, self.w_down)):
            names.add("gemv_cluster")  # (steps of 17 to 64 tokens with weights this small)
        if ops.FUSED_FEED_FORWARD and ops.mlp_decode_supported(1, self.hidden_size, self.intermediate_size):
            names.add("mlp_decode")
        if any(ops.streams_through_shared_memory(1, w.shape[0], w.shape[1]) for w in (self.w_gate_up, self.w_down)):
            names.add("gemv_tma")
        return names


register_part("feed_forward", "swiglu", SwiGLU)
