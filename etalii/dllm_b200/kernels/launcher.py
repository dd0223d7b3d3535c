"""The C++ host side of prefill-sized steps (csrc/step_launcher.cu): one call issues every launch of every layer.

A model whose layers are all the pre-norm arrangement of the library's own attention (rotary positions or none),
SwiGLU feed-forward and RMSNorm parts, in bfloat16, gets a table of its layers' weights, sizes and cache entries in
native memory when it is built. A step of more than 64 tokens that is no decode step then runs through
`dllm_prefill_pre_norm_layers` instead of through the parts' Python `forward`s: the same kernels with the same
arguments, chosen by the same rules, launched without the interpreter between them. Any other model, dtype or step
keeps the Python path (parts registered from outside are never asked to have a native twin)."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, byref, c_float, c_int, c_longlong, c_void_p

import torch

from . import ops
from .build import library


class KernelTable(Structure):
    _fields_ = [(name, c_void_p) for name in ("rmsnorm", "gemm_tcgen05", "gemm_tcgen05_qkv_rope", "attention_prefill",
                                              "attention_prefill_tcgen05", "cast_ssq", "gemm_tcgen05_normed",
                                              "gemm_tcgen05_qkv_rope_normed", "gemm_tcgen05_residual_norm")]


class PreNormLayer(Structure):
    _fields_ = [
        ("mixer_norm_weight", c_void_p), ("feed_forward_norm_weight", c_void_p), ("w_qkv", c_void_p),
        ("w_o", c_void_p), ("w_gate_up", c_void_p), ("w_down", c_void_p), ("rotary_table", c_void_p),
        ("cache_base", c_void_p), ("page_table", c_void_p), ("cache_pages", c_longlong),
        ("mixer_norm_eps", c_float), ("feed_forward_norm_eps", c_float), ("scale", c_float),
        ("hidden", c_int), ("heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("intermediate", c_int),
        ("rotary_dim", c_int), ("window", c_int), ("max_pages", c_int), ("page_size", c_int),
        ("tcgen05_attention_from", c_int), ("rotary_positions", c_int),
    ]


class PrefillStep(Structure):
    _fields_ = [
        ("x", c_void_p), ("normed", c_void_p), ("q", c_void_p), ("attended", c_void_p), ("activations", c_void_p),
        ("tok_seq", c_void_p), ("tok_pos", c_void_p), ("slots", c_void_p), ("cu_seqlens", c_void_p),
        ("start", c_void_p), ("tile_seq", c_void_p), ("tile_first", c_void_p), ("status", c_void_p),
        ("row_ssq", c_void_p), ("tokens", c_int), ("tiles", c_int), ("max_context", c_int), ("norms_folded", c_int),
    ]


_STAGES = ("the norm before attention (or the step's first sums of squares)", "the q/k/v product", "attention", "the output product",
           "the norm before the feed-forward", "the gate/up product", "the down product")
ENABLED = True
"""Turn off to drive every step from Python (measurements of the difference, debugging)."""


def _address(lib: str, name: str) -> int:
    return ctypes.cast(ops._fn(lib, name), c_void_p).value


class PreNormLayers:
    """The native table of a model's layers, and the call that runs a step through them."""

    MIN_TOKENS = ops.GEMV_MAX_ROWS + 1

    def __init__(self, layers: list[PreNormLayer], widths: dict, keep: list, norms_folded: bool) -> None:
        self.norms_folded = norms_folded
        self.count = len(layers)
        self.array = (PreNormLayer * self.count)(*layers)
        self.widths = widths
        self._keep = keep  # the tensors whose addresses the table holds
        self._table = None
        self._function = None
        self._uses_tcgen05_attention = any(layer.tcgen05_attention_from >= 0 for layer in layers)
        self._uses_plain_attention = True

    @classmethod
    def build(cls, model) -> "PreNormLayers | None":
        """The table for `model`, or None if one of its layers is not made of the parts this path restates."""
        from ..parts.attention import TCGEN05_ATTENTION_FROM, Attention
        from ..parts.block import PreNormBlock
        from ..parts.feed_forward import SwiGLU
        from ..parts.norm import RMSNorm
        from ..parts.position import RotaryEmbedding

        rt = model.rt
        if rt.dtype != torch.bfloat16 or model.spec.schedule or not model.blocks:
            return None
        layers, keep, folded = [], [], []
        for block, view in zip(model.blocks, model._views):
            if type(block) is not PreNormBlock:
                return None
            mixer, ffn = block.mixer, block.feed_forward
            if type(mixer) is not Attention or type(ffn) is not SwiGLU or type(block.mixer_norm) is not RMSNorm or \
                    type(block.feed_forward_norm) is not RMSNorm:
                return None
            position = mixer.position
            if position is not None and type(position) is not RotaryEmbedding:
                return None
            table = position.table() if position is not None else None
            rotary_dim = position.rotary_dim if position is not None else 0
            if view is None or not ops.gemm_qkv_rope_supported(view, rotary_dim, table is not None) or \
                    not ops.attention_prefill_supported(view):
                return None
            from_context = TCGEN05_ATTENTION_FROM.get(mixer.head_dim, 512) \
                if ops.attention_prefill_tcgen05_supported(view) else -1
            by_pair = ops.table_by_pair(table) if table is not None else None  # (as the tile product reads it)
            layers.append(PreNormLayer(
                block.mixer_norm.weight.data_ptr(), block.feed_forward_norm.weight.data_ptr(),
                mixer.w_qkv.data_ptr(), mixer.w_o.data_ptr(), ffn.w_gate_up.data_ptr(), ffn.w_down.data_ptr(),
                by_pair.data_ptr() if by_pair is not None else None, view.base_ptr, view.page_table.data_ptr(),
                view.storage.shape[0], block.mixer_norm.eps, block.feed_forward_norm.eps, mixer.scale,
                mixer.hidden_size, mixer.num_heads, mixer.num_kv_heads, mixer.head_dim, ffn.intermediate_size,
                rotary_dim, mixer.window or 0, view.max_pages, view.page_size, from_context,
                table.shape[0] if table is not None else 0))
            keep += [block.mixer_norm.weight, block.feed_forward_norm.weight, mixer.w_qkv, mixer.w_o, ffn.w_gate_up,
                     ffn.w_down, table, by_pair, view]
            if ffn.hidden_size != mixer.hidden_size:
                return None
            folded.append(bool(getattr(block.mixer_norm, "folded", False)) and
                          bool(getattr(block.feed_forward_norm, "folded", False)) and mixer.hidden_size % 16 == 0)
        if any(folded) and not all(folded) or len({layer.hidden for layer in layers}) > 1 and any(folded):
            return None  # (a model that mixes folded and unfolded norms, or widths, keeps the Python path)
        widths = {"hidden": max(layer.hidden for layer in layers),
                  "q": max(layer.heads * layer.head_dim for layer in layers),
                  "intermediate": max(layer.intermediate for layer in layers)}
        return cls(layers, widths, keep, norms_folded=all(folded))

    def libraries(self) -> set[str]:
        names = {"step_launcher", "elementwise", "gemm_tcgen05", "attention_prefill"}
        if self._uses_tcgen05_attention:
            names.add("attention_prefill_tcgen05")
        return names

    def takes(self, batch) -> bool:
        return ENABLED and ops.trace is None and not batch.is_decode and batch.n_tokens >= self.MIN_TOKENS

    def _bind(self) -> None:
        self._table = KernelTable(
            _address("elementwise", "dllm_rmsnorm"), _address("gemm_tcgen05", "dllm_gemm_tcgen05"),
            _address("gemm_tcgen05", "dllm_gemm_tcgen05_qkv_rope"),
            _address("attention_prefill", "dllm_attention_prefill"),
            _address("attention_prefill_tcgen05", "dllm_attention_prefill_tcgen05")
            if self._uses_tcgen05_attention else None,
            _address("elementwise", "dllm_cast_ssq"), _address("gemm_tcgen05", "dllm_gemm_tcgen05_normed"),
            _address("gemm_tcgen05", "dllm_gemm_tcgen05_qkv_rope_normed"),
            _address("gemm_tcgen05", "dllm_gemm_tcgen05_residual_norm"))
        function = library("step_launcher").dllm_prefill_pre_norm_layers
        function.argtypes = [POINTER(KernelTable), POINTER(PreNormLayer), c_int, POINTER(PrefillStep), POINTER(c_int),
                             POINTER(c_int), c_void_p]
        function.restype = c_int
        self._function = function

    def run(self, x: torch.Tensor, batch, rt) -> None:
        """Runs every layer on the float32 residual stream `x` [tokens, hidden] in place."""
        if self._function is None:
            self._bind()
        n = batch.n_tokens
        ws = rt.ws
        step = PrefillStep(
            x.data_ptr(), ws.buffer("normed", (n, self.widths["hidden"]), torch.bfloat16).data_ptr(),
            ws.buffer("q", (n, self.widths["q"]), torch.bfloat16).data_ptr(),
            ws.buffer("attended", (n, self.widths["q"]), torch.bfloat16).data_ptr(),
            ws.buffer("ffn_act", (n, self.widths["intermediate"]), torch.bfloat16).data_ptr(),
            batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.slots.data_ptr(), batch.cu_seqlens.data_ptr(),
            batch.start.data_ptr(), batch.tile_seq.data_ptr(), batch.tile_first.data_ptr(),
            ops._status_word().data_ptr(),
            ws.buffer("row_ssq", (n, -(-self.widths["hidden"] // 16)), torch.float32).data_ptr()
            if self.norms_folded else None,
            n, batch.n_tiles, batch.max_context, 1 if self.norms_folded else 0)
        launched, failed_at = c_int(0), c_int(-1)
        status = self._function(byref(self._table), self.array, self.count, byref(step), byref(launched),
                                byref(failed_at), ops._stream())
        ops.launches += launched.value
        if status != 0:
            layer, stage = divmod(failed_at.value, 16)
            raise ops.KernelError(f"layer {layer}, {_STAGES[stage]}: {ops._STATUS.get(status, status)}")
