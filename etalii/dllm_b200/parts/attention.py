"""Grouped-query attention over the cache: fused q/k/v projection, position encoding fused with the cache write,
attention of every token over its own sequence, output projection with the residual add in its epilogue
(reference: src/etalii_dllm/transformer.py:497-543, cpp/include/dllm/nn.hpp:535-569, 733-796)."""
from __future__ import annotations

import torch

from ..cache.paged import CacheNeed
from ..kernels import ops
from .norm import NormedInput, fuses_norm, project, row_rule
from .registry import build_part, register_part
from .spec import ParamSpec


def decode_chunk(sequences: int, kv_heads: int, max_context: int, head_dim: int = 0) -> int:
    """Keys per block of the decode kernel. Head sizes the tensor-core kernel takes (multiples of 16 up to 128) use
    its fixed 256; otherwise small chunks spread few sequences over the whole device and larger ones keep the
    number of blocks (one per chunk, kv head and sequence) in bounds."""
    if head_dim and head_dim % 16 == 0 and head_dim <= 128:
        return 256
    for chunk in (64, 128, 256, 512):
        if -(-max_context // chunk) * kv_heads * sequences <= 8192:
            return chunk
    return 1024


KV_REQUEST_LIMIT = 32 << 20
"""The decode q/k/v kernel asks L2 for the layer's cache pages only while they are at most this many bytes."""

TCGEN05_ATTENTION_FROM = {64: 512, 128: 192}
"""Prefill steps whose longest context is above this (by head size) take the tcgen05 attention kernel. Measured: with
heads of 128 it leads from 256 keys on (1.4 to 1.8 times from 384 on, one prompt or eight); with heads of 64 it leads
from about 768 keys per query on, 1.3 to 1.6 times at 2,048 and more, while on shorter prompts a block's fixed costs
weigh more and the mma.sync kernel with its tiles of 64 queries is as fast or a little faster."""


class Attention:
    accepts_pending_norm = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 window: int | None = None, position=None) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.scale = int(head_dim), float(scale)
        self.window = int(window) if window else None
        self.position = build_part("position", position) if position is not None else None
        self.w_qkv = self.w_o = None

    @staticmethod
    def parameters(hidden_size, num_heads, num_kv_heads, head_dim, **_) -> dict[str, ParamSpec]:
        q, kv = int(num_heads) * int(head_dim), int(num_kv_heads) * int(head_dim)
        return {"q": ParamSpec((q, hidden_size)), "k": ParamSpec((kv, hidden_size)),
                "v": ParamSpec((kv, hidden_size)), "o": ParamSpec((hidden_size, q))}

    def supports(self, rt) -> str | None:
        """None, or why the attention kernels cannot run these sizes (asked before weights go to the device)."""
        hd, group = self.head_dim, self.num_heads // self.num_kv_heads
        if hd % 8 or hd > 256:
            return f"head_dim {hd}: the attention kernels take multiples of 8 up to 256"
        if rt.dtype == torch.bfloat16 and (hd % 16 or hd > 128) and group > 64:
            return (f"{group} query heads per key/value head with head_dim {hd}: the decode kernel for head sizes "
                    f"that are no multiple of 16 up to 128 takes at most 64")
        return row_rule(rt, hidden_size=self.hidden_size, **{"heads x head_dim": self.num_heads * hd})

    def cache_need(self) -> CacheNeed:
        return CacheNeed("kv", kv_heads=self.num_kv_heads, head_dim=self.head_dim, window=self.window)

    def bind(self, tensors, rt) -> None:
        # one projection for q, k and v: the rows of the three matrices one after another
        fused = torch.cat([tensors["q"].to(rt.dtype), tensors["k"].to(rt.dtype), tensors["v"].to(rt.dtype)], dim=0)
        self.w_qkv = fused.contiguous().to(rt.device)
        self.w_o = rt.to_device(tensors["o"], rt.dtype)
        if self.position is not None:
            self.position.bind({}, rt)

    def absorb_input_scale(self, scale: torch.Tensor) -> bool:
        """Takes a per-input-feature scale (the weight of the norm in front) into the columns of the q/k/v matrix.
        Only in bfloat16, where products round anyway; the float32 path keeps the norm's own multiplication."""
        if self.w_qkv is None or self.w_qkv.dtype != torch.bfloat16:
            return False
        self.w_qkv = (self.w_qkv.float() * scale.to(self.w_qkv.device).float()[None, :]).to(torch.bfloat16).contiguous()
        return True

    def forward(self, h: torch.Tensor, residual: torch.Tensor, batch, cache, rt, write_cache: bool = True) -> None:
        """h: normed activations [tokens, hidden]; adds the attention output to `residual` (float32) in place."""
        n = batch.n_tokens
        q_size = self.num_heads * self.head_dim
        q = rt.ws.buffer("q", (n, q_size), rt.dtype)
        table = self.position.table() if self.position is not None else None
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        split = ops.reduction_split(n, *self.w_qkv.shape) if rt.dtype == torch.bfloat16 else 1
        if split > 1:
            # 33 to 64 tokens against a large W of few rows: the reduction is cut so that the whole device reads W,
            # and the rotation sums the partial results
            hidden = h.tensor() if isinstance(h, NormedInput) else h
            ops.rope_cache_write(ops.gemm_parts(hidden, self.w_qkv, split), q, cache, table, rotary_dim,
                                 self.num_heads, batch, write_cache)
        elif rt.dtype == torch.bfloat16 and n <= ops.GEMV_MAX_ROWS and self.head_dim % 16 == 0 and rotary_dim % 16 == 0:
            # decode-sized: norm, projection, rotation and cache write in one kernel
            if isinstance(h, NormedInput) and not fuses_norm(self.w_qkv):
                h = h.tensor()
            pending = isinstance(h, NormedInput)
            # (in a decode step of a few sequences whose keys and values are a small part of L2, it also asks L2 for
            # the pages the attention kernel is about to read: measured, it gains 2 % of the step at the 135M shape
            # with eight sequences and costs 3 to 4 % with one sequence or where a layer's pages are tens of MB)
            pages_bytes = n * batch.max_context * 4 * self.num_kv_heads * self.head_dim
            ask = batch.is_decode and 2 <= n <= 16 and pages_bytes <= KV_REQUEST_LIMIT
            ops.gemv_qkv_rope(h.x if pending else h, self.w_qkv, q, cache, table, rotary_dim, self.num_heads, batch,
                              write_cache, norm_weight=h.weight if pending else None, eps=h.eps if pending else 0.0,
                              prefetch_window=(self.window or 0) if ask else -1)
        elif rt.dtype == torch.bfloat16 and ops.gemm_qkv_rope_supported(cache, rotary_dim, table is not None):
            # prefill-sized: the tile product ends in rotation and cache write
            hidden = h.tensor() if isinstance(h, NormedInput) else h
            ops.gemm_qkv_rope(hidden, self.w_qkv, q, cache, table, rotary_dim, self.num_heads, batch, write_cache)
        else:
            qkv = rt.ws.buffer("qkv", (n, q_size + 2 * self.num_kv_heads * self.head_dim), torch.float32)
            project(qkv, h, self.w_qkv, ops.EPI_STORE_F32)
            ops.rope_cache_write(qkv, q, cache, table, rotary_dim, self.num_heads, batch, write_cache)
        attended = rt.ws.buffer("attended", (n, q_size), rt.dtype)
        if batch.is_decode and rt.dtype == torch.bfloat16 and ops.attention_decode_cluster_supported(cache):
            ops.attention_decode_cluster(attended, q, cache, self.num_heads, self.scale, self.window or 0, batch)
        elif batch.is_decode and rt.dtype == torch.bfloat16:
            chunk = decode_chunk(batch.n_seqs, self.num_kv_heads, batch.max_context, self.head_dim)
            scratch = rt.ws.buffer("attention_scratch", (ops.attention_decode_scratch(
                batch.n_seqs, self.num_heads, self.head_dim, chunk, batch.max_context),), torch.float32)
            tickets = rt.ws.zeros("attention_tickets", batch.n_seqs * self.num_kv_heads, torch.int32)
            ops.attention_decode(attended, q, cache, self.num_heads, self.scale, self.window or 0, batch, chunk,
                                 scratch, tickets)
        elif not batch.is_decode and ops.attention_prefill_tcgen05_supported(cache) and \
                batch.max_context > TCGEN05_ATTENTION_FROM.get(self.head_dim, 512):
            ops.attention_prefill_tcgen05(attended, q, cache, self.num_heads, self.scale, self.window or 0, batch)
        elif not batch.is_decode and ops.attention_prefill_supported(cache):
            ops.attention_prefill(attended, q, cache, self.num_heads, self.scale, self.window or 0, batch)
        elif ops.attention_blocks_supported(cache):
            # the float32 path, and bfloat16 heads the tensor-core kernels do not take: one kernel for every cut
            ops.attention_blocks(attended, q, cache, self.num_heads, self.scale, self.window or 0, batch)
        else:
            ops.attention_general(attended, q, cache, self.num_heads, self.scale, self.window or 0, batch)
        ops.gemm(residual, attended, self.w_o, ops.EPI_RESIDUAL)


    def kernel_libraries(self, rt) -> set[str]:
        """The kernel libraries this part's steps call (built together when the model loads)."""
        if rt.dtype != torch.bfloat16:
            return {"gemm_simt", "elementwise", "attention"}
        hd = self.head_dim
        names = {"gemv", "gemm_tcgen05", "elementwise"}
        if any(ops.splits_over_clusters(64, w.shape[0], w.shape[1]) for w in (self.w_qkv, self.w_o)):
            names.add("gemv_cluster")  # (steps of 17 to 64 tokens with weights this small)
        names.add("attention_decode_cluster" if hd % 16 == 0 and hd <= 128 else "attention_decode")
        if hd in (64, 128):
            names.add("attention_prefill_tcgen05")  # (long prompts; short ones take the mma.sync kernel)
        if hd % 16 == 0 and hd <= 128:
            names.add("attention_prefill")
        else:
            names.add("attention")
        return names


register_part("mixer", "attention", Attention)
