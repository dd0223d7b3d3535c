"""Python entry points of the hand-written kernels. Each takes torch CUDA tensors, checks what the kernel assumes
(device, dtype, contiguity, sizes), launches on torch's current stream and raises on a refused argument. There is
no CPU path and no library fallback: a tensor that is not on a CUDA device is an error."""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_longlong, c_void_p

import torch

from .build import library

EPI_STORE_F32, EPI_STORE_T, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_STATUS = {-1: "bad argument", -2: "unsupported size", -3: "kernel launch failed"}
_EPILOGUE_NAMES = {0: "store_f32", 1: "store", 2: "residual", 3: "swiglu"}


class KernelError(RuntimeError):
    pass


_prototypes = {
    ("elementwise", "dllm_embed"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ("elementwise", "dllm_rmsnorm"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    ("elementwise", "dllm_rope_cache_write"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                               c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                               c_int, c_int, c_longlong, c_void_p],
    ("elementwise", "dllm_copy_to_device"): [c_void_p, c_void_p, c_longlong, c_void_p],
    ("elementwise", "dllm_add_residual"): [c_void_p, c_void_p, c_longlong, c_int, c_void_p],
    ("elementwise", "dllm_sum_parts_residual"): [c_void_p, c_void_p, c_int, c_longlong, c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05_split"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                  c_void_p, c_void_p],
    ("elementwise", "dllm_decode_advance"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                             c_void_p],
    ("elementwise", "dllm_mask_tokens"): [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p],
    ("gemm_simt", "dllm_gemm_f32"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("gemm_bf16", "dllm_gemm_bf16"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                            c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05_qkv_rope"): [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                                     c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int,
                                                     c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05_normed"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                                                   c_int, c_float, c_void_p, c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05_residual_norm"): [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                          c_int, c_int, c_int, c_void_p, c_void_p],
    ("gemm_tcgen05", "dllm_gemm_tcgen05_qkv_rope_normed"): [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                            c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                                            c_void_p, c_int, c_float, c_void_p, c_void_p],
    ("elementwise", "dllm_cast_ssq"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
    ("gemv", "dllm_gemv_bf16"): [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int,
                                 c_void_p, c_longlong, c_void_p],
    ("gemv_cluster", "dllm_gemv_cluster"): [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_int,
                                            c_int, c_void_p, c_longlong, c_void_p],
    ("gemv_cluster", "dllm_gemv_cluster_qkv_rope"): [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p,
                                                     c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                                     c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                     c_void_p, c_longlong, c_void_p],
    ("mlp_decode", "dllm_mlp_decode"): [c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                        c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p],
    ("gemv", "dllm_argmax_candidates"): [c_void_p, c_void_p, c_int, c_int, c_void_p],
    ("gemv_tma", "dllm_gemv_tma"): [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    ("gemv", "dllm_gemv_qkv_rope"): [c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                     c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p,
                                     c_void_p, c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p],
    ("attention", "dllm_attention_general"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                              c_int, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int,
                                              c_void_p],
    ("attention", "dllm_attention_blocks"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int,
                                             c_void_p],
    ("attention_decode", "dllm_attention_decode"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                    c_int, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_int,
                                                    c_void_p, c_void_p, c_void_p],
    ("attention_decode_cluster", "dllm_attention_decode_cluster"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                                    c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                                                    c_int, c_float, c_int, c_int, c_void_p],
    ("attention_prefill", "dllm_attention_prefill"): [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                                      c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                                      c_int, c_float, c_int, c_void_p],
    ("attention_prefill_tcgen05", "dllm_attention_prefill_tcgen05"): [
        c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p,
        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p],
    ("sampling", "dllm_sample"): [c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                  c_float, c_int, c_double, c_double, c_void_p],
    ("sampling", "dllm_seed_rng"): [c_void_p, c_void_p, c_void_p, c_int, c_void_p],
}
_functions: dict[tuple[str, str], ctypes._CFuncPtr] = {}


launches = 0
"""How many kernels this module has launched (every call below launches exactly one)."""

trace: list | None = None
"""A list while a measurement wants every launch timed: each launch appends (name, CUDA event recorded behind it).
On one stream the time between consecutive events is the kernel's (plus the gap before it)."""


def _fn(lib: str, name: str):
    key = (lib, name)
    found = _functions.get(key)
    if found is None:
        found = getattr(library(lib), name)
        found.argtypes = _prototypes[key]
        found.restype = c_int
        _functions[key] = found
    return found


def _check(status: int, what: str, detail="") -> None:
    """Counts the launch; a refusal raises. `detail` may be a callable that makes the text (only then is it made:
    formatting a message costs a launch's worth of host time)."""
    global launches
    launches += 1
    if callable(what):
        what = what()
    if trace is not None and status == 0:
        event = torch.cuda.Event(enable_timing=True)
        event.record()
        trace.append((what, event))
    if status != 0:
        if callable(detail):
            detail = detail()
        raise KernelError(f"{what}: {_STATUS.get(status, status)}{(' (' + detail + ')') if detail else ''}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle (the raw getter costs a fraction of a microsecond; the Stream object ten times
    that, once per launch)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise KernelError("kernels take contiguous CUDA tensors only (there is no CPU path)")


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported (float32 and bfloat16 are)") from None


def embed(out: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, status: torch.Tensor | None = None) -> None:
    """out[r] = float32(table[tokens[r]]); a token outside the table gives a zero row and sets the status word
    (`status`: an int32 word the device can write; default: the pinned word that `raise_if_failed` reads)."""
    _cuda(out, table, tokens)
    if status is None:
        status = _status_word()
    assert out.dtype == torch.float32 and tokens.dtype == torch.int32 and status.dtype == torch.int32
    rows, hidden = out.shape
    assert tokens.numel() >= rows and table.shape[1] == hidden
    _check(_fn("elementwise", "dllm_embed")(out.data_ptr(), table.data_ptr(), tokens.data_ptr(), rows, hidden,
                                            table.shape[0], _code(table.dtype), status.data_ptr(), _stream()),
           "embed")


def copy_to_device(dst_ptr: int, src_ptr: int, nbytes: int) -> None:
    """Copies `nbytes` from pinned host memory to device memory on the current stream, without a host wait (the
    caller keeps the source alive and unchanged until the copy has run: an event behind it tells)."""
    status = _fn("elementwise", "dllm_copy_to_device")(dst_ptr, src_ptr, int(nbytes), _stream())
    if status != 0:
        raise KernelError(f"copy to the device: {_STATUS.get(status, status)}")


def rmsnorm(out: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float,
            rows: torch.Tensor | None = None) -> None:
    """out[r] = norm(x[rows[r]] if rows is given else x[r]) * weight; x and weight float32."""
    _cuda(out, x, weight, rows)
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == x.shape[-1]
    n = out.shape[0]
    assert out.shape[-1] == x.shape[-1] and (rows is not None or x.shape[0] >= n)
    assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= n)
    _check(_fn("elementwise", "dllm_rmsnorm")(out.data_ptr(), x.data_ptr(), weight.data_ptr(),
                                              rows.data_ptr() if rows is not None else None, n, x.shape[-1],
                                              float(eps), _code(out.dtype), _stream()), "rmsnorm")


prefetch_hints: dict[int, torch.Tensor] = {}
"""Weight tensor (by address) -> the weight tensor a later kernel of the step streams. A decode-sized product whose
weights are a key asks the L2 cache for the value while it runs. The model fills this from its run order."""


PREFETCH_LIMIT = 16 << 20
"""Larger weights are not asked into L2 ahead of time: four products of them would not fit there anyway."""


PREFETCH_SLICED_LIMIT = 64 << 20
"""A step's last matrix (the head's) up to this size is asked into L2 in slices by the products before it."""


def _prefetch_of(w: torch.Tensor):
    hint = prefetch_hints.get(w.data_ptr())
    if hint is None or hint.numel() * hint.element_size() > PREFETCH_LIMIT:
        return (None, 0)
    return (hint.data_ptr(), hint.numel() * hint.element_size())


_async_status = None


def _status_word() -> torch.Tensor:
    """A pinned host word that kernels with bounded waits set when a wait runs out; the host can read it at any
    time without a synchronisation."""
    global _async_status
    if _async_status is None:
        _async_status = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _async_status


def raise_if_failed() -> None:
    """Raises if a kernel has set the status word since the last look: a bounded wait on an mbarrier ran out
    (codes 2-5 the tile product, 12-21 the tcgen05 attention, 32-33 the product that streams through shared memory)
    or the embedding met a token outside its table (64). Results computed since are not valid. The word lives in
    pinned host memory, so the look costs no synchronisation; it is meaningful after the host has waited for the
    kernels in question (a `.tolist()`, a copy to the host, a synchronize)."""
    if _async_status is not None and int(_async_status[0]) != 0:
        code = int(_async_status[0])
        _async_status[0] = 0
        if code == 64:
            raise KernelError("the embedding was given a token outside its table; the step's results are invalid")
        raise KernelError(f"a kernel gave up waiting on an mbarrier (role code {code}); the step's results are invalid")


GEMV_MAX_ROWS = 64
"""The weight-streaming kernel takes at most this many activation rows."""


CLUSTER_SPLIT_BYTES = (1 << 20, 16 << 20)
CLUSTER_NARROW_ROWS = 8192


def splits_over_clusters(rows: int, outputs: int, inner: int) -> bool:
    """Whether a product with 9 to 64 rows of activations takes the kernel that splits the reduction over the
    blocks of a thread-block cluster (`gemv_cluster.cu`): weights of a few megabytes, where bringing the activations
    to the multiprocessors is the cost and a block per 16 rows of W reads them far too often. Measured at the layer
    sizes of a 576-wide model, as links of a chain of dependent launches: with 64 rows 4.0 to 7.4 µs against 4.9 to
    10.8; with 16 rows 3.2 to 3.6 against 3.8 to 4.5, but 2.5 against 2.3 for the smallest matrix (576 x 576); with 8
    rows the kernel with a block per 16 rows of W wins everywhere (1.5 to 2.5 against 2.4 to 3.3).
    With 17 to 64 rows it also takes larger weights of few rows (at most 8,192: 6144 x 4096 with 32 rows 16.6 µs
    against 21.1 for a block per 16 rows and 23.7 for the tile kernel, with 64 rows 22.3 against 47.3 and 23.9;
    4096 x 14336 with 32 rows 29.9 against 40.0 and 73.9), where the tile kernel has too few tiles for the device."""
    size = 2 * outputs * inner
    if 16 < rows <= GEMV_MAX_ROWS:
        return size <= CLUSTER_SPLIT_BYTES[1] or outputs <= CLUSTER_NARROW_ROWS
    return 8 < rows <= 16 and CLUSTER_SPLIT_BYTES[0] <= size <= CLUSTER_SPLIT_BYTES[1]


def streams(rows: int, outputs: int, inner: int | None = None) -> bool:
    """Whether a bfloat16 product of `rows` activation rows and `outputs` weight rows (of `inner` values, if given)
    runs in one of the weight-streaming kernels, which can take an RMSNorm in front: always up to 16 rows; up to 64
    rows where the weights are small enough for the kernel that splits the reduction over a cluster, or unless the
    matrix has so many rows that its blocks (16 weight rows each) would together re-read the activations far more
    often than the weights."""
    if rows <= 16:
        return True
    if inner is not None and splits_over_clusters(rows, outputs, inner):
        return True
    if rows <= 32:
        return outputs <= 4096
    # 33 to 64 rows: measured at 576-wide layers, the tile kernel (with a separate norm) wins from 2,048 weight rows
    # on (gate/up 3072 x 576 with 48 rows: 9.0 against 10.6 µs), the streaming kernel below that
    return rows <= GEMV_MAX_ROWS and outputs < 2048


TMA_STREAM_BYTES = 48 << 20


def streams_through_shared_memory(rows: int, outputs: int, inner: int) -> bool:
    """Whether a decode-sized product takes the kernel that streams W through a ring of shared-memory stages.
    Measured against the kernel that streams through registers: it wins (0.71 to 0.97 of the HBM rate against 0.65 to
    0.89) for few rows of activations, long rows of W (its copies are 2 KB pieces of a row) and matrices of tens of
    megabytes; with more rows the copies of the activations cost it the lead."""
    if inner % 64 or 2 * outputs * inner < TMA_STREAM_BYTES:
        return False
    # (up to 4 rows its lead holds, 6144 x 4096: 11.3 µs against 12.2; up to 8 rows only for very long rows of W,
    # 4096 x 14336: 24.2 against 28.8)
    return (rows <= 4 and inner >= 4096) or (rows <= 8 and inner >= 8192)


def takes_weights_as_rows(rows: int, outputs: int, inner: int) -> bool:
    """Whether a product with 3 to 64 rows of activations runs the other way round on the tile kernel (W as the
    128-row operand, read once). Measured: it wins where W has at least as many 128-row tiles as the device has
    multiprocessors (28672 x 4096 with 64 rows: 49 µs against 89 µs for the tile kernel and 187 µs for the streaming
    one; 16384 x 2048: 17 against 25); with fewer tiles a block's rate is bound by its one lane issuing products."""
    if not (outputs >= 16384 and 2 * outputs * inner >= (32 << 20)):
        return False
    # with 3 to 16 rows (the tile kernel's time does not depend on the rows): from 9 rows on, where the streaming
    # kernels need a second fragment of tokens (16384 x 2048 with 16 rows: 16.6 µs against 19.6; 49152 x 2048: 39.0
    # against 47.1), and from 3 rows on for rows of W of 4,096 values or more (128256 x 4096 with 8 rows: 176 against
    # 194; 28672 x 4096: 43.8 against 46.6; with rows of 2,048 values and up to 8 rows the streaming kernel reads at
    # 0.9 to 1.0 of the memory rate and keeps them)
    return 16 < rows <= 64 or (8 < rows <= 16 and inner >= 2048) or (3 <= rows <= 8 and inner >= 4096)


SPLIT_MIN_BYTES = 16 << 20
MAX_REDUCTION_SPLIT = 8


B200_MULTIPROCESSORS = 148


_sm_count = 0


def _multiprocessors() -> int:
    """The device's multiprocessors (a B200's where no device is present: the rules are plain functions of sizes)."""
    global _sm_count
    if _sm_count == 0:
        _sm_count = (torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
                     if torch.cuda.is_available() else B200_MULTIPROCESSORS)
    return _sm_count


def reduction_split(rows: int, outputs: int, inner: int, multiprocessors: int | None = None) -> int:
    """Into how many stretches the reduction of a residual product with 33 to 64 rows of activations is cut, 1 for
    not at all. A W of few rows and a long reduction (an output or down projection: 4096 x 14336, 2048 x 8192) has
    fewer 128-row tiles than the device has multiprocessors, and a multiprocessor takes in about 80 GB/s: with 32
    tiles the whole device reads W at a quarter of its memory rate. Cut, the tiles of every stretch run side by side
    and a second small kernel sums their partial results in order. Measured with 64 rows, both kernels together,
    against the best of the other kernels: 4096 x 14336 29.3 µs against 73.3, 4096 x 4096 12.9 against 20.0,
    2048 x 8192 13.4 against 19.1; with 32 rows and fewer, and for weights under 16 MB, the kernel that splits the
    reduction over a cluster is as fast or faster (2048 x 2048 with 64 rows: 7.6 against 8.9)."""
    if not (32 < rows <= GEMV_MAX_ROWS) or inner % 8 or outputs % 4 or 2 * outputs * inner <= SPLIT_MIN_BYTES:
        return 1
    multiprocessors = multiprocessors or _multiprocessors()
    tiles, k_tiles = -(-outputs // 128), -(-inner // 64)
    if tiles >= multiprocessors:
        return 1
    # doubled while the work items stay within two a multiprocessor and a stretch keeps eight k tiles or more
    split = 1
    while split < MAX_REDUCTION_SPLIT and tiles * split <= multiprocessors and k_tiles // (split * 2) >= 8:
        split *= 2
    return split


_parts: dict = {}


def _parts_buffer(device, floats: int) -> torch.Tensor:
    """Scratch for partial results, one buffer per size for the life of the process: a captured graph may hold its
    address. Like the work buffers, it serves one stream: a product's parts are read by the kernel behind it."""
    key = (str(device), floats)
    if key not in _parts:
        _parts[key] = torch.empty(floats, device=device, dtype=torch.float32)
    return _parts[key]


def gemm_parts(a: torch.Tensor, w: torch.Tensor, split: int) -> torch.Tensor:
    """The product a[M,K] @ w[N,K]^T (bfloat16, M <= 64) as `split` partial results over stretches of the reduction:
    a float32 tensor [split, M, N] in scratch that the next call of the same width overwrites. The tile kernel runs
    it with W as the 128-row operand; whoever reads the parts sums them in order."""
    _cuda(a, w)
    m, k = a.shape
    n = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[1] == k
    assert 0 < m <= GEMV_MAX_ROWS and 1 <= split <= MAX_REDUCTION_SPLIT
    parts = _parts_buffer(a.device, MAX_REDUCTION_SPLIT * GEMV_MAX_ROWS * n)
    _check(_fn("gemm_tcgen05", "dllm_gemm_tcgen05_split")(
        parts.data_ptr(), w.data_ptr(), a.data_ptr(), n, m, k, split, 32 if m <= 32 else 64,
        _status_word().data_ptr(), _stream()), "gemm_parts",
        lambda: f"M={m} N={n} K={k} (multiple of 8) in {split} stretches (at most one per 64 values of K)")
    return parts[:split * m * n].view(split, m, n)


def gemm(c: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int = EPI_STORE_T, kernel: int = 0,
         norm_weight: torch.Tensor | None = None, eps: float = 0.0, tile_n: int = 0, cluster: int = 0) -> None:
    """c = a[M,K] @ w[N,K]^T with float32 accumulation, then the epilogue: EPI_STORE_F32 (c float32), EPI_STORE_T
    (c in the weights' dtype), EPI_RESIDUAL (c float32 += product), EPI_SWIGLU (w interleaves gate and up rows;
    c[M,N/2] = silu(gate) * up). float32 weights run the true 32-bit kernel; bfloat16 the tcgen05/TMA tile kernel
    or, for M <= 64, a weight-streaming kernel (`kernel`: 0 chooses by the sizes, 1 forces the mma.sync tile kernel,
    2 forces streaming through registers, 3 forces tcgen05, 4 forces streaming through shared memory, 5 forces
    tcgen05 with W as the 128-row operand (for at most 256 rows of `a`), 6 forces the reduction split over a cluster
    (`cluster` blocks, 0 chooses), 7 forces W as the 128-row operand with the reduction cut into `cluster` stretches
    (residual epilogue, at most 64 rows; 0 chooses); `tile_n` picks the tcgen05 tile width).
    With `norm_weight` (streaming kernel only), `a` is the float32 residual stream and is RMS-normed on the way in."""
    _cuda(c, a, w, norm_weight)
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k, (a.shape, w.shape)
    want_cols = n // 2 if epilogue == EPI_SWIGLU else n
    want_dtype = torch.float32 if epilogue in (EPI_STORE_F32, EPI_RESIDUAL) else w.dtype
    assert tuple(c.shape) == (m, want_cols) and c.dtype == want_dtype, (c.shape, c.dtype, m, want_cols, want_dtype)
    def detail() -> str:
        return (f"M={m} N={n} K={k}: K must be a multiple of {4 if w.dtype == torch.float32 else 8}; N even for the "
                f"SwiGLU epilogue; the weight-streaming kernel takes M up to {GEMV_MAX_ROWS}")
    if w.dtype == torch.float32:
        assert a.dtype == torch.float32 and norm_weight is None
        status = _fn("gemm_simt", "dllm_gemm_f32")(c.data_ptr(), a.data_ptr(), w.data_ptr(), m, n, k, epilogue,
                                                   _stream())
    elif w.dtype == torch.bfloat16:
        streaming = (kernel == 2 and m <= GEMV_MAX_ROWS) or (kernel == 0 and streams(m, n, k))
        split = reduction_split(m, n, k) if (kernel == 0 and epilogue == EPI_RESIDUAL and norm_weight is None) else 1
        if kernel == 7 or split > 1:
            # W as the 128-row operand, the reduction cut into stretches, the parts summed into c by a second kernel
            assert a.dtype == torch.bfloat16 and norm_weight is None and epilogue == EPI_RESIDUAL and m <= 64
            split = split if kernel == 0 else max(1, int(cluster) or reduction_split(m, n, k))
            parts = gemm_parts(a, w, split)
            status = _fn("elementwise", "dllm_sum_parts_residual")(c.data_ptr(), parts.data_ptr(), split, m * n,
                                                                   _stream())
        elif kernel == 5 or (kernel == 0 and norm_weight is None and takes_weights_as_rows(m, n, k)):
            # the product the other way round: W is the 128-row operand, the tokens are the tile's columns
            assert a.dtype == torch.bfloat16 and norm_weight is None and m <= 256
            width = 32 if m <= 32 else (64 if m <= 64 else (128 if m <= 128 else 256))
            status = _fn("gemm_tcgen05", "dllm_gemm_tcgen05")(
                c.data_ptr(), w.data_ptr(), a.data_ptr(), n, m, k, epilogue + 5, width, _status_word().data_ptr(),
                _stream())
        elif kernel == 4 or (kernel == 0 and norm_weight is None and streams_through_shared_memory(m, n, k)):
            assert a.dtype == torch.bfloat16 and norm_weight is None
            status = _fn("gemv_tma", "dllm_gemv_tma")(c.data_ptr(), a.data_ptr(), w.data_ptr(), m, n, k, epilogue,
                                                      _status_word().data_ptr(), _stream())
        elif (kernel == 6 and m <= GEMV_MAX_ROWS) or (kernel == 0 and streaming and splits_over_clusters(m, n, k)):
            if norm_weight is not None:
                assert a.dtype == torch.float32 and norm_weight.dtype == torch.float32 and norm_weight.numel() == k
            else:
                assert a.dtype == torch.bfloat16
            status = _fn("gemv_cluster", "dllm_gemv_cluster")(
                c.data_ptr(), a.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps),
                w.data_ptr(), m, n, k, epilogue, int(cluster), *_prefetch_of(w), _stream())
        elif streaming:
            if norm_weight is not None:
                assert a.dtype == torch.float32 and norm_weight.dtype == torch.float32 and norm_weight.numel() == k
            else:
                assert a.dtype == torch.bfloat16
            status = _fn("gemv", "dllm_gemv_bf16")(
                c.data_ptr(), a.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps),
                w.data_ptr(), m, n, k, epilogue, *_prefetch_of(w), _stream())
        elif kernel == 1:
            assert a.dtype == torch.bfloat16 and norm_weight is None
            status = _fn("gemm_bf16", "dllm_gemm_bf16")(c.data_ptr(), a.data_ptr(), w.data_ptr(), m, n, k, epilogue,
                                                        _stream())
        else:
            assert a.dtype == torch.bfloat16 and norm_weight is None
            status = _fn("gemm_tcgen05", "dllm_gemm_tcgen05")(
                c.data_ptr(), a.data_ptr(), w.data_ptr(), m, n, k, epilogue, tile_n, _status_word().data_ptr(),
                _stream())
    else:
        raise KernelError(f"gemm: dtype {w.dtype} is not supported")
    _check(status, (lambda: f"gemm {_EPILOGUE_NAMES[epilogue]} M={m} N={n} K={k}"
                    + (" +norm" if norm_weight is not None else "")) if trace is not None else "gemm", detail)


MLP_DECODE_MAX_ROWS = 16
FUSED_FEED_FORWARD = False
"""Whether decode steps take the one-kernel feed-forward (`mlp_decode`) where it fits. Off: measured on a B200 at the
SmolLM2-135M layer sizes with 8 tokens, as one link of a chain of dependent launches in a CUDA graph, the fused kernel
takes 7.4 us against 4.7 us for the two kernels it replaces. Its gate/up part costs 2.65 us, the exchange inside the
cluster 0.6 us, the down product 0.8 us, and the fixed-order sum of the clusters' partial results through global
memory (fence, ticket, fence, loads) 3.3 us: more than the second launch it saves. The kernel stays as a tested
option."""


def mlp_decode_supported(rows: int, hidden: int, intermediate: int) -> bool:
    """Whether the feed-forward of a decode step may run as one kernel: up to 16 tokens and an intermediate size
    that slices of 16 tile."""
    return 0 < rows <= MLP_DECODE_MAX_ROWS and intermediate % 16 == 0 and hidden % 8 == 0


def mlp_decode_scratch(rows: int, hidden: int, intermediate: int) -> int:
    """Floats of scratch `mlp_decode` needs: a partial result [8 or 16 tokens, hidden] per cluster of blocks."""
    cluster = next(c for c in (8, 4, 2, 1) if intermediate % (16 * c) == 0)
    return (intermediate // (16 * cluster)) * (8 if rows <= 8 else 16) * hidden


def mlp_decode(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, w_gate_up: torch.Tensor, w_down: torch.Tensor,
               scratch: torch.Tensor, tickets: torch.Tensor) -> None:
    """x (float32 residual [rows, hidden]) += down(silu(gate(h)) * up(h)), h = RMSNorm(x) rounded to bfloat16, in one
    kernel. w_gate_up [2 * intermediate, hidden] interleaves gate and up rows; w_down is [hidden, intermediate].
    `scratch`: `mlp_decode_scratch` floats; `tickets`: 8 int32 zeros (the kernel leaves them zero)."""
    _cuda(x, norm_weight, w_gate_up, w_down, scratch, tickets)
    rows, hidden = x.shape
    intermediate = w_down.shape[1]
    assert x.dtype == torch.float32 and norm_weight.dtype == torch.float32 and norm_weight.numel() == hidden
    assert w_gate_up.dtype == torch.bfloat16 and w_down.dtype == torch.bfloat16
    assert tuple(w_gate_up.shape) == (2 * intermediate, hidden) and w_down.shape[0] == hidden
    assert scratch.dtype == torch.float32 and scratch.numel() >= mlp_decode_scratch(rows, hidden, intermediate)
    assert tickets.dtype == torch.int32 and tickets.numel() >= 8
    _check(_fn("mlp_decode", "dllm_mlp_decode")(
        x.data_ptr(), norm_weight.data_ptr(), float(eps), w_gate_up.data_ptr(), w_down.data_ptr(), rows, hidden,
        intermediate, scratch.data_ptr(), tickets.data_ptr(), *_prefetch_of(w_gate_up), *_prefetch_of(w_down),
        _stream()), "mlp_decode",
        lambda: f"rows={rows} (at most 16), hidden={hidden} (multiple of 8), intermediate={intermediate} (multiple of 16)")


EPI_ARGMAX = 9
ARGMAX_MAX_ROWS = 16


def head_argmax_supported(rows: int, w: torch.Tensor) -> bool:
    """Whether the greedy choice can be made inside the head product: bfloat16 weights and a step small enough for
    the weight-streaming kernel (up to 16 rows)."""
    return w.dtype == torch.bfloat16 and 0 < rows <= ARGMAX_MAX_ROWS and w.shape[1] % 8 == 0


def head_argmax_scratch(rows: int, outputs: int) -> int:
    """Floats of scratch: a (value, feature) candidate per token and tile of 16 output features."""
    return 2 * rows * (-(-outputs // 16))


def head_argmax(out_tokens: torch.Tensor, a: torch.Tensor, w: torch.Tensor, scratch: torch.Tensor,
                norm_weight: torch.Tensor | None = None, eps: float = 0.0) -> None:
    """out_tokens[r] = the index of the largest of a[r] @ w^T (the lowest index on ties; 0 if no value is above
    -inf), without the logits ever being stored: the product's tiles leave one candidate each, a second small
    kernel picks the winner. With `norm_weight`, `a` is the float32 residual stream, RMS-normed on the way in."""
    _cuda(out_tokens, a, w, scratch, norm_weight)
    m, k = a.shape
    n = w.shape[0]
    assert head_argmax_supported(m, w) and w.shape[1] == k and out_tokens.dtype == torch.int32
    assert scratch.dtype == torch.float32 and scratch.numel() >= head_argmax_scratch(m, n)
    assert a.dtype == (torch.float32 if norm_weight is not None else torch.bfloat16)
    _check(_fn("gemv", "dllm_gemv_bf16")(
        scratch.data_ptr(), a.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps),
        w.data_ptr(), m, n, k, EPI_ARGMAX, *_prefetch_of(w), _stream()), "head_argmax product",
        lambda: f"M={m} N={n} K={k}")
    _check(_fn("gemv", "dllm_argmax_candidates")(out_tokens.data_ptr(), scratch.data_ptr(), m, -(-n // 16),
                                                 _stream()), "head_argmax choice")


def cast_ssq(copy: torch.Tensor, ssq: torch.Tensor, x: torch.Tensor) -> None:
    """copy = bfloat16(x) and ssq[r] = sum of x[r]^2: what a norm folded around the next tile product needs of rows
    that no product's epilogue has written (a step's first rows)."""
    _cuda(copy, ssq, x)
    rows, hidden = x.shape
    assert x.dtype == torch.float32 and copy.dtype == torch.bfloat16 and tuple(copy.shape) == (rows, hidden)
    assert ssq.dtype == torch.float32 and ssq.numel() >= rows
    _check(_fn("elementwise", "dllm_cast_ssq")(copy.data_ptr(), ssq.data_ptr(), x.data_ptr(), rows, hidden, _stream()),
           "cast_ssq", lambda: f"hidden={hidden} must be a multiple of 4")


def gemm_normed(c: torch.Tensor, a: torch.Tensor, w: torch.Tensor, epilogue: int, ssq: torch.Tensor, parts: int,
                eps: float) -> None:
    """c = epilogue((a @ w^T) * 1 / sqrt(sum(ssq[:parts, row]) / K + eps)): the tile product with an RMSNorm folded
    around it. `a` is the bfloat16 copy of the un-normed rows, `w` carries the norm's weight in its columns;
    epilogues EPI_STORE_F32, EPI_STORE_T and EPI_SWIGLU."""
    _cuda(c, a, w, ssq)
    m, k = a.shape
    n = w.shape[0]
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ssq.dtype == torch.float32
    assert ssq.numel() >= m * parts
    _check(_fn("gemm_tcgen05", "dllm_gemm_tcgen05_normed")(
        c.data_ptr(), a.data_ptr(), w.data_ptr(), m, n, k, epilogue, ssq.data_ptr(), int(parts), float(eps),
        _status_word().data_ptr(), _stream()), "gemm_normed", lambda: f"M={m} N={n} K={k}")


def gemm_residual_norm(x: torch.Tensor, copy: torch.Tensor, ssq: torch.Tensor, a: torch.Tensor,
                       w: torch.Tensor) -> int:
    """x (float32) += a @ w^T; copy = bfloat16(new x); ssq[tile, row] = the sum of the squares of the new values of
    the row in each half tile of columns. Returns the number of parts (the reader's `parts`). N a multiple of 16."""
    _cuda(x, copy, ssq, a, w)
    m, k = a.shape
    n = w.shape[0]
    assert x.dtype == torch.float32 and tuple(x.shape) == (m, n) and copy.dtype == torch.bfloat16
    assert tuple(copy.shape) == (m, n) and ssq.dtype == torch.float32 and ssq.numel() >= m * (-(-n // 16))
    parts = c_int(0)
    _check(_fn("gemm_tcgen05", "dllm_gemm_tcgen05_residual_norm")(
        x.data_ptr(), copy.data_ptr(), ssq.data_ptr(), ctypes.addressof(parts), a.data_ptr(), w.data_ptr(), m, n, k,
        _status_word().data_ptr(), _stream()), "gemm_residual_norm", lambda: f"M={m} N={n} (multiple of 16) K={k}")
    return parts.value


def gemm_qkv_rope_supported(cache, rotary_dim: int, has_table: bool) -> bool:
    """Whether the tile kernel can end in the rotation and cache write: one head per tile, full rotation."""
    return cache.dtype == torch.bfloat16 and cache.head_dim in (32, 64, 128) and \
        (not has_table or rotary_dim == cache.head_dim)


_tables_by_pair: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}


def table_by_pair(table: torch.Tensor) -> torch.Tensor:
    """The rotary table [positions, pairs, (cos, sin)] laid out pair by pair, [pairs, positions, (cos, sin)], as the
    tile product reads it (a warp's tokens, at consecutive positions, then read consecutive bytes). Made once per
    table and kept with it."""
    found = _tables_by_pair.get(table.data_ptr())
    if found is None or found[0] is not table:
        if len(_tables_by_pair) > 64:
            _tables_by_pair.clear()
        found = _tables_by_pair[table.data_ptr()] = (table, table.transpose(0, 1).contiguous())
    return found[1]


def gemm_qkv_rope(a: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cache, table: torch.Tensor | None,
                  rotary_dim: int, heads: int, batch, write_cache: bool = True) -> None:
    """The q/k/v projection of a prefill-sized step in the tcgen05 tile kernel, ending in the rotation of q and k and
    the write of k and v into the paged cache (no float32 q/k/v in memory, no separate rotation kernel)."""
    _cuda(a, w, q_out, table)
    m, k = batch.n_tokens, a.shape[1]
    assert gemm_qkv_rope_supported(cache, rotary_dim, table is not None)
    assert a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16
    assert w.shape == ((heads + 2 * cache.kv_heads) * cache.head_dim, k) and a.shape[0] >= m
    if table is not None:
        assert table.dtype == torch.float32 and table.shape[0] > batch.max_position, "position beyond the table"
        assert table.shape[1] == rotary_dim // 2 and table.shape[2] == 2
    by_pair = table_by_pair(table) if table is not None else None  # (the layout this kernel reads)
    _check(_fn("gemm_tcgen05", "dllm_gemm_tcgen05_qkv_rope")(
        a.data_ptr(), w.data_ptr(), m, k, q_out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(),
        cache.max_pages, cache.page_size, heads, cache.kv_heads, cache.head_dim,
        by_pair.data_ptr() if by_pair is not None else None, rotary_dim if table is not None else 0,
        table.shape[0] if table is not None else 0,
        batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(), batch.slots.data_ptr(), 1 if write_cache else 0,
        _status_word().data_ptr(), _stream()), "gemm_qkv_rope", lambda: f"M={m} K={k} head_dim={cache.head_dim}")


def gemv_qkv_rope(a: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, cache, table: torch.Tensor | None,
                  rotary_dim: int, heads: int, batch, write_cache: bool = True,
                  norm_weight: torch.Tensor | None = None, eps: float = 0.0, prefetch_window: int = -1,
                  kernel: int = 0, cluster: int = 0) -> None:
    """The q/k/v projection of at most 64 tokens in one kernel (bfloat16): optional RMSNorm of the float32 residual
    in front, rotation of q and k, q to q_out, k and v into the paged cache. With `prefetch_window` >= 0 the kernel
    also asks L2 for the cached keys and values of the tokens' sequences (0: all of them, w: the last w), which the
    attention kernel behind it reads. `kernel`: 0 chooses, 2 forces a block per 16 rows of W, 6 the reduction split
    over a cluster (`cluster` blocks, 0 chooses)."""
    _cuda(a, w, q_out, table, norm_weight)
    m, k = batch.n_tokens, a.shape[1]
    assert w.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and q_out.dtype == torch.bfloat16
    assert w.shape == ((heads + 2 * cache.kv_heads) * cache.head_dim, k) and a.shape[0] >= m
    assert a.dtype == (torch.float32 if norm_weight is not None else torch.bfloat16)
    if table is not None:
        assert table.dtype == torch.float32 and table.shape[0] > batch.max_position, "position beyond the table"
        assert table.shape[1] == rotary_dim // 2 and table.shape[2] == 2
    if kernel == 6 or (kernel == 0 and splits_over_clusters(m, w.shape[0], k)):
        _check(_fn("gemv_cluster", "dllm_gemv_cluster_qkv_rope")(
            a.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps), w.data_ptr(), m, k,
            q_out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size, heads,
            cache.kv_heads, cache.head_dim, table.data_ptr() if table is not None else None,
            rotary_dim if table is not None else 0, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(),
            batch.slots.data_ptr(), 1 if write_cache else 0, int(prefetch_window), int(cluster), *_prefetch_of(w),
            _stream()),
            "gemv_cluster_qkv_rope",
            lambda: f"M={m} (at most 64), K={k} (multiple of 8), head_dim and rotary_dim multiples of 16")
        return
    _check(_fn("gemv", "dllm_gemv_qkv_rope")(
        a.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps), w.data_ptr(), m, k,
        q_out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size, heads,
        cache.kv_heads, cache.head_dim, table.data_ptr() if table is not None else None,
        rotary_dim if table is not None else 0, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(),
        batch.slots.data_ptr(), 1 if write_cache else 0, int(prefetch_window), *_prefetch_of(w), _stream()),
        "gemv_qkv_rope", lambda: f"M={m} (at most 64), K={k} (multiple of 8), head_dim and rotary_dim multiples of 16")


def rope_cache_write(qkv: torch.Tensor, q_out: torch.Tensor, cache, table: torch.Tensor | None, rotary_dim: int,
                     heads: int, batch, write_cache: bool = True) -> None:
    """Rotates queries and keys of qkv (float32 [tokens, (heads + 2 kv_heads) * head_dim]) by the table's angle for
    each token's position; queries go to q_out, keys and values into the token's place in the paged cache. A qkv
    of three dimensions is partial results [parts, tokens, ...] (`gemm_parts`), summed in order on the way in."""
    _cuda(qkv, q_out, table)
    tokens = batch.n_tokens
    assert qkv.dtype == torch.float32 and q_out.dtype == cache.dtype
    n_parts, part_stride = 1, 0
    if qkv.dim() == 3:
        assert qkv.is_contiguous()
        n_parts, part_stride = qkv.shape[0], qkv.shape[1] * qkv.shape[2]
        qkv = qkv[0]
    assert qkv.shape[0] >= tokens and qkv.shape[1] == (heads + 2 * cache.kv_heads) * cache.head_dim
    if table is not None:
        assert table.dtype == torch.float32 and table.shape[0] > batch.max_position, "position beyond the table"
        assert table.shape[1] == rotary_dim // 2 and table.shape[2] == 2
    _check(_fn("elementwise", "dllm_rope_cache_write")(
        qkv.data_ptr(), q_out.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages,
        cache.page_size, heads, cache.kv_heads, cache.head_dim, table.data_ptr() if table is not None else None,
        rotary_dim if table is not None else 0, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(),
        batch.slots.data_ptr(), tokens, 1 if write_cache else 0, _code(cache.dtype), n_parts, part_stride,
        _stream()), "rope_cache_write")


def attention_general(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int,
                      batch) -> None:
    """Causal attention of every token in the batch over its own sequence's cache (keys up to its position, the
    last `window` of them if window > 0). out, q: [tokens, heads * head_dim] in the cache's dtype."""
    _cuda(out, q)
    assert q.dtype == cache.dtype and out.dtype == cache.dtype
    _check(_fn("attention", "dllm_attention_general")(
        out.data_ptr(), q.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, cache.head_dim, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(),
        batch.slots.data_ptr(), batch.n_tokens, float(scale), int(window or 0), _code(cache.dtype), _stream()),
        "attention", lambda: f"head_dim={cache.head_dim} must be a multiple of 8, at most 256")


def attention_blocks_supported(cache) -> bool:
    return cache.page_size == 64 and cache.head_dim % 8 == 0 and cache.head_dim <= 256


def attention_blocks(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int, batch) -> None:
    """`attention_general` blockwise: the keys and values of a kv head go through shared memory page by page and
    serve every (token, head) pair of a run of tokens at once. Without a window a pair's result has the same bits
    as `attention_general` gives; with one the same formula is rounded in other places. The float32 path's attention,
    for whole prompts and single tokens alike."""
    _cuda(out, q)
    assert q.dtype == cache.dtype and out.dtype == cache.dtype and attention_blocks_supported(cache)
    _check(_fn("attention", "dllm_attention_blocks")(
        out.data_ptr(), q.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, cache.head_dim, batch.tok_seq.data_ptr(), batch.tok_pos.data_ptr(),
        batch.slots.data_ptr(), batch.n_tokens, int(batch.max_new), float(scale), int(window or 0),
        _code(cache.dtype), _stream()), "attention_blocks",
        lambda: f"head_dim={cache.head_dim} must be a multiple of 8, at most 256; pages of 64")


def add_residual(residual: torch.Tensor, update: torch.Tensor) -> None:
    """residual (float32) += update, summed in float32."""
    _cuda(residual, update)
    assert residual.dtype == torch.float32 and residual.numel() == update.numel()
    _check(_fn("elementwise", "dllm_add_residual")(residual.data_ptr(), update.data_ptr(), residual.numel(),
                                                   _code(update.dtype), _stream()), "add_residual")


def sample_scratch(rows: int, vocab: int) -> int:
    """Floats of scratch that temperature sampling needs: a float and a double per logit."""
    return 3 * rows * vocab + 2


def sample(out_tokens: torch.Tensor, logits: torch.Tensor, scratch: torch.Tensor | None, rng: torch.Tensor | None,
           rng_rows: torch.Tensor | None, temperature: float, top_k: int = 0, top_p: float = 1.0,
           min_p: float = 0.0) -> None:
    """One token per row of logits (float32 [rows, vocab]); see csrc/sampling.cu for the rule."""
    _cuda(out_tokens, logits, scratch, rng, rng_rows)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and out_tokens.dtype == torch.int32 and out_tokens.numel() >= rows
    if temperature > 0:
        assert scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= sample_scratch(rows, vocab)
        assert scratch.data_ptr() % 8 == 0
        assert rng is not None and rng.dtype == torch.int64 and rng_rows.dtype == torch.int32
    _check(_fn("sampling", "dllm_sample")(
        out_tokens.data_ptr(), logits.data_ptr(), logits.stride(0), rows, vocab,
        scratch.data_ptr() if scratch is not None else None, rng.data_ptr() if rng is not None else None,
        rng_rows.data_ptr() if rng_rows is not None else None, float(temperature), int(top_k), float(top_p),
        float(min_p), _stream()), "sample")


def seed_rng(rng: torch.Tensor, rows: torch.Tensor, seeds: torch.Tensor) -> None:
    """rng[rows[i]] = xoshiro256** state seeded with seeds[i] (int64 bit patterns of unsigned 64-bit seeds)."""
    _cuda(rng, rows, seeds)
    assert rng.dtype == torch.int64 and rows.dtype == torch.int32 and seeds.dtype == torch.int64
    _check(_fn("sampling", "dllm_seed_rng")(rng.data_ptr(), rows.data_ptr(), seeds.data_ptr(), rows.numel(),
                                            _stream()), "seed_rng")


def decode_advance(tokens: torch.Tensor, tok_pos: torch.Tensor, start: torch.Tensor, chosen: torch.Tensor,
                   history: torch.Tensor, counter: torch.Tensor, batch: int) -> None:
    """tokens = chosen; positions and cached lengths + 1; history[counter] = chosen; counter + 1 (all int32)."""
    _cuda(tokens, tok_pos, start, chosen, history, counter)
    _check(_fn("elementwise", "dllm_decode_advance")(
        tokens.data_ptr(), tok_pos.data_ptr(), start.data_ptr(), chosen.data_ptr(), history.data_ptr(),
        counter.data_ptr(), batch, history.numel() // batch, _stream()), "decode_advance")


def mask_tokens(logits: torch.Tensor, ids: torch.Tensor, produced: torch.Tensor, steps: torch.Tensor | None,
                min_tokens: int) -> None:
    """logits[:, ids] = -inf in every row while produced[0] + steps[0] < min_tokens (float32 logits [rows, vocab];
    ids, produced and steps int32 on the device; `steps` may be None). Ids outside the vocabulary are skipped."""
    _cuda(logits, ids, produced)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous()
    assert ids.dtype == torch.int32 and produced.dtype == torch.int32
    assert steps is None or (steps.is_cuda and steps.dtype == torch.int32)
    _check(_fn("elementwise", "dllm_mask_tokens")(
        logits.data_ptr(), logits.shape[0], logits.shape[1], ids.data_ptr(), ids.numel(), produced.data_ptr(),
        steps.data_ptr() if steps is not None else None, int(min_tokens), _stream()), "mask_tokens")


def attention_decode_scratch(sequences: int, heads: int, head_dim: int, chunk: int, max_context: int) -> int:
    """Floats of scratch `attention_decode` needs."""
    return sequences * heads * (-(-max_context // chunk)) * (head_dim + 2)


def attention_decode(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int, batch,
                     chunk: int, scratch: torch.Tensor, tickets: torch.Tensor) -> None:
    """Attention for a batch in which every sequence brings one token (bfloat16): keys are split into chunks of
    `chunk` positions across blocks, every block serves all query heads of its kv head, partial results are combined
    in chunk order by the block that finishes last. Serves any length up to batch.max_context. `tickets`: int32
    zeros, one per (sequence, kv head); the kernel leaves them zero."""
    _cuda(out, q, scratch, tickets)
    assert tickets.dtype == torch.int32 and tickets.numel() >= batch.n_seqs * cache.kv_heads
    assert cache.dtype == torch.bfloat16 and q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert batch.n_tokens == batch.n_seqs and scratch.dtype == torch.float32
    assert scratch.numel() >= attention_decode_scratch(batch.n_seqs, heads, cache.head_dim, chunk, batch.max_context)
    _check(_fn("attention_decode", "dllm_attention_decode")(
        out.data_ptr(), q.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, cache.head_dim, batch.tok_pos.data_ptr(), batch.slots.data_ptr(), batch.n_seqs,
        float(scale), int(window or 0), int(chunk), int(batch.max_context), scratch.data_ptr(),
        tickets.data_ptr(), _stream()),
        "attention_decode", lambda: f"head_dim={cache.head_dim} must be a multiple of 8, at most 256")


def attention_prefill_supported(cache) -> bool:
    return cache.dtype == torch.bfloat16 and cache.head_dim % 16 == 0 and cache.head_dim <= 128 \
        and cache.page_size == 64


def attention_prefill(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int,
                      batch) -> None:
    """Blockwise causal attention of the batch's new tokens over their sequences' caches on the tensor cores
    (bfloat16, head_dim a multiple of 16 up to 128, pages of 64 positions)."""
    _cuda(out, q)
    assert attention_prefill_supported(cache) and q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    _check(_fn("attention_prefill", "dllm_attention_prefill")(
        out.data_ptr(), q.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, cache.head_dim, batch.tile_seq.data_ptr(), batch.tile_first.data_ptr(),
        batch.cu_seqlens.data_ptr(), batch.start.data_ptr(), batch.slots.data_ptr(), batch.n_tiles, float(scale),
        int(window or 0), _stream()), "attention_prefill",
        lambda: f"head_dim={cache.head_dim} must be a multiple of 16, at most 128; pages of 64")


def attention_prefill_tcgen05_supported(cache) -> bool:
    return cache.dtype == torch.bfloat16 and cache.head_dim in (64, 128) and cache.page_size == 64


def attention_prefill_tcgen05(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int,
                              batch) -> None:
    """Blockwise causal attention of the batch's new tokens over their sequences' caches on the 5th-generation
    tensor cores (bfloat16, head_dim 64 or 128, pages of 64 positions): tiles of 128 queries, scores and outputs in tensor
    memory, pages of keys and values by TMA."""
    _cuda(out, q)
    assert attention_prefill_tcgen05_supported(cache) and q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    _check(_fn("attention_prefill_tcgen05", "dllm_attention_prefill_tcgen05")(
        out.data_ptr(), q.data_ptr(), q.shape[0], cache.base_ptr, cache.storage.shape[0],
        cache.page_table.data_ptr(), cache.max_pages, cache.page_size, heads, cache.kv_heads, cache.head_dim,
        batch.tile_seq.data_ptr(), batch.tile_first.data_ptr(), batch.cu_seqlens.data_ptr(), batch.start.data_ptr(),
        batch.slots.data_ptr(), batch.n_tiles, float(scale), int(window or 0), _status_word().data_ptr(),
        _stream()), "attention_prefill_tcgen05", lambda: f"head_dim={cache.head_dim} must be 64 or 128; pages of 64")


def attention_decode_cluster_supported(cache) -> bool:
    return cache.dtype == torch.bfloat16 and cache.head_dim % 16 == 0 and cache.head_dim <= 128 \
        and cache.page_size == 64


DECODE_CLUSTER_SHAPES = 5
"""Launch shapes of the cluster decode kernel: 0..3 are 1, 2, 4, 8 blocks per (sequence, kv head) pair, of four warps
(two when head_dim is above 64); 4 is eight blocks of four warps at any head_dim."""


def attention_decode_cluster(out: torch.Tensor, q: torch.Tensor, cache, heads: int, scale: float, window: int,
                             batch, shape: int = -1) -> None:
    """Attention for a batch in which every sequence brings one token (bfloat16, head_dim a multiple of 16 up to
    128): the blocks of a cluster split the keys of a (sequence, kv head) pair and combine through distributed
    shared memory; no scratch, and a launch shape that does not depend on the context length. shape -1 lets the
    kernel choose by the number of pairs; 0..4 name one of DECODE_CLUSTER_SHAPES."""
    _cuda(out, q)
    assert attention_decode_cluster_supported(cache) and q.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert batch.n_tokens == batch.n_seqs
    _check(_fn("attention_decode_cluster", "dllm_attention_decode_cluster")(
        out.data_ptr(), q.data_ptr(), cache.base_ptr, cache.page_table.data_ptr(), cache.max_pages, cache.page_size,
        heads, cache.kv_heads, cache.head_dim, batch.tok_pos.data_ptr(), batch.slots.data_ptr(), batch.n_seqs,
        float(scale), int(window or 0), int(shape), _stream()), "attention_decode_cluster",
        lambda: f"head_dim={cache.head_dim} must be a multiple of 16, at most 128; pages of 64")
