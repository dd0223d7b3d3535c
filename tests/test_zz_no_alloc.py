"""The allocation-free decode attention (`dllm_attention_decode_static`), called through its exported C symbol the
way a caller without an allocator would: inputs and outputs only. Its result must equal the regular entry point's,
on two calls in a row (the built-in scratch keeps the first call's contents), it must agree with a plain attention
computed from the same inputs, and a call must leave the device's free memory as it found it. This file is collected
last on purpose."""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from helpers import rel_error

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _entry_point():
    from etalii.dllm_b200.kernels.build import library

    function = library("attention_decode_static").dllm_attention_decode_static
    function.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                         c_int, c_float, c_int, c_int, c_int, c_void_p]
    function.restype = c_int
    return function


def _case(heads, kv_heads, head_dim, lengths, seed):
    from etalii.dllm_b200.cache.paged import CacheNeed, PagedCache
    from etalii.dllm_b200.engine.batch import BatchBuffers

    cache = PagedCache([CacheNeed("kv", kv_heads, head_dim)], max_tokens=64 * 40, max_length=1024,
                       dtype=torch.bfloat16, device=DEV)
    slots = cache.acquire(len(lengths))
    for slot, n in zip(slots, lengths):
        cache.reserve(slot, n)
        cache.advance(slot, n)
    cache.sync_tables()
    view = cache.kv_view(0)
    g = torch.Generator().manual_seed(seed)
    view.storage.copy_(torch.randn(view.storage.shape, generator=g).to(torch.bfloat16))
    batch = BatchBuffers(DEV).fill(slots, [[1]] * len(lengths), [n - 1 for n in lengths], [[] for _ in lengths])
    batch.max_context = 1024
    q = torch.randn((len(lengths), heads * head_dim), generator=g).to(torch.bfloat16).to(DEV)
    return cache, view, batch, q


@pytest.mark.parametrize("heads,kv_heads,head_dim,chunk", [(9, 3, 64, 256), (6, 3, 24, 64)])
def test_static_scratch_entry_point_matches_the_regular_one(heads, kv_heads, head_dim, chunk):
    from etalii.dllm_b200.kernels import ops

    function = _entry_point()
    stream = torch.cuda.current_stream().cuda_stream
    for call, lengths in enumerate(([700, 64, 65, 1, 300], [130, 999])):  # two calls in a row, different shapes
        cache, view, batch, q = _case(heads, kv_heads, head_dim, lengths, seed=call)
        n = len(lengths)
        want = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16, device=DEV)
        scratch = torch.empty(ops.attention_decode_scratch(n, heads, head_dim, chunk, 1024), dtype=torch.float32,
                              device=DEV)
        tickets = torch.zeros(n * kv_heads, dtype=torch.int32, device=DEV)
        ops.attention_decode(want, q, view, heads, 0.3, 0, batch, chunk, scratch, tickets)
        got = torch.zeros_like(want)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0] if call == 1 else None  # (the first call may load the library)
        status = function(got.data_ptr(), q.data_ptr(), view.base_ptr, view.page_table.data_ptr(), view.max_pages,
                          view.page_size, heads, kv_heads, head_dim, batch.tok_pos.data_ptr(), batch.slots.data_ptr(),
                          n, 0.3, 0, chunk, 1024, stream)
        assert status == 0
        torch.cuda.synchronize()
        if free_before is not None:  # what the entry point exists for: the call took no device memory
            assert torch.cuda.mem_get_info()[0] == free_before
        assert rel_error(got.float().cpu(), want.float().cpu()) <= 8e-3
        assert torch.equal(got, want)  # the same kernels in the same order: the same bits
        # and the numbers themselves, against the plain attention of the same queries, keys and values
        import plain_kernels as PK

        plain = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16)
        view_cpu = type(view)(view.storage.cpu(), view.page_table.cpu(), view.page_size, kv_heads, head_dim, None)
        cpu_batch = type("B", (), {"n_tokens": n, "tok_pos": batch.tok_pos.cpu(), "tok_seq": batch.tok_seq.cpu(),
                                   "slots": batch.slots.cpu()})
        PK.attention_general(plain, q.cpu(), view_cpu, heads, 0.3, 0, cpu_batch)
        assert rel_error(got.float().cpu(), plain.float()) <= 8e-3


def test_static_scratch_entry_point_refuses_what_does_not_fit(capfd):
    function = _entry_point()
    cache, view, batch, q = _case(9, 3, 64, [5], seed=0)
    out = torch.zeros_like(q)
    # 4096 sequences of 9 heads with 32 chunks would need far more than the built-in 2 Mi floats
    status = function(out.data_ptr(), q.data_ptr(), view.base_ptr, view.page_table.data_ptr(), view.max_pages,
                      view.page_size, 9, 3, 64, batch.tok_pos.data_ptr(), batch.slots.data_ptr(), 4096, 0.3, 0, 256,
                      8192, torch.cuda.current_stream().cuda_stream)
    assert status == -4
    assert "scratch is too small" in capfd.readouterr().err
