"""Each kernel alone against its plain reference (tests/plain_kernels.py), at sizes other than the engine's."""
import numpy as np
import pytest
import torch

import plain_kernels as PK
from helpers import rel_error

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ops():
    from etalii.dllm_b200.kernels import ops as module

    return module


def _randn(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    table = _randn((37, 72), dtype, 0)
    tokens = torch.tensor([0, 36, 5, 5, 17], dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty((5, 72), dtype=torch.float32, device=DEV)
    ops().embed(out, table, tokens, status)
    assert torch.equal(out, table[tokens.long()].float()) and int(status[0]) == 0
    bad = torch.tensor([3, 37, -1], dtype=torch.int32, device=DEV)
    out3 = torch.empty((3, 72), dtype=torch.float32, device=DEV)
    ops().embed(out3, table, bad, status)
    assert int(status[0]) == 64 and torch.equal(out3[1], torch.zeros(72, device=DEV))
    assert torch.equal(out3[0], table[3].float())
    # without a status argument the kernels' shared pinned word is set, and the host raises when it looks
    ops().raise_if_failed()
    ops().embed(out3, table, bad)
    torch.cuda.synchronize()
    with pytest.raises(ops().KernelError, match="outside its table"):
        ops().raise_if_failed()
    ops().raise_if_failed()  # looked at once, the word is clear again


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("hidden,eps", [(72, 1e-5), (1000, 1e-6), (4096, 1e-2)])
def test_rmsnorm(dtype, tol, hidden, eps):
    x = _randn((9, hidden), torch.float32, 1, 3.0)
    w = _randn((hidden,), torch.float32, 2) + 1
    out = torch.empty((9, hidden), dtype=dtype, device=DEV)
    ref = torch.empty_like(out)
    ops().rmsnorm(out, x, w, eps)
    PK.rmsnorm(ref, x, w, eps)
    assert rel_error(out.float().cpu(), ref.float().cpu()) <= tol
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    out3 = torch.empty((3, hidden), dtype=dtype, device=DEV)
    ops().rmsnorm(out3, x, w, eps, rows)
    assert torch.equal(out3, out[rows.long()])  # a gathered row has the same bits as the row in place


GEMM_SHAPES = [(1, 64, 64), (3, 130, 72), (16, 96, 144), (17, 200, 136), (40, 576, 1536), (64, 130, 72), (77, 384, 160), (130, 66, 1544), (300, 258, 576)]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_gemm_f32(m, n, k, epilogue):
    a, w = _randn((m, k), torch.float32, 3), _randn((n, k), torch.float32, 4, 0.2)
    cols = n // 2 if epilogue == 3 else n
    c = _randn((m, cols), torch.float32, 5)
    ref = c.clone()
    ops().gemm(c, a, w, epilogue)
    PK.gemm(ref, a, w, epilogue)
    assert rel_error(c.cpu(), ref.cpu()) <= 2e-6


def test_gemm_f32_rows_do_not_depend_on_the_batch():
    a, w = _randn((150, 136), torch.float32, 6), _randn((200, 136), torch.float32, 7)
    whole = torch.empty((150, 200), dtype=torch.float32, device=DEV)
    ops().gemm(whole, a, w, 0)
    # one row and three (the kernel for a few rows), twenty (64 x 64 tiles), 149 of 150 (128 x 128 tiles)
    for rows in ([149], [0, 64, 65], list(range(70, 90)), list(range(1, 150))):
        part = torch.empty((len(rows), 200), dtype=torch.float32, device=DEV)
        ops().gemm(part, a[rows].contiguous(), w, 0)
        assert torch.equal(part, whole[rows])
    # the epilogues too: the SwiGLU of sixteen rows is the SwiGLU of those rows among 150
    act = torch.empty((150, 100), dtype=torch.float32, device=DEV)
    ops().gemm(act, a, w, 3)
    few = torch.empty((16, 100), dtype=torch.float32, device=DEV)
    ops().gemm(few, a[40:56].contiguous(), w, 3)
    assert torch.equal(few, act[40:56])


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
@pytest.mark.parametrize("kernel", [1, 2])
def test_gemm_bf16(m, n, k, epilogue, kernel):
    if kernel == 2 and m > 64:
        pytest.skip("the weight-streaming kernel takes at most 64 rows")
    a, w = _randn((m, k), torch.bfloat16, 3), _randn((n, k), torch.bfloat16, 4, 0.2)
    cols = n // 2 if epilogue == 3 else n
    c = _randn((m, cols), torch.float32 if epilogue in (0, 2) else torch.bfloat16, 5)
    ref = c.clone()
    ops().gemm(c, a, w, epilogue, kernel)
    PK.gemm(ref, a, w, epilogue)
    assert rel_error(c.float().cpu(), ref.float().cpu()) <= (2e-5 if epilogue in (0, 2) else 8e-3)


ODD_SHAPES = [(5, 131, 72), (16, 61, 40), (70, 61, 40), (200, 257, 136), (64, 1001, 64)]


@pytest.mark.parametrize("m,n,k", ODD_SHAPES)
@pytest.mark.parametrize("epilogue", [0, 1, 2])
@pytest.mark.parametrize("kernel", ["f32", 1, 2, 3])
def test_gemm_with_an_odd_number_of_outputs(m, n, k, epilogue, kernel):
    if kernel == 2 and m > 64:
        pytest.skip("the weight-streaming kernel takes at most 64 rows")
    dtype = torch.float32 if kernel == "f32" else torch.bfloat16
    a, w = _randn((m, k), dtype, 3), _randn((n, k), dtype, 4, 0.2)
    c = _randn((m, n), torch.float32 if epilogue in (0, 2) else dtype, 5)
    ref = c.clone()
    ops().gemm(c, a, w, epilogue, 0 if kernel == "f32" else kernel)
    torch.cuda.synchronize()
    ops().raise_if_failed()
    PK.gemm(ref, a, w, epilogue)
    tol = 2e-6 if kernel == "f32" else (2e-5 if epilogue in (0, 2) else 8e-3)
    assert rel_error(c.float().cpu(), ref.float().cpu()) <= tol


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(64, 64), (130, 576), (1001, 1088), (4100, 512), (9500, 192), (96, 2624)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_gemm_streaming_through_shared_memory(m, n, k, epilogue):
    """The bulk-copy ring kernel: tiles of 16 and 32 rows, several trips round the ring, a short last stage, rows of
    W beyond N, fewer tokens than the fragment holds."""
    if epilogue == 3 and n % 2:
        n += 1
    a, w = _randn((m, k), torch.bfloat16, 3), _randn((n, k), torch.bfloat16, 4, 0.2)
    cols = n // 2 if epilogue == 3 else n
    c = _randn((m, cols), torch.float32 if epilogue in (0, 2) else torch.bfloat16, 5)
    ref = c.clone()
    ops().gemm(c, a, w, epilogue, kernel=4)
    torch.cuda.synchronize()
    ops().raise_if_failed()
    PK.gemm(ref, a, w, epilogue)
    assert rel_error(c.float().cpu(), ref.float().cpu()) <= (2e-5 if epilogue in (0, 2) else 8e-3)
    again = ref.clone()  # the same starting values as c had
    again.copy_(_randn((m, cols), c.dtype, 5))
    ops().gemm(again, a, w, epilogue, kernel=4)
    assert torch.equal(again, c)


@pytest.mark.parametrize("m", [1, 17, 33, 64, 100, 256])
@pytest.mark.parametrize("n,k", [(128, 64), (130, 576), (1001, 1088), (4100, 512), (300, 2240), (19000, 128)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_gemm_with_weights_as_rows(m, n, k, epilogue):
    """The tile kernel the other way round (W as the 128-row operand, the accumulator tile is C^T): every width of
    the token tile, features beyond the last tile of W, tokens beyond the tile, fewer and more tiles than blocks."""
    if epilogue == 3 and n % 2:
        n += 1
    a, w = _randn((m, k), torch.bfloat16, 3), _randn((n, k), torch.bfloat16, 4, 0.2)
    cols = n // 2 if epilogue == 3 else n
    c = _randn((m, cols), torch.float32 if epilogue in (0, 2) else torch.bfloat16, 5)
    ref = c.clone()
    ops().gemm(c, a, w, epilogue, kernel=5)
    torch.cuda.synchronize()
    ops().raise_if_failed()
    PK.gemm(ref, a, w, epilogue)
    assert rel_error(c.float().cpu(), ref.float().cpu()) <= (2e-5 if epilogue in (0, 2) else 8e-3)


@pytest.mark.parametrize("m", [1, 17, 33, 64])
@pytest.mark.parametrize("n,k,split", [(128, 1024, 2), (132, 576, 8), (1000, 1088, 3), (4100, 512, 4), (300, 2240, 5),
                                       (2048, 1088, 1), (520, 8200, 8)])
def test_gemm_with_the_reduction_cut(m, n, k, split):
    """The tile kernel with W as the 128-row operand and the reduction cut into stretches whose partial results a
    second kernel adds to the residual in order: stretches of unequal length, more and fewer items than blocks,
    features beyond the last tile; twice the same bits."""
    a, w = _randn((m, k), torch.bfloat16, 3), _randn((n, k), torch.bfloat16, 4, 0.2)
    c = _randn((m, n), torch.float32, 5)
    ref, again = c.clone(), c.clone()
    ops().gemm(c, a, w, 2, kernel=7, cluster=split)
    ops().gemm(again, a, w, 2, kernel=7, cluster=split)
    torch.cuda.synchronize()
    ops().raise_if_failed()
    PK.gemm(ref, a, w, 2)
    assert rel_error(c.cpu(), ref.cpu()) <= 2e-5
    assert torch.equal(again, c)


def test_gemm_streaming_through_shared_memory_refuses_what_it_cannot_run():
    from etalii.dllm_b200.kernels.ops import KernelError

    for m, k in ((17, 64), (4, 72)):
        a, w = _randn((m, k), torch.bfloat16, 1), _randn((32, k), torch.bfloat16, 2)
        with pytest.raises(KernelError):
            ops().gemm(torch.empty((m, 32), dtype=torch.bfloat16, device=DEV), a, w, 1, kernel=4)


def test_swiglu_refuses_an_odd_number_of_rows():
    from etalii.dllm_b200.kernels.ops import KernelError

    for dtype, kernel in ((torch.float32, 0), (torch.bfloat16, 1), (torch.bfloat16, 2), (torch.bfloat16, 3)):
        a, w = _randn((4, 64), dtype, 1), _randn((9, 64), dtype, 2)
        with pytest.raises(KernelError, match="N even"):
            ops().gemm(torch.empty((4, 4), dtype=dtype, device=DEV), a, w, 3, kernel)


@pytest.mark.parametrize("m,n,k", [(3, 5008, 2112), (16, 4800, 4160), (40, 9552, 2240), (1, 300, 6400)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_streaming_products_with_long_rows(m, n, k, epilogue):
    """Rows of more than 2,048 values: the variants that ask for the next stretch early, and whose blocks walk over
    several tiles when there are more tiles than blocks fit on the device."""
    a, w = _randn((m, k), torch.bfloat16, 3), _randn((n, k), torch.bfloat16, 4, 0.05)
    cols = n // 2 if epilogue == 3 else n
    c = _randn((m, cols), torch.float32 if epilogue in (0, 2) else torch.bfloat16, 5)
    ref = c.clone()
    ops().gemm(c, a, w, epilogue, kernel=2)
    PK.gemm(ref, a, w, epilogue)
    assert rel_error(c.float().cpu(), ref.float().cpu()) <= (2e-5 if epilogue in (0, 2) else 8e-3)
    worst = (c.float().cpu() - ref.float().cpu()).abs().max(dim=0).values  # per output column: no tile left out
    assert float(worst.max()) <= 2e-2 * float(ref.float().abs().max()), int(worst.argmax())


def test_gemm_refuses_sizes_it_cannot_run():
    from etalii.dllm_b200.kernels.ops import KernelError

    a, w = _randn((4, 12), torch.bfloat16, 1), _randn((8, 12), torch.bfloat16, 2)
    with pytest.raises(KernelError):
        ops().gemm(torch.empty((4, 8), dtype=torch.bfloat16, device=DEV), a, w, 1)
    with pytest.raises(KernelError):
        ops().gemm(torch.empty((4, 8), dtype=torch.float32), a.cpu(), w.cpu(), 0)  # no CPU path


def _cache_and_batch(dtype, kv_heads, head_dim, lengths, new, window=None, seed=0):
    """A cache whose sequences' pages interleave, filled with random keys and values up to each length, and the
    batch of the last `new[b]` tokens of each sequence."""
    from etalii.dllm_b200.cache.paged import CacheNeed, PagedCache
    from etalii.dllm_b200.engine.batch import BatchBuffers

    room = max(64 * 40, sum((n + 63) // 64 * 64 for n in lengths) + 128)
    cache = PagedCache([CacheNeed("kv", kv_heads, head_dim, window)], max_tokens=room,
                       max_length=max(1024, max(lengths)), dtype=dtype, device=DEV)
    slots = cache.acquire(len(lengths) + 1)[1:]  # slot 0 stays unused: slots are not sequence indices
    grown = [0] * len(lengths)
    while any(g < n for g, n in zip(grown, lengths)):  # grow round-robin so pages interleave
        for i, slot in enumerate(slots):
            step = min(50, lengths[i] - grown[i])
            if step > 0:
                cache.reserve(slot, step)
                cache.advance(slot, step)
                grown[i] += step
    cache.sync_tables()
    view = cache.kv_view(0)
    g = torch.Generator().manual_seed(seed)
    view.storage.copy_((torch.randn(view.storage.shape, generator=g)).to(dtype))
    starts = [n - k for n, k in zip(lengths, new)]
    batch = BatchBuffers(DEV).fill(slots, [[1] * k for k in new], starts, [[] for _ in new])
    return cache, view, batch


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-6), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(4, 2, 16, None), (6, 3, 24, None), (9, 3, 64, None),
                                                           (8, 1, 128, 70), (5, 5, 40, 33)])
def test_attention_general(dtype, tol, heads, kv_heads, head_dim, window):
    lengths, new = [130, 67, 1, 200], [130, 1, 1, 9]
    cache, view, batch = _cache_and_batch(dtype, kv_heads, head_dim, lengths, new, window)
    n = batch.n_tokens
    q = _randn((n, heads * head_dim), dtype, 9)
    out = torch.zeros((n, heads * head_dim), dtype=dtype, device=DEV)
    ref = torch.zeros((n, heads * head_dim), dtype=dtype)
    ops().attention_general(out, q, view, heads, 0.3, window or 0, batch)
    view_cpu = type(view)(view.storage.cpu(), view.page_table.cpu(), view.page_size, kv_heads, head_dim, window)
    cpu_batch = type("B", (), {"n_tokens": n, "tok_pos": batch.tok_pos.cpu(), "tok_seq": batch.tok_seq.cpu(),
                               "slots": batch.slots.cpu()})
    PK.attention_general(ref, q.cpu(), view_cpu, heads, 0.3, window or 0, cpu_batch)
    assert rel_error(out.float().cpu(), ref.float()) <= tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 5e-6), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(4, 2, 16, None), (6, 3, 24, None), (9, 3, 64, None),
                                                           (8, 1, 128, 70), (5, 5, 40, 33), (40, 2, 8, None),
                                                           (2, 1, 256, None), (34, 2, 16, 100)])
@pytest.mark.parametrize("decode", [False, True])
def test_attention_blocks(dtype, tol, heads, kv_heads, head_dim, window, decode):
    """The blockwise kernel against the plain attention, and against the warp-per-pair kernel: the same bits where
    there is no window (the tiles of 32 keys are then the same ones), tokens of several sequences in one block,
    whole prompts and single tokens, one and two stages of shared memory, groups of more than sixteen heads."""
    lengths = [130, 67, 1, 200, 64, 65]
    new = [1] * 6 if decode else [130, 1, 1, 9, 3, 65]
    cache, view, batch = _cache_and_batch(dtype, kv_heads, head_dim, lengths, new, window)
    n = batch.n_tokens
    q = _randn((n, heads * head_dim), dtype, 9)
    out = torch.full((n, heads * head_dim), float("nan"), dtype=dtype, device=DEV)
    ops().attention_blocks(out, q, view, heads, 0.3, window or 0, batch)
    ref = torch.zeros((n, heads * head_dim), dtype=dtype)
    view_cpu = type(view)(view.storage.cpu(), view.page_table.cpu(), view.page_size, kv_heads, head_dim, window)
    cpu_batch = type("B", (), {"n_tokens": n, "tok_pos": batch.tok_pos.cpu(), "tok_seq": batch.tok_seq.cpu(),
                               "slots": batch.slots.cpu()})
    PK.attention_general(ref, q.cpu(), view_cpu, heads, 0.3, window or 0, cpu_batch)
    assert rel_error(out.float().cpu(), ref.float()) <= tol
    other = torch.zeros_like(out)
    ops().attention_general(other, q, view, heads, 0.3, window or 0, batch)
    if window is None:
        assert torch.equal(out, other)
    else:
        assert rel_error(out.float().cpu(), other.float().cpu()) <= tol
    if not decode:  # a token alone in its step gets the bits it got among its tile mates
        from etalii.dllm_b200.engine.batch import BatchBuffers

        token = 130 + 1 + 1 + 4  # the fifth of the nine new tokens of the fourth sequence
        single = BatchBuffers(DEV).fill([batch.h_slots[3]], [[1]], [lengths[3] - 9 + 4], [[]])
        alone = torch.zeros((1, heads * head_dim), dtype=dtype, device=DEV)
        ops().attention_blocks(alone, q[token:token + 1].contiguous(), view, heads, 0.3, window or 0, single)
        assert torch.equal(alone[0], out[token])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_a_far_key(dtype):
    """One key among hundreds matches the query: the output must be that key's value, wherever its page lies."""
    heads, kv_heads, hd = 4, 2, 32
    cache, view, batch = _cache_and_batch(dtype, kv_heads, hd, [700], [1])
    view.storage.mul_(0.05)
    slot = batch.h_slots[0]
    for target in (0, 63, 64, 333, 698):
        page = int(view.page_table[slot, target // 64])
        saved = view.storage[page].clone()
        view.storage[page, 0, :, target % 64, :] = 4.0
        view.storage[page, 1, :, target % 64, :] = 7.0
        q = torch.full((1, heads * hd), 4.0, dtype=dtype, device=DEV)
        out = torch.zeros_like(q)
        ops().attention_general(out, q, view, heads, 1.0, 0, batch)
        assert torch.allclose(out.float(), torch.full_like(out, 7.0).float(), atol=0.05), target
        out.zero_()
        ops().attention_blocks(out, q, view, heads, 1.0, 0, batch)
        assert torch.allclose(out.float(), torch.full_like(out, 7.0).float(), atol=0.05), target
        view.storage[page] = saved


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary", [(4, 2, 16, 16), (6, 3, 24, 24), (2, 1, 64, 32)])
def test_rope_cache_write(dtype, tol, heads, kv_heads, head_dim, rotary):
    lengths, new = [70, 5, 129], [70, 1, 3]
    cache, view, batch = _cache_and_batch(dtype, kv_heads, head_dim, lengths, new)
    n = batch.n_tokens
    angles = torch.arange(256, dtype=torch.float64)[:, None] * torch.rand(rotary // 2, dtype=torch.float64)[None]
    table = torch.stack([angles.cos(), angles.sin()], -1).float().to(DEV)
    qkv = _randn((n, (heads + 2 * kv_heads) * head_dim), torch.float32, 4)
    q = torch.zeros((n, heads * head_dim), dtype=dtype, device=DEV)
    before = view.storage.clone()
    ops().rope_cache_write(qkv, q, view, table, rotary, heads, batch, True)
    ref_view = type(view)(before.cpu().clone(), view.page_table.cpu(), view.page_size, kv_heads, head_dim, None)
    ref_q = torch.zeros((n, heads * head_dim), dtype=dtype)
    cpu_batch = type("B", (), {"n_tokens": n, "tok_pos": batch.tok_pos.cpu(), "tok_seq": batch.tok_seq.cpu(),
                               "slots": batch.slots.cpu()})
    PK.rope_cache_write(qkv.cpu(), ref_q, ref_view, table.cpu(), rotary, heads, cpu_batch, True)
    assert rel_error(q.float().cpu(), ref_q.float()) <= tol
    assert rel_error(view.storage.float().cpu(), ref_view.storage.float()) <= tol
    # only the new tokens' rows changed
    changed = (view.storage != before).any(dim=-1).sum().item()
    assert changed <= n * kv_heads * 2
    q2 = torch.zeros_like(q)
    snapshot = view.storage.clone()
    ops().rope_cache_write(qkv, q2, view, table, rotary, heads, batch, False)
    assert torch.equal(q2, q) and torch.equal(view.storage, snapshot)
    # three partial results summed in order on the way in: the bits of their float32 sum
    parts = torch.stack([_randn(tuple(qkv.shape), torch.float32, 10 + i) for i in range(3)]).contiguous()
    summed = (parts[0] + parts[1]) + parts[2]
    q3, q4 = torch.zeros_like(q), torch.zeros_like(q)
    ops().rope_cache_write(parts, q3, view, table, rotary, heads, batch, True)
    from_parts = view.storage.clone()
    ops().rope_cache_write(summed, q4, view, table, rotary, heads, batch, True)
    assert torch.equal(q3, q4) and torch.equal(from_parts, view.storage)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_residual(dtype):
    x = _randn((7, 33), torch.float32, 1)
    u = _randn((7, 33), dtype, 2)
    want = x + u.float()
    ops().add_residual(x, u)
    assert torch.equal(x, want)


def _sample_both(logits, options, seeds):
    """Tokens chosen by the kernel and by the plain sampler for each row, three draws per row."""
    import plain_llama as P

    rows = logits.shape[0]
    dev = logits.to(DEV)
    rng = torch.zeros((rows + 3, 4), dtype=torch.int64, device=DEV)
    stream_rows = torch.arange(rows, dtype=torch.int32, device=DEV) + 2
    wrapped = torch.tensor([((s % 2**64) + 2**63) % 2**64 - 2**63 for s in seeds], dtype=torch.int64, device=DEV)
    ops().seed_rng(rng, stream_rows, wrapped)
    scratch = torch.empty(ops().sample_scratch(rows, logits.shape[1]), dtype=torch.float32, device=DEV)
    got, want = [], []
    randoms = [P.Random(s) for s in seeds]
    for _ in range(3):
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        ops().sample(out, dev, scratch, rng, stream_rows, options["temperature"], options.get("top_k", 0),
                     options.get("top_p", 1.0), options.get("min_p", 0.0))
        got.append(out.tolist())
        want.append([P.sample(logits[r].numpy(), randoms[r], **options) for r in range(rows)])
    return got, want


@pytest.mark.parametrize("options", [
    {"temperature": 0.0}, {"temperature": 0.8}, {"temperature": 1.5, "top_k": 7},
    {"temperature": 1.0, "top_p": 0.6}, {"temperature": 2.0, "min_p": 0.05},
    {"temperature": 1.3, "top_k": 20, "top_p": 0.9, "min_p": 0.02}, {"temperature": 0.3, "top_k": 1},
])
@pytest.mark.parametrize("vocab", [384, 5000, 49153])
def test_sample_matches_plain_sampler(options, vocab):
    g = torch.Generator().manual_seed(vocab)
    logits = torch.randn((6, vocab), generator=g) * 3
    seeds = [0, 1, 2**64 + 5, 12345678901234567890, 7, 99]
    got, want = _sample_both(logits, options, seeds)
    assert got == want


@pytest.mark.parametrize("rows", [19, 40, 80])
@pytest.mark.parametrize("spread", [0.5, 3.0, 12.0])
def test_sample_with_many_rows_and_flat_or_peaked_distributions(rows, spread):
    """More rows mean fewer blocks per row (clusters of 4, 2 and 1); a peaked distribution leaves single candidates
    early in the descent, a flat one crowds the bins to the last bits."""
    g = torch.Generator().manual_seed(rows)
    logits = torch.randn((rows, 1500), generator=g) * spread
    seeds = [11 * r + 3 for r in range(rows)]
    for options in ({"temperature": 0.9}, {"temperature": 1.1, "top_k": 50, "top_p": 0.8, "min_p": 0.01}):
        got, want = _sample_both(logits, options, seeds)
        assert got == want, options


@pytest.mark.parametrize("rows,vocab", [(19, 40001), (40, 20000), (80, 9001)])
def test_sample_where_a_thread_holds_more_of_the_vocabulary_than_it_caches(rows, vocab):
    """With many rows a row has few blocks, and a thread's stripe of a large vocabulary is longer than the eight
    elements it keeps in registers over the passes: those rows re-read their probabilities in every pass."""
    g = torch.Generator().manual_seed(rows + vocab)
    logits = torch.randn((rows, vocab), generator=g) * 2.5
    seeds = [7 * r + 1 for r in range(rows)]
    for options in ({"temperature": 0.8}, {"temperature": 1.2, "top_k": 40, "top_p": 0.85}):
        got, want = _sample_both(logits, options, seeds)
        assert got == want, options


def test_mask_tokens_holds_stop_tokens_back_until_the_output_is_long_enough():
    """logits[:, ids] = -inf while produced + steps < min_tokens, nothing otherwise; ids outside the vocabulary are
    skipped; and the sampler's choice on the masked rows is the plain sampler's choice among the other tokens."""
    import plain_llama as P

    g = torch.Generator().manual_seed(9)
    logits = torch.randn((5, 777), generator=g) * 2
    ids = [3, 776, 400, 5000, -1]
    best = logits.argmax(dim=1).tolist()
    ids[2] = best[1]  # one row's largest logit is held back
    dev_ids = torch.tensor(ids, dtype=torch.int32, device=DEV)
    for produced, steps, min_tokens, masked in ((0, None, 1, True), (2, 1, 4, True), (2, 2, 4, False),
                                                (4, None, 4, False), (0, 0, 0, False)):
        work = logits.to(DEV)
        ops().mask_tokens(work, dev_ids, torch.tensor([produced], dtype=torch.int32, device=DEV),
                          None if steps is None else torch.tensor([steps], dtype=torch.int32, device=DEV), min_tokens)
        want = logits.clone()
        if masked:
            want[:, [3, 776, best[1]]] = float("-inf")
        assert torch.equal(work.cpu(), want), (produced, steps, min_tokens)
    masked_rows = logits.clone()
    masked_rows[:, [3, 776, best[1]]] = float("-inf")
    allowed = [t for t in range(777) if t not in (3, 776, best[1])]
    for options in ({"temperature": 0.0}, {"temperature": 0.9}, {"temperature": 1.2, "top_k": 9, "top_p": 0.8}):
        got, _ = _sample_both(masked_rows, options, [1, 2, 3, 4, 5])
        randoms = [P.Random(s) for s in [1, 2, 3, 4, 5]]
        want = [[P.sample(logits[r].numpy(), randoms[r], allowed=allowed, **options) for r in range(5)]
                for _ in range(3)]
        assert got == want, options


def test_sample_ties_go_to_the_lower_id():
    logits = torch.zeros((4, 1000))
    logits[0, [5, 700]] = 3.0      # two equal maxima
    logits[1, :] = 1.0             # all equal
    logits[2, [999, 0, 500]] = 2.0
    logits[3, 10:20] = 5.0
    got, want = _sample_both(logits, {"temperature": 0.0}, [0, 0, 0, 0])
    assert got == want and got[0] == [5, 0, 0, 10]
    for options in ({"temperature": 1.0}, {"temperature": 1.0, "top_k": 3}, {"temperature": 0.7, "top_p": 0.5},
                    {"temperature": 1.0, "min_p": 1.0}):
        got, want = _sample_both(logits, options, [3, 4, 5, 6])
        assert got == want, options


@pytest.mark.parametrize("rows", [3, 40, 80])
def test_sample_rows_without_a_largest_logit_get_token_zero(rows):
    """A row whose logits are all NaN or all -inf has no largest probability. With min_p > 0 the kernel reads the
    probability at the index of the maximum, so such a row must leave before that: it gets token 0 in the greedy
    and in the sampling path, and its neighbours are chosen as always."""
    import plain_llama as P

    g = torch.Generator().manual_seed(rows)
    vocab = 1000
    logits = torch.randn((rows, vocab), generator=g) * 2
    logits[0, :] = float("nan")
    logits[2, :] = float("-inf")
    seeds = list(range(rows))
    dev = logits.to(DEV)
    rng = torch.zeros((rows, 4), dtype=torch.int64, device=DEV)
    stream_rows = torch.arange(rows, dtype=torch.int32, device=DEV)
    ops().seed_rng(rng, stream_rows, torch.tensor(seeds, dtype=torch.int64, device=DEV))
    scratch = torch.empty(ops().sample_scratch(rows, vocab), dtype=torch.float32, device=DEV)
    for options in ({"temperature": 0.0}, {"temperature": 0.9, "min_p": 0.05},
                    {"temperature": 1.2, "top_k": 5, "top_p": 0.7, "min_p": 0.5}):
        out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
        ops().sample(out, dev, scratch, rng, stream_rows, options["temperature"], options.get("top_k", 0),
                     options.get("top_p", 1.0), options.get("min_p", 0.0))
        got = out.tolist()
        assert got[0] == 0 and got[2] == 0, options
        want = P.sample(logits[1].numpy(), P.Random(1), **options)
        assert got[1] == want, options
        assert all(0 <= t < vocab for t in got)
        if options["temperature"] > 0:  # the next draw of row 1 continues row 1's stream
            ops().seed_rng(rng, stream_rows, torch.tensor(seeds, dtype=torch.int64, device=DEV))


@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(4, 2, 16, None), (6, 3, 24, None), (9, 3, 64, None),
                                                           (8, 1, 128, 70), (5, 5, 40, 33), (12, 1, 256, None),
                                                           (20, 2, 96, 300)])
@pytest.mark.parametrize("chunk", [64, 256])
def test_attention_decode(heads, kv_heads, head_dim, window, chunk):
    lengths = [130, 67, 1, 700, 64, 65]
    cache, view, batch = _cache_and_batch(torch.bfloat16, kv_heads, head_dim, lengths, [1] * len(lengths), window)
    n = batch.n_tokens
    q = _randn((n, heads * head_dim), torch.bfloat16, 9)
    out = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16, device=DEV)
    ref = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16)
    batch.max_context = 1024  # sized for more than any sequence holds, as under a CUDA graph
    scratch = torch.full((ops().attention_decode_scratch(n, heads, head_dim, chunk, 1024),), float("nan"),
                         dtype=torch.float32, device=DEV)
    tickets = torch.zeros(n * kv_heads, dtype=torch.int32, device=DEV)
    ops().attention_decode(out, q, view, heads, 0.3, window or 0, batch, chunk, scratch, tickets)
    again = torch.zeros_like(out)
    ops().attention_decode(again, q, view, heads, 0.3, window or 0, batch, chunk, scratch, tickets)
    assert int(tickets.abs().sum()) == 0 and torch.equal(again, out)  # the counters are back at zero; same bits
    view_cpu = type(view)(view.storage.cpu(), view.page_table.cpu(), view.page_size, kv_heads, head_dim, window)
    cpu_batch = type("B", (), {"n_tokens": n, "tok_pos": batch.tok_pos.cpu(), "tok_seq": batch.tok_seq.cpu(),
                               "slots": batch.slots.cpu()})
    PK.attention_general(ref, q.cpu(), view_cpu, heads, 0.3, window or 0, cpu_batch)
    assert rel_error(out.float().cpu(), ref.float()) <= 8e-3
    general = torch.zeros_like(out)
    ops().attention_general(general, q, view, heads, 0.3, window or 0, batch)
    assert rel_error(out.float().cpu(), general.float().cpu()) <= 8e-3


def test_attention_decode_finds_a_far_key():
    heads, kv_heads, hd = 4, 2, 32
    cache, view, batch = _cache_and_batch(torch.bfloat16, kv_heads, hd, [700], [1])
    view.storage.mul_(0.05)
    slot = batch.h_slots[0]
    scratch = torch.zeros(ops().attention_decode_scratch(1, heads, hd, 64, 700), dtype=torch.float32, device=DEV)
    for target in (0, 63, 64, 333, 698, 699):
        page = int(view.page_table[slot, target // 64])
        saved = view.storage[page].clone()
        view.storage[page, 0, :, target % 64, :] = 4.0
        view.storage[page, 1, :, target % 64, :] = 7.0
        q = torch.full((1, heads * hd), 4.0, dtype=torch.bfloat16, device=DEV)
        out = torch.zeros_like(q)
        ops().attention_decode(out, q, view, heads, 1.0, 0, batch, 64, scratch,
                               torch.zeros(kv_heads, dtype=torch.int32, device=DEV))
        assert torch.allclose(out.float(), torch.full_like(out, 7.0).float(), atol=0.05), target
        view.storage[page] = saved


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (3, 130, 72), (8, 576, 1536), (16, 96, 144), (5, 3072, 576),
                                   (17, 200, 136), (33, 576, 576), (64, 960, 576), (50, 66, 1544)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
def test_gemv_with_the_norm_in_front(m, n, k, epilogue):
    x = _randn((m, k), torch.float32, 3, 2.0)
    nw = _randn((k,), torch.float32, 8) * 0.1 + 1
    w = _randn((n, k), torch.bfloat16, 4, 0.2)
    cols = n // 2 if epilogue == 3 else n
    c = _randn((m, cols), torch.float32 if epilogue in (0, 2) else torch.bfloat16, 5)
    ref = c.clone()
    ops().gemm(c, x, w, epilogue, kernel=2, norm_weight=nw, eps=1e-5)  # the streaming kernel, also above 16 rows
    normed = torch.empty((m, k), dtype=torch.float64, device=DEV)
    PK.rmsnorm(normed, x, nw, 1e-5)
    PK.gemm(ref, normed, w, epilogue)
    # the normed activations are the bfloat16 operand of a tensor-core product (as when the norm runs on its own)
    assert rel_error(c.float().cpu(), ref.float().cpu()) <= 8e-3


@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary", [(4, 2, 16, 16), (6, 3, 48, 32), (2, 1, 64, 32),
                                                           (9, 3, 64, 64), (3, 1, 128, 0)])
@pytest.mark.parametrize("normed", [False, True])
@pytest.mark.parametrize("rows_extra", [1, 40])
def test_gemv_qkv_rope(heads, kv_heads, head_dim, rotary, normed, rows_extra):
    _check_gemv_qkv_rope(heads, kv_heads, head_dim, rotary, normed, rows_extra, 136)


@pytest.mark.parametrize("normed", [False, True])
def test_gemv_qkv_rope_long_rows_and_more_tiles_than_blocks(normed):
    """Rows of W of more than 2,048 values and 448 tiles: the variant whose blocks walk over several tiles."""
    _check_gemv_qkv_rope(40, 8, 128, 128, normed, 3, 2240)


def _check_gemv_qkv_rope(heads, kv_heads, head_dim, rotary, normed, rows_extra, k, kernel=2, cluster=0):
    lengths, new = [70, 5, 129, 64, 200, 33], [1, 1, 3, 2, rows_extra, 1]
    cache, view, batch = _cache_and_batch(torch.bfloat16, kv_heads, head_dim, lengths, new)
    n = batch.n_tokens
    table = None
    if rotary:
        angles = torch.arange(256, dtype=torch.float64)[:, None] * torch.rand(rotary // 2, dtype=torch.float64)[None]
        table = torch.stack([angles.cos(), angles.sin()], -1).float().to(DEV)
    w = _randn(((heads + 2 * kv_heads) * head_dim, k), torch.bfloat16, 4, 0.2 if k < 1000 else 0.05)
    x = _randn((n, k), torch.float32 if normed else torch.bfloat16, 6)
    nw = _randn((k,), torch.float32, 8) * 0.1 + 1
    q = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16, device=DEV)
    before = view.storage.clone()
    # (with the request for the sequences' cached pages into L2, as decode steps make it: a hint, no result changes)
    ops().gemv_qkv_rope(x, w, q, view, table, rotary, heads, batch, True, prefetch_window=0 if normed else 40,
                        norm_weight=nw if normed else None, eps=1e-6, kernel=kernel, cluster=cluster)
    h = x.double()
    if normed:
        h = torch.empty((n, k), dtype=torch.float64, device=DEV)
        PK.rmsnorm(h, x, nw, 1e-6)
    qkv = (h @ w.double().T).float().cpu()
    ref_view = type(view)(before.cpu().clone(), view.page_table.cpu(), view.page_size, kv_heads, head_dim, None)
    ref_q = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16)
    cpu_batch = type("B", (), {"n_tokens": n, "tok_pos": batch.tok_pos.cpu(), "tok_seq": batch.tok_seq.cpu(),
                               "slots": batch.slots.cpu()})
    PK.rope_cache_write(qkv, ref_q, ref_view, table.cpu() if rotary else None, rotary, heads, cpu_batch, True)
    assert rel_error(q.float().cpu(), ref_q.float()) <= 8e-3
    assert rel_error(view.storage.float().cpu(), ref_view.storage.float()) <= 8e-3
    assert (view.storage != before).any(dim=-1).sum().item() <= n * kv_heads * 2
    q2, snapshot = torch.zeros_like(q), view.storage.clone()
    ops().gemv_qkv_rope(x, w, q2, view, table, rotary, heads, batch, False, norm_weight=nw if normed else None,
                        eps=1e-6, kernel=kernel, cluster=cluster)
    assert torch.equal(q2, q) and torch.equal(view.storage, snapshot)


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (3, 130, 72), (16, 96, 144), (17, 200, 136), (33, 576, 576),
                                   (64, 960, 576), (50, 66, 1544), (64, 576, 1536), (40, 3072, 576), (29, 48, 2048)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
@pytest.mark.parametrize("normed", [False, True])
def test_gemv_cluster(m, n, k, epilogue, normed):
    """The product whose reduction is split over the blocks of a cluster, at every cluster size its rows allow:
    against the plain product, and the same bits on a second run (fixed order of the sums)."""
    x = _randn((m, k), torch.float32 if normed else torch.bfloat16, 3, 2.0 if normed else 1.0)
    nw = _randn((k,), torch.float32, 8) * 0.1 + 1
    w = _randn((n, k), torch.bfloat16, 4, 0.2)
    cols = n // 2 if epilogue == 3 else n
    start = _randn((m, cols), torch.float32 if epilogue in (0, 2) else torch.bfloat16, 5)
    ref = start.clone()
    h = x
    if normed:
        h = torch.empty((m, k), dtype=torch.float64, device=DEV)
        PK.rmsnorm(h, x, nw, 1e-5)
    PK.gemm(ref, h, w, epilogue)
    most = 4 if m <= 16 else 8
    for cluster in [c for c in (0, 1, 2, 4, 8) if c <= most]:
        c = start.clone()
        ops().gemm(c, x, w, epilogue, kernel=6, cluster=cluster, norm_weight=nw if normed else None, eps=1e-5)
        assert rel_error(c.float().cpu(), ref.float().cpu()) <= 8e-3, cluster
        again = start.clone()
        ops().gemm(again, x, w, epilogue, kernel=6, cluster=cluster, norm_weight=nw if normed else None, eps=1e-5)
        assert torch.equal(again, c), cluster
    with pytest.raises(Exception):
        ops().gemm(start.clone(), x, w, epilogue, kernel=6, cluster=3, norm_weight=nw if normed else None, eps=1e-5)


@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary", [(4, 2, 16, 16), (6, 3, 48, 32), (2, 1, 64, 32),
                                                           (9, 3, 64, 64), (3, 1, 128, 0)])
@pytest.mark.parametrize("normed", [False, True])
@pytest.mark.parametrize("rows_extra,cluster", [(1, 0), (1, 4), (12, 2), (24, 8), (40, 0), (40, 1), (40, 8), (56, 4)])
def test_gemv_cluster_qkv_rope(heads, kv_heads, head_dim, rotary, normed, rows_extra, cluster):
    _check_gemv_qkv_rope(heads, kv_heads, head_dim, rotary, normed, rows_extra, 136, kernel=6, cluster=cluster)


@pytest.mark.parametrize("normed", [False, True])
def test_gemv_cluster_qkv_rope_long_rows(normed):
    _check_gemv_qkv_rope(40, 8, 128, 128, normed, 30, 2240, kernel=6)


@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(4, 2, 16, None), (9, 3, 64, None), (8, 1, 128, 70),
                                                           (6, 2, 48, 33), (5, 5, 32, None), (2, 2, 96, 130)])
def test_attention_prefill(heads, kv_heads, head_dim, window):
    """Whole prompts, prompts that go on from a cached prefix, single tokens and tile edges, in one batch."""
    lengths, new = [130, 200, 1, 64, 65, 300, 77], [130, 9, 1, 64, 65, 128, 1]
    cache, view, batch = _cache_and_batch(torch.bfloat16, kv_heads, head_dim, lengths, new, window)
    n = batch.n_tokens
    q = _randn((n, heads * head_dim), torch.bfloat16, 9)
    out = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16, device=DEV)
    ref = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16)
    ops().attention_prefill(out, q, view, heads, 0.3, window or 0, batch)
    view_cpu = type(view)(view.storage.cpu(), view.page_table.cpu(), view.page_size, kv_heads, head_dim, window)
    cpu_batch = type("B", (), {"n_tokens": n, "tok_pos": batch.tok_pos.cpu(), "tok_seq": batch.tok_seq.cpu(),
                               "slots": batch.slots.cpu()})
    PK.attention_general(ref, q.cpu(), view_cpu, heads, 0.3, window or 0, cpu_batch)
    assert rel_error(out.float().cpu(), ref.float()) <= 8e-3
    worst = (out.float().cpu() - ref.float()).abs().max(dim=1).values
    assert worst.max() <= 8e-3 * ref.float().abs().max(), int(worst.argmax())


def test_attention_prefill_finds_a_far_key_and_ignores_what_lies_beyond():
    heads, kv_heads, hd = 4, 2, 32
    cache, view, batch = _cache_and_batch(torch.bfloat16, kv_heads, hd, [700], [100])
    view.storage.mul_(0.05)
    slot = batch.h_slots[0]
    last_page = int(view.page_table[slot, 699 // 64])
    view.storage[last_page, :, :, 700 % 64:, :] = 1e4  # rows of the last page beyond the sequence's length
    for target in (0, 63, 64, 333, 599):
        page = int(view.page_table[slot, target // 64])
        saved = view.storage[page].clone()
        view.storage[page, 0, :, target % 64, :] = 4.0
        view.storage[page, 1, :, target % 64, :] = 7.0
        q = torch.full((100, heads * hd), 4.0, dtype=torch.bfloat16, device=DEV)
        out = torch.zeros_like(q)
        ops().attention_prefill(out, q, view, heads, 1.0, 0, batch)
        assert torch.allclose(out.float(), torch.full_like(out, 7.0).float(), atol=0.05), target
        view.storage[page] = saved


@pytest.mark.parametrize("heads,kv_heads,window", [(9, 3, None), (4, 4, 70), (8, 1, 33), (6, 2, 200), (1, 1, None)])
@pytest.mark.parametrize("head_dim", [64, 128])
def test_attention_prefill_tcgen05(heads, kv_heads, window, head_dim):
    """Whole prompts, prompts that go on from a cached prefix, single tokens and tile edges, in one batch."""
    lengths, new = [130, 200, 1, 64, 65, 300, 77, 128, 129, 390], [130, 9, 1, 64, 65, 128, 1, 128, 129, 257]
    cache, view, batch = _cache_and_batch(torch.bfloat16, kv_heads, head_dim, lengths, new, window)
    n = batch.n_tokens
    q = _randn((n, heads * head_dim), torch.bfloat16, 9)
    out = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16, device=DEV)
    ref = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16)
    ops().attention_prefill_tcgen05(out, q, view, heads, 0.3, window or 0, batch)
    torch.cuda.synchronize()
    ops().raise_if_failed()
    view_cpu = type(view)(view.storage.cpu(), view.page_table.cpu(), view.page_size, kv_heads, head_dim, window)
    cpu_batch = type("B", (), {"n_tokens": n, "tok_pos": batch.tok_pos.cpu(), "tok_seq": batch.tok_seq.cpu(),
                               "slots": batch.slots.cpu()})
    PK.attention_general(ref, q.cpu(), view_cpu, heads, 0.3, window or 0, cpu_batch)
    worst = (out.float().cpu() - ref.float()).abs().max(dim=1).values
    assert worst.max() <= 8e-3 * ref.float().abs().max(), int(worst.argmax())
    assert rel_error(out.float().cpu(), ref.float()) <= 8e-3
    again = torch.zeros_like(out)
    ops().attention_prefill_tcgen05(again, q, view, heads, 0.3, window or 0, batch)
    assert torch.equal(again, out)


@pytest.mark.parametrize("window", [None, 1000])
@pytest.mark.parametrize("head_dim", [64, 128])
def test_attention_prefill_tcgen05_long(window, head_dim):
    """Thousands of keys per query (many trips round the rings of stages and buffers), against the mma.sync kernel."""
    heads, kv_heads = 6, 2
    lengths, new = [2500, 4100, 700], [2500, 1030, 700]
    cache, view, batch = _cache_and_batch(torch.bfloat16, kv_heads, head_dim, lengths, new, window)
    n = batch.n_tokens
    q = _randn((n, heads * head_dim), torch.bfloat16, 9)
    out, ref = (torch.zeros((n, heads * head_dim), dtype=torch.bfloat16, device=DEV) for _ in range(2))
    ops().attention_prefill_tcgen05(out, q, view, heads, 0.3, window or 0, batch)
    ops().attention_prefill(ref, q, view, heads, 0.3, window or 0, batch)
    torch.cuda.synchronize()
    ops().raise_if_failed()
    worst = (out.float() - ref.float()).abs().max(dim=1).values
    assert float(worst.max()) <= 8e-3 * float(ref.float().abs().max()), int(worst.argmax())


@pytest.mark.parametrize("hd", [64, 128])
def test_attention_prefill_tcgen05_finds_a_far_key_and_ignores_what_lies_beyond(hd):
    heads, kv_heads = 4, 2
    cache, view, batch = _cache_and_batch(torch.bfloat16, kv_heads, hd, [700], [200])
    view.storage.mul_(0.05)
    slot = batch.h_slots[0]
    last_page = int(view.page_table[slot, 699 // 64])
    view.storage[last_page, :, :, 700 % 64:, :] = 1e4  # rows of the last page beyond the sequence's length
    for target in (0, 63, 64, 333, 499):
        page = int(view.page_table[slot, target // 64])
        saved = view.storage[page].clone()
        view.storage[page, 0, :, target % 64, :] = 4.0
        view.storage[page, 1, :, target % 64, :] = 7.0
        q = torch.full((200, heads * hd), 4.0, dtype=torch.bfloat16, device=DEV)
        out = torch.zeros_like(q)
        ops().attention_prefill_tcgen05(out, q, view, heads, 1.0, 0, batch)
        assert torch.allclose(out.float(), torch.full_like(out, 7.0).float(), atol=0.05), target
        view.storage[page] = saved


def test_attention_prefill_tcgen05_refuses_other_head_sizes():
    from etalii.dllm_b200.kernels.ops import KernelError

    cache, view, batch = _cache_and_batch(torch.bfloat16, 2, 32, [70], [70])
    q = _randn((70, 4 * 32), torch.bfloat16, 9)
    with pytest.raises((KernelError, AssertionError)):
        ops().attention_prefill_tcgen05(torch.zeros_like(q), q, view, 4, 0.3, 0, batch)


def test_gemv_qkv_rope_refuses_head_sizes_it_cannot_pair():
    from etalii.dllm_b200.kernels.ops import KernelError

    cache, view, batch = _cache_and_batch(torch.bfloat16, 3, 24, [5], [1])
    w = _randn(((6 + 6) * 24, 64), torch.bfloat16, 1)
    with pytest.raises(KernelError, match="multiples of 16"):
        ops().gemv_qkv_rope(_randn((1, 64), torch.bfloat16, 2), w, torch.zeros((1, 144), dtype=torch.bfloat16,
                            device=DEV), view, None, 0, 6, batch)


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES + [(2048, 576, 576), (1000, 960, 1536), (64, 3072, 576), (129, 192, 72),
                                                 (5000, 1024, 264), (300, 4608, 136)])
@pytest.mark.parametrize("epilogue", [0, 1, 2, 3])
@pytest.mark.parametrize("tile_n", [32, 64, 128, 256])
def test_gemm_tcgen05(m, n, k, epilogue, tile_n):
    a, w = _randn((m, k), torch.bfloat16, 3), _randn((n, k), torch.bfloat16, 4, 0.2)
    cols = n // 2 if epilogue == 3 else n
    c = _randn((m, cols), torch.float32 if epilogue in (0, 2) else torch.bfloat16, 5)
    ref = c.clone()
    ops().gemm(c, a, w, epilogue, kernel=3, tile_n=tile_n)
    torch.cuda.synchronize()
    ops().raise_if_failed()
    PK.gemm(ref, a, w, epilogue)
    assert rel_error(c.float().cpu(), ref.float().cpu()) <= (2e-5 if epilogue in (0, 2) else 8e-3)


@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary,wide", [
    (9, 3, 64, 64, False), (4, 2, 32, 32, False), (5, 1, 128, 128, False), (3, 3, 64, 0, False),
    (21, 6, 64, 64, True), (13, 2, 128, 128, True), (29, 3, 64, 0, True)])
def test_gemm_qkv_rope(heads, kv_heads, head_dim, rotary, wide):
    """`wide`: enough rows, columns and a long enough reduction that a tile holds four heads of 64 or two of 128
    (head counts that are no multiples of that: the last tile ends beyond the last head, tiles straddle q, k and v)."""
    lengths, new, k = ([900, 70, 5, 129], [900, 70, 1, 129], 1032) if wide else ([300, 70, 5, 129], [300, 70, 1, 9], 136)
    cache, view, batch = _cache_and_batch(torch.bfloat16, kv_heads, head_dim, lengths, new)
    n = batch.n_tokens
    table = None
    if rotary:
        angles = torch.arange(1024, dtype=torch.float64)[:, None] * torch.rand(rotary // 2, dtype=torch.float64)[None]
        table = torch.stack([angles.cos(), angles.sin()], -1).float().to(DEV)
    w = _randn(((heads + 2 * kv_heads) * head_dim, k), torch.bfloat16, 4, 0.05 if wide else 0.2)
    x = _randn((n, k), torch.bfloat16, 6)
    q = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16, device=DEV)
    before = view.storage.clone()
    ops().gemm_qkv_rope(x, w, q, view, table, rotary, heads, batch, True)
    torch.cuda.synchronize()
    ops().raise_if_failed()
    qkv = (x.double() @ w.double().T).float().cpu()
    ref_view = type(view)(before.cpu().clone(), view.page_table.cpu(), view.page_size, kv_heads, head_dim, None)
    ref_q = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16)
    cpu_batch = type("B", (), {"n_tokens": n, "tok_pos": batch.tok_pos.cpu(), "tok_seq": batch.tok_seq.cpu(),
                               "slots": batch.slots.cpu()})
    PK.rope_cache_write(qkv, ref_q, ref_view, table.cpu() if rotary else None, rotary, heads, cpu_batch, True)
    assert rel_error(q.float().cpu(), ref_q.float()) <= 8e-3
    assert rel_error(view.storage.float().cpu(), ref_view.storage.float()) <= 8e-3
    assert (view.storage != before).any(dim=-1).sum().item() <= n * kv_heads * 2
    q2, snapshot = torch.zeros_like(q), view.storage.clone()
    ops().gemm_qkv_rope(x, w, q2, view, table, rotary, heads, batch, False)
    assert torch.equal(q2, q) and torch.equal(view.storage, snapshot)


@pytest.mark.parametrize("heads,kv_heads,head_dim,window", [(4, 2, 16, None), (9, 3, 64, None), (8, 1, 128, 70),
                                                           (6, 2, 48, 33), (34, 2, 32, None), (20, 2, 96, 300)])
@pytest.mark.parametrize("lengths", [[130, 67, 1, 700, 64, 65], [2100, 2048, 2049, 4500],
                                     [1 + (37 * i * i) % 190 for i in range(130)]],
                         ids=["short", "long", "many"])
def test_attention_decode_cluster(heads, kv_heads, head_dim, window, lengths):
    from etalii.dllm_b200.cache.paged import CacheNeed, PagedCache
    from etalii.dllm_b200.engine.batch import BatchBuffers

    cache = PagedCache([CacheNeed("kv", kv_heads, head_dim, window)], max_tokens=64 * 420, max_length=8192,
                       dtype=torch.bfloat16, device=DEV)
    slots = cache.acquire(len(lengths))
    for slot, n in zip(slots, lengths):
        cache.reserve(slot, n)
        cache.advance(slot, n)
    cache.sync_tables()
    view = cache.kv_view(0)
    g = torch.Generator().manual_seed(3)
    view.storage.copy_(torch.randn(view.storage.shape, generator=g).to(torch.bfloat16))
    batch = BatchBuffers(DEV).fill(slots, [[1]] * len(lengths), [n - 1 for n in lengths], [[] for _ in lengths])
    n = batch.n_tokens
    q = _randn((n, heads * head_dim), torch.bfloat16, 9)
    out = torch.zeros((n, heads * head_dim), dtype=torch.bfloat16, device=DEV)
    general = torch.zeros_like(out)
    ops().attention_general(general, q, view, heads, 0.3, window or 0, batch)  # itself checked against the plain one
    for shape in range(-1, ops().DECODE_CLUSTER_SHAPES):  # the kernel's own choice, then every launch shape by name
        out.zero_()
        ops().attention_decode_cluster(out, q, view, heads, 0.3, window or 0, batch, shape)
        assert rel_error(out.float().cpu(), general.float().cpu()) <= 8e-3, shape
        worst = (out.float() - general.float()).abs().max(dim=1).values
        assert float(worst.max()) <= 8e-3 * float(general.float().abs().max()), (shape, int(worst.argmax()))
        again = torch.zeros_like(out)
        ops().attention_decode_cluster(again, q, view, heads, 0.3, window or 0, batch, shape)
        assert torch.equal(again, out), shape


def test_attention_decode_cluster_finds_a_far_key():
    heads, kv_heads, hd = 4, 2, 32
    cache, view, batch = _cache_and_batch(torch.bfloat16, kv_heads, hd, [700], [1])
    view.storage.mul_(0.05)
    slot = batch.h_slots[0]
    for target in (0, 63, 64, 333, 698, 699):
        page = int(view.page_table[slot, target // 64])
        saved = view.storage[page].clone()
        view.storage[page, 0, :, target % 64, :] = 4.0
        view.storage[page, 1, :, target % 64, :] = 7.0
        q = torch.full((1, heads * hd), 4.0, dtype=torch.bfloat16, device=DEV)
        for shape in range(-1, ops().DECODE_CLUSTER_SHAPES):
            out = torch.zeros_like(q)
            ops().attention_decode_cluster(out, q, view, heads, 1.0, 0, batch, shape)
            assert torch.allclose(out.float(), torch.full_like(out, 7.0).float(), atol=0.05), (target, shape)
        view.storage[page] = saved


def test_a_bounded_wait_that_runs_out_is_reported_and_hangs_nothing():
    """The tcgen05 kernels wait on mbarriers with a limit; when it runs out they set the pinned status word and
    return. Here a one-thread kernel of the test, built from the same header with a limit of 100,000 cycles, waits
    on a barrier nobody arrives at: it must come back within milliseconds, and the host must raise."""
    import ctypes
    import os
    import time

    from etalii.dllm_b200.kernels.build import compile_extra

    source = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "bounded_wait_probe.cu")
    lib = compile_extra(source, flags=("-DDLLM_WAIT_LIMIT_CYCLES=100000ll",))
    lib.probe_wait_limit.restype = ctypes.c_longlong
    assert lib.probe_wait_limit() == 100000
    lib.probe_wait_that_runs_out.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    lib.probe_wait_that_runs_out.restype = ctypes.c_int
    module = ops()
    module.raise_if_failed()
    word = module._status_word()
    cycles = torch.zeros(1, dtype=torch.int64, device=DEV)
    torch.cuda.synchronize()
    began = time.perf_counter()
    assert lib.probe_wait_that_runs_out(word.data_ptr(), cycles.data_ptr(), module._stream()) == 0
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - began
    assert elapsed < 0.5, f"the wait took {elapsed:.3f} s"
    assert 100000 < int(cycles[0]) < 50_000_000
    with pytest.raises(module.KernelError, match="gave up waiting"):
        module.raise_if_failed()
    module.raise_if_failed()  # reported once
    # the context is as usable as before
    x = torch.arange(8, device=DEV, dtype=torch.float32)
    assert float((x * 2).sum()) == 56.0


@pytest.mark.parametrize("m,hidden,inter", [(1, 64, 160), (8, 576, 1536), (3, 144, 384), (16, 40, 48), (12, 72, 208),
                                            (5, 2048, 1024), (9, 576, 1536), (8, 104, 16)])
def test_mlp_decode_fused_feed_forward(m, hidden, inter):
    """The one-kernel feed-forward of decode steps against the plain computation (float64 from the same inputs) and
    against the two separate kernels it replaces; a repeated launch gives the same bits (the clusters' partial sums
    are added in a fixed order) and the tickets are left at zero."""
    x0 = _randn((m, hidden), torch.float32, 1, 2.0)
    norm_w = _randn((hidden,), torch.float32, 2, 0.1) + 1
    w_gu = _randn((2 * inter, hidden), torch.bfloat16, 3, 0.08)
    w_d = _randn((hidden, inter), torch.bfloat16, 4, 0.08)
    eps = 1e-5
    scratch = torch.full((ops().mlp_decode_scratch(m, hidden, inter),), float("nan"), dtype=torch.float32, device=DEV)
    tickets = torch.zeros(8, dtype=torch.int32, device=DEV)
    want = x0.clone()
    PK.mlp_decode(want, norm_w, eps, w_gu, w_d)
    got = x0.clone()
    ops().mlp_decode(got, norm_w, eps, w_gu, w_d, scratch, tickets)
    update = (want - x0).abs().max().item()
    assert (got - want).abs().max().item() <= 1.5e-2 * update
    assert int(tickets.abs().sum()) == 0
    again = x0.clone()
    ops().mlp_decode(again, norm_w, eps, w_gu, w_d, scratch, tickets)
    assert torch.equal(again, got)
    # the two kernels it replaces: the same roundings (normed input and activations in bfloat16), other sum orders
    act = torch.empty((m, inter), dtype=torch.bfloat16, device=DEV)
    ops().gemm(act, x0, w_gu, ops().EPI_SWIGLU, norm_weight=norm_w, eps=eps, kernel=2)
    two = x0.clone()
    ops().gemm(two, act, w_d, ops().EPI_RESIDUAL, kernel=2)
    assert (got - two).abs().max().item() <= 4e-3 * update
    # a row's result does not depend on its batch mates
    if m > 1:
        alone = x0[m - 1:].clone()
        ops().mlp_decode(alone, norm_w, eps, w_gu, w_d, scratch, tickets)
        assert torch.equal(alone[0], got[m - 1])


@pytest.mark.parametrize("m,n,k,normed", [(1, 384, 64, True), (8, 49153, 576, True), (16, 1000, 136, False),
                                          (5, 17, 72, False), (9, 4096, 2240, True)])
def test_head_argmax_chooses_what_the_logits_would(m, n, k, normed):
    """The greedy choice made inside the head product against the argmax of the stored logits of the same kernel
    (the same sums, so the same winner, ties included), at vocabularies that are no multiple of 16."""
    x = _randn((m, k), torch.float32 if normed else torch.bfloat16, 1)
    w = _randn((n, k), torch.bfloat16, 2, 0.1)
    w[n // 2] = w[3]            # two features with equal logits in every row ...
    x[0] = 0                    # ... and a row whose logits are all equal (zero): the lowest index wins
    if m > 2:
        x[2, 0] = float("nan")  # a row without any number: token 0, as the sampler answers it
    nw = _randn((k,), torch.float32, 3, 0.1) + 1 if normed else None
    logits = torch.empty((m, n), dtype=torch.float32, device=DEV)
    ops().gemm(logits, x, w, ops().EPI_STORE_F32, kernel=2, norm_weight=nw, eps=1e-5)
    want = torch.empty(m, dtype=torch.int32, device=DEV)
    ops().sample(want, logits, None, None, None, 0.0)
    got = torch.full((m,), -1, dtype=torch.int32, device=DEV)
    scratch = torch.full((ops().head_argmax_scratch(m, n),), float("nan"), dtype=torch.float32, device=DEV)
    ops().head_argmax(got, x, w, scratch, norm_weight=nw, eps=1e-5)
    assert got.tolist() == want.tolist()
    assert got[0].item() == 0 and (m <= 2 or got[2].item() == 0)
    finite = [r for r in range(m) if r not in (0, 2)]
    assert got[finite].tolist() == logits[finite].argmax(dim=1).tolist()


@pytest.mark.parametrize("m,hidden,inner,outputs", [
    (130, 576, 1536, 256), (300, 144, 96, 256), (2048, 576, 576, 256), (65, 2048, 512, 256),
    (2048, 2048, 256, 3072),   # 256-wide tiles for both products: their epilogues go through shared memory
    (4100, 576, 320, 256),     # more 64-wide tiles than blocks: persistent blocks, the rows staged behind the ring
])
def test_tile_products_with_the_norm_folded_around_them(m, hidden, inner, outputs):
    """x += a W^T with the bfloat16 copy and the sums of squares of the new rows from the epilogue, then a product
    that reads the copy and scales its rows: together RMSNorm(x) W2^T without a norm kernel. Against float64."""
    x0 = _randn((m, hidden), torch.float32, 1, 2.0)
    a = _randn((m, inner), torch.bfloat16, 2)
    w = _randn((hidden, inner), torch.bfloat16, 3, 0.05)
    x = x0.clone()
    copy = torch.full((m, hidden), float("nan"), dtype=torch.bfloat16, device=DEV)
    ssq = torch.full((m * (-(-hidden // 16)),), float("nan"), dtype=torch.float32, device=DEV)
    parts = ops().gemm_residual_norm(x, copy, ssq, a, w)
    want_x = x0.double() + a.double() @ w.double().T
    assert rel_error(x.cpu(), want_x.cpu()) <= 2e-5
    assert torch.equal(copy, x.to(torch.bfloat16))
    sums = ssq[: m * parts].view(parts, m).sum(dim=0)
    assert rel_error(sums.cpu(), (x.double() ** 2).sum(dim=1).cpu()) <= 1e-5
    # the reader: SwiGLU and plain stores of (norm(x) * weight) @ w2^T with the weight folded into w2's columns
    eps = 1e-5
    norm_w = _randn((hidden,), torch.float32, 4, 0.1) + 1
    w2 = _randn((outputs, hidden), torch.bfloat16, 5, 0.05)
    folded = (w2.float() * norm_w[None, :]).to(torch.bfloat16)
    normed = x.double() / torch.sqrt((x.double() ** 2).mean(dim=1, keepdim=True) + eps)
    prod = normed @ folded.double().T
    got = torch.empty((m, outputs), dtype=torch.float32, device=DEV)
    ops().gemm_normed(got, copy, folded, ops().EPI_STORE_F32, ssq, parts, eps)
    assert rel_error(got.cpu(), prod.float().cpu()) <= 8e-3
    act = torch.empty((m, outputs // 2), dtype=torch.bfloat16, device=DEV)
    ops().gemm_normed(act, copy, folded, ops().EPI_SWIGLU, ssq, parts, eps)
    gate, up = prod[:, 0::2], prod[:, 1::2]
    assert rel_error(act.float().cpu(), (gate * torch.sigmoid(gate) * up).float().cpu()) <= 1.2e-2
    # a step's first rows: the cast kernel gives the copy and one sum a row
    copy1 = torch.empty_like(copy)
    ssq1 = torch.empty(m, dtype=torch.float32, device=DEV)
    ops().cast_ssq(copy1, ssq1, x)
    assert torch.equal(copy1, copy) and rel_error(ssq1.cpu(), sums.cpu()) <= 1e-6
    again = torch.empty_like(got)
    ops().gemm_normed(again, copy1, folded, ops().EPI_STORE_F32, ssq1, 1, eps)
    assert rel_error(again.cpu(), got.cpu()) <= 1e-5
    ops().raise_if_failed()
