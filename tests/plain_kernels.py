"""Plain PyTorch restatements of each kernel, with the kernels' own signatures (etalii/dllm_b200/kernels/ops.py).
They compute in float64 from the given inputs and round once to the output type; the GPU tests compare every kernel
with its function here, at sizes other than the engine's. They share no code with the kernels."""
from __future__ import annotations

import torch

import plain_llama as P

EPI_STORE_F32, EPI_STORE_T, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3


def embed(out, table, tokens, status):
    ids = tokens[: out.shape[0]].long()
    bad = (ids < 0) | (ids >= table.shape[0])
    if bad.any():
        status[0] = 64
    rows = table[ids.clamp(0, table.shape[0] - 1)].float()
    rows[bad] = 0
    out.copy_(rows)


def rmsnorm(out, x, weight, eps, rows=None):
    src = x if rows is None else x[rows[: out.shape[0]].long()]
    src = src[: out.shape[0]].double()
    inv = 1.0 / torch.sqrt((src * src).mean(dim=-1, keepdim=True) + eps)
    out.copy_((src * inv * weight.double()).to(out.dtype))


def gemm(c, a, w, epilogue=EPI_STORE_T, kernel=0, norm_weight=None, eps=0.0):
    if norm_weight is not None:
        normed = torch.empty(a.shape, dtype=torch.float64, device=a.device)
        rmsnorm(normed, a, norm_weight, eps)
        a = normed
    prod = a.double() @ w.double().T
    if epilogue == EPI_RESIDUAL:
        c.copy_((c.double() + prod).float())
    elif epilogue == EPI_SWIGLU:
        gate, up = prod[:, 0::2], prod[:, 1::2]
        act = (gate * torch.sigmoid(gate)).float()
        c.copy_((act * up.float()).to(c.dtype))
    else:
        c.copy_(prod.to(c.dtype))


def mlp_decode_supported(rows, hidden, intermediate):
    return False


def mlp_decode(x, norm_weight, eps, w_gate_up, w_down, scratch=None, tickets=None):
    """x += down(silu(gate(h)) * up(h)) with h = RMSNorm(x): in float64 from the inputs, rounded once."""
    xd = x.double()
    h = xd / torch.sqrt((xd * xd).mean(dim=-1, keepdim=True) + eps) * norm_weight.double()
    prod = h @ w_gate_up.double().T
    gate, up = prod[:, 0::2], prod[:, 1::2]
    x.copy_((xd + (gate * torch.sigmoid(gate) * up) @ w_down.double().T).float())


def _kv(cache):
    return cache.storage  # [pages, 2, kv_heads, page_size, head_dim]


def rope_cache_write(qkv, q_out, cache, table, rotary_dim, heads, batch, write_cache=True):
    n, hd, nkv = batch.n_tokens, cache.head_dim, cache.kv_heads
    x = qkv[:n].double().view(n, heads + 2 * nkv, hd)
    pos = batch.tok_pos[:n].long()
    rotated = x.clone()
    if table is not None:
        half = rotary_dim // 2
        cs = table[pos].double()  # [n, half, 2]
        c, s = cs[:, None, :, 0], cs[:, None, :, 1]
        a, b = x[:, : heads + nkv, :half], x[:, : heads + nkv, half:rotary_dim]
        rotated[:, : heads + nkv, :half] = a * c - b * s
        rotated[:, : heads + nkv, half:rotary_dim] = a * s + b * c
    q_out[:n].copy_(rotated[:, :heads].reshape(n, heads * hd).to(q_out.dtype))
    if not write_cache:
        return
    slots = batch.slots[batch.tok_seq[:n].long()].long()
    pages = cache.page_table[slots, pos // cache.page_size].long()
    row = pos % cache.page_size
    store = _kv(cache)
    store[pages, 0, :, row] = rotated[:, heads:heads + nkv].to(store.dtype)
    store[pages, 1, :, row] = rotated[:, heads + nkv:].to(store.dtype)


def attention_general(out, q, cache, heads, scale, window, batch):
    n, hd, nkv = batch.n_tokens, cache.head_dim, cache.kv_heads
    group = heads // nkv
    store = _kv(cache).double()
    qd = q[:n].double().view(n, heads, hd)
    for t in range(n):
        pos = int(batch.tok_pos[t])
        slot = int(batch.slots[int(batch.tok_seq[t])])
        end = pos + 1
        first = end - window if window and end > window else 0
        js = torch.arange(first, end)
        pages = cache.page_table[slot, js // cache.page_size].long()
        rows = js % cache.page_size
        keys = store[pages, 0, :, rows]  # [count, nkv, hd]
        values = store[pages, 1, :, rows]
        for h in range(heads):
            g = h // group
            scores = (keys[:, g] @ qd[t, h]) * scale
            p = torch.softmax(scores, dim=0)
            out[t, h * hd:(h + 1) * hd] = (p @ values[:, g]).to(out.dtype)


def add_residual(residual, update):
    residual.add_(update.float().view_as(residual))


class _Rng:
    """Device-side state layout of the sampler: 4 words per row, as signed 64-bit patterns."""

    @staticmethod
    def load(rng, row):
        r = P.Random(0)
        r.s = [int(v) % (1 << 64) for v in rng[row].tolist()]
        return r

    @staticmethod
    def store(rng, row, r):
        rng[row] = torch.tensor([v - (1 << 64) if v >= (1 << 63) else v for v in r.s], dtype=torch.int64)


def sample(out_tokens, logits, scratch, rng, rng_rows, temperature, top_k=0, top_p=1.0, min_p=0.0):
    for r in range(logits.shape[0]):
        row = logits[r].float().cpu().numpy()
        if temperature == 0:
            out_tokens[r] = P.argmax(row)
            continue
        state_row = int(rng_rows[r])
        random = _Rng.load(rng.cpu(), state_row)
        out_tokens[r] = P.sample(row, random, temperature, top_k, top_p, min_p)
        fresh = rng.cpu()
        _Rng.store(fresh, state_row, random)
        rng.copy_(fresh)


def seed_rng(rng, rows, seeds):
    fresh = rng.cpu()
    for row, seed in zip(rows.tolist(), seeds.tolist()):
        _Rng.store(fresh, row, P.Random(int(seed) % (1 << 64)))
    rng.copy_(fresh)


def decode_advance(tokens, tok_pos, start, chosen, history, counter, batch):
    row = int(counter[0])
    tokens[:batch] = chosen[:batch]
    tok_pos[:batch] += 1
    start[:batch] += 1
    if row < history.numel() // batch:
        history[row * batch:(row + 1) * batch] = chosen[:batch]
    counter[0] = row + 1


def gemv_qkv_rope(a, w, q_out, cache, table, rotary_dim, heads, batch, write_cache=True, norm_weight=None, eps=0.0,
                  prefetch_window=-1):
    n = batch.n_tokens
    qkv = torch.empty((n, w.shape[0]), dtype=torch.float32, device=a.device)
    gemm(qkv, a[:n], w, EPI_STORE_F32, norm_weight=norm_weight, eps=eps)
    rope_cache_write(qkv, q_out, cache, table, rotary_dim, heads, batch, write_cache)


def attention_decode(out, q, cache, heads, scale, window, batch, chunk, scratch, tickets):
    attention_general(out, q, cache, heads, scale, window, batch)


def attention_prefill(out, q, cache, heads, scale, window, batch):
    attention_general(out, q, cache, heads, scale, window, batch)


def attention_prefill_supported(cache):
    return False


def gemm_qkv_rope(a, w, q_out, cache, table, rotary_dim, heads, batch, write_cache=True):
    gemv_qkv_rope(a, w, q_out, cache, table, rotary_dim, heads, batch, write_cache)


def gemm_qkv_rope_supported(cache, rotary_dim, has_table):
    return False


DECODE_CLUSTER_SHAPES = 5


def attention_decode_cluster(out, q, cache, heads, scale, window, batch, shape=-1):
    attention_general(out, q, cache, heads, scale, window, batch)


def attention_prefill_tcgen05(out, q, cache, heads, scale, window, batch):
    attention_general(out, q, cache, heads, scale, window, batch)


def attention_prefill_tcgen05_supported(cache):
    return False


def attention_blocks_supported(cache):
    return True


def attention_blocks(out, q, cache, heads, scale, window, batch):
    attention_general(out, q, cache, heads, scale, window, batch)


def attention_decode_cluster_supported(cache):
    return False


def streams(rows, outputs):
    return rows <= 16 or (rows <= 32 and outputs <= 4096) or (rows <= 64 and outputs < 2048)


def takes_weights_as_rows(rows, outputs, inner):
    return False


def streams_through_shared_memory(rows, outputs, inner):
    return False


def sample_scratch(rows, vocab):
    return 3 * rows * vocab + 2
