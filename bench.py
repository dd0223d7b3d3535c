"""Measures decode and prefill throughput of the engine on one B200 and prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--repeats R] [--layers L] [--impl ours|reference]
                    [--shape smollm2-135m|smollm2-1.7b|llama-3.1-8b] [--batch B] [--no-points]
                    [--profile decode|prefill|kernels|ablate|ablate-fused|feed-forward|gemm|attention|stream|cluster|cut|sampling]

Default workload: the SmolLM2-135M shape (30 layers, hidden 576, 9 heads, 3 kv heads, head_dim 64, intermediate 1536,
vocabulary 49152, tied head) with seeded random bfloat16 weights; a batch of 8 sequences with unequal prompt lengths
(128 to 2,048 seeded random tokens) inside a context of 8,192. A "step" is one decode step of the whole batch
(model, greedy token choice, feedback), replayed as a CUDA graph. After one untimed run, R runs of exactly K steps are
timed with CUDA events, each from a fresh cache; `value` is decoded tokens per second at the mean step time, `sd` the
standard deviation over the runs (the reference's method: benchmarks/benchmark.py:209-216).
`e2e` is generated tokens per second of whole `Engine.generate` calls (wall clock around the call: prompt step,
decoding, host token lists in and out), mean and sd of R calls, with the call's prompt and decode parts.
`prefill` is one 2,048-token prompt in one step: `ms` as a user calls it, `host_ms` until the last launch is issued,
`device_ms` the same launches replayed as a CUDA graph. `roofline` relates the decode step to HBM bandwidth: every
weight read once plus the cache of the live sequences, over the step's time. `points` repeats the decode at batch 1
and 64, the end-to-end run with temperature sampling, and decode and prefill of the true 32-bit path (`fp32_*`, against
twice the bytes). `kernels` lists where the decode step's time goes, kind of launch by kind of launch.
`--impl reference` tries the reference's own pure-NumPy implementation on the same configuration (see `reference_arm`).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SMOLLM2_135M = {
    "model_type": "llama", "num_hidden_layers": 30, "hidden_size": 576, "num_attention_heads": 9,
    "num_key_value_heads": 3, "head_dim": 64, "intermediate_size": 1536, "vocab_size": 49152,
    "rope_theta": 100000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 8192,
    "hidden_act": "silu", "bos_token_id": 1, "eos_token_id": 2,
}
SHAPES = {
    "smollm2-135m": ("SmolLM2-135M", SMOLLM2_135M),
    # the two larger shapes of the same architecture (not the default run; `--layers` keeps a slice of them small)
    "smollm2-1.7b": ("SmolLM2-1.7B", dict(
        SMOLLM2_135M, num_hidden_layers=24, hidden_size=2048, num_attention_heads=32, num_key_value_heads=32,
        head_dim=64, intermediate_size=8192, rope_theta=130000.0)),
    "llama-3.1-8b": ("Llama-3.1-8B", dict(
        SMOLLM2_135M, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
        head_dim=128, intermediate_size=14336, vocab_size=128256, rope_theta=500000.0, tie_word_embeddings=False,
        rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                      "original_max_position_embeddings": 8192})),
}
FULL_LAYERS = SMOLLM2_135M["num_hidden_layers"]
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as handle:
            data = json.load(handle)
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]), "source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.process = [], None

    def __enter__(self):
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            self.samples.append([part.strip() for part in line.split(",")])

    def __exit__(self, *exc):
        if self.process is not None:
            time.sleep(0.15)
            self.process.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        clocks = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({name for s in self.samples if len(s) >= 6
                          for name, flag in zip(names, s[2:6]) if flag.lower().startswith("active")})
        top = max((int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()), default=None)
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None, "sm_max_mhz": top, "reasons": reasons,
                "samples": len(clocks)}


def make_prompts(batch, vocab, seed):
    import numpy as np

    rng = np.random.default_rng(seed)
    lengths = rng.integers(128, PREFILL_TOKENS + 1, batch).tolist()
    lengths[0] = PREFILL_TOKENS if batch > 1 else 1088  # the longest length is always present; batch 1: the mean
    return [rng.integers(0, vocab, n).tolist() for n in lengths]


def decode_run(engine, prompts, steps, warmup):
    """Device-timed decode: returns (milliseconds for `steps` steps, launches per step, cached tokens at the end)."""
    import torch

    from etalii.dllm_b200 import SamplingOptions

    slots = engine.open(len(prompts))
    tokens = []
    for begin in range(0, len(prompts), 8):  # prompts enter the cache eight at a time
        part = slice(begin, begin + 8)
        logits = engine.step(slots[part], prompts[part])
        tokens += engine.sampler.choose(logits, engine.last_batch.slots, SamplingOptions()).tolist()
    longest = max(len(p) for p in prompts) + warmup + steps + 1
    graph = engine._decode_graph(len(prompts), SamplingOptions(), longest)
    done = 0
    while done < warmup:  # warm-up steps (the first run also captures the graph)
        n = min(graph.CAPACITY, warmup - done)
        tokens = engine.decode(slots, tokens, n)[-1]
        done += n
    total_ms, done = 0.0, 0
    while done < steps:
        n = min(graph.CAPACITY, steps - done)
        engine.decode_start(graph, slots, tokens, n)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay(n)
        end.record()
        torch.cuda.synchronize()
        total_ms += begin.elapsed_time(end)
        tokens = graph.tokens(n)[-1]
        done += n
    cached = sum(engine.cache.length(s) for s in slots)
    engine.close(slots)
    return total_ms, graph.launches_per_step, cached


def prefill_run(engine, vocab, warmup, repeats=5):
    import numpy as np
    import torch

    prompt = np.random.default_rng(7).integers(0, vocab, PREFILL_TOKENS).tolist()
    times = []
    for index in range(warmup + repeats):
        slot = engine.open(1)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        engine.step(slot, [prompt])
        end.record()
        torch.cuda.synchronize()
        engine.close(slot)
        if index >= warmup:
            times.append(begin.elapsed_time(end))
    return sorted(times)[len(times) // 2]  # the median: the step is launched from Python, host jitter shows in the mean


def gemm_table() -> int:
    """Times the tile products alone (CUDA events around a CUDA graph of 20 dependent launches, warm) at layer shapes
    of the three model sizes: the tcgen05 kernel at each tile width and the mma.sync kernel, in TFLOP/s."""
    import torch

    from etalii.dllm_b200.kernels import ops

    def run(m, n, k, epilogue, tile_n, kernel):
        a = torch.randn(m, k, device="cuda:0").bfloat16()
        w = (torch.randn(n, k, device="cuda:0") * 0.05).bfloat16()
        cols = n // 2 if epilogue == ops.EPI_SWIGLU else n
        dtype = torch.float32 if epilogue in (ops.EPI_STORE_F32, ops.EPI_RESIDUAL) else torch.bfloat16
        c = torch.zeros(m, cols, device="cuda:0", dtype=dtype)
        for _ in range(3):
            ops.gemm(c, a, w, epilogue, kernel=kernel, tile_n=tile_n)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()  # 20 dependent launches without the host between them
        with torch.cuda.graph(graph):
            for _ in range(20):
                ops.gemm(c, a, w, epilogue, kernel=kernel, tile_n=tile_n)
        graph.replay()
        torch.cuda.synchronize()
        best = None
        for _ in range(3):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            ms = begin.elapsed_time(end) / 20
            best = ms if best is None else min(best, ms)
        ops.raise_if_failed()
        return best * 1e3, 2 * m * n * k / best / 1e9

    shapes = [(2048, 576, 576, ops.EPI_RESIDUAL), (2048, 576, 1536, ops.EPI_RESIDUAL), (2048, 3072, 576, ops.EPI_SWIGLU),
              (2048, 2048, 8192, ops.EPI_RESIDUAL), (2048, 16384, 2048, ops.EPI_SWIGLU),
              (2048, 4096, 4096, ops.EPI_RESIDUAL), (2048, 28672, 4096, ops.EPI_SWIGLU),
              (2048, 4096, 14336, ops.EPI_RESIDUAL), (8192, 4096, 4096, ops.EPI_STORE_T)]
    print("M N K epilogue | tcgen05 tile 32 | 64 | 128 | 256 | chosen | mma.sync   (microseconds, TFLOP/s)")
    for m, n, k, epilogue in shapes:
        cells = []
        for tile_n in (32, 64, 128, 256, 0):
            if tile_n and n % tile_n:
                cells.append("-")
                continue
            us, tf = run(m, n, k, epilogue, tile_n, 3)
            cells.append(f"{us:.1f} us {tf:.0f}")
        us, tf = run(m, n, k, epilogue, 0, 1)
        print(f"{m} {n} {k} {epilogue} | " + " | ".join(cells) + f" | {us:.1f} us {tf:.0f}")
    return 0


def attention_table() -> int:
    """Times the attention kernels alone (CUDA events; several caches in turn, larger than L2 together for the decode
    rows): the two prefill kernels on whole prompts, and the cluster decode kernel at every launch shape."""
    import torch

    from etalii.dllm_b200.cache.paged import CacheNeed, PagedCache
    from etalii.dllm_b200.engine.batch import BatchBuffers
    from etalii.dllm_b200.kernels import ops

    device = torch.device("cuda:0")

    def setup(heads, kv_heads, head_dim, lengths, new, layers):
        total = sum((n + 63) // 64 * 64 for n in lengths)
        cache = PagedCache([CacheNeed("kv", kv_heads, head_dim, None)] * layers, max_tokens=total + 64,
                           max_length=max(lengths) + 64, dtype=torch.bfloat16, device=device)
        slots = cache.acquire(len(lengths))
        for slot, n in zip(slots, lengths):
            cache.reserve(slot, n)
            cache.advance(slot, n)
        cache.sync_tables()
        views = [cache.kv_view(i) for i in range(layers)]
        for view in views:
            view.storage.normal_()
        batch = BatchBuffers(device).fill(slots, [[1] * k for k in new], [n - k for n, k in zip(lengths, new)],
                                          [[] for _ in lengths])
        q = torch.randn((batch.n_tokens, heads * head_dim), device=device).to(torch.bfloat16)
        return views, batch, q, torch.zeros_like(q)

    def time_us(call, views, reps=5):
        for _ in range(2):
            for view in views:
                call(view)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(reps):
            for view in views:
                call(view)
        end.record()
        torch.cuda.synchronize()
        ops.raise_if_failed()
        return begin.elapsed_time(end) * 1e3 / (reps * len(views))

    print("prefill: heads kv_heads head_dim prompts | mma.sync us | tcgen05 us, TFLOP/s")
    for heads, kv_heads, head_dim, lengths in (
            (9, 3, 64, [2048]), (9, 3, 64, [512]), (9, 3, 64, [8192]), (32, 8, 64, [2048]), (32, 8, 64, [4096, 4096]),
            (9, 3, 64, [300] * 16), (32, 8, 128, [512]), (32, 8, 128, [2048]), (32, 8, 128, [8192])):
        views, batch, q, out = setup(heads, kv_heads, head_dim, lengths, lengths, 4 if head_dim > 64 else 8)
        old = time_us(lambda v: ops.attention_prefill(out, q, v, heads, 0.125, 0, batch), views)
        new = time_us(lambda v: ops.attention_prefill_tcgen05(out, q, v, heads, 0.125, 0, batch), views)
        flops = sum(4 * heads * head_dim * n * (n + 1) / 2 for n in lengths)
        shown = lengths if len(lengths) < 4 else f"{len(lengths)} x {lengths[0]}"
        print(f"{heads} {kv_heads} {head_dim} {shown} | {old:.1f} | {new:.1f}, {flops / new / 1e6:.0f}")
    print("decode: heads kv_heads head_dim batch, MB of keys and values, us at the measured HBM rate | "
          "chosen shape us | shapes 0..4 us")
    bandwidth = peaks()["hbm_gbs"]
    for heads, kv_heads, head_dim in ((9, 3, 64), (32, 8, 128), (32, 32, 64)):
        for size in (1, 8, 64, 128):
            g = torch.Generator().manual_seed(size)
            lengths = [int(x) for x in torch.randint(128, 2304, (size,), generator=g)]
            layers = max(2, min(16, int(300e6 / (size * 1200 * 4 * kv_heads * head_dim)) + 1))
            views, batch, q, out = setup(heads, kv_heads, head_dim, lengths, [1] * size, layers)
            kv_bytes = sum(lengths) * 4 * kv_heads * head_dim
            cells = [time_us(lambda v: ops.attention_decode_cluster(out, q, v, heads, 0.125, 0, batch, shape), views)
                     for shape in range(-1, ops.DECODE_CLUSTER_SHAPES)]
            print(f"{heads} {kv_heads} {head_dim} {size}, {kv_bytes / 1e6:.1f} MB, {kv_bytes / bandwidth / 1e3:.1f} us | "
                  f"{cells[0]:.1f} | " + " ".join(f"{c:.1f}" for c in cells[1:]))
    return 0


def stream_table() -> int:
    """Times the decode products alone at layer shapes of the larger models, every kernel that can run them, as
    fractions of the measured HBM rate (a CUDA graph of 20 launches over several copies of W, so that W comes from
    HBM): the rules in `kernels/ops.py` that choose among them rest on these tables."""
    import torch

    from etalii.dllm_b200.kernels import ops

    device = "cuda:0"
    rate = peaks()["hbm_gbs"]

    def run(m, n, k, epilogue, kernel, cluster=0):
        copies = max(2, int(300e6 // (n * k * 2)) + 1)
        ws = [(torch.randn(n, k, device=device) * 0.05).bfloat16() for _ in range(copies)]
        x = torch.randn(m, k, device=device).bfloat16()
        cols = n // 2 if epilogue == ops.EPI_SWIGLU else n
        dtype = torch.float32 if epilogue in (ops.EPI_STORE_F32, ops.EPI_RESIDUAL) else torch.bfloat16
        c = torch.zeros(m, cols, device=device, dtype=dtype)
        for i in range(3):
            ops.gemm(c, x, ws[i % copies], epilogue, kernel=kernel, cluster=cluster)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(20):
                ops.gemm(c, x, ws[i % copies], epilogue, kernel=kernel, cluster=cluster)
        graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        ops.raise_if_failed()
        us = begin.elapsed_time(end) / 20 * 1e3
        return us, n * k * 2 / us / 1e3 / rate

    shapes = [(6144, 4096, ops.EPI_STORE_T), (4096, 4096, ops.EPI_RESIDUAL), (28672, 4096, ops.EPI_SWIGLU),
              (4096, 14336, ops.EPI_RESIDUAL), (128256, 4096, ops.EPI_STORE_F32), (6144, 2048, ops.EPI_STORE_T),
              (16384, 2048, ops.EPI_SWIGLU), (2048, 8192, ops.EPI_RESIDUAL), (49152, 2048, ops.EPI_STORE_F32),
              (49152, 576, ops.EPI_STORE_F32)]

    def cell(m, n, k, epilogue, kernel):
        us, fraction = run(m, n, k, epilogue, kernel)
        return f"{us:.1f} {fraction:.2f}"

    print("rows of activations, W rows x row length, epilogue | registers: us, of HBM | shared memory | tile kernel, "
          "W as its rows")
    for m in (1, 4, 8, 16):
        for n, k, epilogue in shapes:
            ring = cell(m, n, k, epilogue, 4) if k % 64 == 0 else "-"
            print(f"{m} {n} x {k} {epilogue} | {cell(m, n, k, epilogue, 2)} | {ring} | {cell(m, n, k, epilogue, 5)}")
    # 32 and 64 rows against matrices of few rows: a block per 16 rows of W, the tile kernel, the same with W as its
    # rows, the reduction split over a cluster, and W as rows with the reduction cut (residual products only)
    print("rows, W | registers | tile kernel | W as its rows | cluster | reduction cut in 2 | 4 | 8")
    narrow = [(4096, 4096, ops.EPI_RESIDUAL), (4096, 14336, ops.EPI_RESIDUAL), (2048, 2048, ops.EPI_RESIDUAL),
              (2048, 8192, ops.EPI_RESIDUAL), (6144, 4096, ops.EPI_STORE_T), (6144, 2048, ops.EPI_STORE_T)]
    for m in (32, 64):
        for n, k, epilogue in narrow:
            cells = [cell(m, n, k, epilogue, kernel) for kernel in (2, 3, 5, 6)]
            if epilogue == ops.EPI_RESIDUAL:
                for split in (2, 4, 8):
                    us, fraction = run(m, n, k, epilogue, 7, split)
                    cells.append(f"{us:.1f} {fraction:.2f}")
            print(f"{m} {n} x {k} {epilogue} | " + " | ".join(cells))
    return 0


def cut_reduction_case() -> int:
    """One narrow product with a long reduction and 64 rows (4096 x 14336, the residual epilogue) as the tile kernel
    runs it with the reduction cut into 8 stretches: a few launches over three copies of W, a small case for ncu."""
    import torch

    from etalii.dllm_b200.kernels import ops

    device = "cuda:0"
    m, n, k, split = 64, 4096, 14336, 8
    ws = [(torch.randn(n, k, device=device) * 0.05).bfloat16() for _ in range(3)]
    x = torch.randn(m, k, device=device).bfloat16()
    c = torch.zeros(m, n, device=device, dtype=torch.float32)
    for i in range(3):
        ops.gemm(c, x, ws[i % 3], ops.EPI_RESIDUAL, kernel=7, cluster=split)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for i in range(3):
        ops.gemm(c, x, ws[i % 3], ops.EPI_RESIDUAL, kernel=7, cluster=split)
    end.record()
    torch.cuda.synchronize()
    ops.raise_if_failed()
    us = begin.elapsed_time(end) / 3 * 1e3
    print(f"profile cut: {m} x {n} x {k} in {split} stretches, {us:.1f} us a product with its sum (launched one by "
          f"one), {n * k * 2 / us / 1e3:.0f} GB/s of weights")
    return 0


def sampling_table() -> int:
    """Times the token-choice kernel alone: rows of seeded random logits (standard deviation 3, or 12 for a peaked
    distribution), greedy and at temperature 0.8 without and with top-p and top-k, as 20 launches in a CUDA graph."""
    import torch

    from etalii.dllm_b200.kernels import ops

    device = "cuda:0"

    def run(rows, vocab, temperature, top_k=0, top_p=1.0, spread=3.0):
        generator = torch.Generator(device=device).manual_seed(rows + vocab)
        logits = torch.randn(rows, vocab, device=device, generator=generator) * spread
        out = torch.zeros(rows, dtype=torch.int32, device=device)
        scratch = torch.empty(ops.sample_scratch(rows, vocab), dtype=torch.float32, device=device)
        rng = torch.zeros(rows, 4, dtype=torch.int64, device=device)
        rng_rows = torch.arange(rows, dtype=torch.int32, device=device)
        ops.seed_rng(rng, rng_rows, torch.arange(rows, dtype=torch.int64, device=device) + 5)
        for _ in range(3):
            ops.sample(out, logits, scratch, rng, rng_rows, temperature, top_k, top_p)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(20):
                ops.sample(out, logits, scratch, rng, rng_rows, temperature, top_k, top_p)
        graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / 20 * 1e3

    print("rows x vocabulary | greedy | temperature 0.8 | + top-p 0.9 | + top-k 50 | temperature 0.8, peaked   (us)")
    for rows in (1, 8, 64):
        for vocab in (49152, 128256):
            print(f"{rows} x {vocab} | {run(rows, vocab, 0.0):.1f} | {run(rows, vocab, 0.8):.1f} | "
                  f"{run(rows, vocab, 0.8, 0, 0.9):.1f} | {run(rows, vocab, 0.8, 50):.1f} | "
                  f"{run(rows, vocab, 0.8, spread=12.0):.1f}", flush=True)
    return 0


def cluster_table(rows: int) -> int:
    """Times the products of a step of 9 to 64 rows at the layer shapes of a 576-wide model, as links of a chain of
    30 dependent launches in a CUDA graph: the kernel with a block per 16 rows of W against the one that splits the
    reduction over a thread-block cluster, at every cluster size."""
    import torch

    from etalii.dllm_b200.kernels import ops

    device = "cuda:0"
    shapes = [("output", 576, 576, ops.EPI_RESIDUAL, False), ("down", 576, 1536, ops.EPI_RESIDUAL, False),
              ("gate/up + norm", 3072, 576, ops.EPI_SWIGLU, True), ("960 x 576 + norm", 960, 576, ops.EPI_STORE_T, True)]
    links = 30
    print(f"{rows} rows | a block per 16 rows of W | cluster of 1 | 2 | 4 | 8   (microseconds per launch)")
    for name, n, k, epilogue, normed in shapes:
        ws = [(torch.randn(n, k, device=device) * 0.05).bfloat16() for _ in range(8)]
        x = torch.randn(rows, k, device=device)
        x = x if normed else x.bfloat16()
        norm_weight = torch.ones(k, device=device) if normed else None
        cols = n // 2 if epilogue == ops.EPI_SWIGLU else n
        dtype = torch.float32 if epilogue == ops.EPI_RESIDUAL else torch.bfloat16
        c = torch.zeros(rows, cols, device=device, dtype=dtype)
        cells = []
        for kernel, cluster in ((2, 0), (6, 1), (6, 2), (6, 4), (6, 8)):
            if cluster > (4 if rows <= 16 else 8):
                continue

            def chain():
                for i in range(links):
                    ops.gemm(c, x, ws[i % 8], epilogue, kernel=kernel, cluster=cluster, norm_weight=norm_weight,
                             eps=1e-5)

            chain()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                chain()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            for _ in range(20):
                graph.replay()
            end.record()
            torch.cuda.synchronize()
            cells.append(f"{begin.elapsed_time(end) * 1e3 / (20 * links):.2f}")
        print(f"{name} {n} x {k} | " + " | ".join(cells))
    ops.raise_if_failed()
    return 0


def model_numbers(config, layers):
    h, i, v = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    nh, nkv, hd = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    per_layer = h * (nh + 2 * nkv) * hd + nh * hd * h + 3 * h * i
    matrix_params = layers * per_layer
    norm_params = (2 * layers + 1) * h
    kv_values_per_token = layers * 2 * nkv * hd
    t = PREFILL_TOKENS
    prefill_flops = 2 * matrix_params * t + layers * 4 * hd * nh * t * (t + 1) // 2 + 2 * h * v
    return {"matrix_params": matrix_params, "head_params": v * h, "norm_params": norm_params,
            "kv_values_per_token": kv_values_per_token, "prefill_flops": prefill_flops}


def step_bytes(numbers, element_bytes, cached_tokens):
    """Bytes a decode step has to read: every weight once (matrices and head in the model's dtype, norms float32)
    and the keys and values of the live sequences."""
    weights = element_bytes * (numbers["matrix_params"] + numbers["head_params"]) + 4 * numbers["norm_params"]
    return weights, weights + cached_tokens * numbers["kv_values_per_token"] * element_bytes


def decode_point(engine, prompts, steps, warmup, repeats):
    """`repeats` device-timed runs of `steps` decode steps after one untimed run (the reference's method,
    benchmarks/benchmark.py:209-216: one warm-up, mean and sd of the repetitions, a fresh cache each time)."""
    from etalii.dllm_b200.measure import mean_sd

    decode_run(engine, prompts, min(4, steps), 3)  # builds kernels, work buffers and the graph before anything is timed
    runs = [decode_run(engine, prompts, steps, warmup) for _ in range(repeats)]
    ms, sd = mean_sd([r[0] / steps for r in runs])
    return {"ms_per_step": ms, "sd_ms": sd, "launches_per_step": runs[-1][1], "cached": runs[-1][2],
            "tokens_per_s": len(prompts) / (ms / 1e3),
            "sd": mean_sd([len(prompts) * steps / (r[0] / 1e3) for r in runs])[1]}


def prefill_point(engine, vocab, warmup, repeats=5):
    """One prompt of PREFILL_TOKENS tokens in one step: device time by CUDA events around the step as a user calls
    it (median of `repeats`), the host's time until the last launch is issued, and the device time of the same
    launches replayed as a CUDA graph (no host between the kernels)."""
    import numpy as np
    import torch

    prompt = np.random.default_rng(7).integers(0, vocab, PREFILL_TOKENS).tolist()
    times, host = [], []
    for index in range(warmup + repeats):
        slot = engine.open(1)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        began = time.perf_counter()
        begin.record()
        engine.step(slot, [prompt])
        issued = time.perf_counter()
        end.record()
        torch.cuda.synchronize()
        engine.close(slot)
        if index >= warmup:
            times.append(begin.elapsed_time(end))
            host.append((issued - began) * 1e3)
    slot = engine.open(1)
    engine.step(slot, [prompt])
    batch = engine.last_batch
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        engine.model.forward(batch)
    device = []
    for _ in range(repeats + 1):
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        device.append(begin.elapsed_time(end))
    engine.close(slot)
    engine.check()
    median = lambda values: sorted(values)[len(values) // 2]  # noqa: E731
    return {"ms": median(times), "host_ms": median(host), "device_ms": median(device[1:])}


def kernel_shares(engine, prompts, steps=3):
    """Where a decode step's time goes, kernel by kernel: the step run launch by launch (no graph) with a CUDA event
    behind every launch; the share of each kind of launch in the sum, and its mean time (an event between two
    kernels keeps the second from starting under the first's tail, so the sum is above the graph's step time)."""
    import torch

    from etalii.dllm_b200 import SamplingOptions
    from etalii.dllm_b200.engine.decode import DecodeGraph
    from etalii.dllm_b200.kernels import ops

    slots = engine.open(len(prompts))
    tokens = []
    for begin in range(0, len(prompts), 8):
        part = slice(begin, begin + 8)
        logits = engine.step(slots[part], prompts[part])
        tokens += engine.sampler.choose(logits, engine.last_batch.slots, SamplingOptions()).tolist()
    run = DecodeGraph(engine, len(prompts), SamplingOptions(), use_graph=False,
                      max_context=max(len(p) for p in prompts) + 64)
    engine.decode_start(run, slots, tokens, steps + 2)
    run.replay(2)
    torch.cuda.synchronize()
    totals, counts = {}, {}
    for _ in range(steps):
        # The stream is held busy first (a kernel that spins for about 10 ms) while the host issues the whole step
        # with an event behind every launch; the step's kernels then run back to back, as in a graph, and the
        # events are as far apart as the kernels take, not as the host needs to launch them.
        torch.cuda._sleep(20_000_000)
        ops.trace = []
        before = torch.cuda.Event(enable_timing=True)
        before.record()
        run.replay(1)
        torch.cuda.synchronize()
        events, ops.trace = ops.trace, None
        for name, event in events:
            totals[name] = totals.get(name, 0.0) + before.elapsed_time(event)
            counts[name] = counts.get(name, 0) + 1
            before = event
    engine.close(slots)
    whole = sum(totals.values())
    return {name: {"share": round(totals[name] / whole, 4), "launches_per_step": round(counts[name] / steps, 1),
                   "us": round(totals[name] / counts[name] * 1e3, 2)}
            for name in sorted(totals, key=lambda n: -totals[n])}


def ablation_table(engine, prompts, layers, fused_feed_forward=False) -> int:
    """What each kind of launch costs inside the decode step: the step's CUDA graph timed whole and with one kind of
    launch left out (the results are then wrong, the timing is what is read). Printed per layer."""
    from etalii.dllm_b200.kernels import ops

    ops.FUSED_FEED_FORWARD = fused_feed_forward
    real = {name: getattr(ops, name) for name in ("gemv_qkv_rope", "attention_decode_cluster", "gemm", "mlp_decode",
                                                  "head_argmax")}

    def run(label):
        engine._graphs.clear()
        ms, launches, _ = decode_run(engine, prompts, 64, 3)
        print(f"{label}: {ms / 64 * 1e3:.1f} us per step, {launches} launches", flush=True)
        return ms / 64 * 1e3

    full = run("full step")

    def without(label, per=layers, **patch):
        for name, function in patch.items():
            setattr(ops, name, function)
        try:
            t = run("without " + label)
        finally:
            for name in patch:
                setattr(ops, name, real[name])
        print(f"   -> {label}: {(full - t) / per:.2f} us per {'layer' if per == layers else 'step'}", flush=True)

    def nothing(*args, **kwargs):
        return None

    def gemm_without(leave_out):
        def gemm(c, a, w, epilogue=1, **kwargs):
            if leave_out(w, epilogue):
                return None
            return real["gemm"](c, a, w, epilogue, **kwargs)
        return gemm

    hidden = engine.model.hidden_size
    without("attention", attention_decode_cluster=nothing)
    without("q/k/v product", gemv_qkv_rope=nothing)
    without("output product", gemm=gemm_without(lambda w, e: e == ops.EPI_RESIDUAL and w.shape[1] == hidden))
    if fused_feed_forward:
        without("feed-forward (one kernel)", mlp_decode=nothing)
    else:
        without("gate/up product", gemm=gemm_without(lambda w, e: e == ops.EPI_SWIGLU))
        without("down product", gemm=gemm_without(lambda w, e: e == ops.EPI_RESIDUAL and w.shape[1] != hidden))
    without("head product and choice", per=1, head_argmax=nothing)
    ops.FUSED_FEED_FORWARD = False
    return 0


def feed_forward_chain(config_dict, rows=8, links=30) -> int:
    """The one-kernel feed-forward against the two kernels it replaces, each as a chain of `links` dependent launches
    with weights of their own (more than L2 holds together) in a CUDA graph: microseconds per link."""
    import torch

    from etalii.dllm_b200.kernels import ops

    device = "cuda:0"
    hidden, inter = config_dict["hidden_size"], config_dict["intermediate_size"]
    torch.manual_seed(0)
    x = torch.randn(rows, hidden, device=device)
    norm_w = torch.ones(hidden, device=device)
    gate_up = [(torch.randn(2 * inter, hidden, device=device) * 0.05).bfloat16() for _ in range(links)]
    down = [(torch.randn(hidden, inter, device=device) * 0.05).bfloat16() for _ in range(links)]
    scratch = torch.zeros(ops.mlp_decode_scratch(rows, hidden, inter), device=device)
    tickets = torch.zeros(8, dtype=torch.int32, device=device)
    act = torch.zeros(rows, inter, device=device, dtype=torch.bfloat16)

    def timed(body, name):
        for _ in range(2):
            body()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            body()
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(5):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end) * 1e3 / links)
        print(f"{name}: {min(times):.2f} us per link ({rows} rows, hidden {hidden}, intermediate {inter})", flush=True)

    def two_kernels():
        for i in range(links):
            ops.gemm(act, x, gate_up[i], ops.EPI_SWIGLU, norm_weight=norm_w, eps=1e-5)
            ops.gemm(x, act, down[i], ops.EPI_RESIDUAL)

    def one_kernel():
        for i in range(links):
            ops.mlp_decode(x, norm_w, 1e-5, gate_up[i], down[i], scratch, tickets)

    timed(two_kernels, "norm + gate/up + SwiGLU, then down + residual (two kernels)")
    timed(one_kernel, "the same in one kernel")
    return 0


REFERENCE_BUDGET_S = 150.0


def reference_worker(budget_s: float) -> int:
    """Runs in a process of its own with only the reference's sources on the path: the reference's pure-NumPy
    second implementation (`etalii_dllm.reference.ReferenceTransformer`, its stock code path) on the benchmark's
    configuration, float32, the same eight prompts; prints one JSON line of what it managed within the budget."""
    import numpy as np

    import etalii_dllm.reference as ref
    from etalii_dllm.architecture import TransformerConfig

    c = SMOLLM2_135M
    config = TransformerConfig(
        family="llama", vocabulary_size=c["vocab_size"], hidden_size=c["hidden_size"],
        intermediate_size=c["intermediate_size"], layers=c["num_hidden_layers"], heads=c["num_attention_heads"],
        kv_heads=c["num_key_value_heads"], head_dim=c["head_dim"], context_length=c["max_position_embeddings"],
        rms_norm_eps=c["rms_norm_eps"], rope_theta=c["rope_theta"], rope_scaling=None,
        tie_word_embeddings=c["tie_word_embeddings"], eos_token_ids=(c["eos_token_id"],))
    rng = np.random.default_rng(0)
    tensors = {}
    for name, shape in config.tensor_shapes().items():
        norm = name.endswith("norm.weight")
        tensors[name] = (rng.standard_normal(shape, dtype=np.float32) * np.float32(0.01 if norm else 0.02)
                         + np.float32(1.0 if norm else 0.0))
    model = ref.ReferenceTransformer(config, tensors)
    prompts = make_prompts(8, c["vocab_size"], seed=1)
    began = time.perf_counter()
    fed, decoded, decode_s = 0, 0, 0.0
    # the reference holds one sequence at a time: prompt by prompt, shortest first, 16 tokens a call
    for prompt in sorted(prompts, key=len):
        model.reset()
        for at in range(0, len(prompt), 16):
            if time.perf_counter() - began > budget_s:
                break
            logits = model.forward(prompt[at:at + 16])
            fed += len(prompt[at:at + 16])
        else:
            token = int(np.argmax(logits))
            while time.perf_counter() - began <= budget_s and decoded < 64:
                t0 = time.perf_counter()
                token = int(np.argmax(model.forward([token])))
                decode_s += time.perf_counter() - t0
                decoded += 1
            continue
        break
    print(json.dumps({"seconds": round(time.perf_counter() - began, 1), "prompt_tokens_fed": fed,
                      "prompt_tokens_total": sum(len(p) for p in prompts), "decoded": decoded,
                      "decode_s": round(decode_s, 3)}))
    return 0


def reference_arm(args) -> int:
    """`--impl reference`: the reference cannot be installed here (its native engine needs nanobind, which the
    offline wheelhouse does not have), but its pure-NumPy second implementation runs from a copy of its sources
    under baseline/_ref. It is tried on the benchmark's configuration with a time budget; what it managed is
    reported. It goes through no file of this library."""
    where = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isfile(os.path.join(where, "etalii_dllm", "reference.py")):
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference does not install offline (pip: no numpy in the wheelhouse; --no-deps: the "
                          "CMake build needs nanobind, which is not installed), and no copy of its Python sources "
                          "is under baseline/_ref"}))
        return 0
    budget = float(os.environ.get("DLLM_B200_REFERENCE_BUDGET_S", REFERENCE_BUDGET_S))
    env = dict(os.environ, PYTHONPATH=where)
    began = time.perf_counter()
    try:
        done = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-worker",
                               "--budget", str(budget)], env=env, capture_output=True, text=True,
                              timeout=budget + 240)
        report = json.loads(done.stdout.strip().splitlines()[-1])
    except Exception as error:  # a failed import, a timeout, no JSON
        print(json.dumps({"impl": "reference", "unavailable":
                          f"the reference's pure-NumPy implementation did not run: {type(error).__name__}: "
                          f"{str(error)[:160]} (after {time.perf_counter() - began:.0f} s)"}))
        return 0
    if report["decoded"] >= 8 and report["prompt_tokens_fed"] >= report["prompt_tokens_total"]:
        # every prompt was fed and decoded: one sequence at a time is how the reference's second implementation
        # runs, so the batch's tokens per second is its single-sequence rate
        value = report["decoded"] / report["decode_s"]
        print(json.dumps({
            "impl": "reference (pure-NumPy second implementation, CPU, float32, one sequence at a time)",
            "metric": "decode tokens/s (SmolLM2-135M shape, batch 8, random weights)", "value": round(value, 3),
            "unit": "tokens/s", "n_gpus": args.gpus, "steps": report["decoded"], "warmup": 0,
            "ms_per_step": round(1e3 / value, 1), "higher_is_better": True, "dtype": "float32", "same_config": True,
            "data": "synthetic"}))
        return 0
    rate = report["prompt_tokens_fed"] / max(report["seconds"], 1e-9)
    hours = report["prompt_tokens_total"] / max(rate, 1e-9) / 3600
    print(json.dumps({"impl": "reference", "unavailable":
                      f"the reference's native engine does not install offline (no nanobind); its pure-NumPy second "
                      f"implementation (etalii_dllm.reference.ReferenceTransformer, float32, CPU) was run on the "
                      f"benchmark's configuration and cut after {report['seconds']:.0f} s: it had fed "
                      f"{report['prompt_tokens_fed']} of the batch's {report['prompt_tokens_total']} prompt tokens "
                      f"({rate:.2f} tokens/s, about {hours:.1f} h for the prompts alone) and decoded "
                      f"{report['decoded']} tokens of its shortest prompt"
                      + (f" at {report['decoded'] / report['decode_s']:.2f} tokens/s (one sequence; it holds one at a "
                         f"time)" if report["decoded"] and report["decode_s"] > 0 else "")}))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--repeats", type=int, default=5, help="timed repetitions of the decode run (mean and sd)")
    parser.add_argument("--shape", default="smollm2-135m", choices=sorted(SHAPES),
                        help="layer sizes: the default is the benchmark's; the others are larger shapes of the family")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the full model (named in config)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference", "reference-worker"))
    parser.add_argument("--budget", type=float, default=REFERENCE_BUDGET_S, help=argparse.SUPPRESS)
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 and the float32 points")
    parser.add_argument("--profile", choices=("decode", "prefill", "gemm", "attention", "stream", "cluster", "cut", "sampling", "kernels",
                                              "ablate", "ablate-fused", "feed-forward"),
                        help="run only a few decode steps (or one prefill) and print no JSON: a small case for ncu")
    args = parser.parse_args()
    if args.impl == "reference-worker":
        return reference_worker(args.budget)
    if args.impl == "reference":
        return reference_arm(args)
    if args.profile == "gemm":
        return gemm_table()
    if args.profile == "attention":
        return attention_table()
    if args.profile == "stream":
        return stream_table()
    if args.profile == "cluster":
        return cluster_table(args.batch if args.batch > 8 else 64)
    if args.profile == "cut":
        return cut_reduction_case()
    if args.profile == "sampling":
        return sampling_table()
    if args.gpus != 1:
        print(f"bench.py measures one GPU: --gpus {args.gpus} is not supported (this library runs on a single device)")
        return 2
    warmup = max(3, args.warmup)

    from etalii.dllm_b200 import SamplingOptions
    from etalii.dllm_b200.config.registry import config_from_dict
    from etalii.dllm_b200.engine.engine import Engine
    from etalii.dllm_b200.measure import measure_generation

    shape_name, shape = SHAPES[args.shape]
    full_layers = shape["num_hidden_layers"]
    args.layers = args.layers or full_layers
    config_dict = dict(shape, num_hidden_layers=args.layers)
    config = config_from_dict(config_dict)
    numbers = model_numbers(config_dict, args.layers)
    cache_tokens = 64 * (PREFILL_TOKENS + 64 * ((warmup + args.steps) // 64 + 3))
    engine = Engine.from_random(config, seed=0, dtype="bfloat16", device="cuda:0", max_tokens=cache_tokens,
                                max_length=config_dict["max_position_embeddings"])
    peak = peaks()
    vocab = config_dict["vocab_size"]

    prompts = make_prompts(args.batch, vocab, seed=1)
    if args.profile == "decode":
        ms, launches, _ = decode_run(engine, prompts, args.steps, 3)
        print(f"profile decode: {args.steps} steps, {ms / args.steps:.4f} ms per step, {launches} launches per step")
        return 0
    if args.profile == "prefill":
        print(f"profile prefill: {prefill_run(engine, vocab, warmup=1, repeats=1):.4f} ms")
        return 0
    if args.profile in ("ablate", "ablate-fused"):
        return ablation_table(engine, prompts, args.layers, fused_feed_forward=args.profile == "ablate-fused")
    if args.profile == "feed-forward":
        return feed_forward_chain(config_dict, rows=args.batch)
    if args.profile == "kernels":
        for name, row in kernel_shares(engine, prompts).items():
            print(f"{row['share'] * 100:5.1f} %  {row['launches_per_step']:5.1f} x {row['us']:7.2f} us  {name}")
        return 0
    with ClockSampler() as clocks:
        point = decode_point(engine, prompts, args.steps, warmup, args.repeats)
    ms_per_step = point["ms_per_step"]
    mean_cached = point["cached"] - args.batch * args.steps / 2  # halfway through the timed steps
    weight_bytes, bytes_per_step = step_bytes(numbers, 2, mean_cached)
    achieved = bytes_per_step / (ms_per_step / 1e3) / 1e9

    measured = prefill_point(engine, vocab, warmup=3)
    prefill = {"value": round(PREFILL_TOKENS / (measured["ms"] / 1e3), 1), "tokens": PREFILL_TOKENS,
               "ms": round(measured["ms"], 4),
               "frac": round(numbers["prefill_flops"] / (measured["ms"] / 1e3) / (peak["bf16_tflops"] * 1e12), 5),
               "host_ms": round(measured["host_ms"], 4), "device_ms": round(measured["device_ms"], 4)}

    # end to end through the public entry point: host token lists in, host token lists out, the wall clock around
    # the whole call (prompt step, decoding, results)
    whole = measure_generation(engine, prompts, args.steps + 1, SamplingOptions(), repeats=args.repeats)
    graph = next(g for g in engine._graphs.values() if g.b == args.batch)
    prompt_bytes = 4 * sum(len(p) for p in prompts)
    e2e = {"value": round(whole["tokens_per_s"], 1), "sd": round(whole["sd"], 1), "unit": "tokens/s",
           "what": "generated tokens / wall time of Engine.generate (prompts of 128-2048 tokens included)",
           "call_s": round(whole["call_s"], 5), "prefill_s": round(whole["prefill_s"], 5),
           "decode_s": round(whole["decode_s"], 5), "decode_only": round(whole["decode_tokens_per_s"], 1),
           # (no stop tokens in this run: the decode steps go in runs of up to DecodeGraph.CAPACITY, one load each)
           "h2d_bytes_per_step": round((prompt_bytes + graph.host.numel() * 4 * -(-args.steps // graph.CAPACITY))
                                       / (args.steps + 1), 1),
           "d2h_bytes_per_step": args.batch * 4}

    points = {}
    if not args.no_points:
        # the same end-to-end run with sampling on the device instead of greedy choice
        sampled = measure_generation(engine, prompts, args.steps + 1, SamplingOptions(temperature=0.8, seed=1),
                                     repeats=2)
        points["e2e_temperature_0.8"] = round(sampled["tokens_per_s"], 1)
        for name, batch in (("decode_b1", 1), ("decode_b64", 64)):
            other = decode_point(engine, make_prompts(batch, vocab, seed=2 + batch), args.steps, warmup, 3)
            points[name] = round(other["tokens_per_s"], 1)
            cached = other["cached"] - batch * args.steps / 2
            points[name + "_hbm_frac"] = round(step_bytes(numbers, 2, cached)[1] / (other["ms_per_step"] / 1e3) / 1e9
                                               / peak["hbm_gbs"], 4)
        kernels = kernel_shares(engine, prompts)
        del engine
        import gc

        import torch

        gc.collect()
        torch.cuda.empty_cache()
        # the true 32-bit path of the same model: float32 weights, cache and products (no tensor cores)
        steps32 = min(args.steps, 64)
        engine32 = Engine.from_random(config, seed=0, dtype="float32", device="cuda:0", max_tokens=cache_tokens,
                                      max_length=config_dict["max_position_embeddings"])
        for name, batch in (("fp32_decode_b1", 1), ("fp32_decode_b8", 8), ("fp32_decode_b64", 64)):
            other = decode_point(engine32, make_prompts(batch, vocab, seed=1 if batch == 8 else 2 + batch), steps32,
                                 3, 3)
            points[name] = round(other["tokens_per_s"], 1)
            cached = other["cached"] - batch * steps32 / 2
            points[name + "_hbm_frac"] = round(step_bytes(numbers, 4, cached)[1] / (other["ms_per_step"] / 1e3) / 1e9
                                               / peak["hbm_gbs"], 4)
        measured32 = prefill_point(engine32, vocab, warmup=1, repeats=3)
        points["fp32_prefill_2048"] = round(PREFILL_TOKENS / (measured32["ms"] / 1e3), 1)
        points["fp32_prefill_ms"] = round(measured32["ms"], 3)
    else:
        kernels = kernel_shares(engine, prompts)

    line = {
        "metric": f"decode tokens/s ({shape_name} shape, batch {args.batch}, bf16, random weights)",
        "value": round(point["tokens_per_s"], 1), "sd": round(point["sd"], 1), "repeats": args.repeats,
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms_per_step, 5), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random token ids, seeded random weights N(0, 0.02)",
        "config": {
            "model": f"{shape_name} shape (llama)", "global_batch": args.batch,
            "seq_len": config_dict["max_position_embeddings"],
            "parallelism": "single GPU", "layers": args.layers, "layers_full_model": full_layers,
            "hidden": config_dict["hidden_size"], "heads": config_dict["num_attention_heads"],
            "kv_heads": config_dict["num_key_value_heads"], "head_dim": config_dict["head_dim"],
            "intermediate": config_dict["intermediate_size"], "vocab": vocab,
            "prompt_lengths": "128-2048 unequal", "mean_cached_tokens_per_seq": round(mean_cached / args.batch, 1),
            "l2": f"inputs larger than L2 (weights {weight_bytes / 1e6:.0f} MB + cache per step)",
            "sampling": "greedy, on device",
            "decode": "CUDA graph per batch size", "peaks": peak["source"],
        },
        "clocks": clocks.summary(),
        "e2e": e2e,
        "gpu_launches": int(point["launches_per_step"] * args.steps),
        "launches_per_step": point["launches_per_step"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
        "kernels": kernels,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
