"""Measures decode and prefill throughput of the engine on one B200 and prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
                    [--shape smollm2-135m|smollm2-1.7b|llama-3.1-8b] [--batch B] [--no-points]
                    [--profile decode|prefill|gemm|attention|stream]

Default workload: the SmolLM2-135M shape (30 layers, hidden 576, 9 heads, 3 kv heads, head_dim 64, intermediate 1536,
vocabulary 49152, tied head) with seeded random bfloat16 weights; a batch of 8 sequences with unequal prompt lengths
(128 to 2,048 seeded random tokens) inside a context of 8,192. A "step" is one decode step of the whole batch
(model, greedy token choice, feedback), replayed as a CUDA graph; `value` is decoded tokens per second over exactly K
steps timed with CUDA events. `e2e` is the same through `Engine.generate` with host token lists in and out.
`prefill` is one 2,048-token prompt in one step. `roofline` relates the decode step to HBM bandwidth: every weight
read once plus the cache of the live sequences, over the step's time. `points` repeats the decode at batch 1 and 64, and the end-to-end run with temperature sampling.
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
    """Times the tile products alone (CUDA events, 20 launches after 3) at layer shapes of the three model sizes:
    the tcgen05 kernel at each tile width and the mma.sync kernel, in TFLOP/s."""
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
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(20):
            ops.gemm(c, a, w, epilogue, kernel=kernel, tile_n=tile_n)
        end.record()
        torch.cuda.synchronize()
        ops.raise_if_failed()
        ms = begin.elapsed_time(end) / 20
        return ms * 1e3, 2 * m * n * k / ms / 1e9

    shapes = [(2048, 576, 576, ops.EPI_RESIDUAL), (2048, 576, 1536, ops.EPI_RESIDUAL), (2048, 3072, 576, ops.EPI_SWIGLU),
              (2048, 2048, 8192, ops.EPI_RESIDUAL), (2048, 16384, 2048, ops.EPI_SWIGLU),
              (2048, 4096, 4096, ops.EPI_RESIDUAL), (2048, 28672, 4096, ops.EPI_SWIGLU),
              (2048, 4096, 14336, ops.EPI_RESIDUAL), (8192, 4096, 4096, ops.EPI_STORE_T)]
    print("M N K epilogue | tcgen05 tile 64 | 128 | 256 | chosen | mma.sync   (microseconds, TFLOP/s)")
    for m, n, k, epilogue in shapes:
        cells = []
        for tile_n in (64, 128, 256, 0):
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
    """Times the decode products alone at layer shapes of the larger models: the kernel that streams W through
    registers against the one that streams it through shared memory, as fractions of the measured HBM rate (a CUDA
    graph of 20 launches over several copies of W, so that W comes from HBM)."""
    import torch

    from etalii.dllm_b200.kernels import ops

    device = "cuda:0"
    rate = peaks()["hbm_gbs"]

    def run(m, n, k, epilogue, kernel):
        copies = max(2, int(300e6 // (n * k * 2)) + 1)
        ws = [(torch.randn(n, k, device=device) * 0.05).bfloat16() for _ in range(copies)]
        x = torch.randn(m, k, device=device).bfloat16()
        cols = n // 2 if epilogue == ops.EPI_SWIGLU else n
        dtype = torch.float32 if epilogue in (ops.EPI_STORE_F32, ops.EPI_RESIDUAL) else torch.bfloat16
        c = torch.zeros(m, cols, device=device, dtype=dtype)
        for i in range(3):
            ops.gemm(c, x, ws[i % copies], epilogue, kernel=kernel)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(20):
                ops.gemm(c, x, ws[i % copies], epilogue, kernel=kernel)
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
    print("rows of activations, W rows x row length, epilogue | registers: us, of HBM | shared memory: us, of HBM")
    for m in (1, 8, 16):
        for n, k, epilogue in shapes:
            a, b = run(m, n, k, epilogue, 2), run(m, n, k, epilogue, 4)
            print(f"{m} {n} x {k} {epilogue} | {a[0]:.1f} {a[1]:.2f} | {b[0]:.1f} {b[1]:.2f}")
    return 0


def model_numbers(config, layers):
    h, i, v = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    nh, nkv, hd = config["num_attention_heads"], config["num_key_value_heads"], config["head_dim"]
    per_layer = h * (nh + 2 * nkv) * hd + nh * hd * h + 3 * h * i
    matrix_params = layers * per_layer
    norm_params = (2 * layers + 1) * h
    kv_bytes_per_token = layers * 2 * nkv * hd * 2
    t = PREFILL_TOKENS
    prefill_flops = 2 * matrix_params * t + layers * 4 * hd * nh * t * (t + 1) // 2 + 2 * h * v
    return {"matrix_params": matrix_params, "head_params": v * h, "norm_params": norm_params,
            "kv_bytes_per_token": kv_bytes_per_token, "prefill_flops": prefill_flops}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=256)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--shape", default="smollm2-135m", choices=sorted(SHAPES),
                        help="layer sizes: the default is the benchmark's; the others are larger shapes of the family")
    parser.add_argument("--layers", type=int, default=0, help="fewer layers than the full model (named in config)")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 decode points")
    parser.add_argument("--profile", choices=("decode", "prefill", "gemm", "attention", "stream"),
                        help="run only a few decode steps (or one prefill) and print no JSON: a small case for ncu")
    args = parser.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference does not install offline: pip finds no numpy in the wheelhouse, and with "
                          "--no-deps its wheel build fails in CMake because nanobind is not installed"}))
        return 0
    if args.profile == "gemm":
        return gemm_table()
    if args.profile == "attention":
        return attention_table()
    if args.profile == "stream":
        return stream_table()
    if args.gpus != 1:
        print(f"bench.py measures one GPU: --gpus {args.gpus} is not supported (this library runs on a single device)")
        return 2
    warmup = max(3, args.warmup)

    import torch

    from etalii.dllm_b200 import SamplingOptions
    from etalii.dllm_b200.config.registry import config_from_dict
    from etalii.dllm_b200.engine.engine import Engine
    from etalii.dllm_b200.kernels import ops

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
    decode_run(engine, prompts, 4, 3)  # builds kernels, work buffers and the graph before anything is timed
    with ClockSampler() as clocks:
        ms, launches_per_step, cached = decode_run(engine, prompts, args.steps, warmup)
    ms_per_step = ms / args.steps
    value = args.batch * args.steps / (ms / 1e3)

    weight_bytes = 2 * (numbers["matrix_params"] + numbers["head_params"]) + 4 * numbers["norm_params"]
    mean_cached = cached - args.batch * args.steps / 2  # halfway through the timed steps
    step_bytes = weight_bytes + mean_cached * numbers["kv_bytes_per_token"]
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9

    prefill_ms = prefill_run(engine, vocab, warmup=3)
    prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 4),
               "frac": round(numbers["prefill_flops"] / (prefill_ms / 1e3) / (peak["bf16_tflops"] * 1e12), 5)}

    # end to end through the public entry point: host token lists in, host token lists out
    engine.generate(prompts, 20, SamplingOptions(), ignore_eos=True)
    engine.generate(prompts, args.steps + 1, SamplingOptions(), ignore_eos=True)
    stats = engine.stats
    graph = next(g for g in engine._graphs.values() if g.b == args.batch)
    e2e = {"value": round(stats["decode_tokens"] / stats["decode_s"], 1), "unit": "tokens/s",
           "h2d_bytes_per_step": round(graph.host.numel() * 4 / engine.decode_chunk, 1),
           "d2h_bytes_per_step": args.batch * 4}

    points = {}
    if not args.no_points:
        # the same end-to-end run with sampling on the device instead of greedy choice
        sampled = SamplingOptions(temperature=0.8, seed=1)
        engine.generate(prompts, 20, sampled, ignore_eos=True)
        engine.generate(prompts, args.steps + 1, sampled, ignore_eos=True)
        points["e2e_temperature_0.8"] = round(engine.stats["decode_tokens"] / engine.stats["decode_s"], 1)
        for name, batch in (("decode_b1", 1), ("decode_b64", 64)):
            batch_prompts = make_prompts(batch, vocab, seed=2 + batch)
            decode_run(engine, batch_prompts, 4, 3)
            point_ms, _, _ = decode_run(engine, batch_prompts, args.steps, warmup)
            points[name] = round(batch * args.steps / (point_ms / 1e3), 1)

    line = {
        "metric": f"decode tokens/s ({shape_name} shape, batch {args.batch}, bf16, random weights)",
        "value": round(value, 1),
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
        "gpu_launches": int(launches_per_step * args.steps),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
