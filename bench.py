"""Benchmark of the fused-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload (one "step"): the Llama-3-8B-shaped prefill of the reference's config list — GQA
with fused RoPE, B=4, Hq=32, Hkv=8, N=4096, D=128, causal, bf16, theta=5e5 — on synthetic seeded
N(0,1) inputs.  `value` is attention TFLOP/s (4*B*Hq*N^2*D/2 flop per step) with inputs resident in
HBM; `e2e` is the same metric through the public call with pinned HOST buffers (H2D of Q/K/V and D2H
of the packed [O|LSE] inside the timed region).  With N GPUs every rank runs its own batch (weak
scaling, no collective on the data path) and `value` is the whole-job aggregate.  The paged-decode
half of the metric (64 sequences, ctx U[512,8192], page 16) is reported in the `decode` object as
HBM GB/s, the backward and chunked-prefill configs in `backward` / `chunked_prefill`.

`--impl reference` times the reference's own CPU implementation of the path: its scalar oracle,
restated in C++ under oracle/ (no Rust toolchain exists on these machines), on all host threads,
each step a bounded sample of query rows of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))

# DRAM bytes (read + written) per launch of each leg's dominant kernel(s) on exactly the workloads timed below, taken from
# one `ncu --set full` capture each; the summaries and their commands are under profiles/.  The profiler cannot run inside
# this script, so the figures are carried as constants and change only when a kernel changes.
NCU_TRAFFIC = {
    "forward": 304_634_112 + 102_786_304,  # fwd_sm100_kernel<128,false>, C2
    "decode": 1_110_867_000 + 4_535_296,  # decode_mma_kernel<128>, C3
    "backward": 1_229_615_000 + 110_039_296 + 643_880_000 + 235_303_936,  # dK/dV kernel + dQ kernel, C5
}
sys.path.insert(0, ROOT)

C2 = dict(B=4, Hq=32, Hkv=8, N=4096, D=128, theta=500000.0)
C3 = dict(S=64, Hq=32, Hkv=8, D=128, page=16, lo=512, hi=8192, theta=500000.0)
C5 = dict(B=2, Hq=32, Hkv=8, N=8192, D=128)


def prefill_flops(c):
    return 4 * c["B"] * c["Hq"] * c["N"] * c["N"] * c["D"] // 2


def bind_to_gpu_cpus(local_rank):
    """Pin this rank's process to the host cores next to its GPU (NVML's ideal CPU set), before any pinned host
    buffer is allocated: the end-to-end leg moves hundreds of MB per step over PCIe, and with eight ranks on a
    two-socket host, buffers on the far socket would cross the inter-socket link.  Reads NVML only; changes no GPU
    setting.  Returns the number of cores bound, or None if NVML or the affinity call is unavailable."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, device_index, period_s=0.004):
        self.idx, self.period = device_index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._err = None

    def _run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.idx)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                     "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                     "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                     "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
            while not self._stop.is_set():
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                time.sleep(self.period)
        except Exception as e:  # NVML missing: report it, never fail the bench
            self._err = repr(e)

    def start(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        time.sleep(0.02)

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)
        sm = sorted(self.samples)
        out = {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz, "samples": len(sm),
               "reasons": sorted(self.reasons)}
        if self._err:
            out["error"] = self._err
        return out


def make_c2_inputs(torch, rank):
    c = C2
    q = torch.randn(c["B"], c["Hq"], c["N"], c["D"], generator=torch.Generator().manual_seed(1 + 1000 * rank)).bfloat16()
    k = torch.randn(c["B"], c["Hkv"], c["N"], c["D"], generator=torch.Generator().manual_seed(2 + 1000 * rank)).bfloat16()
    v = torch.randn(c["B"], c["Hkv"], c["N"], c["D"], generator=torch.Generator().manual_seed(3 + 1000 * rank)).bfloat16()
    return q, k, v


def oracle_rows_c2(ob, np, q, k, v, rows, threads):
    """Oracle O/LSE on sampled (b, h, row) of the C2 workload: RoPE materialised with the oracle
    formula, then the grouped oracle (bit-identical route to the fused oracle)."""
    c = C2
    B, Hq, Hkv, N, D, theta = c["B"], c["Hq"], c["Hkv"], c["N"], c["D"], c["theta"]
    qf, kf, vf = q.float().numpy(), k.float().numpy(), v.float().numpy()
    rk = ob.rotate_rows(kf, D, np.tile(np.arange(N, dtype=np.uint64), B * Hkv), theta)
    rq = qf.reshape(B, Hq, N, D).copy()
    for (b, h, r) in rows:
        rq[b, h, r] = ob.rotate_rows(rq[b, h, r], D, [r], theta)
    t0 = time.perf_counter()
    eo, el = ob.forward_rows(rq, rk, vf, ob._shape(B, Hq, Hkv, N, N, D), ob.HEAD_MAJOR, rows, True, threads=threads)
    return eo, el, time.perf_counter() - t0


def sample_rows(np, count, seed):
    c = C2
    rng = np.random.default_rng(seed)
    return [(int(rng.integers(c["B"])), int(rng.integers(c["Hq"])), int(rng.integers(c["N"]))) for _ in range(count)]


def rows_flops(rows):
    return sum(4 * C2["D"] * (r + 1) for (_, _, r) in rows)


def run_reference(args, rank, world):
    """Reference arm: the scalar CPU oracle (C++ restatement) on all host threads."""
    if rank != 0:
        return
    import numpy as np
    import torch
    from oracle import binding as ob
    ob.build()
    threads = os.cpu_count() or 1
    q, k, v = make_c2_inputs(torch, 0)
    per_step = 256 * threads
    warm = sample_rows(np, 64, 99)
    for _ in range(max(args.warmup, 1)):
        oracle_rows_c2(ob, np, q, k, v, warm, threads)
    total_flops, total_t = 0, 0.0
    for s in range(args.steps):
        rows = sample_rows(np, per_step, 100 + s)
        _, _, dt = oracle_rows_c2(ob, np, q, k, v, rows, threads)
        total_flops += rows_flops(rows)
        total_t += dt
    tflops = total_flops / total_t / 1e12
    line = {
        "impl": "reference", "metric": "prefill_attention_tflops", "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total_t / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C2 GQA+RoPE causal prefill B=4 Hq=32 Hkv=8 N=4096 D=128 bf16-quantised inputs",
                   "sample": f"{per_step} random (batch, q_head, row) query rows per step"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": f"{per_step} query rows per step, {args.steps} steps, oracle restated in C++ "
                                   "(no Rust toolchain on this machine)"},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def timed_region(torch, dist, world, fn, steps):
    """barrier + synchronize, K steps between CUDA events, max over ranks (milliseconds)."""
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


def write_manifest(torch, fa, ctx, args, c, step):
    """Benchmark manifest (BenchmarkManifest, src/benchmark_manifest.rs:46-199) of the headline workload: per-step device
    latencies of up to 101 further steps, median and p95 in integer nanoseconds, canonical JSON from the library."""
    import importlib
    import platform
    import subprocess
    tel = importlib.import_module("flat_attention_b200.telemetry")
    n = max(1, min(args.steps, 101))
    events = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1)]
    torch.cuda.synchronize()
    for i in range(n):
        events[i].record()
        step()
    events[n].record()
    torch.cuda.synchronize()
    lat = sorted(int(round(events[i].elapsed_time(events[i + 1]) * 1e6)) for i in range(n))
    median = lat[n // 2]
    p95 = max(median, lat[min(n - 1, (95 * n + 99) // 100 - 1)])
    sha = args.commit_sha
    if not sha:
        try:
            sha = subprocess.run(["git", "-C", ROOT, "rev-parse", "HEAD"], capture_output=True, text=True, timeout=10).stdout.strip()
        except Exception:
            sha = ""
    if len(sha) != 40:
        sha = "0" * 40
    fp = tel.device_fingerprint(ctx)
    tokens = c["B"] * c["N"]
    m = tel.BenchmarkManifest(
        commit_sha=sha, benchmark_id="c2-gqa-rope-causal-prefill", command="python bench.py " + " ".join(sys.argv[1:]),
        device=fp.name.decode(), backend=fp.backend.decode(), driver=fp.driver.decode() + "; " + fp.driver_info.decode(),
        os=platform.system(), arch=platform.machine(), precision="bf16", batch=c["B"], q_heads=c["Hq"], kv_heads=c["Hkv"],
        query_len=c["N"], kv_len=c["N"], head_dim=c["D"], causal=True, warmup_iterations=args.warmup, measured_iterations=n,
        median_latency_ns=median, p95_latency_ns=p95, tokens_per_second_milli=tokens * 1_000_000_000_000 // max(median, 1))
    text = m.canonical_json()
    os.makedirs(os.path.dirname(os.path.abspath(args.manifest)), exist_ok=True)
    with open(args.manifest, "w") as f:
        f.write(text + "\n")
    return {"path": args.manifest, "result_checksum": m.result_checksum(), "median_latency_ns": median, "p95_latency_ns": p95,
            "device_fingerprint": "%016x" % tel.fingerprint_stable(fp)}


def bench_decode(torch, np, fa, ctx, peaks, steps, warmup):
    """Config 3: batched paged decode, HBM GB/s of the algorithmic bytes."""
    c = C3
    S, Hq, Hkv, D, ps = c["S"], c["Hq"], c["Hkv"], c["D"], c["page"]
    rng = np.random.default_rng(5)
    lens = (c["lo"] + rng.integers(0, c["hi"] - c["lo"] + 1, S)).astype(np.int32)
    pages_per = (lens + ps - 1) // ps
    pool = int(pages_per.sum()) + 64
    perm = np.random.default_rng(6).permutation(pool).astype(np.int32)
    maxp = int(pages_per.max())
    tables = np.zeros((S, maxp), np.int32)
    at = 0
    for s in range(S):
        tables[s, :pages_per[s]] = perm[at:at + pages_per[s]]
        at += pages_per[s]
    g = torch.Generator(device="cuda").manual_seed(7)
    K = torch.randn(pool * ps, Hkv * D, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    V = torch.randn(pool * ps, Hkv * D, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    Q = torch.randn(S, Hq * D, generator=g, device="cuda", dtype=torch.float32).bfloat16()
    qpos = (lens - 1).astype(np.int32)
    d_tab, d_len, d_pos = torch.from_numpy(tables).cuda(), torch.from_numpy(lens).cuda(), torch.from_numpy(qpos).cuda()
    out = ctx.empty_bytes(S * Hq * D * 2 + S * Hq * 4)
    cfg = fa.config(True)

    def step():
        ctx.decode_paged_batched(fa.BF16, S, Hq, Hkv, D, ps, pool, maxp, d_tab, d_len, d_pos, tables, lens, qpos, cfg,
                                 c["theta"], Q, K, V, out)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        step()
    ctx.set_kernel_timing(True)
    ctx.take_kernel_time()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(steps):
        # flush L2 (256 MiB write) so every step streams K/V from HBM; the events sit right behind the
        # flush in stream order, so host-side validation of the call overlaps the flush, as it overlaps
        # the previous step in a serving loop
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    kms, kn = ctx.take_kernel_time()
    ctx.set_kernel_timing(False)
    kv_bytes = int(lens.sum()) * Hkv * D * 2 * 2
    other = S * Hq * D * 2 * 2 + S * Hq * 4 + int(pages_per.sum()) * 4
    alg = kv_bytes + other
    ms = total / steps
    kernel_ms = kms / max(kn, 1)
    return {
        "metric": "paged_decode_hbm_gbs", "value": alg / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms,
        "algorithmic_bytes": alg, "sequences": S, "context_tokens": int(lens.sum()),
        "roofline": {"bound": "hbm", "achieved": alg / (kernel_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": alg / (kernel_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC["decode"],
                     "traffic_source": "dram bytes read+written per launch, one ncu capture of this workload (profiles/)",
                     "kernel": "decode_mma_kernel<128>", "kernel_ms": kernel_ms, "peak_source": peaks["source"]},
        "l2": "flushed between steps (256 MiB write)",
    }


def bench_backward(torch, fa, ctx, peaks, steps, warmup):
    """Config 5: grouped backward recompute, TFLOP/s of the 5 algorithmic GEMMs (10*B*Hq*N^2*D/2 flop)."""
    c = C5
    B, Hq, Hkv, N, D = c["B"], c["Hq"], c["Hkv"], c["N"], c["D"]
    g = torch.Generator(device="cuda").manual_seed(11)
    q = torch.randn(B, Hq, N, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, Hkv, N, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, Hkv, N, D, generator=g, device="cuda").bfloat16()
    do = torch.randn(B, Hq, N, D, generator=g, device="cuda").bfloat16()
    shp = fa.shape(B, Hq, Hkv, N, N, D)
    FL, L = fa.forward_layout(fa.BF16, shp), fa.backward_layout(fa.BF16, shp)
    fwd = ctx.create_output_buffer(fa.BF16, shp)
    ctx.forward_grouped(fa.BF16, shp, fa.config(True), q, k, v, fwd)
    packed = ctx.empty_bytes(L.input_bytes)
    for off, t in ((L.q_offset, q), (L.k_offset, k), (L.v_offset, v), (L.d_out_offset, do)):
        packed[off:off + t.numel() * 2] = t.view(torch.uint8).reshape(-1)
    packed[L.out_offset:L.out_offset + FL.q_bytes] = fwd[:FL.q_bytes]
    packed[L.lse_offset:L.lse_offset + 4 * FL.lse_elements] = fwd[FL.lse_byte_offset:FL.lse_byte_offset + 4 * FL.lse_elements]
    grads = ctx.empty_bytes(L.output_bytes)
    cfg = fa.config(True)
    for _ in range(warmup):
        ctx.backward_grouped(fa.BF16, shp, cfg, packed, grads)
    ctx.set_kernel_timing(True)
    ctx.take_kernel_time()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        ctx.backward_grouped(fa.BF16, shp, cfg, packed, grads)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    kms, kn = ctx.take_kernel_time()
    ctx.set_kernel_timing(False)
    flops = 10 * B * Hq * N * N * D // 2
    kernel_ms = kms / steps  # the two tensor-core kernels of one call
    return {"metric": "grouped_backward_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
            "flop_per_step": flops, "workload": "C5 B=2 Hq=32 Hkv=8 N=8192 D=128 causal bf16, f32 gradients",
            "roofline": {"bound": "tensor", "achieved": flops / (kernel_ms * 1e-3) / 1e12, "peak": peaks["bf16_sustained"] or peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": flops / (kernel_ms * 1e-3) / 1e12 / (peaks["bf16_sustained"] or peaks["bf16_tflops"]),
                         "traffic": NCU_TRAFFIC["backward"], "traffic_source": "dram bytes read+written, both kernels, one ncu capture of this workload (profiles/)",
                         "kernel": "bwd_sm100_kernel<128> + bwd_dq_sm100_kernel<128>",
                         "kernel_ms": kernel_ms, "peak_source": peaks["source"] + " (sustained cuBLAS bf16: the step runs for milliseconds)",
                         "note": "7 GEMM units are executed for 5 algorithmic ones (scores recomputed in both kernels)"}}


def bench_prefill_variants(torch, fa, ctx, peaks, steps, warmup):
    """The C2 prefill shape through the two widened modes of the forward: the ALiBi score bias on the rectangular
    projection entry point (bf16) and IEEE binary16 storage (GQA + RoPE, head-major).  Same flops as the headline."""
    c = C2
    B, Hq, Hkv, N, D, theta = c["B"], c["Hq"], c["Hkv"], c["N"], c["D"], c["theta"]
    shp, cfg, rot = fa.shape(B, Hq, Hkv, N, N, D), fa.config(True), fa.rotary(theta, 0)
    flops = prefill_flops(c)
    peak = peaks["bf16_tflops"]
    results = {}

    def timed(name, kernel, fn, note):
        for _ in range(warmup):
            fn()
        ctx.set_kernel_timing(True)
        ctx.take_kernel_time()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        kms, kn = ctx.take_kernel_time()
        ctx.set_kernel_timing(False)
        kms /= max(kn, 1)
        results[name] = {"value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "workload": note,
                         "roofline": {"bound": "tensor", "achieved": flops / (kms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                                      "frac": flops / (kms * 1e-3) / 1e12 / peak, "traffic": None, "kernel": kernel,
                                      "kernel_ms": kms, "peak_source": peaks["source"] + " (burst cuBLAS bf16)"}}

    g = torch.Generator(device="cuda").manual_seed(21)
    q = torch.randn(B, N, Hq, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, N, Hkv, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, N, Hkv, D, generator=g, device="cuda").bfloat16()
    out = ctx.create_output_buffer(fa.BF16, shp)
    slopes = [2.0 ** -(8.0 * (h + 1) / Hq) for h in range(Hq)]
    timed("alibi", "fwd_sm100_kernel<128,false,ALIBI>",
          lambda: ctx.forward_projection_rope_asymmetric_alibi(fa.BF16, shp, cfg, rot, slopes, 0, 0, q, k, v, out),
          "C2 shape, projection layout, bf16, RoPE + ALiBi (slopes 2^(-8(h+1)/Hq))")
    q16, k16, v16 = (x.transpose(1, 2).contiguous().half() for x in (q, k, v))
    out16 = ctx.create_output_buffer(fa.F16, shp)
    timed("binary16", "fwd_sm100_kernel<128,false,false,F16IO>",
          lambda: ctx.forward_grouped_rope(fa.F16, shp, cfg, rot, q16, k16, v16, out16),
          "C2 shape, head-major, IEEE binary16 storage, RoPE")
    return results


def bench_chunked_prefill(torch, fa, ctx, peaks, warmup):
    """Config 4 (prefill part): one 32768-token sequence fed in 2048-token chunks into a growing paged cache."""
    Hq, Hkv, D, N, chunk, ps, theta = 64, 8, 128, 32768, 2048, 16, 500000.0
    g = torch.Generator(device="cuda").manual_seed(13)
    q = torch.randn(N, Hq * D, generator=g, device="cuda").bfloat16()
    k = torch.randn(N, Hkv * D, generator=g, device="cuda").bfloat16()
    v = torch.randn(N, Hkv * D, generator=g, device="cuda").bfloat16()
    cache = fa.CudaPagedKvCache(ctx, fa.BF16, ps, N // ps + 8, Hkv, D)
    out = ctx.empty_bytes(chunk * Hq * D * 2 + Hq * chunk * 4)
    cfg = fa.config(True)

    def run():
        cache.reset()
        for start in range(0, N, chunk):
            ctx.chunked_prefill_paged(cache, Hq, chunk, cfg, theta, 0, q[start:start + chunk], k[start:start + chunk],
                                      v[start:start + chunk], out)
    for _ in range(max(1, warmup - 2)):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 3
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    flops = 4 * Hq * D * N * N // 2
    return {"metric": "chunked_prefill_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_sequence": ms,
            "flop_per_sequence": flops, "frac_of_peak": flops / (ms * 1e-3) / 1e12 / (peaks["bf16_sustained"] or peaks["bf16_tflops"]),
            "workload": "C4 1 x 32768 tokens in 2048-token chunks, Hq=64 Hkv=8 D=128 causal bf16, page 16, RoPE fused "
                        "into the cache append (K) and into the attention kernel (Q)"}


def bench_splitkv_128k(torch, np, dist, fa, ctx, rank, world, steps, warmup):
    """Config 4 (decode part): one 131072-token sequence, KV axis split across the ranks; every rank
    decodes its slice, the (O, LSE) partials are all-gathered over NCCL and merged on every rank."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("flat_distributed", os.path.join(ROOT, "flat-attention_b200", "distributed.py"))
    fd = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(fd)
    Hq, Hkv, D, ps, theta, n = 64, 8, 128, 16, 500000.0, 131072
    first, count = fd.shard_pages(n, ps, world, rank)
    pages = count // ps
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    K = torch.randn(pages * ps, Hkv * D, generator=g, device="cuda").bfloat16()
    V = torch.randn(pages * ps, Hkv * D, generator=g, device="cuda").bfloat16()
    Q = torch.randn(1, Hq * D, generator=torch.Generator(device="cuda").manual_seed(99), device="cuda").bfloat16()
    tab = np.random.default_rng(rank).permutation(pages).astype(np.int32).reshape(1, pages)
    lens, qpos = np.array([count], np.int32), np.array([n - 1], np.int32)
    args = dict(num_seqs=1, q_heads=Hq, kv_heads=Hkv, head_dim=D, page_size=ps, physical_pages=pages, max_pages_per_seq=pages,
                page_tables_dev=torch.from_numpy(tab).cuda(), context_lens_dev=torch.from_numpy(lens).cuda(),
                q_rope_positions_dev=torch.from_numpy(qpos).cuda(), host_page_tables=None, host_context_lens=lens,
                cfg=fa.config(True), theta=theta, q=Q, k=K, v=V)
    out = ctx.empty_bytes(Hq * D * 2 + Hq * 4)
    partial = torch.empty(Hq * (D + 1), dtype=torch.float32, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def step():
        return fd.splitkv_decode(ctx, fa, fa.BF16, args, Hq, D, out)
    for _ in range(warmup):
        step()
    tot, tot_merge = 0.0, 0.0
    for _ in range(steps):
        flush.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        ctx.decode_paged_batched_partial(fa.BF16, out=partial, **args)
        e1.record()
        gathered = fd.all_gather_partials(partial)
        ctx.splitkv_merge_packed(fa.BF16, world, Hq, D, gathered, out)
        e2.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e2)
        tot_merge += e1.elapsed_time(e2)
    t = torch.tensor([tot / steps, tot_merge / steps], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_merge = float(t[0]), float(t[1])
    kv_bytes = n * Hkv * D * 2 * 2
    return {"metric": "splitkv_decode_128k", "ms_per_step": ms, "gather_merge_ms": ms_merge,
            "aggregate_kv_gbs": kv_bytes / (ms * 1e-3) / 1e9, "per_gpu_kv_gbs": kv_bytes / world / ((ms - ms_merge) * 1e-3) / 1e9,
            "kv_bytes_total": kv_bytes, "gathered_bytes": world * Hq * (D + 1) * 4,
            "workload": "1 sequence x 131072 tokens, Hq=64 Hkv=8 D=128 bf16, page 16, KV split over %d GPUs, NCCL all-gather" % world}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-extras", action="store_true", help="only the headline prefill workload")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU oracle legs (parity gate, cpu_baseline): for profiler runs")
    ap.add_argument("--variants-only", action="store_true", help="run only the ALiBi / binary16 prefill variants (N=1): "
                                                                "a short command for profiler captures")
    ap.add_argument("--manifest", default=None, help="write a schema-1 canonical-JSON benchmark manifest of the headline "
                                                     "workload to this path (rank 0)")
    ap.add_argument("--commit-sha", default=None, help="40-hex source revision recorded in the manifest "
                                                       "(default: git rev-parse HEAD, else zeros)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    fa = load_package()

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    numa = bind_to_gpu_cpus(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = load_peaks()
    ctx = fa.Context(local_rank)
    if args.variants_only:
        if rank == 0:
            print(json.dumps({"prefill_variants": bench_prefill_variants(torch, fa, ctx, peaks, max(1, args.steps), args.warmup)}),
                  flush=True)
        return
    c = C2
    B, Hq, Hkv, N, D, theta = c["B"], c["Hq"], c["Hkv"], c["N"], c["D"], c["theta"]
    shp = fa.shape(B, Hq, Hkv, N, N, D)
    cfg, rot = fa.config(True), fa.rotary(theta, 0)
    q, k, v = make_c2_inputs(torch, rank)
    hq, hk, hv = q.pin_memory(), k.pin_memory(), v.pin_memory()
    dq, dk, dv = hq.cuda(non_blocking=True), hk.cuda(non_blocking=True), hv.cuda(non_blocking=True)
    out = ctx.create_output_buffer(fa.BF16, shp)
    host_out = torch.empty(out.numel(), dtype=torch.uint8).pin_memory()
    flops = prefill_flops(c)

    def step():
        ctx.forward_grouped_rope(fa.BF16, shp, cfg, rot, dq, dk, dv, out)

    def step_e2e():
        # the public host-slice call: pinned host Q/K/V in, pinned host [O | LSE] out, blocks until the result is readable
        ctx.forward_host(fa.BF16, fa.HEAD_MAJOR, shp, cfg, rot, hq, hk, hv, host_out)

    for i in range(args.warmup):
        step()
        if i == 0:
            # a kernel whose bounded waits gave up reports it here: stop at once instead of timing a broken path
            st = ctx.device_status()
            if st != 0:
                raise SystemExit(f"bench: the forward kernel reported device status {st} on its first launch")
    torch.cuda.synchronize()

    # parity gate before timing (reference bench protocol): a few sampled rows against the oracle
    parity = None
    if rank == 0 and not args.no_cpu:
        from oracle import binding as ob
        rows = [(0, 0, 0), (0, 0, 129), (B - 1, Hq - 1, N - 1)] + sample_rows(np, 13, 3)
        eo, el, _ = oracle_rows_c2(ob, np, q, k, v, rows, min(8, os.cpu_count() or 1))
        o, l = ctx.split_output(out, fa.BF16, shp)
        ao = np.stack([o[b, h, r].float().cpu().numpy() for (b, h, r) in rows])
        al = np.array([float(l[b, h, r]) for (b, h, r) in rows])
        parity = {"rows": len(rows), "max_abs_o": float(np.abs(ao - eo).max()), "max_abs_lse": float(np.abs(al - el).max())}
        parity["ok"] = parity["max_abs_o"] <= 2e-2 and parity["max_abs_lse"] <= 2e-3

    sampler = ClockSampler(local_rank)
    launches0 = ctx.launch_count()
    ctx.set_kernel_timing(True)
    ctx.take_kernel_time()
    if rank == 0:
        sampler.start()
    ms = timed_region(torch, dist, world, step, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    kernel_ms, kernel_n = ctx.take_kernel_time()
    ctx.set_kernel_timing(False)
    launches = ctx.launch_count() - launches0

    for _ in range(2):
        step_e2e()
    ms_e2e = timed_region(torch, dist, world, step_e2e, max(3, min(args.steps, 10)))
    e2e_steps = max(3, min(args.steps, 10))
    status = ctx.device_status()

    ms_per_step = ms / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12
    kms = kernel_ms / max(kernel_n, 1)
    # denominator: the sustained cuBLAS figure when the timed loop ran into the power cap (back-to-back
    # steps for a good fraction of a second), the burst figure when it did not
    capped = bool(clocks and "sw_power_cap" in (clocks.get("reasons") or []))
    # back-to-back tensor-core kernels for a tenth of a second or more are a sustained load whether or not a 4 ms NVML
    # sample caught the power-cap flag
    long_loop = ms >= 100.0
    sustained = capped or long_loop
    peak = (peaks["bf16_sustained"] or peaks["bf16_tflops"]) if sustained else peaks["bf16_tflops"]
    line = {
        "metric": "prefill_attention_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "C2 GQA+RoPE causal prefill (Llama-3-8B shape): B=4 per GPU, Hq=32, Hkv=8, N=4096, D=128, "
                               "bf16, theta=5e5, O + f32 LSE", "flop_per_step_per_gpu": flops,
                   "inputs": "seeded N(0,1) rounded to bf16; 192 MiB of Q/K/V + 32 MiB of rotated K + 136 MiB of O and LSE per step "
                             "exceed the 126 MB L2", "sharding": "independent batches per rank, no collective",
                   "host_cores_bound": numa},
        "e2e": {"value": world * flops / (ms_e2e / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": int(hq.numel() + hk.numel() + hv.numel()) * 2, "d2h_bytes_per_step": int(out.numel()),
                "ms_per_step": ms_e2e / e2e_steps},
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "achieved": flops / (kms * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                     "frac": flops / (kms * 1e-3) / 1e12 / peak, "traffic": NCU_TRAFFIC["forward"],
                     "traffic_source": "dram bytes read+written per launch, one ncu capture of this workload (profiles/)",
                     "kernel": "fwd_sm100_kernel<128,false>",
                     "kernel_ms": kms,
                     "peak_source": peaks["source"] + (" (sustained cuBLAS bf16: sw_power_cap was active during the timed loop)" if capped
                                                       else " (sustained cuBLAS bf16: the timed loop kept the tensor cores busy for %.0f ms)" % ms
                                                       if long_loop else " (burst cuBLAS bf16)")},
        "clocks": clocks,
        "parity": parity,
        "device_status": status,
    }
    if rank == 0 and args.manifest:
        line["manifest"] = write_manifest(torch, fa, ctx, args, c, step)
    if rank == 0 and world == 1 and not args.no_cpu:
        from oracle import binding as ob
        rows = sample_rows(np, 40000, 11)
        _, _, dt = oracle_rows_c2(ob, np, q, k, v, rows, 1)
        line["cpu_baseline"] = {"value": rows_flops(rows) / dt / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
                                "sample": "40000 random (batch, q_head, row) query rows of the same workload, scalar oracle "
                                          "restated in C++, %.1f s" % dt}
    if rank == 0 and world == 1:
        if not args.skip_extras:
            line["decode"] = bench_decode(torch, np, fa, ctx, peaks, max(5, min(args.steps, 20)), args.warmup)
            line["backward"] = bench_backward(torch, fa, ctx, peaks, max(3, min(args.steps, 10)), args.warmup)
            line["chunked_prefill"] = bench_chunked_prefill(torch, fa, ctx, peaks, args.warmup)
            line["prefill_variants"] = bench_prefill_variants(torch, fa, ctx, peaks, max(5, min(args.steps, 20)), args.warmup)
    if world > 1 and not args.skip_extras:
        extra = bench_splitkv_128k(torch, np, dist, fa, ctx, rank, world, max(5, min(args.steps, 20)), args.warmup)
        line["splitkv_decode_128k"] = extra
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
