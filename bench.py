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
HBM GB/s, the backward and chunked-prefill configs in `backward` / `chunked_prefill`.  Every leg is gated
by the CPU oracle on sampled rows before it is timed and prints no throughput if the gate fails.

Roofline denominators follow one rule for every leg: the burst cuBLAS bf16 figure, unless that leg's own
timed loop ran for 100 ms or more or NVML reported sw_power_cap during it, in which case the sustained
figure; both fractions are printed (`frac_burst`, `frac_sustained`) next to the loop's wall time.

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
    "forward": 311_873_792 + 111_970_304,  # fwd_sm100_kernel<128>, C2
    "decode": 1_110_817_000 + 3_957_504,  # decode_mma_kernel<128>, C3
    # the 16 launches of fwd_sm100_kernel<128,paged,shadow> of one C4 sequence, summed (one ncu pass over a whole sequence)
    "chunked": 4196745216 + 500366592,
    # dK/dV kernel (reads, dS writes) + dQ kernel (dS reads, writes), captured on one eighth of C5 and scaled by 8
    "backward": 8 * (60_724_736 + 507_990_528 + 554_259_712 + 22_141_696),
}
sys.path.insert(0, ROOT)
BACKWARD_KERNELS = "bwd_sm100_kernel<128,spill> + bwd_dq_spill_kernel<128>"
BACKWARD_NOTE = ("5 GEMM units, the algorithmic count: the dK/dV kernel writes its bf16 dS tiles to scratch (causal C5: "
                 "4.3 GB) and the dQ kernel streams them back against K, so that kernel is HBM-bound, not tensor-bound")

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


SUSTAINED_LOOP_MS = 100.0


def tensor_roofline(peaks, flops, kernel_ms, loop_ms, reasons, kernel, traffic=None, traffic_source=None, note=None):
    """Roofline object of a tensor-bound leg.  One rule for every leg: `frac` is against the burst cuBLAS bf16 peak
    unless the leg's own timed loop kept the tensor cores busy for SUSTAINED_LOOP_MS or more, or NVML reported
    sw_power_cap during it; then against the sustained peak.  Both fractions are always printed."""
    achieved = flops / (kernel_ms * 1e-3) / 1e12
    burst = peaks["bf16_tflops"]
    sustained = peaks["bf16_sustained"] or burst
    capped = "sw_power_cap" in (reasons or [])
    long_loop = loop_ms >= SUSTAINED_LOOP_MS
    use_sustained = capped or long_loop
    peak = sustained if use_sustained else burst
    why = ("sustained cuBLAS bf16: sw_power_cap was active during the timed loop" if capped else
           "sustained cuBLAS bf16: the timed loop ran for %.0f ms" % loop_ms if long_loop else "burst cuBLAS bf16")
    out = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
           "frac_burst": achieved / burst, "frac_sustained": achieved / sustained, "loop_ms": loop_ms,
           "traffic": traffic, "kernel": kernel, "kernel_ms": kernel_ms, "peak_source": "%s (%s)" % (peaks["source"], why),
           "peak_rule": "burst unless this leg's timed loop ran >= %.0f ms or saw sw_power_cap" % SUSTAINED_LOOP_MS}
    if traffic_source:
        out["traffic_source"] = traffic_source
    if note:
        out["note"] = note
    return out


def gate(name, parity):
    """A leg whose oracle gate failed prints its parity record and no throughput."""
    return {"metric": name, "parity": parity, "error": "parity gate failed: not timed"}


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
    for (b, h, r) in dict.fromkeys(rows):  # a row listed twice is still rotated once
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


def oracle_decode_row(ob, np, q, k_rows, v_rows, Hq, Hkv, D, theta, q_pos):
    """Oracle of one decode step against pre-rotated K: Q rotation materialised, then the rectangular grouped oracle
    (query_len 1 at offset n - 1).  q [Hq*D], k_rows / v_rows [n, Hkv*D] in logical order."""
    n = k_rows.shape[0]
    rq = ob.rotate_rows(q, D, np.full(Hq, q_pos, np.uint64), theta)
    kh = np.ascontiguousarray(k_rows.reshape(n, Hkv, D).transpose(1, 0, 2))
    vh = np.ascontiguousarray(v_rows.reshape(n, Hkv, D).transpose(1, 0, 2))
    return ob.forward_reference_grouped_asymmetric(rq, kh, vh, ob._shape(1, Hq, Hkv, 1, n, D, n - 1), True)


def bench_decode(torch, np, fa, ctx, peaks, steps, warmup, ob=None):
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
    L = fa.decode_layout(fa.BF16, S, Hq, D)
    out = ctx.empty_bytes(L.combined_bytes)
    cfg = fa.config(True)

    def step():
        ctx.decode_paged_batched(fa.BF16, S, Hq, Hkv, D, ps, pool, maxp, d_tab, d_len, d_pos, tables, lens, qpos, cfg,
                                 c["theta"], Q, K, V, out)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        step()
    parity = None
    if ob is not None:
        # oracle gate: the shortest, the longest and one other sequence
        o, l = ctx.split_decode_output(out, fa.BF16, S, Hq, D)
        worst_o = worst_l = 0.0
        picks = sorted({int(np.argmin(lens)), int(np.argmax(lens)), 17})
        for sq in picks:
            rows = torch.from_numpy(np.array([tables[sq, t // ps] * ps + t % ps for t in range(lens[sq])])).cuda()
            eo, el = oracle_decode_row(ob, np, Q[sq].float().cpu().numpy(), K[rows].float().cpu().numpy(),
                                       V[rows].float().cpu().numpy(), Hq, Hkv, D, c["theta"], int(qpos[sq]))
            worst_o = max(worst_o, float(np.abs(o[sq].float().cpu().numpy().reshape(-1) - eo).max()))
            worst_l = max(worst_l, float(np.abs(l[sq].cpu().numpy() - el).max()))
        parity = {"sequences": len(picks), "max_abs_o": worst_o, "max_abs_lse": worst_l,
                  "ok": worst_o <= 2e-2 and worst_l <= 2e-3 and ctx.device_status() == 0}
        if not parity["ok"]:
            return gate("paged_decode_hbm_gbs", parity)
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
        "l2": "flushed between steps (256 MiB write)", "parity": parity,
    }


def bench_backward(torch, np, fa, ctx, peaks, steps, warmup, ob=None, dims=None, device_index=0):
    """Config 5: grouped backward recompute, TFLOP/s of the 5 algorithmic GEMMs (10*B*Hq*N^2*D/2 flop).  `dims`
    overrides (B, Hq, Hkv) for a rank's share of the fixed problem (strong scaling)."""
    c = C5
    B, Hq, Hkv = dims if dims else (c["B"], c["Hq"], c["Hkv"])
    N, D = c["N"], c["D"]
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
    parity = None
    if ob is not None:
        # oracle gate: sampled dQ rows and dK/dV rows (first / last rows, a tile border, random)
        rng = np.random.default_rng(0)
        qr = [(0, 0, 0), (0, 0, 128), (B - 1, Hq - 1, N - 1)] + \
             [(int(rng.integers(B)), int(rng.integers(Hq)), int(rng.integers(N))) for _ in range(5)]
        kr = [(0, 0, 0), (B - 1, Hkv - 1, N - 1), (0, Hkv // 2, 127)] + \
             [(int(rng.integers(B)), int(rng.integers(Hkv)), int(rng.integers(N))) for _ in range(3)]
        o, l = ctx.split_output(fwd, fa.BF16, shp)
        edq, edk, edv = ob.backward_rows(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                                         do.float().cpu().numpy(), o.float().cpu().numpy(), l.cpu().numpy(), B, Hq, Hkv, N, D,
                                         qr, kr, True, threads=min(8, os.cpu_count() or 1))
        gq = grads[L.dq_offset:L.dq_offset + L.q_elements * 4].view(torch.float32).view(B, Hq, N, D)
        gk = grads[L.dk_offset:L.dk_offset + L.kv_elements * 4].view(torch.float32).view(B, Hkv, N, D)
        gv = grads[L.dv_offset:L.dv_offset + L.kv_elements * 4].view(torch.float32).view(B, Hkv, N, D)
        err = {"max_abs_dq": float(np.abs(np.stack([gq[i].cpu().numpy() for i in qr]) - edq).max()),
               "max_abs_dk": float(np.abs(np.stack([gk[i].cpu().numpy() for i in kr]) - edk).max()),
               "max_abs_dv": float(np.abs(np.stack([gv[i].cpu().numpy() for i in kr]) - edv).max())}
        parity = dict(err, dq_rows=len(qr), dkv_rows=len(kr), ok=max(err.values()) <= 2e-2 and ctx.device_status() == 0)
        if not parity["ok"]:
            return gate("grouped_backward_tflops", parity)
    sampler = ClockSampler(device_index)
    ctx.set_kernel_timing(True)
    ctx.take_kernel_time()
    torch.cuda.synchronize()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        ctx.backward_grouped(fa.BF16, shp, cfg, packed, grads)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    loop_ms = e0.elapsed_time(e1)
    ms = loop_ms / steps
    kms, kn = ctx.take_kernel_time()
    ctx.set_kernel_timing(False)
    flops = 10 * B * Hq * N * N * D // 2
    kernel_ms = kms / steps  # the tensor-core kernels of one call
    traffic = NCU_TRAFFIC.get("backward") if not dims else None
    return {"metric": "grouped_backward_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms,
            "flop_per_step": flops, "workload": "C5 B=%d Hq=%d Hkv=%d N=8192 D=128 causal bf16, f32 gradients" % (B, Hq, Hkv),
            "roofline": tensor_roofline(peaks, flops, kernel_ms, loop_ms, clocks.get("reasons"), BACKWARD_KERNELS,
                                        traffic, "dram bytes read+written, both kernels of one call: 8 x one ncu capture of "
                                                 "one eighth of this workload (profiles/)" if traffic else None, BACKWARD_NOTE),
            "clocks": clocks, "parity": parity}


def c2_rows_oracle(ob, np, q, k, v, rows, layout, threads, slopes=None):
    """Oracle O/LSE of sampled (b, h, row) of a C2-shaped call in either layout (host f32 arrays of the de-quantised
    inputs): RoPE materialised with the oracle formula, then the row oracle, with the ALiBi bias when slopes are given."""
    c = C2
    B, Hq, Hkv, N, D, theta = c["B"], c["Hq"], c["Hkv"], c["N"], c["D"], c["theta"]
    shp = ob._shape(B, Hq, Hkv, N, N, D)
    if layout == ob.HEAD_MAJOR:
        rk = ob.rotate_rows(k, D, np.tile(np.arange(N, dtype=np.uint64), B * Hkv), theta).reshape(B, Hkv, N, D)
        rq = q.reshape(B, Hq, N, D).copy()
        for (b, h, r) in dict.fromkeys(rows):  # a row listed twice is still rotated once
            rq[b, h, r] = ob.rotate_rows(rq[b, h, r], D, [r], theta)
    else:
        rk = ob.rotate_rows(k, D, np.repeat(np.tile(np.arange(N, dtype=np.uint64), B), Hkv), theta).reshape(B, N, Hkv, D)
        rq = q.reshape(B, N, Hq, D).copy()
        for (b, h, r) in dict.fromkeys(rows):
            rq[b, r, h] = ob.rotate_rows(rq[b, r, h], D, [r], theta)
    if slopes is None:
        return ob.forward_rows(rq, rk, v, shp, layout, rows, True, threads=threads)
    return ob.forward_rows_alibi(rq, rk, v, shp, layout, rows, slopes, 0, 0, True, threads=threads)


def bench_prefill_variants(torch, np, fa, ctx, peaks, steps, warmup, ob=None, device_index=0):
    """The C2 prefill shape through the two widened modes of the forward: the ALiBi score bias on the rectangular
    projection entry point (bf16) and IEEE binary16 storage (GQA + RoPE, head-major).  Same flops as the headline."""
    c = C2
    B, Hq, Hkv, N, D, theta = c["B"], c["Hq"], c["Hkv"], c["N"], c["D"], c["theta"]
    shp, cfg, rot = fa.shape(B, Hq, Hkv, N, N, D), fa.config(True), fa.rotary(theta, 0)
    flops = prefill_flops(c)
    results = {}
    rows = [(0, 0, 0), (0, 1, 129), (B - 1, Hq - 1, N - 1)] + sample_rows(np, 5, 23)

    def timed(name, kernel, fn, note, check):
        for _ in range(warmup):
            fn()
        parity = check() if ob is not None else None
        if parity is not None and not parity["ok"]:
            results[name] = gate(name, parity)
            return
        sampler = ClockSampler(device_index)
        ctx.set_kernel_timing(True)
        ctx.take_kernel_time()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        sampler.start()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        loop_ms = e0.elapsed_time(e1)
        ms = loop_ms / steps
        kms, kn = ctx.take_kernel_time()
        ctx.set_kernel_timing(False)
        kms /= max(kn, 1)
        results[name] = {"value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "workload": note,
                         "roofline": tensor_roofline(peaks, flops, kms, loop_ms, clocks.get("reasons"), kernel),
                         "parity": parity}

    g = torch.Generator(device="cuda").manual_seed(21)
    q = torch.randn(B, N, Hq, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, N, Hkv, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, N, Hkv, D, generator=g, device="cuda").bfloat16()
    out = ctx.create_output_buffer(fa.BF16, shp)
    slopes = [2.0 ** -(8.0 * (h + 1) / Hq) for h in range(Hq)]

    def check_alibi():
        eo, el = c2_rows_oracle(ob, np, q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), rows,
                                ob.PROJECTION, min(8, os.cpu_count() or 1), np.array(slopes, np.float32))
        o, l = ctx.split_output(out, fa.BF16, shp, fa.PROJECTION)
        o = o.view(B, N, Hq, D)
        ao = np.stack([o[b, r, h].float().cpu().numpy() for (b, h, r) in rows])
        al = np.array([float(l[b, h, r]) for (b, h, r) in rows])
        par = {"rows": len(rows), "max_abs_o": float(np.abs(ao - eo).max()), "max_abs_lse": float(np.abs(al - el).max())}
        par["ok"] = par["max_abs_o"] <= 2e-2 and par["max_abs_lse"] <= 2e-3
        return par

    timed("alibi", "fwd_sm100_kernel<128,false,ALIBI>",
          lambda: ctx.forward_projection_rope_asymmetric_alibi(fa.BF16, shp, cfg, rot, slopes, 0, 0, q, k, v, out),
          "C2 shape, projection layout, bf16, RoPE + ALiBi (slopes 2^(-8(h+1)/Hq))", check_alibi)
    q16, k16, v16 = (x.transpose(1, 2).contiguous().half() for x in (q, k, v))
    out16 = ctx.create_output_buffer(fa.F16, shp)

    def check_f16():
        eo, el = c2_rows_oracle(ob, np, q16.float().cpu().numpy(), k16.float().cpu().numpy(), v16.float().cpu().numpy(), rows,
                                ob.HEAD_MAJOR, min(8, os.cpu_count() or 1))
        o, l = ctx.split_output(out16, fa.F16, shp)
        ao = np.stack([o[b, h, r].float().cpu().numpy() for (b, h, r) in rows])
        al = np.array([float(l[b, h, r]) for (b, h, r) in rows])
        par = {"rows": len(rows), "max_abs_o": float(np.abs(ao - eo).max()), "max_abs_lse": float(np.abs(al - el).max())}
        par["ok"] = par["max_abs_o"] <= 2e-2 and par["max_abs_lse"] <= 2e-3
        return par

    timed("binary16", "fwd_sm100_kernel<128,false,false,F16IO>",
          lambda: ctx.forward_grouped_rope(fa.F16, shp, cfg, rot, q16, k16, v16, out16),
          "C2 shape, head-major, IEEE binary16 storage, RoPE", check_f16)
    return results


def bench_chunked_prefill(torch, np, fa, ctx, peaks, warmup, ob=None, device_index=0, reps=3, shadow=True):
    """Config 4 (prefill part): one 32768-token sequence fed in 2048-token chunks into a growing paged cache."""
    Hq, Hkv, D, N, chunk, ps, theta = 64, 8, 128, 32768, 2048, 16, 500000.0
    g = torch.Generator(device="cuda").manual_seed(13)
    q = torch.randn(N, Hq * D, generator=g, device="cuda").bfloat16()
    k = torch.randn(N, Hkv * D, generator=g, device="cuda").bfloat16()
    v = torch.randn(N, Hkv * D, generator=g, device="cuda").bfloat16()
    cache = fa.CudaPagedKvCache(ctx, fa.BF16, ps, N // ps + 8, Hkv, D)
    if shadow:
        cache.enable_prefill_shadow()
    out = ctx.empty_bytes(chunk * Hq * D * 2 + Hq * chunk * 4)
    cfg = fa.config(True)
    keep = {}

    def run(capture=None):
        cache.reset()
        for start in range(0, N, chunk):
            ctx.chunked_prefill_paged(cache, Hq, chunk, cfg, theta, 0, q[start:start + chunk], k[start:start + chunk],
                                      v[start:start + chunk], out)
            if capture and start in capture:
                o = out[:chunk * Hq * D * 2].view(torch.bfloat16).view(chunk, Hq, D)
                l = out[chunk * Hq * D * 2:].view(torch.float32).view(Hq, chunk)
                keep[start] = (torch.stack([o[r, h] for (h, r) in capture[start]]).float().cpu().numpy(),
                               np.array([float(l[h, r]) for (h, r) in capture[start]], np.float32))
    parity = None
    if ob is not None:
        # oracle gate: first, middle and last chunk; first / last row, a tile border and a page border, random rows
        rng = np.random.default_rng(14)
        capture = {st: list(dict.fromkeys((int(rng.integers(Hq)), r) for r in (0, 15, 16, 127, 128, chunk - 1, int(rng.integers(chunk)))))
                   for st in (0, 7 * chunk, N - chunk)}
        run(capture)
        torch.cuda.synchronize()
        Kc, Vc = cache.download()
        entries = np.array(cache.table().export(), np.int64)
        logical = (entries[:, None] * ps + np.arange(ps)[None, :]).reshape(-1)[:N]
        kc, vc = Kc.float().numpy()[logical], Vc.float().numpy()[logical]
        worst_o = worst_l = 0.0
        for st, pairs in capture.items():
            rq = q[st:st + chunk].float().cpu().numpy().reshape(chunk, Hq, D)
            for (h, r) in pairs:
                rq[r, h] = ob.rotate_rows(rq[r, h], D, [st + r], theta)
            eo, el = ob.forward_rows(rq, kc[:st + chunk], vc[:st + chunk], ob._shape(1, Hq, Hkv, chunk, st + chunk, D, st),
                                     ob.PROJECTION, [(0, h, r) for (h, r) in pairs], True, threads=min(8, os.cpu_count() or 1))
            worst_o = max(worst_o, float(np.abs(keep[st][0] - eo).max()))
            worst_l = max(worst_l, float(np.abs(keep[st][1] - el).max()))
        parity = {"rows": sum(len(p) for p in capture.values()), "chunks": len(capture), "max_abs_o": worst_o,
                  "max_abs_lse": worst_l, "ok": worst_o <= 2e-2 and worst_l <= 2e-3 and ctx.device_status() == 0}
        if not parity["ok"]:
            return gate("chunked_prefill_tflops", parity)
    for _ in range(max(1, warmup - 2)):
        run()
    sampler = ClockSampler(device_index)
    ctx.set_kernel_timing(True)
    ctx.take_kernel_time()
    torch.cuda.synchronize()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    loop_ms = e0.elapsed_time(e1)
    ms = loop_ms / reps
    kms, kn = ctx.take_kernel_time()
    ctx.set_kernel_timing(False)
    kernel_ms = kms / reps  # the 16 attention launches of one sequence
    flops = 4 * Hq * D * N * N // 2
    return {"metric": "chunked_prefill_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_sequence": ms,
            "flop_per_sequence": flops,
            "roofline": tensor_roofline(peaks, flops, kernel_ms, loop_ms, clocks.get("reasons"),
                                        "fwd_sm100_kernel<128,paged" + ("" if shadow else ",CONVK") + "> x 16 chunks", NCU_TRAFFIC.get("chunked"),
                                        "dram bytes read+written of the last chunk's launch scaled by flops to 16 chunks, one "
                                        "ncu capture (profiles/)" if NCU_TRAFFIC.get("chunked") else None),
            "clocks": clocks, "parity": parity,
            "workload": "C4 1 x 32768 tokens in 2048-token chunks, Hq=64 Hkv=8 D=128 causal bf16, page 16, RoPE fused "
                        "into the cache append (K) and into the attention kernel (Q)" +
                        ("; the cache keeps a binary16 shadow of K (flat_paged_kv_cache_enable_prefill_shadow)" if shadow else
                         "; K tiles converted to binary16 inside the kernel (no shadow)")}


def splitkv_slice(torch, np, fd, rank, world, n, ps, Hkv, D):
    """This rank's slice of the 131072-token sequence: seeded K/V in a slice-local paged cache whose pages are a
    seeded permutation.  Any rank can regenerate any other rank's slice from the seeds (the parity gate does)."""
    first, count = fd.shard_pages(n, ps, world, rank)
    pages = count // ps
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    K = torch.randn(pages * ps, Hkv * D, generator=g, device="cuda").bfloat16()
    V = torch.randn(pages * ps, Hkv * D, generator=g, device="cuda").bfloat16()
    tab = np.random.default_rng(rank).permutation(pages).astype(np.int32).reshape(1, pages)
    return first, count, pages, K, V, tab


def bench_splitkv_128k(torch, np, dist, fa, ctx, peaks, rank, world, steps, warmup, ob=None):
    """Config 4 (decode part): one 131072-token sequence, KV axis split across the ranks; every rank
    decodes its slice, the (O, LSE) partials are all-gathered over NCCL and merged on every rank.  Rank 0 also
    decodes the whole sequence on its own GPU (`one_gpu_ms`) and checks both results against the CPU oracle."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("flat_distributed", os.path.join(ROOT, "flat-attention_b200", "distributed.py"))
    fd = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(fd)
    Hq, Hkv, D, ps, theta, n = 64, 8, 128, 16, 500000.0, 131072
    first, count, pages, K, V, tab = splitkv_slice(torch, np, fd, rank, world, n, ps, Hkv, D)
    Q = torch.randn(1, Hq * D, generator=torch.Generator(device="cuda").manual_seed(99), device="cuda").bfloat16()
    lens, qpos = np.array([count], np.int32), np.array([n - 1], np.int32)
    args = dict(num_seqs=1, q_heads=Hq, kv_heads=Hkv, head_dim=D, page_size=ps, physical_pages=pages, max_pages_per_seq=pages,
                page_tables_dev=torch.from_numpy(tab).cuda(), context_lens_dev=torch.from_numpy(lens).cuda(),
                q_rope_positions_dev=torch.from_numpy(qpos).cuda(), host_page_tables=None, host_context_lens=lens,
                cfg=fa.config(True), theta=theta, q=Q, k=K, v=V)
    out = ctx.create_decode_output_buffer(fa.BF16, 1, Hq, D)
    block = Hq * (D + 1)
    gathered = torch.empty(world * block, dtype=torch.float32, device="cuda")
    partial = gathered[rank * block:(rank + 1) * block]  # this rank's block of the gather buffer (in-place all-gather)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    dist.barrier()  # the communicator exists once the group has run a collective
    comm = fd.nccl_comm_ptr()
    abi = {k: v for k, v in args.items() if k not in ("cfg", "theta", "q", "k", "v")}

    def step():
        # the whole step through the C ABI: partial, in-place ncclAllGather, local merge
        ctx.splitkv_decode_nccl(comm, rank, world, fa.BF16, cfg=args["cfg"], theta=theta, q=Q, k=K, v=V, gathered=gathered,
                                out=out, **abi)
    for _ in range(warmup):
        step()

    # rank 0: the whole sequence in one cache on one GPU (the other ranks' slices regenerated from their seeds)
    one_gpu, parity = None, None
    if rank == 0:
        Ks, Vs = [], []
        for r in range(world):
            _, _, _, Kr, Vr, tr = splitkv_slice(torch, np, fd, r, world, n, ps, Hkv, D)
            rows = torch.from_numpy((tr.reshape(-1, 1).astype(np.int64) * ps + np.arange(ps)[None, :]).reshape(-1)).cuda()
            Ks.append(Kr[rows])
            Vs.append(Vr[rows])
            del Kr, Vr
        Kf, Vf = torch.cat(Ks), torch.cat(Vs)  # logical order, [n, Hkv*D]
        del Ks, Vs
        full_tab = np.random.default_rng(77).permutation(n // ps).astype(np.int32).reshape(1, -1)
        phys = torch.from_numpy((full_tab.reshape(-1, 1).astype(np.int64) * ps + np.arange(ps)[None, :]).reshape(-1)).cuda()
        Kp, Vp = torch.empty_like(Kf), torch.empty_like(Vf)
        Kp[phys], Vp[phys] = Kf, Vf
        flens = np.array([n], np.int32)
        d_tab, d_len, d_pos = torch.from_numpy(full_tab).cuda(), torch.from_numpy(flens).cuda(), torch.from_numpy(qpos).cuda()
        out1 = ctx.create_decode_output_buffer(fa.BF16, 1, Hq, D)

        def step1():
            ctx.decode_paged_batched(fa.BF16, 1, Hq, Hkv, D, ps, n // ps, n // ps, d_tab, d_len, d_pos, None, flens, qpos,
                                     fa.config(True), theta, Q, Kp, Vp, out1)
        for _ in range(warmup):
            step1()
        ctx.set_kernel_timing(True)
        ctx.take_kernel_time()
        tot1 = 0.0
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step1()
            e1.record()
            torch.cuda.synchronize()
            tot1 += e0.elapsed_time(e1)
        kms1, kn1 = ctx.take_kernel_time()
        ctx.set_kernel_timing(False)
        one_gpu = {"ms_per_step": tot1 / steps, "kernel_ms": kms1 / max(kn1, 1)}
        if ob is not None:
            # oracle over all 131072 tokens, one KV head (its group of query heads) at a time
            o8, l8 = ctx.split_decode_output(out, fa.BF16, 1, Hq, D)
            o1, l1 = ctx.split_decode_output(out1, fa.BF16, 1, Hq, D)
            G = Hq // Hkv
            qf = Q[0].float().cpu().numpy().reshape(Hq, D)
            err = {"max_abs_o": 0.0, "max_abs_lse": 0.0, "one_gpu_max_abs_o": 0.0, "one_gpu_max_abs_lse": 0.0}
            for kvh in range(Hkv):
                kh = Kf[:, kvh * D:(kvh + 1) * D].float().cpu().numpy()
                vh = Vf[:, kvh * D:(kvh + 1) * D].float().cpu().numpy()
                eo, el = oracle_decode_row(ob, np, qf[kvh * G:(kvh + 1) * G].reshape(-1), kh, vh, G, 1, D, theta, n - 1)
                eo = eo.reshape(G, D)
                for tag, (o, l) in (("", (o8, l8)), ("one_gpu_", (o1, l1))):
                    err[tag + "max_abs_o"] = max(err[tag + "max_abs_o"],
                                                 float(np.abs(o[0, kvh * G:(kvh + 1) * G].float().cpu().numpy() - eo).max()))
                    err[tag + "max_abs_lse"] = max(err[tag + "max_abs_lse"],
                                                   float(np.abs(l[0, kvh * G:(kvh + 1) * G].cpu().numpy() - el).max()))
            parity = dict(err, heads=Hq, tokens=n,
                          ok=max(err["max_abs_o"], err["one_gpu_max_abs_o"]) <= 2e-2 and
                          max(err["max_abs_lse"], err["one_gpu_max_abs_lse"]) <= 2e-3 and ctx.device_status() == 0)
        del Kf, Vf  # (the one-GPU cache Kp / Vp stays: its step is replayed from a graph below)
    ok = torch.tensor([1 if (parity is None or parity["ok"]) else 0], device="cuda")
    dist.broadcast(ok, 0)
    if int(ok.item()) == 0:
        return dict(gate("splitkv_decode_128k", parity), one_gpu=one_gpu)

    ctx.set_kernel_timing(True)
    ctx.take_kernel_time()
    tot, tot_merge = 0.0, 0.0
    for _ in range(steps):
        flush.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        ctx.decode_paged_batched_partial(fa.BF16, out=partial, **args)
        e1.record()
        ctx.splitkv_merge_nccl(comm, rank, world, fa.BF16, Hq, D, gathered, out)
        e2.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e2)
        tot_merge += e1.elapsed_time(e2)
    kms, kn = ctx.take_kernel_time()
    ctx.set_kernel_timing(False)

    # The same step replayed from a CUDA graph: a decode step is a handful of short kernels plus one small collective, so
    # the event window above is mostly the host's time to enqueue them; a serving loop captures the step once.  The
    # library calls only enqueue (scratch sized, plan cached), and NCCL collectives can be captured.
    def graph_ms(fn, reps):
        side = torch.cuda.Stream()
        main = ctx.stream
        try:
            ctx.set_stream(side)
            with torch.cuda.stream(side):
                fn()
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                fn()
            total = 0.0
            for _ in range(reps):
                flush.zero_()
                torch.cuda.synchronize()
                if world > 1:
                    dist.barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                g.replay()
                b.record()
                torch.cuda.synchronize()
                total += a.elapsed_time(b)
            return total / reps, None
        except Exception as e:  # a capture that fails is reported, never fatal
            return None, repr(e)[:300]
        finally:
            torch.cuda.synchronize()
            ctx.set_stream(main)
    g_ms, g_err = graph_ms(step, steps)
    g1_ms = g1_err = None
    if rank == 0 and one_gpu is not None:
        world_saved, world = world, 1  # the single-GPU replay has no barrier partner
        try:
            g1_ms, g1_err = graph_ms(step1, steps)
        finally:
            world = world_saved
        one_gpu["graph_ms_per_step"], one_gpu["graph_error"] = g1_ms, g1_err
    # The same step over NVLink peer memory (flat_splitkv_decode_peer): the partial, then ONE kernel that stores it into
    # every rank's buffer, waits for the others' flags and merges.  Same bits as the NCCL route (checked).
    peer = {}
    xchg = None
    try:
        xchg = fa.SplitKvPeerExchange(ctx, rank, world, Hq, D)
    except Exception as e:
        peer["error"] = repr(e)[:300]
    made = torch.tensor([1 if xchg is not None else 0], device="cuda")
    dist.all_reduce(made, op=dist.ReduceOp.MIN)  # the ranks agree before anyone enters the handle exchange
    if int(made.item()) == 0:
        if xchg is not None:
            xchg.close()
        xchg = None
        peer.setdefault("error", "another rank could not create its exchange buffer")
    else:
        try:
            fd.connect_peer_exchange(xchg)
        except Exception as e:  # raised on every rank or on none
            peer["error"] = repr(e)[:300]
            xchg.close()
            xchg = None
    p_ms = pg_ms = -1.0
    if xchg is not None:
        out_p = ctx.create_decode_output_buffer(fa.BF16, 1, Hq, D)

        def step_peer():
            ctx.splitkv_decode_peer(xchg, fa.BF16, cfg=args["cfg"], theta=theta, q=Q, k=K, v=V, out=out_p, **abi)
        for _ in range(warmup):
            step_peer()
        tot_p = 0.0
        for _ in range(steps):
            flush.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step_peer()
            b.record()
            torch.cuda.synchronize()
            tot_p += a.elapsed_time(b)
        p_ms = tot_p / steps
        peer["same_bits_as_nccl_route"] = bool(torch.equal(out_p, out)) and ctx.device_status() == 0
        pg, peer["graph_error"] = graph_ms(step_peer, steps)
        pg_ms = pg if pg is not None else -1.0
        torch.cuda.synchronize()
        dist.barrier()  # nobody unmaps a buffer a peer may still store into
        xchg.close()
    t = torch.tensor([tot / steps, tot_merge / steps, kms / max(kn, 1), g_ms if g_ms is not None else -1.0, p_ms, pg_ms],
                     device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_merge, kernel_ms = float(t[0]), float(t[1]), float(t[2])
    graph_step_ms = float(t[3]) if g_ms is not None else None
    if xchg is not None:
        same = torch.tensor([1 if peer["same_bits_as_nccl_route"] else 0], device="cuda")
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        peer.update(ms_per_step=float(t[4]), graph_ms_per_step=float(t[5]) if float(t[5]) > 0 else None,
                    same_bits_as_nccl_route=bool(int(same.item())),
                    what="flat_splitkv_decode_peer: partial decode, then one kernel: 16-byte peer stores of the 33 KB block "
                         "into every rank's buffer, flag, bounded wait for the others' flags, merge")
        if one_gpu:
            peer["speedup_vs_one_gpu"] = one_gpu["ms_per_step"] / peer["ms_per_step"]
            if one_gpu.get("graph_ms_per_step") and peer["graph_ms_per_step"]:
                peer["graph_speedup_vs_one_gpu"] = one_gpu["graph_ms_per_step"] / peer["graph_ms_per_step"]
    kv_bytes = n * Hkv * D * 2 * 2
    per_gpu_gbs = kv_bytes / world / (kernel_ms * 1e-3) / 1e9
    return {"metric": "splitkv_decode_128k", "ms_per_step": ms, "gather_merge_ms": ms_merge,
            "partial_kernel_ms": kernel_ms, "one_gpu": one_gpu,
            "graph_ms_per_step": graph_step_ms, "graph_error": g_err, "peer": peer,
            "speedup_vs_one_gpu": (one_gpu["ms_per_step"] / ms) if one_gpu else None,
            "graph_speedup_vs_one_gpu": (one_gpu["graph_ms_per_step"] / graph_step_ms)
            if one_gpu and one_gpu.get("graph_ms_per_step") and graph_step_ms else None,
            "aggregate_kv_gbs": kv_bytes / (ms * 1e-3) / 1e9, "per_gpu_kv_gbs": per_gpu_gbs,
            "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": per_gpu_gbs / peaks["hbm_gbs"], "kernel": "decode_mma_kernel<128> (one rank's slice)",
                         "kernel_ms": kernel_ms, "peak_source": peaks["source"]},
            "kv_bytes_total": kv_bytes, "gathered_bytes": world * Hq * (D + 1) * 4, "parity": parity,
            "workload": "1 sequence x 131072 tokens, Hq=64 Hkv=8 D=128 bf16, page 16, KV split over %d GPUs, in-place ncclAllGather "
                        "issued by the library (flat_splitkv_merge_nccl); "
                        "ms_per_step = partial + gather + merge between CUDA events, max over ranks; partial_kernel_ms = the "
                        "decode kernel alone" % world}


def bench_strong(torch, np, dist, fa, ctx, peaks, rank, world, steps, warmup, fd):
    """Strong scaling of the two fixed tensor-bound problems: the 32 (batch, kv_head) units of the C2 prefill and the 16
    units of the C5 backward are dealt to the ranks in contiguous blocks (distributed.shard_units); no collective on
    the data path.  A unit with its query-head group is independent of every other, so a rank's block runs as one call
    with batch 1 and the block's heads.  Aggregate = the whole problem's flop / the slowest rank's time."""
    c = C2
    N, D, theta, G = c["N"], c["D"], c["theta"], c["Hq"] // c["Hkv"]
    units = fd.shard_units(c["B"] * c["Hkv"], world, rank)
    u = len(units)
    res = {}
    if u > 0:
        g = torch.Generator(device="cuda").manual_seed(500 + rank)
        q = torch.randn(1, u * G, N, D, generator=g, device="cuda").bfloat16()
        k = torch.randn(1, u, N, D, generator=g, device="cuda").bfloat16()
        v = torch.randn(1, u, N, D, generator=g, device="cuda").bfloat16()
        shp = fa.shape(1, u * G, u, N, N, D)
        out = ctx.create_output_buffer(fa.BF16, shp)
        cfg, rot = fa.config(True), fa.rotary(theta, 0)

        def step():
            ctx.forward_grouped_rope(fa.BF16, shp, cfg, rot, q, k, v, out)
    else:
        def step():
            pass
    for _ in range(warmup):
        step()
    ctx.set_kernel_timing(True)
    ctx.take_kernel_time()
    ms = timed_region(torch, dist, world, step, steps) / steps
    kms, kn = ctx.take_kernel_time()
    ctx.set_kernel_timing(False)
    t = torch.tensor([kms / max(kn, 1)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    flops = prefill_flops(c)
    res["prefill_c2"] = {"units_total": c["B"] * c["Hkv"], "units_this_rank": u, "ms_per_step": ms,
                         "slowest_rank_kernel_ms": float(t[0]), "aggregate_tflops": flops / (ms * 1e-3) / 1e12}
    b5 = C5
    units5 = fd.shard_units(b5["B"] * b5["Hkv"], world, rank)
    u5 = len(units5)
    G5 = b5["Hq"] // b5["Hkv"]
    leg = bench_backward(torch, np, fa, ctx, peaks, max(3, min(steps, 10)), warmup, None, (1, u5 * G5, u5)) if u5 > 0 else None
    t = torch.tensor([leg["ms_per_step"] if leg else 0.0, leg["roofline"]["kernel_ms"] if leg else 0.0], device="cuda",
                     dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    flops5 = 10 * b5["B"] * b5["Hq"] * b5["N"] * b5["N"] * b5["D"] // 2
    res["backward_c5"] = {"units_total": b5["B"] * b5["Hkv"], "units_this_rank": u5, "ms_per_step": float(t[0]),
                          "slowest_rank_kernel_ms": float(t[1]), "aggregate_tflops": flops5 / (float(t[0]) * 1e-3) / 1e12}
    return res


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
    ap.add_argument("--no-shadow", action="store_true", help="chunked prefill without the binary16 K shadow of the paged cache")
    ap.add_argument("--chunked-only", action="store_true", help="run only the chunked prefill against the paged cache "
                                                               "(N=1; --steps = timed passes): a short command for profiler captures")
    ap.add_argument("--backward-only", default=None, metavar="B,HQ,HKV", help="run only the grouped backward of config 5 with this "
                    "batch and head counts (N=8192, D=128 as in config 5; '2,32,8' is config 5 itself): a short command "
                    "for profiler captures, which want a scratch of a few hundred MB rather than config 5's 4.3 GB")
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
            print(json.dumps({"prefill_variants": bench_prefill_variants(torch, np, fa, ctx, peaks, max(1, args.steps), args.warmup)}),
                  flush=True)
        return
    if args.backward_only:
        if rank == 0:
            dims = tuple(int(x) for x in args.backward_only.split(","))
            ob_b = None
            if not args.no_cpu:
                from oracle import binding as ob_b
            print(json.dumps({"backward": bench_backward(torch, np, fa, ctx, peaks, max(1, args.steps), args.warmup, ob_b,
                                                         None if dims == (C5["B"], C5["Hq"], C5["Hkv"]) else dims, local_rank)}),
                  flush=True)
        return
    if args.chunked_only:
        if rank == 0:
            ob_c = None
            if not args.no_cpu:
                from oracle import binding as ob_c
            print(json.dumps({"chunked_prefill": bench_chunked_prefill(torch, np, fa, ctx, peaks, args.warmup, ob_c, local_rank,
                                                                       reps=max(1, args.steps), shadow=not args.no_shadow)}), flush=True)
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
        # (inputs validated like the reference's forward: the non-finite scan runs on the device as the chunks land)
        ctx.forward_host(fa.BF16, fa.HEAD_MAJOR, shp, cfg, rot, hq, hk, hv, host_out, check_finite=True)

    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()

    def step_copy_floor():
        # the same bytes as one end-to-end step, from and to the same pinned buffers, upload and download on two
        # streams, no kernel: what the host link alone allows at this number of ranks
        cur = torch.cuda.current_stream()
        copy_in.wait_stream(cur)
        copy_out.wait_stream(cur)
        with torch.cuda.stream(copy_in):
            dq.copy_(hq, non_blocking=True)
            dk.copy_(hk, non_blocking=True)
            dv.copy_(hv, non_blocking=True)
        with torch.cuda.stream(copy_out):
            host_out.copy_(out, non_blocking=True)
        cur.wait_stream(copy_in)
        cur.wait_stream(copy_out)

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

    gate_ok = parity is None or parity["ok"]
    if world > 1:
        flag = torch.tensor([1 if gate_ok else 0], device="cuda")
        dist.broadcast(flag, 0)
        gate_ok = bool(flag.item())
    if not gate_ok:
        # a kernel whose results differ from the oracle's is not timed
        if rank == 0:
            print(json.dumps({"metric": "prefill_attention_tflops", "parity": parity, "n_gpus": world,
                              "error": "parity gate failed: no throughput is reported"}), flush=True)
        raise SystemExit(1)

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
    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e = timed_region(torch, dist, world, step_e2e, e2e_steps)
    for _ in range(2):
        step_copy_floor()
    ms_floor = timed_region(torch, dist, world, step_copy_floor, e2e_steps)
    status = ctx.device_status()

    ms_per_step = ms / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12
    kms = kernel_ms / max(kernel_n, 1)
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
                "ms_per_step": ms_e2e / e2e_steps, "check_finite": True,
                "call": "flat_forward_host: pinned host Q/K/V in, device-side non-finite scan, attention, pinned host [O|LSE] out"},
        "e2e_floor": {"ms_per_step": ms_floor / e2e_steps, "e2e_over_floor": ms_e2e / ms_floor,
                      "what": "the same H2D and D2H bytes from the same pinned buffers on two streams, no kernel, max over ranks"},
        "gpu_launches": int(launches),
        "roofline": tensor_roofline(peaks, flops, kms, ms, (clocks or {}).get("reasons"), "fwd_sm100_kernel<128,false>",
                                    NCU_TRAFFIC["forward"],
                                    "dram bytes read+written per launch, one ncu capture of this workload (profiles/)"),
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
    ob_gate = None
    if not args.no_cpu:
        from oracle import binding as ob_gate
    if rank == 0 and world == 1:
        if not args.skip_extras:
            line["decode"] = bench_decode(torch, np, fa, ctx, peaks, max(5, min(args.steps, 20)), args.warmup, ob_gate)
            line["backward"] = bench_backward(torch, np, fa, ctx, peaks, max(3, min(args.steps, 10)), args.warmup, ob_gate,
                                              device_index=local_rank)
            line["chunked_prefill"] = bench_chunked_prefill(torch, np, fa, ctx, peaks, args.warmup, ob_gate, local_rank,
                                                            shadow=not args.no_shadow)
            line["prefill_variants"] = bench_prefill_variants(torch, np, fa, ctx, peaks, max(5, min(args.steps, 20)), args.warmup,
                                                              ob_gate, local_rank)
    if world > 1 and not args.skip_extras:
        extra = bench_splitkv_128k(torch, np, dist, fa, ctx, peaks, rank, world, max(5, min(args.steps, 20)), args.warmup,
                                   ob_gate if rank == 0 else None)
        line["splitkv_decode_128k"] = extra
        import importlib.util
        spec = importlib.util.spec_from_file_location("flat_distributed", os.path.join(ROOT, "flat-attention_b200", "distributed.py"))
        fd = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(fd)
        strong = bench_strong(torch, np, dist, fa, ctx, peaks, rank, world, max(5, min(args.steps, 20)), args.warmup, fd)
        # one GPU's time for the whole fixed problem: the weak-scaling step above is exactly that for C2; C5 is timed here
        full5 = bench_backward(torch, np, fa, ctx, peaks, max(3, min(args.steps, 10)), args.warmup, None)
        t5 = torch.tensor([full5["ms_per_step"]], device="cuda", dtype=torch.float64)
        dist.all_reduce(t5, op=dist.ReduceOp.MAX)
        strong["prefill_c2"]["one_gpu_ms"] = ms_per_step
        strong["prefill_c2"]["efficiency"] = ms_per_step / (world * strong["prefill_c2"]["ms_per_step"])
        strong["backward_c5"]["one_gpu_ms"] = float(t5[0])
        strong["backward_c5"]["efficiency"] = float(t5[0]) / (world * strong["backward_c5"]["ms_per_step"])
        strong["what"] = ("the fixed C2 / C5 problems dealt to the ranks by (batch, kv_head) unit, no collective; efficiency = "
                          "one-GPU time / (N x slowest rank's time)")
        line["strong"] = strong
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
