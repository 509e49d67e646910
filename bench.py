#!/usr/bin/env python
"""Benchmark of the causal self-attention forward+backward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" = one forward + one backward pass over one batch of the workload.  Default workload: the 7B-class GQA
configuration (B=2, Hq=28, Hkv=4, S=8192, D=128, bf16), the one the headline metric is quoted on.  With N > 1
(launched by torch.distributed.run, one rank per GPU) every rank runs the same per-GPU batch on its own shard of
batch x KV-head groups -- the path needs no communication -- so scaling is weak and `value` is the sum of all
ranks' FLOPs over the slowest rank's time.

Prints ONE JSON line (rank 0).  `value` is device-resident throughput; `e2e` goes through the public host-buffer
call (pinned host memory -> device -> results back to the host inside the timed region).
`--impl reference` times the reference project's own OpenMP CPU attention (oracle/_ref, built from the reference
sources) on a bounded sample of the same workload on this box's host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "causal attention fwd+bwd TFLOP/s (causal-adjusted 7*B*Hq*S^2*D), aggregate over GPUs"
UNIT = "TFLOP/s"
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}
# DRAM bytes (read + write) of one launch of the dominant kernel per batch element, from the ncu capture summarised in
# profiles/attn_bwd_tc_kernel_gqa7b_d128.md (captured on the full workload, batch 2; traffic grows in proportion to the batch)
NCU_DRAM_BYTES_PER_BATCH = {"gqa7b_d128": (1823.955e6 + 987.866e6) / 2}
# the same for the cache-mode forward kernel, one new token, no window (profiles/attn_fwd_tc_kernel_cache_mode_gqa7b_d128.md,
# captured at batch 16)
NCU_CACHED_DRAM_BYTES_PER_BATCH = {"gqa7b_d128": (268640768 + 5306880) / 16.0}


class stdout_to_stderr:
    """File-descriptor-level redirect of standard output to standard error.  NCCL prints a version banner on standard
    output when the first communicator of a process is made; this program's standard output carries ONE JSON line, so
    communicator set-up runs inside this."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)
        return self

    def __exit__(self, *a):
        sys.stdout.flush()
        os.dup2(self.saved, 1)
        os.close(self.saved)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period, self.samples, self.reasons, self.max_mhz = index, period_s, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


EXTRA_LEGS_LIMIT_S = 300      # strong-scaling + ring legs (N > 1) or the other workloads (N = 1) together
CPU_SAMPLE_MAX_SEQ = 8192     # one head at S = 8192 keeps two S x S fp32 matrices (2 x 268 MB): the largest length sampled
CPU_SAMPLE_PASSES = 3         # about 4 s per pass at S = 8192 on 16-32 cores


def _host_cores() -> int:
    try:
        import psutil
        n = psutil.cpu_count(logical=False)
        if n:
            return int(n)
    except Exception:
        pass
    return os.cpu_count() or 1


def _set_openmp_threads(n: int) -> None:
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its children; the CPU baseline is meant to use every core,
    so the thread count is set explicitly in the OpenMP runtime the checker libraries link."""
    import ctypes
    os.environ["OMP_NUM_THREADS"] = str(n)
    try:
        ctypes.CDLL("libgomp.so.1", mode=ctypes.RTLD_GLOBAL).omp_set_num_threads(int(n))
    except OSError:
        pass


def cpu_reference_sample(workload):
    """Times the reference's own CPU attention (attention core only) on ONE query head of ONE sequence of the
    workload's own length (capped at 8192: the reference keeps whole S x S score matrices); the causal FLOP formula
    is applied to the sample so the unit matches the GPU metric.  One warm-up pass, then CPU_SAMPLE_PASSES timed
    passes, on all physical cores.  The product arm's `cpu_baseline` and `--impl reference` both call this."""
    import numpy as np
    from oracle import cpu
    _set_openmp_threads(_host_cores())
    if not cpu.ref_available():
        cpu.build()
    kind = "reference" if cpu.ref_available() else "port"
    S = min(workload.seq, CPU_SAMPLE_MAX_SEQ)
    D = workload.head_dim
    rng = np.random.default_rng(20261125)
    q = (rng.standard_normal((1, 1, S, D)) * workload.qk_std).astype(np.float32)
    k = (rng.standard_normal((1, 1, S, D)) * workload.qk_std).astype(np.float32)
    v = (rng.standard_normal((1, 1, S, D)) * workload.v_std).astype(np.float32)
    do = (rng.standard_normal((1, 1, S, D)) * workload.do_std).astype(np.float32)
    flops = 7.0 * S * S * D
    times = []
    for i in range(1 + CPU_SAMPLE_PASSES):
        t0 = time.perf_counter()
        if kind == "reference":
            _, _, _, _, secs = cpu.ref_core_fwd_bwd(q, k, v, do, want_outputs=False)
            dt = secs[0] + secs[1]
        else:
            cpu.attn_fwd(q, k, v)
            cpu.attn_bwd(q, k, v, do)
            dt = time.perf_counter() - t0
        if i >= 1:
            times.append(dt)
    mean = sum(times) / len(times)
    cores = cpu.ref_threads() if kind == "reference" else cpu.oracle_threads()
    note = "" if S == workload.seq else f" (the workload's S = {workload.seq} does not fit the reference's dense S x S matrices)"
    return {"value": flops / mean / 1e12, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"1 sequence x 1 query head of the workload, S={S}{note}, D={D}, fp32, attention core only (dense S^2 work), "
                      f"1 warm-up + {len(times)} timed passes of {mean:.3f} s (passes capped at {CPU_SAMPLE_PASSES} whatever --steps says)",
            "ms_per_step": mean * 1e3}


def reference_cuda_sample(workload, q, k, v, do):
    """The reference's own CUDA flash kernels (oracle/_ref, rebuilt for sm_100a) on the same tensors, where they can run."""
    from oracle import cpu
    if workload.head_dim > 64:
        return {"unavailable": "the reference flash kernels stop at head_dim 64 (CudaFlashAttention.hpp:16)"}
    if not cpu.ref_cuda_available():
        return {"unavailable": "oracle/_ref/libsentinel_ref_cuda.so not built"}
    qf, kf, vf, dof = (t.float().numpy() for t in (q, k, v, do))
    _, _, _, _, _, ms = cpu.ref_cuda_flash(qf, kf, vf, dof, reps=5)
    total = ms[0] + ms[1]
    return {"value": workload.flops / (total * 1e-3) / 1e12, "unit": UNIT, "fwd_ms": ms[0], "bwd_ms": ms[1],
            "note": "fp32 tensors, fp16 WMMA operands, K/V repeated to the query heads as at its call site (repeat not timed)"}


def run_reference_arm(args, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    res = cpu_reference_sample(workload)
    line = {"impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            # the product arm's workload keys, value for value; what the CPU actually ran is in cpu_baseline.sample
            "config": {"workload": workload.name, "B_per_gpu": workload.batch, "global_batch": workload.batch * max(1, args.gpus),
                       "Hq": workload.q_heads, "Hkv": workload.kv_heads, "S": workload.seq, "D": workload.head_dim, "causal": True,
                       "parallelism": "host cores of rank 0 only (OpenMP); the other ranks exit without work"},
            "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": res["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_cached_forward(args, w):
    """Auxiliary mode (--cached-tokens T): T new tokens per sequence against a KV cache of the workload's length, the
    reference's decode step (CudaCausalSelfAttention.cu:318-341).  HBM-bound: the algorithmic bytes of one call are the
    K and V rows in use (read once per KV head) plus Q, O and LSE; prints its own JSON line."""
    import torch
    import sentinel_b200 as sb
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200 GPU: there is no CPU fallback for the product path")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    sb._lib.load()
    T, L = args.cached_tokens, w.seq
    B = w.batch
    g = torch.Generator(device="cpu").manual_seed(20261125 + w.index)
    mk = lambda h, s_, std: (torch.randn(B, h, s_, w.head_dim, generator=g) * std).to(torch.bfloat16).to(dev)
    q, kc, vc = mk(w.q_heads, T, w.qk_std), mk(w.kv_heads, L, w.qk_std), mk(w.kv_heads, L, w.v_std)
    o = torch.empty_like(q)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=dev)
    mask = dict(window=args.window, global_tokens=args.global_tokens) if args.window > 0 else {}

    def step():
        sb.attention_cached_forward(q, kc, vc, L, out=o, lse=lse, **mask)

    for _ in range(args.warmup):
        step()
    launches0 = sb.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clocks:
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    launches = sb.launch_count() - launches0
    keys = L if args.window <= 0 else min(L, args.window + T - 1 + args.global_tokens)
    kv_bytes = 2.0 * B * w.kv_heads * keys * w.head_dim * 2
    io_bytes = kv_bytes + 2.0 * q.numel() * 2 + 4.0 * lse.numel()
    peaks = load_peaks()
    peak = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    achieved = io_bytes / (ms * 1e-3) / 1e9
    line = {"metric": "attention_cached_fwd_hbm_gbs", "value": achieved, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w.name + "_cached", "B": B, "Hq": w.q_heads, "Hkv": w.kv_heads, "cache_length": L,
                       "new_tokens": T, "D": w.head_dim, "l2": f"K/V in use {kv_bytes / 1e6:.0f} MB per call",
                       "kernel_path": sb.last_path(), **mask},
            "tokens_per_s": B * T / (ms * 1e-3),
            "roofline": {"bound": "hbm", "kernel": "cache-mode forward kernel + split merge (timed as one call)", "achieved": achieved,
                         "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": f"{peaks['_source']} hbm_gbs",
                         "traffic": (NCU_CACHED_DRAM_BYTES_PER_BATCH[w.name] * B
                                     if w.name in NCU_CACHED_DRAM_BYTES_PER_BATCH and T == 1 and not mask else None),
                         "algorithmic_bytes": io_bytes},
            "gpu_launches": int(launches), "clocks": clocks.summary(), "device_status": sb.poll_device_status()}
    print(json.dumps(line), flush=True)


def run_pack_heads(args, w):
    """Auxiliary mode (--pack-heads): the boundary kernels on the workload's Q tensor -- fp32 feature-major -> rotated
    bf16 token-major (pack) and back with the inverse rotation (unpack).  HBM-bound: 6 bytes per element each way."""
    import torch
    import sentinel_b200 as sb
    from oracle import cpu
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200 GPU: there is no CPU fallback for the product path")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    sb._lib.load()
    B, H, S, D = w.batch, w.q_heads, w.seq, w.head_dim
    g = torch.Generator(device="cpu").manual_seed(20261125 + w.index)
    matrix = torch.randn(H * D, B * S, generator=g, dtype=torch.float32).to(dev)
    cos_t, sin_t = (torch.from_numpy(t).to(dev) for t in cpu.rope_tables(D, S, w.rope_base or 10000.0))
    packed = torch.empty(B, H, S, D, dtype=torch.bfloat16, device=dev)
    back = torch.empty_like(matrix)

    def pack():
        sb.pack_heads(matrix, B, H, S, D, cos_table=cos_t, sin_table=sin_t, out=packed)

    def unpack():
        sb.unpack_heads(packed, back, cos_table=cos_t, sin_table=sin_t, inverse=True)

    def ms_of(fn):
        for _ in range(args.warmup):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / args.steps

    launches0 = sb.launch_count()
    with ClockSampler(0) as clocks:
        t_pack, t_unpack = ms_of(pack), ms_of(unpack)
    n = matrix.numel()
    peaks = load_peaks()
    peak = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    gbs = lambda ms: 6.0 * n / (ms * 1e-3) / 1e9
    line = {"metric": "attention_pack_heads_hbm_gbs", "value": gbs(t_pack), "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t_pack, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32->bf16", "data": "synthetic",
            "config": {"workload": w.name + "_pack_heads", "B": B, "H": H, "S": S, "D": D, "elements": n,
                       "l2": f"{6 * n / 1e6:.0f} MB moved per call, larger than the 126 MB L2"},
            "roofline": {"bound": "hbm", "kernel": "pack64_kernel (rotary embedding + cast + relayout)", "achieved": gbs(t_pack),
                         "peak": peak, "unit": "GB/s", "frac": gbs(t_pack) / peak, "peak_source": f"{peaks['_source']} hbm_gbs",
                         "traffic": None, "algorithmic_bytes": 6.0 * n},
            "unpack": {"ms": t_unpack, "achieved": gbs(t_unpack), "frac": gbs(t_unpack) / peak,
                       "kernel": "unpack64_kernel (inverse rotation)"},
            "gpu_launches": int(sb.launch_count() - launches0), "clocks": clocks.summary()}
    print(json.dumps(line), flush=True)


def _make_timed(torch, dist, dev, world, local):
    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    def timed(fn, n):
        """n calls of fn between CUDA events on the current stream; returns max-over-ranks milliseconds."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        e1.synchronize()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    return barrier, timed


def copy_bound(torch, dist, dev, world, host_in, host_out_like, timed):
    """The plain transfer time of one e2e step: pinned H2D of Q, K, V, dO and D2H of O, LSE, dQ, dK, dV, one
    cudaMemcpyAsync per tensor, both directions at once on two streams, no kernels.  With N ranks all of them copy
    at the same time (they share the host's memory and PCIe root ports), so this is the ceiling the e2e figure of the
    same N can reach."""
    dev_in = [torch.empty(t.shape, dtype=t.dtype, device=dev) for t in host_in]
    dev_out = [torch.empty(t.shape, dtype=t.dtype, device=dev) for t in host_out_like]
    host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in host_out_like]
    up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def step():
        cur = torch.cuda.current_stream(dev)
        up.wait_stream(cur)
        down.wait_stream(cur)
        with torch.cuda.stream(up):
            for h, d in zip(host_in, dev_in):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(down):
            for d, h in zip(dev_out, host_out):
                h.copy_(d, non_blocking=True)
        cur.wait_stream(up)
        cur.wait_stream(down)

    step()
    return timed(step, 5) / 5


def run_other_workload(torch, sb, name, dev, peaks, steps=20):
    """fwd+bwd of another configuration on this GPU (device-resident), so that its figure is in the record too."""
    from sentinel_b200.workloads import WORKLOADS, make_inputs
    w = WORKLOADS[name]
    q, k, v, do = (t.to(dev) for t in make_inputs(w))
    o = torch.empty_like(q)
    lse = torch.empty(q.shape[:3], dtype=torch.float32, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)

    def fwd():
        sb.attention_forward(q, k, v, out=o, lse=lse)

    def bwd():
        sb.attention_backward(q, k, v, o, lse, do, dq=dq, dk=dk, dv=dv)

    def ms_of(fn):
        for _ in range(5):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / steps

    t_step = ms_of(lambda: (fwd(), bwd()))
    t_fwd, t_bwd = ms_of(fwd), ms_of(bwd)
    tf = w.flops / (t_step * 1e-3) / 1e12
    return {"workload": name, "B": w.batch, "Hq": w.q_heads, "Hkv": w.kv_heads, "S": w.seq, "D": w.head_dim, "value": tf,
            "unit": UNIT, "ms_per_step": t_step, "fwd_ms": t_fwd, "bwd_ms": t_bwd,
            "frac_of_burst_peak": tf / float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"])),
            "kernel_path": sb.last_path()}


def run_strong_scaling(torch, dist, sb, w, dev, rank, world, timed, steps, weak_ms_per_step):
    """The workload's OWN global batch cut over the ranks at (batch element, KV group) granularity, no communication:
    with 8 ranks every GPU gets one KV group (7 query heads) of the 7B-class configuration."""
    from sentinel_b200.workloads import make_inputs, shard_units
    units = shard_units(w.batch, w.kv_heads, rank, world)
    if not units or any(b != units[0][0] for b, _ in units):
        return {"unavailable": "a rank's units span more than one batch element"}
    g = w.q_heads // w.kv_heads
    b, hk0, hk1 = units[0][0], units[0][1], units[-1][1] + 1
    q, k, v, do = make_inputs(w)          # every rank draws the same global tensors and keeps its slice
    qs, dos = (t[b:b + 1, hk0 * g:hk1 * g].contiguous().to(dev) for t in (q, do))
    ks, vs = (t[b:b + 1, hk0:hk1].contiguous().to(dev) for t in (k, v))
    del q, k, v, do
    o = torch.empty_like(qs)
    lse = torch.empty(qs.shape[:3], dtype=torch.float32, device=dev)
    dq, dk, dv = torch.empty_like(qs), torch.empty_like(ks), torch.empty_like(vs)

    def step():
        sb.attention_forward(qs, ks, vs, out=o, lse=lse)
        sb.attention_backward(qs, ks, vs, o, lse, dos, dq=dq, dk=dk, dv=dv)

    for _ in range(3):
        step()
    ms = timed(step, steps) / steps
    value = w.flops / (ms * 1e-3) / 1e12
    return {"value": value, "unit": UNIT, "ms_per_step": ms, "scaling": "strong",
            "config": {"global_batch": w.batch, "units_total": w.batch * w.kv_heads, "units_per_gpu": len(units),
                       "query_heads_per_gpu": len(units) * g},
            "efficiency_vs_one_gpu": weak_ms_per_step / (world * ms),
            "one_gpu_ms_per_step": weak_ms_per_step}


def ring_oracle_check(torch, w_local, rank, world, o, lse, dq, dk, dv):
    """Sampled fp64 oracle of the FULL sequence against this rank's shard of the ring's results: a few query rows of
    one head (O, LSE, dQ) and, on the last rank, a few of the latest key columns of one KV head (dK, dV; early key
    columns need every later query, S^2 work the CPU cannot do at this length)."""
    import numpy as np
    from oracle import cpu
    from sentinel_b200.workloads import make_inputs
    _set_openmp_threads(_host_cores())
    S_local = w_local.seq
    h, hk = 5 % w_local.q_heads, 1 % w_local.kv_heads
    g = w_local.q_heads // w_local.kv_heads
    hq0 = hk * g
    qs, ks, vs, dos = [], [], [], []
    for r in range(world):                 # the full-sequence tensors of the heads sampled, shard by shard as the ranks drew them
        q, k, v, do = make_inputs(w_local, seed_offset=r)
        hs = sorted({h, *range(hq0, hq0 + g)})
        qs.append(q[:, hs].float().numpy()); dos.append(do[:, hs].float().numpy())
        ks.append(k[:, [h // g, hk]].float().numpy()); vs.append(v[:, [h // g, hk]].float().numpy())
    hs = sorted({h, *range(hq0, hq0 + g)})
    qf, dof, kf, vf = (np.concatenate(x, axis=2) for x in (qs, dos, ks, vs))
    base = rank * S_local
    out = {}
    # rows: head h against its KV head (index 0 of the kept pair)
    # The bound is stated for whole tensors, and dQ's norm is far from uniform over the rows: a row with n visible keys
    # has |dQ|^2 ~ 1/n, so the first rows of the sequence carry much of it (and, with two or three keys and no averaging
    # of the bf16 roundings of P and dS, the largest relative error).  A stratified sample estimates the whole-shard
    # figure without bias: every one of the first 256 rows of the sequence (weight 1; they cost next to nothing) plus
    # uniformly spaced rows of the rest, each standing for the rows between it and the next (weight = spacing).
    # A row costs (its position) x D oracle work: many rows on the early shards, fewer at the end of a long sequence.
    n_uniform = 256 if base + S_local <= 32768 else 90
    head_rows = np.arange(min(256, S_local)) if rank == 0 else np.zeros(0, dtype=np.int64)
    lo = len(head_rows)
    uni = np.unique(np.linspace(lo, S_local - 1, n_uniform).astype(np.int64))
    rows = (np.concatenate([head_rows, uni]) + base).astype(np.int32)
    weights = np.concatenate([np.ones(lo), np.full(len(uni), (S_local - lo) / len(uni))])
    hi = hs.index(h)
    wo, wl, wdq = cpu.attn_rows(qf[:, hi:hi + 1], kf[:, 0:1], vf[:, 0:1], dof[:, hi:hi + 1], 0, 0, rows)
    loc = rows - base
    got_o, got_dq = o[0, h, loc].float().cpu().numpy(), dq[0, h, loc].float().cpu().numpy()
    got_l = lse[0, h, loc].float().cpu().numpy()

    def errs(got, want, w=None):
        d2 = ((got - want) ** 2).sum(axis=-1)
        r2 = (want ** 2).sum(axis=-1)
        w = np.ones(len(d2)) if w is None else w
        return {"max_abs": float(np.abs(got - want).max()), "rel_l2": float(np.sqrt((w * d2).sum() / max((w * r2).sum(), 1e-60)))}

    out["o"], out["dq"] = errs(got_o, wo, weights), errs(got_dq, wdq, weights)
    out["lse_max_abs"] = float(np.abs(got_l - wl).max())
    out["rows_sampled"] = int(len(rows))
    if rank == world - 1:
        S = S_local * world
        cols = np.array([S - 385, S - 130, S - 1], dtype=np.int32)
        gi = [hs.index(x) for x in range(hq0, hq0 + g)]
        wdk, wdv = cpu.attn_cols(qf[:, gi], kf[:, 1:2], vf[:, 1:2], dof[:, gi], 0, 0, cols)
        locc = cols - base
        out["dk"] = errs(dk[0, hk, locc].float().cpu().numpy(), wdk)
        out["dv"] = errs(dv[0, hk, locc].float().cpu().numpy(), wdv)
        out["cols"] = [int(x) for x in cols]
    vals = [out[n] for n in ("o", "dq", "dk", "dv") if n in out]
    out["within_tolerance"] = bool(all(e["max_abs"] <= 2e-2 and e["rel_l2"] <= 5e-3 for e in vals) and out["lse_max_abs"] <= 2e-2)
    return out


def run_ring(torch, dist, sb, dev, rank, world, timed, steps, per_gpu_value):
    """The long-context workload: 16384 tokens per rank (131072 at 8 ranks), K/V chunks travelling round the ring."""
    import dataclasses
    from sentinel_b200.ring import GpuBackend, RingAttention
    from sentinel_b200.workloads import WORKLOADS, make_inputs
    w = WORKLOADS["longctx_ring"]
    shard = w.seq // w.seq_shards
    w_local = dataclasses.replace(w, seq=shard, seq_shards=1)
    q, k, v, do = (t.to(dev) for t in make_inputs(w_local, seed_offset=rank))
    from sentinel_b200.ring import NativeRing
    S = shard * world
    flops = 7.0 * w.batch * w.q_heads * float(S) ** 2 * w.head_dim

    def measure(ring):
        res = {}

        def fwd():
            res["o"], res["lse"] = ring.forward(q, k, v, keep_state=True)

        def bwd():
            res["g"] = ring.backward(q, k, v, res["o"], res["lse"], do, use_saved_state=True)

        for _ in range(2):
            fwd(); bwd()
        total = timed(lambda: (fwd(), bwd()), steps) / steps
        fwd_ms = timed(fwd, steps) / steps
        return res, total, fwd_ms

    # the schedule as the library runs it behind the C ABI (sntl_ring_attn_fwd / _bwd: NCCL from C++, no allocation)
    native = NativeRing()
    res, total, fwd_ms = measure(native)
    bwd_ms = total - fwd_ms                # the backward consumes the state its forward kept, so it is not timed alone
    # the same calls for a host that keeps its shards in the zigzag order (SNTL_FLAG_RING_ZIGZAG): nothing is redistributed.
    # The same device tensors serve (which tokens they stand for does not change the time).
    zz = NativeRing(zigzag_layout=True)
    _, zz_total, zz_fwd_ms = measure(zz)
    zz.close()
    # the same schedule driven from Python over torch.distributed (the form the CPU tests pin), and one profiled step of it
    py_res, py_total, py_fwd_ms = measure(RingAttention(GpuBackend()))
    prof = RingAttention(GpuBackend(), profile=True)
    for _ in range(2):                     # the second pass is the one kept: the first pays for this object's first allocations
        prof.timings.clear()
        o_, l_ = prof.forward(q, k, v, keep_state=True)
        prof.backward(q, k, v, o_, l_, do, use_saved_state=True)
    value = flops / (total * 1e-3) / 1e12
    check = ring_oracle_check(torch, w_local, rank, world, res["o"], res["lse"], *res["g"]) if rank in (0, world - 1) else None
    gathered = [None] * world
    dist.all_gather_object(gathered, check)
    kv_bytes = 2 * 2 * w.batch * w.kv_heads * (shard // 2) * w.head_dim * 2          # K and V, two chunks, bf16
    acc_bytes = 2 * 2 * w.batch * w.kv_heads * (shard // 2) * w.head_dim * 4         # dK and dV accumulators, fp32
    return {"workload": "longctx_ring", "S": S, "tokens_per_gpu": shard, "value": value, "unit": UNIT, "ms_per_step": total,
            "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "efficiency_vs_n_times_one_gpu": value / (world * per_gpu_value),
            "bytes_sent_per_gpu_per_step": {"forward": (world - 1) * kv_bytes, "backward": (world - 1) * kv_bytes + world * acc_bytes,
                                            "redistribution": "one of the two half-shards of Q,K,V,O,dO,LSE each way, once"},
            "driver": "sntl_ring_attn_fwd / sntl_ring_attn_bwd (C ABI, NCCL send/recv issued by the library)",
            "zigzag_layout": {"value": flops / (zz_total * 1e-3) / 1e12, "ms_per_step": zz_total, "fwd_ms": zz_fwd_ms,
                              "bwd_ms": zz_total - zz_fwd_ms,
                              "efficiency_vs_n_times_one_gpu": flops / (zz_total * 1e-3) / 1e12 / (world * per_gpu_value),
                              "note": "shards passed and returned in the zigzag order (SNTL_FLAG_RING_ZIGZAG): no redistribution round"},
            "python_schedule": {"value": flops / (py_total * 1e-3) / 1e12, "ms_per_step": py_total, "fwd_ms": py_fwd_ms,
                                "bwd_ms": py_total - py_fwd_ms, "compute_stream_breakdown_ms": prof.timings},
            "oracle": {"first_rank": gathered[0], "last_rank": gathered[world - 1],
                       "bound": "max abs <= 2e-2 and relative L2 <= 5e-3 against the fp64 oracle over the full sequence"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="gqa7b_d128")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override the workload's per-GPU batch (profiling captures)")
    ap.add_argument("--skip-e2e", action="store_true", help="skip the host-buffer leg (profiling captures)")
    ap.add_argument("--lean", action="store_true",
                    help="headline timing only: no sustained loop, other workloads, strong-scaling or ring legs (profiling captures)")
    ap.add_argument("--cached-tokens", type=int, default=0,
                    help="auxiliary mode: this many new tokens per sequence against a KV cache of the workload's length")
    ap.add_argument("--pack-heads", action="store_true",
                    help="auxiliary mode: the rotary + cast + relayout boundary kernels on the workload's Q tensor")
    ap.add_argument("--window", type=int, default=0, help="sliding window (keys per query); 0 = the workload's plain causal mask")
    ap.add_argument("--global-tokens", type=int, default=0, help="always-visible first keys (with --window)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    from sentinel_b200.workloads import WORKLOADS, make_inputs
    w = WORKLOADS[args.workload]
    if args.batch > 0:
        import dataclasses
        w = dataclasses.replace(w, batch=args.batch)
    if args.impl == "reference":
        run_reference_arm(args, w)
        return
    if args.cached_tokens > 0:
        run_cached_forward(args, w)
        return
    if args.pack_heads:
        run_pack_heads(args, w)
        return

    import torch
    import torch.distributed as dist
    import sentinel_b200 as sb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200 GPU: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        with stdout_to_stderr():
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier(device_ids=[local])       # the communicator exists (and has said so) before anything is printed
            torch.cuda.synchronize()
    sb._lib.load()
    barrier, timed = _make_timed(torch, dist, dev, world, local)

    ring = None
    if w.seq_shards > 1:
        # sequence-sharded workload: every rank holds seq/seq_shards tokens; with N ranks the sequence is N shards long
        # (the full 131072 tokens at N = 8) and K/V chunks travel round the ring over NCCL
        import dataclasses
        from sentinel_b200.ring import NativeRing
        shard = w.seq // w.seq_shards
        ring = NativeRing() if world > 1 else None
        w_local = dataclasses.replace(w, seq=shard, seq_shards=1)
        w = dataclasses.replace(w, seq=shard * world)
        q, k, v, do = (t.pin_memory() for t in make_inputs(w_local, seed_offset=rank))
    else:
        # per-rank batch: the workload's own batch; each rank draws its own shard (different seed offset)
        q, k, v, do = (t.pin_memory() for t in make_inputs(w, seed_offset=rank))
    qd, kd, vd, dod = (t.to(dev, non_blocking=True) for t in (q, k, v, do))
    o = torch.empty_like(qd)
    lse = torch.empty(qd.shape[:3], dtype=torch.float32, device=dev)
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    torch.cuda.synchronize()

    state = {}

    mask = dict(window=args.window, global_tokens=args.global_tokens) if args.window > 0 else {}
    if mask and ring is not None:
        raise SystemExit("--window applies to the unsharded workloads")

    def fwd():
        if ring is not None:
            state["o"], state["lse"] = ring.forward(qd, kd, vd, keep_state=True)
        else:
            sb.attention_forward(qd, kd, vd, out=o, lse=lse, **mask)

    def bwd():
        if ring is not None:
            ring.backward(qd, kd, vd, state["o"], state["lse"], dod, use_saved_state=True)
        else:
            sb.attention_backward(qd, kd, vd, o, lse, dod, dq=dq, dk=dk, dv=dv, **mask)

    def step():
        fwd()
        bwd()

    for _ in range(args.warmup):
        step()
    status = sb.poll_device_status()
    if status != 0:
        raise SystemExit(f"device-side wait timed out during warm-up (status word {status:#x})")

    launches0 = sb.launch_count()
    with ClockSampler(local) as clocks:
        total_ms = timed(step, args.steps)
        launches = sb.launch_count() - launches0
        if ring is not None:
            fwd_ms = timed(fwd, args.steps) / args.steps
            bwd_ms = total_ms / args.steps - fwd_ms       # the ring backward consumes the state its forward kept
        else:
            fwd_ms = timed(fwd, args.steps) / args.steps
            bwd_ms = timed(bwd, args.steps) / args.steps
    ms_per_step = total_ms / args.steps
    flops_rank = w.flops / world if ring is not None else w.flops     # the ring workload's FLOPs are for the whole sequence
    if mask:
        # 7 GEMM-shaped products of 2*D flops per visible (query, key) pair; the plain causal figure is the same rule
        # with S*S/2 pairs
        import numpy as np
        qi = np.arange(w.seq, dtype=np.int64)
        pairs = np.minimum(qi + 1, args.window) + np.clip(np.minimum(args.global_tokens, qi - args.window + 1), 0, None)
        flops_rank = 14.0 * w.head_dim * w.batch * w.q_heads * float(pairs.sum())
    value = flops_rank * world / (ms_per_step * 1e-3) / 1e12
    peaks = load_peaks()
    burst = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    sustained_peak = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
    clock_summary = clocks.summary()

    # the same loop for at least two seconds: what the 1000 W cap leaves of the burst figure
    sustained = None
    if not args.lean and ring is None:
        n_sus = max(args.steps, int(2200.0 / ms_per_step) + 1)
        with ClockSampler(local) as sus_clocks:
            sus_ms = timed(step, n_sus) / n_sus
        sc = sus_clocks.summary()
        sus_tf = flops_rank / (sus_ms * 1e-3) / 1e12
        sustained = {"value": sus_tf * world, "unit": UNIT, "per_gpu": sus_tf, "steps": n_sus, "seconds": sus_ms * n_sus * 1e-3,
                     "ms_per_step": sus_ms, "sm_mhz_median": sc["sm_mhz"], "reasons": sc["reasons"],
                     "mcycles_per_step": (sus_ms * 1e-3 * sc["sm_mhz"]) if sc["sm_mhz"] else None,
                     "frac_of_sustained_peak": sus_tf / sustained_peak, "frac_of_burst_peak": sus_tf / burst}

    # end to end through the host-buffer call: H2D of Q,K,V,dO, forward+backward, D2H of O,LSE,dQ,dK,dV
    def e2e_step():
        if ring is not None:
            sh = [t.to(dev, non_blocking=True) for t in (q, k, v, do)]
            o_, lse_ = ring.forward(sh[0], sh[1], sh[2], keep_state=True)
            grads = ring.backward(sh[0], sh[1], sh[2], o_, lse_, sh[3], use_saved_state=True)
            outs = [t.to("cpu", non_blocking=True) for t in (o_, lse_) + tuple(grads)]
            torch.cuda.current_stream().synchronize()
        else:
            sb.attention_forward_backward_host(q, k, v, do, device=dev, **mask)

    copy_ms = None
    if args.skip_e2e:
        e2e_ms = float("nan")
    else:
        for _ in range(2):
            e2e_step()
        e2e_steps = max(3, min(args.steps, 10))
        e2e_ms = timed(e2e_step, e2e_steps) / e2e_steps
        if not args.lean:
            copy_ms = copy_bound(torch, dist, dev, world, [q, k, v, do], [q, lse.cpu(), q, k, v], timed)
    esz = q.element_size()
    h2d = esz * (2 * q.numel() + 2 * k.numel())
    d2h = esz * (2 * q.numel() + 2 * k.numel()) + 4 * lse.numel()
    e2e_value = None if args.skip_e2e else flops_rank * world / (e2e_ms * 1e-3) / 1e12
    status = sb.poll_device_status()

    # roofline of the dominant call.  The denominator follows the length of the timed region: a kernel timed in a
    # burst (< 1 s) is read against the burst cuBLAS figure, one timed inside a seconds-long loop against the sustained one
    region_s = total_ms * 1e-3
    use_burst = region_s < 1.0
    peak = burst if use_burst else sustained_peak
    bwd_flops = flops_rank * 5.0 / 7.0
    achieved = bwd_flops / (bwd_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "attention backward (delta pass + dK/dV/dQ kernel + dQ convert, timed as one call)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": f"{peaks['_source']} {'bf16_tflops (burst)' if use_burst else 'bf16_tflops_sustained'}: the timed region of "
                               f"{args.steps} steps lasted {region_s:.3f} s at a median {clock_summary['sm_mhz']} MHz",
                "frac_of_burst_peak": achieved / burst, "frac_of_sustained_peak": achieved / sustained_peak,
                "traffic": (NCU_DRAM_BYTES_PER_BATCH[w.name] * w.batch
                            if w.name in NCU_DRAM_BYTES_PER_BATCH and ring is None and not mask else None),
                "fwd": {"achieved": flops_rank * 2.0 / 7.0 / (fwd_ms * 1e-3) / 1e12, "ms": fwd_ms,
                        "frac_of_burst_peak": flops_rank * 2.0 / 7.0 / (fwd_ms * 1e-3) / 1e12 / burst},
                "bwd_ms": bwd_ms,
                "fwd_bwd_frac_of_burst_peak": flops_rank / (ms_per_step * 1e-3) / 1e12 / burst}

    def make_line(extras, status_now):
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16" if w.dtype == "bf16" else "f32", "data": "synthetic",
                "config": {"workload": w.name, "B_per_gpu": w.batch, "global_batch": (w.batch if ring is not None else w.batch * world), "Hq": w.q_heads,
                           "Hkv": w.kv_heads, "S": w.seq, "D": w.head_dim, "causal": True,
                           "parallelism": (f"sequence split into {world} contiguous shards, zigzag-balanced ring of K/V chunks over NCCL"
                                           if ring is not None else f"batch x KV-group sharding over {world} GPU(s), no communication"),
                           "l2": "per-step working set (Q,K,V,O,dO,dQ,dK,dV,dQ-accumulator) > 0.8 GB, larger than the 126 MB L2",
                           "kernel_path": "tcgen05" if w.dtype == "bf16" else "simt_f32",
                           **({"window": args.window, "global_tokens": args.global_tokens,
                               "flop_rule": "14*D per visible (query, key) pair"} if mask else {})},
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": None if args.skip_e2e else e2e_ms,
                        "copy_bound_ms": copy_ms,
                        "frac_of_copy_bound": (copy_ms / e2e_ms) if (copy_ms and not args.skip_e2e) else None,
                        "copy_bound": "the same bytes as plain pinned copies, both directions at once, all ranks at once, no kernels"},
                "gpu_launches": int(launches), "clocks": clock_summary, "roofline": roofline,
                "device_status": status_now}
        if sustained is not None:
            line["sustained"] = sustained
        line.update(extras)
        return line

    # The extra legs (other workloads; strong scaling and the ring at N > 1) come after every number of the headline
    # line is in hand.  Should one of them stall -- a peer that died, an NCCL set-up problem on the box -- a watchdog
    # prints the headline line without it and ends the process, so that the main measurement is never lost to them.
    extras = {}
    done = threading.Event()

    def watchdog():
        if done.wait(EXTRA_LEGS_LIMIT_S):
            return
        if rank == 0:
            late = dict(extras)
            late["extra_legs"] = {"unavailable": f"not finished within {EXTRA_LEGS_LIMIT_S} s; the headline figures above are complete"}
            print(json.dumps(make_line(late, status)), flush=True)
        os._exit(0)

    threading.Thread(target=watchdog, daemon=True).start()
    plain_headline = ring is None and not mask and args.batch == 0 and not args.lean
    if plain_headline and world == 1:
        extras["other_workloads"] = [run_other_workload(torch, sb, n, dev, peaks) for n in ("llama1b_gqa", "gpt2_small")]
    if plain_headline and world > 1:
        try:
            extras["strong"] = run_strong_scaling(torch, dist, sb, w, dev, rank, world, timed, args.steps, ms_per_step)
        except Exception as exc:
            extras["strong"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
        try:
            extras["ring"] = run_ring(torch, dist, sb, dev, rank, world, timed, max(3, min(args.steps, 5)), value / world)
        except Exception as exc:
            extras["ring"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
    status = status or sb.poll_device_status()
    done.set()

    if rank == 0:
        line = make_line(extras, status)
        if not args.no_cpu_baseline and world == 1:
            try:
                r = cpu_reference_sample(w)
                line["cpu_baseline"] = {kk: r[kk] for kk in ("value", "unit", "cores", "kind", "sample")}
            except Exception as exc:  # the checker is optional for the bench line, never for the product path
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"unavailable: {exc}"}
        if world == 1 and ring is None and not args.no_cpu_baseline:
            try:
                line["reference_cuda"] = reference_cuda_sample(w, q, k, v, do)
            except Exception as exc:
                line["reference_cuda"] = {"unavailable": str(exc)}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
