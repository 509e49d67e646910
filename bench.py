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
NCU_DRAM_BYTES_PER_BATCH = {"gqa7b_d128": (1870.9e6 + 988.1e6) / 2}
# the same for the cache-mode forward kernel, one new token, no window (profiles/attn_fwd_tc_kernel_cache_mode_gqa7b_d128.md,
# captured at batch 16)
NCU_CACHED_DRAM_BYTES_PER_BATCH = {"gqa7b_d128": (268640768 + 5306880) / 16.0}


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


def cpu_reference_sample(workload, steps: int, warmup: int):
    """Times the reference's own CPU attention (attention core only) on ONE query head of ONE sequence at a reduced
    length; the causal FLOP formula is applied to the sample so the unit matches the GPU metric."""
    import numpy as np
    from oracle import cpu
    if not cpu.ref_available():
        cpu.build()
    kind = "reference" if cpu.ref_available() else "port"
    S = min(workload.seq, 2048)
    D = workload.head_dim
    rng = np.random.default_rng(20261125)
    q = (rng.standard_normal((1, 1, S, D)) * workload.qk_std).astype(np.float32)
    k = (rng.standard_normal((1, 1, S, D)) * workload.qk_std).astype(np.float32)
    v = (rng.standard_normal((1, 1, S, D)) * workload.v_std).astype(np.float32)
    do = (rng.standard_normal((1, 1, S, D)) * workload.do_std).astype(np.float32)
    flops = 7.0 * S * S * D
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        if kind == "reference":
            _, _, _, _, secs = cpu.ref_core_fwd_bwd(q, k, v, do, want_outputs=False)
            dt = secs[0] + secs[1]
        else:
            cpu.attn_fwd(q, k, v)
            cpu.attn_bwd(q, k, v, do)
            dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    mean = sum(times) / len(times)
    cores = cpu.ref_threads() if kind == "reference" else cpu.oracle_threads()
    return {"value": flops / mean / 1e12, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"1 sequence x 1 query head, S={S}, D={D}, fp32, attention core only (dense S^2 work), "
                      f"{len(times)} timed passes of {mean:.3f} s", "ms_per_step": mean * 1e3}


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
    res = cpu_reference_sample(workload, max(1, args.steps), max(1, min(args.warmup, 2)))
    line = {"impl": "reference", "metric": METRIC, "value": res["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload.name, "B": workload.batch, "Hq": workload.q_heads, "Hkv": workload.kv_heads,
                       "S": workload.seq, "D": workload.head_dim, "causal": True},
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
    ap.add_argument("--cached-tokens", type=int, default=0,
                    help="auxiliary mode: this many new tokens per sequence against a KV cache of the workload's length")
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
        dist.init_process_group("nccl", device_id=dev)
    sb._lib.load()

    ring = None
    if w.seq_shards > 1:
        # sequence-sharded workload: every rank holds seq/seq_shards tokens; with N ranks the sequence is N shards long
        # (the full 131072 tokens at N = 8) and K/V chunks travel round the ring over NCCL
        import dataclasses
        from sentinel_b200.ring import GpuBackend, RingAttention
        shard = w.seq // w.seq_shards
        ring = RingAttention(GpuBackend()) if world > 1 else None
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
            state["o"], state["lse"] = ring.forward(qd, kd, vd)
        else:
            sb.attention_forward(qd, kd, vd, out=o, lse=lse, **mask)

    def bwd():
        if ring is not None:
            ring.backward(qd, kd, vd, state["o"], state["lse"], dod)
        else:
            sb.attention_backward(qd, kd, vd, o, lse, dod, dq=dq, dk=dk, dv=dv, **mask)

    def step():
        fwd()
        bwd()

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

    for _ in range(args.warmup):
        step()
    status = sb.poll_device_status()
    if status != 0:
        raise SystemExit(f"device-side wait timed out during warm-up (status word {status:#x})")

    launches0 = sb.launch_count()
    with ClockSampler(local) as clocks:
        total_ms = timed(step, args.steps)
        launches = sb.launch_count() - launches0
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

    # end to end through the host-buffer call: H2D of Q,K,V,dO, forward+backward, D2H of O,LSE,dQ,dK,dV
    def e2e_step():
        if ring is not None:
            sh = [t.to(dev, non_blocking=True) for t in (q, k, v, do)]
            o_, lse_ = ring.forward(sh[0], sh[1], sh[2])
            grads = ring.backward(sh[0], sh[1], sh[2], o_, lse_, sh[3])
            outs = [t.to("cpu", non_blocking=True) for t in (o_, lse_) + tuple(grads)]
            torch.cuda.current_stream().synchronize()
        else:
            sb.attention_forward_backward_host(q, k, v, do, device=dev, **mask)

    if args.skip_e2e:
        e2e_ms = float("nan")
    else:
        for _ in range(2):
            e2e_step()
        e2e_steps = max(3, min(args.steps, 10))
        e2e_ms = timed(e2e_step, e2e_steps) / e2e_steps
    esz = q.element_size()
    h2d = esz * (2 * q.numel() + 2 * k.numel())
    d2h = esz * (2 * q.numel() + 2 * k.numel()) + 4 * lse.numel()
    e2e_value = None if args.skip_e2e else flops_rank * world / (e2e_ms * 1e-3) / 1e12
    status = sb.poll_device_status()

    peaks = load_peaks()
    peak = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
    bwd_flops = flops_rank * 5.0 / 7.0
    achieved = bwd_flops / (bwd_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "attention backward (delta pass + dK/dV/dQ kernel + dQ convert, timed as one call)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": f"{peaks['_source']} bf16_tflops_sustained (kernel timed inside a seconds-long loop)",
                "traffic": (NCU_DRAM_BYTES_PER_BATCH[w.name] * w.batch
                            if w.name in NCU_DRAM_BYTES_PER_BATCH and ring is None and not mask else None),
                "fwd": {"achieved": flops_rank * 2.0 / 7.0 / (fwd_ms * 1e-3) / 1e12, "ms": fwd_ms},
                "bwd_ms": bwd_ms,
                "fwd_bwd_frac_of_burst_peak": flops_rank / (ms_per_step * 1e-3) / 1e12 / float(peaks.get("bf16_tflops", 1590.0))}

    if rank == 0:
        cpu_base = None
        if world == 1 and not args.no_cpu_baseline:
            try:
                r = cpu_reference_sample(w, 3, 1)
                cpu_base = {kk: r[kk] for kk in ("value", "unit", "cores", "kind", "sample")}
            except Exception as exc:  # the checker is optional for the bench line, never for the product path
                cpu_base = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": f"unavailable: {exc}"}
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16" if w.dtype == "bf16" else "f32", "data": "synthetic",
                "config": {"workload": w.name, "B_per_gpu": w.batch, "global_batch": (w.batch if ring is not None else w.batch * world), "Hq": w.q_heads,
                           "Hkv": w.kv_heads, "S": w.seq, "D": w.head_dim, "causal": True,
                           "parallelism": (f"sequence split into {world} contiguous shards, zigzag-balanced ring of K/V chunks over NCCL"
                                           if ring is not None else f"batch x KV-group sharding over {world} GPU(s), no communication"),
                           "l2": "per-step working set (Q,K,V,O,dO,dQ,dK,dV,dQ-accumulator) > 0.8 GB, larger than the 126 MB L2",
                           "kernel_path": sb.last_path(),
                           **({"window": args.window, "global_tokens": args.global_tokens,
                               "flop_rule": "14*D per visible (query, key) pair"} if mask else {})},
                "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "ms_per_step": None if args.skip_e2e else e2e_ms},
                "gpu_launches": int(launches), "clocks": clocks.summary(), "roofline": roofline,
                "device_status": status}
        if cpu_base is not None:
            line["cpu_baseline"] = cpu_base
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
