"""Forward + backward on HOST tensors with the transfers overlapped with the kernels.

A caller that keeps its activations in host memory pays for 538 MB of PCIe traffic per step of the headline workload,
several times the kernels' own time.  This module hides as much of it as the dependencies allow:

* an upload stream, a download stream (the two PCIe directions run concurrently) and two compute streams;
* the problem is cut into chunks of whole (batch element, KV group) units -- every chunk is a complete attention
  problem, contiguous in memory, so nothing is exchanged between chunks -- and chunk c+1 uploads while chunk c computes
  and chunk c-1 downloads;
* chunks alternate between the two compute streams: a chunk's backward ends with a few long-running CTAs (the first
  key tiles visit every query tile), and the next chunk's kernels fill the SMs those leave idle;
* inside a chunk the forward starts as soon as Q, K, V are on the device (dO follows during the forward), O and LSE
  go back while the backward runs, and the gradients go back while the next chunk computes -- on a download stream
  of their own, so that the next chunk's O does not queue behind this chunk's backward.

Device staging buffers, streams and events are cached per shape, so steady-state calls allocate and create nothing.
Host tensors should be pinned (``tensor.pin_memory()``); pageable memory works but makes the copies synchronous.
"""
from __future__ import annotations

import torch

from . import flash_attention as fa

_cache: dict = {}


def _buffers(q, k, dev):
    key = (tuple(q.shape), tuple(k.shape), q.dtype, dev.index)
    buf = _cache.get(key)
    if buf is None:
        mk = lambda like: torch.empty(like.shape, dtype=like.dtype, device=dev)
        buf = {
            "q": mk(q), "k": mk(k), "v": mk(k), "do": mk(q), "o": mk(q), "dq": mk(q), "dk": mk(k), "dv": mk(k),
            "lse": torch.empty(q.shape[:3], dtype=torch.float32, device=dev),
            "h_o": torch.empty(q.shape, dtype=q.dtype).pin_memory(), "h_dq": torch.empty(q.shape, dtype=q.dtype).pin_memory(),
            "h_dk": torch.empty(k.shape, dtype=k.dtype).pin_memory(), "h_dv": torch.empty(k.shape, dtype=k.dtype).pin_memory(),
            "h_lse": torch.empty(q.shape[:3], dtype=torch.float32).pin_memory(),
            "up": torch.cuda.Stream(device=dev), "down": torch.cuda.Stream(device=dev),
            "down_grads": torch.cuda.Stream(device=dev),
            "compute": [torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)],
            "events": {},       # chunk index -> (qkv uploaded, dO uploaded, forward done, backward done), reused every call
        }
        _cache.clear()          # one shape at a time: the staging buffers are as large as the problem
        _cache[key] = buf
    return buf


def _chunk_slices(B, Hq, Hkv, chunks):
    """Cuts the B x Hkv independent (batch element, KV group) units into chunks that are contiguous in memory:
    a chunk is a run of KV groups inside one batch element (with the query heads of those groups), or -- when there
    are fewer chunks than batch elements -- a run of whole batch elements."""
    g = Hq // Hkv
    if chunks is None:
        # Eight equal chunks measured best on the headline shape (7.3 ms against 7.4 with four and 7.7-8.2 with unequal
        # plans): both PCIe directions stay busy, and the backward cuts its long key tiles by query head when a chunk
        # is small, so small chunks cost little.
        chunks = min(B * Hkv, 8)
    chunks = max(1, min(chunks, B * Hkv))
    if chunks <= B:
        return [(slice(c * B // chunks, (c + 1) * B // chunks), slice(0, Hq), slice(0, Hkv)) for c in range(chunks)]
    per_b = max(1, min(Hkv, -(-chunks // B)))
    out = []
    for b in range(B):
        for c in range(per_b):
            k0, k1 = c * Hkv // per_b, (c + 1) * Hkv // per_b
            out.append((slice(b, b + 1), slice(k0 * g, k1 * g), slice(k0, k1)))
    return out


def forward_backward_host(q, k, v, dout, *, causal=True, scale=None, flags=0, device="cuda", chunks=None, window=0,
                          global_tokens=0, out=None):
    """Returns host tensors (O, LSE, dQ, dK, dV).  ``chunks`` = number of pipeline chunks (default: up to 8, cut along
    batch elements first and KV groups second; every chunk is a complete attention problem).

    Without ``out`` the five returned tensors are this module's cached pinned staging buffers: they stay valid only
    until the next call (which overwrites them, or drops them when the shape changes) -- copy what must be kept.
    ``out`` = (O, LSE, dQ, dK, dV) host tensors of the caller (pinned for asynchronous copies) receives the results
    instead and is returned.  Raises if a device-side wait timed out during the call."""
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    B, Hq, Hkv = q.shape[0], q.shape[1], k.shape[1]
    buf = _buffers(q, k, dev)
    if out is None:
        h_o, h_lse, h_dq, h_dk, h_dv = (buf[n] for n in ("h_o", "h_lse", "h_dq", "h_dk", "h_dv"))
    else:
        h_o, h_lse, h_dq, h_dk, h_dv = out
        for t, like in ((h_o, buf["h_o"]), (h_lse, buf["h_lse"]), (h_dq, buf["h_dq"]), (h_dk, buf["h_dk"]), (h_dv, buf["h_dv"])):
            if t.shape != like.shape or t.dtype != like.dtype or t.is_cuda:
                raise ValueError("out must be host tensors shaped (O, LSE, dQ, dK, dV)")
    caller = torch.cuda.current_stream(dev)
    up, down, down_g, lanes = buf["up"], buf["down"], buf["down_grads"], buf["compute"]
    for st in (up, down, down_g, *lanes):
        st.wait_stream(caller)      # earlier users of the staging buffers are done
    for c, (sb, sq, sk) in enumerate(_chunk_slices(B, Hq, Hkv, chunks)):
        qs, ks = (sb, sq), (sb, sk)
        comp = lanes[c % len(lanes)]
        evs = buf["events"].get(c)
        if evs is None:
            evs = buf["events"][c] = tuple(torch.cuda.Event() for _ in range(4))
        ev_qkv, ev_do, ev_fwd, ev_bwd = evs
        with torch.cuda.stream(up):
            buf["q"][qs].copy_(q[qs], non_blocking=True)
            buf["k"][ks].copy_(k[ks], non_blocking=True)
            buf["v"][ks].copy_(v[ks], non_blocking=True)
            ev_qkv.record(up)
            buf["do"][qs].copy_(dout[qs], non_blocking=True)
            ev_do.record(up)
        with torch.cuda.stream(comp):
            comp.wait_event(ev_qkv)
            fa.attention_forward(buf["q"][qs], buf["k"][ks], buf["v"][ks], causal=causal, scale=scale, flags=flags,
                                 out=buf["o"][qs], lse=buf["lse"][qs], window=window, global_tokens=global_tokens)
            ev_fwd.record(comp)
        with torch.cuda.stream(down):
            down.wait_event(ev_fwd)
            h_o[qs].copy_(buf["o"][qs], non_blocking=True)
            h_lse[qs].copy_(buf["lse"][qs], non_blocking=True)
        with torch.cuda.stream(comp):
            comp.wait_event(ev_do)
            fa.attention_backward(buf["q"][qs], buf["k"][ks], buf["v"][ks], buf["o"][qs], buf["lse"][qs], buf["do"][qs],
                                  causal=causal, scale=scale, flags=flags, dq=buf["dq"][qs], dk=buf["dk"][ks],
                                  dv=buf["dv"][ks], window=window, global_tokens=global_tokens)
            ev_bwd.record(comp)
        with torch.cuda.stream(down_g):    # a stream of their own: O of the next chunk must not queue behind this backward
            down_g.wait_event(ev_bwd)
            h_dq[qs].copy_(buf["dq"][qs], non_blocking=True)
            h_dk[ks].copy_(buf["dk"][ks], non_blocking=True)
            h_dv[ks].copy_(buf["dv"][ks], non_blocking=True)
    for st in (up, down, down_g, *lanes):
        caller.wait_stream(st)     # a timed region (events on the caller's stream) ends after the last download
    with torch.cuda.device(dev):
        fa.raise_if_device_wait_timed_out()     # synchronises the caller's stream: the call's one synchronisation point
    return h_o, h_lse, h_dq, h_dk, h_dv
