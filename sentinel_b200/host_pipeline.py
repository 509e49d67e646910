"""Forward + backward on HOST tensors with the transfers overlapped with the kernels.

A caller that keeps its activations in host memory pays for 538 MB of PCIe traffic per step of the headline workload,
several times the kernels' own time.  This module hides as much of it as the dependencies allow:

* three streams: upload, compute, download (the two PCIe directions run concurrently);
* the batch is cut into chunks of whole (batch element) units -- every chunk is a complete attention problem, so
  nothing is exchanged between chunks -- and chunk c+1 uploads while chunk c computes and chunk c-1 downloads;
* inside a chunk the forward starts as soon as Q, K, V are on the device (dO follows during the forward), O and LSE
  go back while the backward runs, and the gradients go back while the next chunk computes.

Device staging buffers are cached per shape, so steady-state calls allocate nothing.  Host tensors should be pinned
(``tensor.pin_memory()``); pageable memory works but makes the copies synchronous.
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
        }
        _cache.clear()          # one shape at a time: the staging buffers are as large as the problem
        _cache[key] = buf
    return buf


def forward_backward_host(q, k, v, dout, *, causal=True, scale=None, flags=0, device="cuda", chunks=None):
    """Returns host tensors (O, LSE, dQ, dK, dV).  ``chunks`` = number of batch chunks (default: one per batch element,
    at most 4)."""
    dev = torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    B = q.shape[0]
    n_chunks = max(1, min(B, 4) if chunks is None else min(chunks, B))
    bounds = [(c * B // n_chunks, (c + 1) * B // n_chunks) for c in range(n_chunks)]
    buf = _buffers(q, k, dev)
    comp = torch.cuda.current_stream(dev)
    up, down = buf["up"], buf["down"]
    up.wait_stream(comp)      # earlier users of the staging buffers are done
    down.wait_stream(comp)
    done = []
    for lo, hi in bounds:
        sl = slice(lo, hi)
        with torch.cuda.stream(up):
            for name, src in (("q", q), ("k", k), ("v", v)):
                buf[name][sl].copy_(src[sl], non_blocking=True)
            ev_qkv = torch.cuda.Event()
            ev_qkv.record(up)
            buf["do"][sl].copy_(dout[sl], non_blocking=True)
            ev_do = torch.cuda.Event()
            ev_do.record(up)
        comp.wait_event(ev_qkv)
        fa.attention_forward(buf["q"][sl], buf["k"][sl], buf["v"][sl], causal=causal, scale=scale, flags=flags,
                             out=buf["o"][sl], lse=buf["lse"][sl])
        ev_fwd = torch.cuda.Event()
        ev_fwd.record(comp)
        with torch.cuda.stream(down):
            down.wait_event(ev_fwd)
            buf["h_o"][sl].copy_(buf["o"][sl], non_blocking=True)
            buf["h_lse"][sl].copy_(buf["lse"][sl], non_blocking=True)
        comp.wait_event(ev_do)
        fa.attention_backward(buf["q"][sl], buf["k"][sl], buf["v"][sl], buf["o"][sl], buf["lse"][sl], buf["do"][sl], causal=causal,
                              scale=scale, flags=flags, dq=buf["dq"][sl], dk=buf["dk"][sl], dv=buf["dv"][sl])
        ev_bwd = torch.cuda.Event()
        ev_bwd.record(comp)
        with torch.cuda.stream(down):
            down.wait_event(ev_bwd)
            buf["h_dq"][sl].copy_(buf["dq"][sl], non_blocking=True)
            buf["h_dk"][sl].copy_(buf["dk"][sl], non_blocking=True)
            buf["h_dv"][sl].copy_(buf["dv"][sl], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(down)
            done.append(ev)
    comp.wait_stream(down)     # the timed region (events on the compute stream) ends after the last download
    comp.synchronize()
    return buf["h_o"], buf["h_lse"], buf["h_dq"], buf["h_dk"], buf["h_dv"]
