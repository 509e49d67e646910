"""Sequence-sharded causal attention over a ring of ranks (the 131072-token workload).

The reference has no sequence-parallel path; this is the multi-GPU schedule built on the single-GPU kernels.

Layout at the interface: the sequence is split into ``W`` equal contiguous shards, rank ``r`` holds tokens
``[r*S/W, (r+1)*S/W)`` of Q, K, V (and O, dO, dQ, dK, dV), each ``[B, H, S/W, D]``.

Schedule
--------
A plain ring over contiguous shards is badly unbalanced under a causal mask (rank r has r+0.5 blocks of work).
So each shard is cut in two half-shards ("chunks", ``2W`` in total) and the chunks are first re-dealt in a zigzag:
rank ``r`` works on chunks ``r`` and ``2W-1-r``.  Then for ``W`` steps the key/value chunks travel round the ring
(rank r sends to r+1).  In every step every rank has exactly two block units of visible (query chunk, key chunk)
pairs -- a pair is visible iff ``key_chunk <= query_chunk``, causal inside iff equal -- so all ranks finish each step
together.

Forward: each visible pair is one call of the attention forward (non-causal, or causal on the diagonal) whose
(O, LSE) partial is folded into fp32 running results with the log-sum-exp merge.

Backward: the work that belongs to a query chunk alone (delta, the rescaled FINAL log-sum-exp, zeroing and converting
its fp32 dQ accumulator) runs once per chunk; each visible pair is then one launch of the tensor-core kernel that adds
its dQ into that accumulator and its dK, dV into a per-pair fp32 partial.  dK/dV of a key chunk are summed in fp32
accumulators that travel with the chunk: after a step's pairs the rank adds its partials to the accumulators that
arrived from the previous rank and passes them on; that hop runs under the NEXT step's kernels (three buffer sets
rotate: being sent, being received, being computed), as does the hop of K/V themselves, so in steady state no
transfer is exposed.  After ``W`` steps one last hop brings the accumulators home.  Results are dealt back to the
contiguous layout at the end.

Communication is ``torch.distributed`` point-to-point (NCCL send/recv over NVLink on GPUs; gloo in the CPU tests).
Every wait on a transfer has a deadline (``timeout_s``): a peer that left, stalled, or posted a different schedule
makes ``RingAttention`` raise ``RingTimeout`` instead of waiting for ever.

The arithmetic is supplied by a *backend* (``GpuBackend`` = this library's kernels).  The schedule itself touches
no tensor values, which is what lets the CPU tests drive it with a reference backend.
"""
from __future__ import annotations

import time
from datetime import timedelta

import torch
import torch.distributed as dist


class RingTimeout(RuntimeError):
    """A point-to-point transfer of the ring did not complete within the deadline."""


def chunk_owner_contiguous(chunk: int) -> int:
    return chunk // 2


def chunk_owner_zigzag(chunk: int, world: int) -> int:
    return chunk if chunk < world else 2 * world - 1 - chunk


def zigzag_chunks(rank: int, world: int):
    """The two chunk ids rank ``rank`` works on, low one first."""
    return (rank, 2 * world - 1 - rank)


def zigzag_shard(x_full, rank: int, world: int):
    """Rank ``rank``'s shard of a whole-sequence tensor ``[B, H, S, ...]`` in the zigzag layout: chunk ``rank`` followed by
    chunk ``2*world-1-rank`` of the ``2*world`` equal chunks of the sequence (what ``zigzag_layout=True`` expects)."""
    chunks = x_full.chunk(2 * world, dim=2)
    a, b = zigzag_chunks(rank, world)
    return torch.cat([chunks[a], chunks[b]], dim=2).contiguous()


def visible_pairs(q_chunks, kv_chunks):
    """[(qi, ki, causal)] over local slot indices for the pairs the causal mask lets through."""
    out = []
    for qi, qc in enumerate(q_chunks):
        for ki, kc in enumerate(kv_chunks):
            if kc < qc:
                out.append((qi, ki, False))
            elif kc == qc:
                out.append((qi, ki, True))
    return out


class GpuBackend:
    """The library's kernels on CUDA tensors."""

    def __init__(self):
        from . import flash_attention as fa
        self.fa = fa

    def fwd(self, q, k, v, causal):
        return self.fa.attention_forward(q, k, v, causal=causal)

    def merge(self, o_acc, lse_acc, o_part, lse_part):
        self.fa.merge_partials(o_acc, lse_acc, o_part, lse_part)

    def bwd_begin(self, q, o, lse, do):
        return self.fa.BackwardPieces(q, o, lse, do)

    def bwd_block(self, handle, k, v, dk_acc, dv_acc, causal):
        handle.block(k, v, dk_acc, dv_acc, causal=causal)

    def bwd_end(self, handle):
        return handle.end()

    def accumulate(self, acc, part):
        self.fa.accumulate(acc, part)

    def zeros_f32(self, like):
        return torch.zeros(like.shape, dtype=torch.float32, device=like.device)

    def neg_inf(self, shape, like):
        return torch.full(shape, float("-inf"), dtype=torch.float32, device=like.device)

    def check(self):
        self.fa.raise_if_device_wait_timed_out()


class RingAttention:
    def __init__(self, backend, group=None, timeout_s: float = 60.0, profile: bool = False, zigzag_layout: bool = False):
        """``zigzag_layout``: every shard passed in (and returned) is already the rank's two zigzag chunks, first half of
        the shard = chunk ``rank``, second half = chunk ``2W-1-rank`` (see ``zigzag_shard``); nothing is redistributed."""
        self.zigzag_layout = zigzag_layout
        self.backend = backend
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.timeout_s = timeout_s
        self.profile = profile and torch.cuda.is_available()
        self.timings: dict = {}
        self._saved = None
        self._side = None        # second compute stream: the two pairs of a step run side by side

    # ------------------------------------------------------------------ transfers
    def _finish(self, works, what):
        """Wait for posted transfers, with a deadline.  With NCCL ``wait()`` only makes the current stream wait (a dead
        peer surfaces through the process group's own timeout); with a host-side backend (gloo) the wait itself takes
        the deadline and its expiry is re-raised as ``RingTimeout``."""
        if not works:
            return
        if torch.cuda.is_available() and dist.get_backend(self.group) == "nccl":
            for w in works:
                w.wait()
            return
        deadline = time.monotonic() + self.timeout_s
        for w in works:
            left = max(deadline - time.monotonic(), 0.001)
            try:
                w.wait(timedelta(seconds=left))
            except RuntimeError as e:
                if "imed out" in str(e) or "imeout" in str(e):
                    raise RingTimeout(f"rank {self.rank}: {what} did not complete within {self.timeout_s} s "
                                      "(a peer left, stalled, or posted a different schedule)") from e
                raise

    def _exchange(self, sends, recvs, what="redistribution"):
        """sends: [(tensor, dst)], recvs: [(tensor, src)]; one batched point-to-point round."""
        ops = [dist.P2POp(dist.isend, t, dst, self.group) for t, dst in sends]
        ops += [dist.P2POp(dist.irecv, t, src, self.group) for t, src in recvs]
        if ops:
            self._finish(dist.batch_isend_irecv(ops), what)

    def to_zigzag_many(self, xs):
        """Contiguous shards [B,H,S_local,...] -> for each, the list of the two chunks this rank works on (zigzag deal).
        All tensors travel in one batched round."""
        r, W = self.rank, self.world
        if self.zigzag_layout:
            return [[x[:, :, :x.shape[2] // 2].contiguous(), x[:, :, x.shape[2] // 2:].contiguous()] for x in xs]
        want = zigzag_chunks(r, W)
        outs, sends, recvs = [], [], []
        for x in xs:
            half = x.shape[2] // 2
            mine = {2 * r: x[:, :, :half].contiguous(), 2 * r + 1: x[:, :, half:].contiguous()}
            out = {c: (mine[c] if c in mine else torch.empty_like(mine[2 * r])) for c in want}
            sends += [(t, chunk_owner_zigzag(c, W)) for c, t in sorted(mine.items()) if chunk_owner_zigzag(c, W) != r]
            recvs += [(out[c], chunk_owner_contiguous(c)) for c in want if chunk_owner_contiguous(c) != r]
            outs.append([out[c] for c in want])
        self._exchange(sends, recvs, "zigzag deal")
        return outs

    def to_zigzag(self, x):
        return self.to_zigzag_many([x])[0]

    def from_zigzag_many(self, chunk_lists):
        """Inverse of ``to_zigzag_many``: per tensor, the two zigzag chunks -> this rank's contiguous shard."""
        r, W = self.rank, self.world
        if self.zigzag_layout:
            return [torch.cat(list(chunks), dim=2) for chunks in chunk_lists]
        want = (2 * r, 2 * r + 1)
        outs, sends, recvs = [], [], []
        for chunks in chunk_lists:
            have = dict(zip(zigzag_chunks(r, W), chunks))
            out = {c: (have[c] if c in have else torch.empty_like(chunks[0])) for c in want}
            sends += [(t.contiguous(), chunk_owner_contiguous(c)) for c, t in sorted(have.items()) if chunk_owner_contiguous(c) != r]
            recvs += [(out[c], chunk_owner_zigzag(c, W)) for c in want if chunk_owner_zigzag(c, W) != r]
            outs.append(out)
        self._exchange(sends, recvs, "deal back")
        return [torch.cat([out[want[0]], out[want[1]]], dim=2) for out in outs]

    def from_zigzag(self, chunks):
        return self.from_zigzag_many([chunks])[0]

    def _rotate_start(self, tensors, buffers):
        """Post the ring shift of ``tensors`` (to rank+1) into ``buffers`` (from rank-1); returns work handles."""
        if self.world == 1:
            return None
        nxt, prv = (self.rank + 1) % self.world, (self.rank - 1) % self.world
        ops = [dist.P2POp(dist.isend, t, nxt, self.group) for t in tensors]
        ops += [dist.P2POp(dist.irecv, b, prv, self.group) for b in buffers]
        return dist.batch_isend_irecv(ops)

    # ------------------------------------------------------------------ two compute lanes
    def _lanes(self, like):
        """(main stream, side stream) on CUDA, (None, None) on CPU."""
        if not like.is_cuda:
            return None, None
        if self._side is None:
            self._side = torch.cuda.Stream(device=like.device)
        return torch.cuda.current_stream(like.device), self._side

    def _mark(self, name):
        if self.profile:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.timings.setdefault("_events", []).append((name, e))

    def _collect(self, prefix):
        """Turns the recorded events into milliseconds: <prefix>_total, <prefix>_exposed_transfer (time the compute
        stream spent waiting for transfers) and <prefix>_redistribution (zigzag deal and deal back)."""
        evs = self.timings.pop("_events", [])
        if not evs:
            return
        torch.cuda.synchronize()
        total = evs[0][1].elapsed_time(evs[-1][1])
        exposed = redis = 0.0
        for (n0, e0), (n1, e1) in zip(evs, evs[1:]):
            if n1 == "wait_done":
                exposed += e0.elapsed_time(e1)
            if n1 in ("dealt", "dealt_back"):
                redis += e0.elapsed_time(e1)
        self.timings[prefix] = {"total_ms": total, "exposed_transfer_ms": exposed, "redistribution_ms": redis,
                                "kernel_ms": total - exposed - redis}

    # ------------------------------------------------------------------ forward
    def forward(self, q, k, v, keep_state: bool = False):
        """q,k,v: this rank's contiguous shards [B,H,S/W,D].  Returns (o, lse) for the same shard.  With ``keep_state``
        the zigzag-dealt Q, K, V, O, LSE are kept so that ``backward(..., use_saved_state=True)`` on the same tensors
        does not deal them again (every rank must make the same choice: it changes what is exchanged)."""
        be, W, r = self.backend, self.world, self.rank
        self._mark("start")
        qz, kz, vz = self.to_zigzag_many([q, k, v])
        self._mark("dealt")
        q_ids = zigzag_chunks(r, W)
        o_acc = [be.zeros_f32(t) for t in qz]
        lse_acc = [be.neg_inf(t.shape[:3], t) for t in qz]
        kv = list(kz) + list(vz)
        # two receive sets; the dealt chunks themselves are only ever read (they may alias the caller's tensors)
        bufs = [[torch.empty_like(t) for t in kv] for _ in range(2 if W > 2 else 1)] if W > 1 else None
        main, side = self._lanes(q)
        for step in range(W):
            src = (r - step) % W
            kv_ids = zigzag_chunks(src, W)
            works = None
            if step + 1 < W:
                works = self._rotate_start(kv, bufs[step % len(bufs)])
            pairs = visible_pairs(q_ids, kv_ids)
            # pairs on different query chunks touch disjoint running results: they run side by side on two streams
            # so that one launch's last, partly filled wave of CTAs is covered by the other's
            by_q = {}
            for qi, ki, causal in pairs:
                by_q.setdefault(qi, []).append((ki, causal))
            lanes = [main, side] if (side is not None and len(by_q) > 1) else [main]
            if len(lanes) > 1:
                side.wait_stream(main)
            for n, (qi, items) in enumerate(sorted(by_q.items())):
                lane = lanes[n % len(lanes)]
                ctx = torch.cuda.stream(lane) if lane is not None else _null()
                with ctx:
                    for ki, causal in items:
                        o_p, lse_p = be.fwd(qz[qi], kv[ki], kv[2 + ki], causal)
                        be.merge(o_acc[qi], lse_acc[qi], o_p, lse_p)
            if len(lanes) > 1:
                main.wait_stream(side)
            if step + 1 < W:
                self._mark("compute_done")
                self._finish(works, "K/V rotation")
                self._mark("wait_done")
                kv = bufs[step % len(bufs)]
        o_z = [t.to(q.dtype) for t in o_acc]
        self._mark("computed")
        o, lse4 = self.from_zigzag_many([o_z, [t.unsqueeze(-1).contiguous() for t in lse_acc]])
        lse = lse4.squeeze(-1)
        self._mark("dealt_back")
        self._saved = {"qz": qz, "kz": kz, "vz": vz, "oz": o_z, "lsez": lse_acc} if keep_state else None
        self._collect("forward")
        return o, lse

    # ------------------------------------------------------------------ backward
    def backward(self, q, k, v, o, lse, do, use_saved_state: bool = False):
        """All arguments are this rank's contiguous shards; returns (dq, dk, dv) for the same shards.
        ``use_saved_state``: q, k, v, o, lse are the tensors of the last ``forward(..., keep_state=True)``."""
        be, W, r = self.backend, self.world, self.rank
        self._mark("start")
        saved = self._saved
        if use_saved_state:
            if saved is None:
                raise ValueError("no saved forward state: call forward(..., keep_state=True) first")
            qz, kz, vz, oz, lsez = saved["qz"], saved["kz"], saved["vz"], saved["oz"], saved["lsez"]
            (doz,) = self.to_zigzag_many([do])
        else:
            qz, kz, vz, oz, doz, lse4 = self.to_zigzag_many([q, k, v, o, do, lse.unsqueeze(-1).contiguous()])
            lsez = [t.squeeze(-1).contiguous() for t in lse4]
        self._saved = None
        self._mark("dealt")
        q_ids = zigzag_chunks(r, W)
        handles = [be.bwd_begin(qz[i], oz[i], lsez[i], doz[i]) for i in range(2)]
        kv = list(kz) + list(vz)
        kv_bufs = [[torch.empty_like(t) for t in kv] for _ in range(2 if W > 2 else 1)] if W > 1 else None
        # fp32 dK/dV: per-pair partials of this step, and the travelling accumulators in three rotating sets
        part = [[be.zeros_f32(kv[0]), be.zeros_f32(kv[0])] for _ in range(3)]     # [pair slot][dk, dv]
        acc = [be.zeros_f32(t) for t in kv]                                      # the set being completed this step
        acc_recv = [torch.empty_like(t) for t in acc] if W > 1 else None
        acc_send = [torch.empty_like(t) for t in acc] if W > 1 else None
        recv_works = send_pending = None
        main, side = self._lanes(q)
        for step in range(W):
            src = (r - step) % W
            kv_ids = zigzag_chunks(src, W)
            kv_works = None
            if step + 1 < W:                          # K/V of the next step move while this step computes
                kv_works = self._rotate_start(kv, kv_bufs[step % len(kv_bufs)])
            pairs = visible_pairs(q_ids, kv_ids)
            lanes = [main, side] if (side is not None and len(pairs) > 1) else [main]
            if len(lanes) > 1:
                side.wait_stream(main)
            for n, (qi, ki, causal) in enumerate(pairs):
                lane = lanes[n % len(lanes)]
                ctx = torch.cuda.stream(lane) if lane is not None else _null()
                with ctx:
                    part[n][0].zero_()
                    part[n][1].zero_()
                    be.bwd_block(handles[qi], kv[ki], kv[2 + ki], part[n][0], part[n][1], causal)
            if len(lanes) > 1:
                main.wait_stream(side)
            self._mark("compute_done")
            # the accumulators of this step's key chunks: zeros at step 0 (the chunks start here), else what the
            # previous rank sent after its own previous step
            if step > 0:
                self._finish(recv_works, "dK/dV accumulator hop")
                acc, acc_recv = acc_recv, acc
            self._mark("wait_done")
            for n, (qi, ki, causal) in enumerate(pairs):
                be.accumulate(acc[ki], part[n][0])
                be.accumulate(acc[2 + ki], part[n][1])
            if W > 1:
                # pass them on; the hop runs under the next step's kernels.  acc_send is free again once the hop
                # posted a step ago has completed (same handles: a batched round completes as a whole)
                acc, acc_send = acc_send, acc
                recv_works = self._rotate_start(acc_send, acc_recv)
            if step + 1 < W:
                self._mark("compute_done")
                self._finish(kv_works, "K/V rotation")
                self._mark("wait_done")
                kv = kv_bufs[step % len(kv_bufs)]
        if W > 1:
            self._mark("compute_done")
            self._finish(recv_works, "dK/dV accumulator hop home")   # the last hop brings this rank's own chunks home
            self._mark("wait_done")
            acc = acc_recv
        dq_z = [be.bwd_end(h) for h in handles]
        self._mark("computed")
        dq, dk, dv = self.from_zigzag_many([dq_z, [t.to(k.dtype) for t in acc[:2]], [t.to(v.dtype) for t in acc[2:]]])
        self._mark("dealt_back")
        self._collect("backward")
        if hasattr(be, "check"):
            be.check()
        return dq, dk, dv


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class NativeRing:
    """The same schedule run by the library itself (``sntl_ring_attn_fwd`` / ``sntl_ring_attn_bwd``): grouped
    ncclSend / ncclRecv issued from C++ on the handle's own communication stream, every buffer carved from one
    workspace, nothing allocated per call.  This is what a C / C++ host binds; here ``torch.distributed`` is only used
    to hand the NCCL unique id from rank 0 to the other ranks.  bf16 ``[B, H, S/W, D]`` CUDA shards, head_dim 64 / 128."""

    def __init__(self, group=None, zigzag_layout: bool = False):
        """``zigzag_layout``: shards come and go as the rank's two zigzag chunks (``SNTL_FLAG_RING_ZIGZAG``,
        ``zigzag_shard``); the library then redistributes nothing."""
        import ctypes as C
        from . import _lib
        self._C, self._lib = C, _lib
        self.zigzag_layout = zigzag_layout
        self.lib = _lib.load()
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        ident = [None]
        if self.rank == 0:
            buf = C.create_string_buffer(128)
            _lib.check(self.lib.sntl_ring_unique_id(buf), "sntl_ring_unique_id")
            ident[0] = buf.raw
        dist.broadcast_object_list(ident, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        handle = C.c_void_p()
        # NCCL may print a version banner on standard output when a communicator is made; programs that print their
        # results there (bench.py's one JSON line) must not get it mixed in, so it goes to standard error
        import os
        import sys
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            rc = self.lib.sntl_ring_comm_create(ident[0], self.rank, self.world, C.byref(handle))
        finally:
            os.dup2(saved, 1)
            os.close(saved)
        _lib.check(rc, "sntl_ring_comm_create")
        self.handle = handle
        self._ws = None

    @staticmethod
    def _check(q, k, v, o=None, lse=None, do=None):
        """The library reads and writes these tensors through raw pointers as bf16 ``[B, H, S/W, D]``: anything else is
        refused here."""
        named = [(q, "q"), (k, "k"), (v, "v")] + [(t, n) for t, n in ((o, "o"), (do, "do")) if t is not None]
        for t, n in named:
            if not t.is_cuda or not t.is_contiguous() or t.dtype != torch.bfloat16 or t.dim() != 4 or t.device != q.device:
                raise ValueError(f"{n} must be a contiguous bf16 [B, H, S, D] CUDA tensor on q's device")
        if k.shape != v.shape or k.shape[0] != q.shape[0] or k.shape[2:] != q.shape[2:]:
            raise ValueError("k and v must share shape and agree with q on batch, shard length and head_dim")
        for t, n in ((o, "o"), (do, "do")):
            if t is not None and t.shape != q.shape:
                raise ValueError(f"{n} must match q")
        if lse is not None and (not lse.is_cuda or not lse.is_contiguous() or lse.dtype != torch.float32
                                or lse.shape != q.shape[:3] or lse.device != q.device):
            raise ValueError("lse must be a contiguous fp32 [B, Hq, S] CUDA tensor on q's device")

    def _desc(self, q, k):
        B, Hq, S, D = q.shape
        flags = self._lib.FLAG_RING_ZIGZAG if self.zigzag_layout else 0
        return self._lib.Desc(self._lib.DTYPE_BF16, self._lib.LAYOUT_BHSD, B, Hq, k.shape[1], S, S, D, float(D ** -0.5), 1, 0, 0, flags, 0, 0)

    def _workspace(self, d, device):
        need = self.lib.sntl_ring_attn_workspace_bytes(self.handle, self._C.byref(d))
        if need == 0:
            self._lib.check(self._lib.ERR_UNSUPPORTED, "sntl_ring_attn_workspace_bytes")
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=device)
        return self._ws, need

    def forward(self, q, k, v, keep_state: bool = False):
        self._check(q, k, v)
        d = self._desc(q, k)
        ws, need = self._workspace(d, q.device)
        o = torch.empty_like(q)
        lse = torch.empty(q.shape[:3], dtype=torch.float32, device=q.device)
        rc = self.lib.sntl_ring_attn_fwd(self.handle, self._C.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                         lse.data_ptr(), ws.data_ptr(), need, torch.cuda.current_stream().cuda_stream)
        self._lib.check(rc, "sntl_ring_attn_fwd")
        return o, lse

    def backward(self, q, k, v, o, lse, do, use_saved_state: bool = False):
        self._check(q, k, v, o, lse, do)
        d = self._desc(q, k)
        ws, need = self._workspace(d, q.device)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        rc = self.lib.sntl_ring_attn_bwd(self.handle, self._C.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                         lse.data_ptr(), do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                         int(bool(use_saved_state)), ws.data_ptr(), need, torch.cuda.current_stream().cuda_stream)
        self._lib.check(rc, "sntl_ring_attn_bwd")
        return dq, dk, dv

    def close(self):
        if self.handle is not None:
            self.lib.sntl_ring_comm_destroy(self.handle)
            self.handle = None
