"""Sequence-sharded causal attention over a ring of ranks (the 131072-token workload).

The reference has no sequence-parallel path; this is the multi-GPU schedule built on the single-GPU kernels.

Layout at the interface: the sequence is split into ``W`` equal contiguous shards, rank ``r`` holds tokens
``[r*S/W, (r+1)*S/W)`` of Q, K, V (and O, dO, dQ, dK, dV), each ``[B, H, S/W, D]``.

Schedule
--------
A plain ring over contiguous shards is badly unbalanced under a causal mask (rank r has r+0.5 blocks of work).
So each shard is cut in two half-shards ("chunks", ``2W`` in total) and the chunks are first re-dealt in a zigzag:
rank ``r`` works on chunks ``r`` and ``2W-1-r``.  Then for ``W`` steps the key/value chunks travel round the ring
(rank r sends to r+1).  In every step every rank has exactly two visible (query chunk, key chunk) pairs -- a pair is
visible iff ``key_chunk <= query_chunk``, causal inside iff equal -- so all ranks finish each step together.
Forward: each visible pair is one call of the attention forward (non-causal, or causal on the diagonal) whose
(O, LSE) partial is folded into fp32 running results with the log-sum-exp merge.  Backward: each visible pair is one
call of the attention backward with the FINAL LSE and O of the query chunk, so its probabilities are already the
global ones; dQ partials add up locally, dK/dV partials add into fp32 accumulators that travel with their key
chunk and arrive home after ``W`` steps.  Results are dealt back to the contiguous layout at the end.

Communication is ``torch.distributed`` point-to-point (NCCL send/recv over NVLink on GPUs; gloo in the CPU tests),
issued for step t+1 before the compute of step t so the transfer overlaps the kernels.

The arithmetic is supplied by a *backend* (``GpuBackend`` = this library's kernels).  The schedule itself touches
no tensor values, which is what lets the CPU tests drive it with a reference backend.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def chunk_owner_contiguous(chunk: int) -> int:
    return chunk // 2


def chunk_owner_zigzag(chunk: int, world: int) -> int:
    return chunk if chunk < world else 2 * world - 1 - chunk


def zigzag_chunks(rank: int, world: int):
    """The two chunk ids rank ``rank`` works on, low one first."""
    return (rank, 2 * world - 1 - rank)


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

    def bwd(self, q, k, v, o, lse, do, causal):
        return self.fa.attention_backward(q, k, v, o, lse, do, causal=causal)

    def merge(self, o_acc, lse_acc, o_part, lse_part):
        self.fa.merge_partials(o_acc, lse_acc, o_part, lse_part)

    def accumulate(self, acc, part):
        self.fa.accumulate(acc, part)

    def zeros_f32(self, like):
        return torch.zeros(like.shape, dtype=torch.float32, device=like.device)

    def neg_inf(self, shape, like):
        return torch.full(shape, float("-inf"), dtype=torch.float32, device=like.device)


class RingAttention:
    def __init__(self, backend, group=None):
        self.backend = backend
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)

    # ------------------------------------------------------------------ redistribution
    def _exchange(self, sends, recvs):
        """sends: [(tensor, dst)], recvs: [(tensor, src)]; one batched point-to-point round."""
        ops = [dist.P2POp(dist.isend, t, dst, self.group) for t, dst in sends]
        ops += [dist.P2POp(dist.irecv, t, src, self.group) for t, src in recvs]
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    def to_zigzag(self, x):
        """[B,H,S_local,D] contiguous shard -> list of the two chunks this rank works on (zigzag deal)."""
        r, W = self.rank, self.world
        half = x.shape[2] // 2
        mine = {2 * r: x[:, :, :half].contiguous(), 2 * r + 1: x[:, :, half:].contiguous()}
        want = zigzag_chunks(r, W)
        out = {c: (mine[c] if c in mine else torch.empty_like(mine[2 * r])) for c in want}
        sends = [(t, chunk_owner_zigzag(c, W)) for c, t in sorted(mine.items()) if chunk_owner_zigzag(c, W) != r]
        recvs = [(out[c], chunk_owner_contiguous(c)) for c in want if chunk_owner_contiguous(c) != r]
        self._exchange(sends, recvs)
        return [out[c] for c in want]

    def from_zigzag(self, chunks):
        """Inverse of ``to_zigzag``: the two zigzag chunks -> this rank's contiguous shard."""
        r, W = self.rank, self.world
        have = dict(zip(zigzag_chunks(r, W), chunks))
        want = (2 * r, 2 * r + 1)
        out = {c: (have[c] if c in have else torch.empty_like(chunks[0])) for c in want}
        sends = [(t.contiguous(), chunk_owner_contiguous(c)) for c, t in sorted(have.items()) if chunk_owner_contiguous(c) != r]
        recvs = [(out[c], chunk_owner_zigzag(c, W)) for c in want if chunk_owner_zigzag(c, W) != r]
        self._exchange(sends, recvs)
        return torch.cat([out[want[0]], out[want[1]]], dim=2)

    def _rotate_start(self, tensors, buffers):
        """Post the ring shift of ``tensors`` (to rank+1) into ``buffers`` (from rank-1); returns work handles."""
        if self.world == 1:
            return None
        nxt, prv = (self.rank + 1) % self.world, (self.rank - 1) % self.world
        ops = [dist.P2POp(dist.isend, t, nxt, self.group) for t in tensors]
        ops += [dist.P2POp(dist.irecv, b, prv, self.group) for b in buffers]
        return dist.batch_isend_irecv(ops)

    @staticmethod
    def _rotate_finish(works):
        if works:
            for w in works:
                w.wait()

    # ------------------------------------------------------------------ forward
    def forward(self, q, k, v):
        """q,k,v: this rank's contiguous shards [B,H,S/W,D].  Returns (o, lse) for the same shard.
        Also returns the zigzag-layout state the backward can reuse."""
        be, W, r = self.backend, self.world, self.rank
        qz, kz, vz = self.to_zigzag(q), self.to_zigzag(k), self.to_zigzag(v)
        q_ids = zigzag_chunks(r, W)
        o_acc = [be.zeros_f32(t) for t in qz]
        lse_acc = [be.neg_inf(t.shape[:3], t) for t in qz]
        kv = list(kz) + list(vz)
        for step in range(W):
            src = (r - step) % W
            kv_ids = zigzag_chunks(src, W)
            works, nxt_kv = None, None
            if step + 1 < W:
                nxt_kv = [torch.empty_like(t) for t in kv]
                works = self._rotate_start(kv, nxt_kv)
            for qi, ki, causal in visible_pairs(q_ids, kv_ids):
                o_p, lse_p = be.fwd(qz[qi], kv[ki], kv[2 + ki], causal)
                be.merge(o_acc[qi], lse_acc[qi], o_p, lse_p)
            if step + 1 < W:
                self._rotate_finish(works)
                kv = nxt_kv
        o_z = [t.to(q.dtype) for t in o_acc]
        o = self.from_zigzag(o_z)
        lse = self.from_zigzag([t.unsqueeze(-1).contiguous() for t in lse_acc]).squeeze(-1)
        return o, lse

    # ------------------------------------------------------------------ backward
    def backward(self, q, k, v, o, lse, do):
        """All arguments are this rank's contiguous shards; returns (dq, dk, dv) for the same shards."""
        be, W, r = self.backend, self.world, self.rank
        qz, kz, vz = self.to_zigzag(q), self.to_zigzag(k), self.to_zigzag(v)
        oz, doz = self.to_zigzag(o), self.to_zigzag(do)
        lsez = [t.squeeze(-1).contiguous() for t in self.to_zigzag(lse.unsqueeze(-1).contiguous())]
        q_ids = zigzag_chunks(r, W)
        dq_acc = [be.zeros_f32(t) for t in qz]
        kv = list(kz) + list(vz)
        dkv = [be.zeros_f32(t) for t in kv]          # travels with its key/value chunk
        for step in range(W):
            src = (r - step) % W
            kv_ids = zigzag_chunks(src, W)
            works, nxt_kv = None, None
            if step + 1 < W:                          # K/V of the next step can move while this step computes
                nxt_kv = [torch.empty_like(t) for t in kv]
                works = self._rotate_start(kv, nxt_kv)
            for qi, ki, causal in visible_pairs(q_ids, kv_ids):
                dq_p, dk_p, dv_p = be.bwd(qz[qi], kv[ki], kv[2 + ki], oz[qi], lsez[qi], doz[qi], causal)
                be.accumulate(dq_acc[qi], dq_p)
                be.accumulate(dkv[ki], dk_p)
                be.accumulate(dkv[2 + ki], dv_p)
            # the gradient accumulators follow their chunk (after this step's contributions), including the last
            # hop that brings them home
            if W > 1:
                nxt_dkv = [torch.empty_like(t) for t in dkv]
                w2 = self._rotate_start(dkv, nxt_dkv)
                self._rotate_finish(w2)
                dkv = nxt_dkv
            if step + 1 < W:
                self._rotate_finish(works)
                kv = nxt_kv
        dq = self.from_zigzag([t.to(q.dtype) for t in dq_acc])
        dk = self.from_zigzag([t.to(k.dtype) for t in dkv[:2]])
        dv = self.from_zigzag([t.to(v.dtype) for t in dkv[2:]])
        return dq, dk, dv
