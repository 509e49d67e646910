"""CPU tests of the multi-rank host logic (gloo, world_size 2 and 4): the sequence-sharded ring schedule and the
batch x KV-group sharding.  The arithmetic is supplied by the fp64 oracle here, so what is under test is the schedule:
zigzag deal, which (query chunk, key chunk) pairs each rank computes at each step, the log-sum-exp merges, the
gradient accumulators that travel with their key chunk, and the deal back to contiguous shards."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


class OracleBackend:
    """Stands in for the CUDA kernels with the CPU oracle (fp32 tensors in, fp32 out)."""

    def __init__(self):
        from oracle import cpu
        self.cpu = cpu
        self.calls = []

    def fwd(self, q, k, v, causal):
        self.calls.append(("fwd", causal))
        o, lse = self.cpu.attn_fwd(q.numpy(), k.numpy(), v.numpy(), causal=causal)
        return torch.from_numpy(o), torch.from_numpy(lse)

    def _bwd(self, q, k, v, o, lse, do, causal):
        # global probabilities from the FINAL lse, exactly what the kernels do: P = exp(scale*qk - lse)
        qn, kn, vn, don = (t.double() for t in (q, k, v, do))
        B, Hq, Sq, D = qn.shape
        g = Hq // kn.shape[1]
        kr, vr = kn.repeat_interleave(g, 1), vn.repeat_interleave(g, 1)
        s = torch.einsum("bhqd,bhkd->bhqk", qn, kr) * D ** -0.5
        p = torch.exp(s - lse.double()[..., None])
        if causal:
            p = p * torch.tril(torch.ones(Sq, kr.shape[2], dtype=torch.float64))
        delta = (o.double() * don).sum(-1, keepdim=True)
        dp = torch.einsum("bhqd,bhkd->bhqk", don, vr)
        ds = p * (dp - delta) * D ** -0.5
        dq = torch.einsum("bhqk,bhkd->bhqd", ds, kr)
        dk = torch.einsum("bhqk,bhqd->bhkd", ds, qn).reshape(B, kn.shape[1], g, -1, D).sum(2)
        dv = torch.einsum("bhqk,bhqd->bhkd", p, don).reshape(B, kn.shape[1], g, -1, D).sum(2)
        return dq.float(), dk.float(), dv.float()

    # the backward in pieces, as the C ABI offers it (sntl_attn_bwd_begin / _block / _end)
    def bwd_begin(self, q, o, lse, do):
        return {"q": q, "o": o, "lse": lse, "do": do, "dq": torch.zeros_like(q, dtype=torch.float32)}

    def bwd_block(self, h, k, v, dk_acc, dv_acc, causal):
        self.calls.append(("bwd", causal))
        dq, dk, dv = self._bwd(h["q"], k, v, h["o"], h["lse"], h["do"], causal)
        h["dq"] += dq
        dk_acc += dk
        dv_acc += dv

    def bwd_end(self, h):
        return h["dq"]

    def merge(self, o_acc, lse_acc, o_part, lse_part):
        m = torch.maximum(lse_acc, lse_part)
        wa, wb = torch.exp(lse_acc - m), torch.exp(lse_part - m)
        o_acc.copy_((o_acc * wa[..., None] + o_part * wb[..., None]) / (wa + wb)[..., None])
        lse_acc.copy_(m + torch.log(wa + wb))

    def accumulate(self, acc, part):
        acc.add_(part.float())

    def zeros_f32(self, like):
        return torch.zeros(like.shape, dtype=torch.float32)

    def neg_inf(self, shape, like):
        return torch.full(shape, float("-inf"), dtype=torch.float32)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ring_worker(rank, world, port, shape, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sentinel_b200.ring import RingAttention, visible_pairs, zigzag_chunks
        B, Hq, Hkv, S, D = shape
        g = torch.Generator().manual_seed(1234)
        q = torch.randn(B, Hq, S, D, generator=g)
        k = torch.randn(B, Hkv, S, D, generator=g)
        v = torch.randn(B, Hkv, S, D, generator=g)
        do = torch.randn(B, Hq, S, D, generator=g)
        sl = slice(rank * S // world, (rank + 1) * S // world)
        be = OracleBackend()
        ring = RingAttention(be)
        o, lse = ring.forward(q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous())
        n_fwd = len(be.calls)
        dq, dk, dv = ring.backward(q[:, :, sl].contiguous(), k[:, :, sl].contiguous(), v[:, :, sl].contiguous(), o, lse,
                                   do[:, :, sl].contiguous())
        # balance: every rank runs the same number of block pairs: 2 per step, 3 at step 0 (two of them diagonal halves)
        assert n_fwd == 2 * world + 1, n_fwd
        assert len(be.calls) - n_fwd == 2 * world + 1
        # the same backward from the state the forward kept (no second deal of Q, K, V, O, LSE): identical results
        qs, ks, vs, dos = (t[:, :, sl].contiguous() for t in (q, k, v, do))
        o2, lse2 = ring.forward(qs, ks, vs, keep_state=True)
        dq2, dk2, dv2 = ring.backward(qs, ks, vs, o2, lse2, dos, use_saved_state=True)
        for a, b_, n in ((o2, o, 'o'), (dq2, dq, 'dq'), (dk2, dk, 'dk'), (dv2, dv, 'dv')):
            assert float((a - b_).abs().max()) <= 1e-6 * float(b_.abs().max()), (n, float((a - b_).abs().max()))
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), o=o.numpy(), lse=lse.numpy(), dq=dq.numpy(), dk=dk.numpy(), dv=dv.numpy())
        # zigzag deal and its inverse are exact permutations
        x = torch.arange(B * Hq * (S // world) * D, dtype=torch.float32).reshape(B, Hq, S // world, D) + 1e6 * rank
        assert torch.equal(ring.from_zigzag(ring.to_zigzag(x)), x)
        # shards handed over in the zigzag layout itself (nothing is redistributed: no exchange before the first step):
        # the same numbers, in that layout
        from sentinel_b200.ring import zigzag_shard
        zring = RingAttention(OracleBackend(), zigzag_layout=True)
        qz, kz, vz, doz = (zigzag_shard(t, rank, world) for t in (q, k, v, do))
        oz, lsez = zring.forward(qz, kz, vz)
        dqz, dkz, dvz = zring.backward(qz, kz, vz, oz, lsez, doz)
        full = {}
        for name, mine in (("o", o), ("lse", lse.unsqueeze(-1)), ("dq", dq), ("dk", dk), ("dv", dv)):
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine.contiguous())
            full[name] = torch.cat(parts, dim=2)
        for name, got in (("o", oz), ("lse", lsez.unsqueeze(-1)), ("dq", dqz), ("dk", dkz), ("dv", dvz)):
            want = zigzag_shard(full[name], rank, world)
            assert float((got - want).abs().max()) <= 1e-6 * max(1.0, float(want.abs().max())), name
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,shape", [(2, (1, 4, 2, 64, 16)), (4, (1, 2, 1, 96, 8))])
def test_ring_schedule_matches_full_sequence_oracle(tmp_path, world, shape, oracle):
    port = _free_port()
    mp.spawn(_ring_worker, args=(world, port, shape, str(tmp_path)), nprocs=world, join=True)
    B, Hq, Hkv, S, D = shape
    g = torch.Generator().manual_seed(1234)
    q = torch.randn(B, Hq, S, D, generator=g).numpy()
    k = torch.randn(B, Hkv, S, D, generator=g).numpy()
    v = torch.randn(B, Hkv, S, D, generator=g).numpy()
    do = torch.randn(B, Hq, S, D, generator=g).numpy()
    wo, wl = oracle.attn_fwd(q, k, v)
    wdq, wdk, wdv, _ = oracle.attn_bwd(q, k, v, do)
    got = {key: np.concatenate([np.load(tmp_path / f"rank{r}.npz")[key] for r in range(world)], axis=2) for key in ("o", "lse", "dq", "dk", "dv")}
    for key, want in (("o", wo), ("lse", wl), ("dq", wdq), ("dk", wdk), ("dv", wdv)):
        assert np.abs(got[key] - want).max() < 2e-5, key


def _failure_worker(rank, world, port, mode, out_dir):
    """Host-made failures only: a rank that never joins the step, a slow rank, a rank that rotates the wrong way."""
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from sentinel_b200.ring import RingAttention, RingTimeout
    B, Hq, Hkv, S, D = 1, 2, 1, 16 * world, 8
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, Hq, S, D, generator=g)
    k = torch.randn(B, Hkv, S, D, generator=g)
    v = torch.randn(B, Hkv, S, D, generator=g)
    sl = slice(rank * S // world, (rank + 1) * S // world)
    args = [t[:, :, sl].contiguous() for t in (q, k, v)]
    outcome = "none"
    t0 = time.monotonic()
    try:
        if mode == "leaves" and rank == world - 1:
            outcome = "left"                    # leaves between steps: nothing of its own is in flight
        else:
            ring = RingAttention(OracleBackend(), timeout_s=10.0 if mode == "slow" else 2.0)
            if mode == "slow" and rank == world - 1:
                time.sleep(1.0)
            if mode == "wrong_way" and rank == world - 1:
                def wrong(tensors, buffers, self=ring):
                    nxt, prv = (self.rank + 1) % self.world, (self.rank - 1) % self.world
                    ops = [dist.P2POp(dist.isend, t, prv, self.group) for t in tensors]
                    ops += [dist.P2POp(dist.irecv, b, nxt, self.group) for b in buffers]
                    return dist.batch_isend_irecv(ops)
                ring._rotate_start = wrong
            ring.forward(*args)
            outcome = "completed"
    except RingTimeout:
        outcome = "timeout"
    except RuntimeError:                        # gloo reports a vanished peer as a connection error
        outcome = "error"
    with open(os.path.join(out_dir, f"outcome{rank}.txt"), "w") as f:
        f.write(f"{outcome} {time.monotonic() - t0:.2f}")
    os._exit(0)                                 # no collective teardown with a peer that may be gone


@pytest.mark.parametrize("mode,world", [("leaves", 2), ("slow", 2), ("wrong_way", 3)])
def test_ring_raises_within_a_deadline_when_a_peer_fails(tmp_path, mode, world):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_failure_worker, args=(r, world, port, mode, str(tmp_path))) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive(), "a rank waited for ever"
    got = [open(tmp_path / f"outcome{r}.txt").read().split() for r in range(world)]
    if mode == "slow":
        assert all(o == "completed" for o, _ in got), got          # a rank that is late but alive is waited for
    else:
        assert got[0][0] in ("timeout", "error"), got               # the healthy rank raised instead of hanging
        assert float(got[0][1]) < 30.0


def test_visible_pairs_cover_the_causal_mask_exactly_once():
    from sentinel_b200.ring import visible_pairs, zigzag_chunks
    for world in (1, 2, 4, 8):
        seen = set()
        per_step = []
        for r in range(world):
            for step in range(world):
                src = (r - step) % world
                qs, ks = zigzag_chunks(r, world), zigzag_chunks(src, world)
                pairs = visible_pairs(qs, ks)
                per_step.append(sum(0.5 if c else 1.0 for _, _, c in pairs))
                for qi, ki, causal in pairs:
                    key = (qs[qi], ks[ki])
                    assert key not in seen
                    assert causal == (key[0] == key[1])
                    seen.add(key)
        n = 2 * world
        assert seen == {(a, b) for a in range(n) for b in range(n) if b <= a}
        assert all(abs(x - 2.0) < 1e-9 for x in per_step)      # perfectly balanced: 2 block units per rank per step


def _shard_worker(rank, world, port, out_dir):
    """Batch x KV-group sharding (workloads 1-4): every (batch, KV head) unit is independent, so ranks just take
    disjoint units and nothing is exchanged on the data path."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import cpu
        from sentinel_b200.workloads import shard_units
        B, Hq, Hkv, S, D = 2, 4, 2, 24, 8
        g = torch.Generator().manual_seed(7)
        q = torch.randn(B, Hq, S, D, generator=g).numpy()
        k = torch.randn(B, Hkv, S, D, generator=g).numpy()
        v = torch.randn(B, Hkv, S, D, generator=g).numpy()
        grp = Hq // Hkv
        res = {}
        for (b, hk) in shard_units(B, Hkv, rank, world):
            o, _ = cpu.attn_fwd(q[b:b + 1, hk * grp:(hk + 1) * grp], k[b:b + 1, hk:hk + 1], v[b:b + 1, hk:hk + 1])
            res[f"{b}_{hk}"] = o
        np.savez(os.path.join(out_dir, f"shard{rank}.npz"), **res)
        count = torch.tensor([len(res)])
        dist.all_reduce(count)          # bookkeeping only: the units add up to the whole job
        assert int(count) == B * Hkv
    finally:
        dist.destroy_process_group()


def test_batch_kv_group_sharding_needs_no_exchange(tmp_path, oracle):
    world = 2
    mp.spawn(_shard_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    B, Hq, Hkv, S, D = 2, 4, 2, 24, 8
    g = torch.Generator().manual_seed(7)
    q = torch.randn(B, Hq, S, D, generator=g).numpy()
    k = torch.randn(B, Hkv, S, D, generator=g).numpy()
    v = torch.randn(B, Hkv, S, D, generator=g).numpy()
    wo, _ = oracle.attn_fwd(q, k, v)
    grp = Hq // Hkv
    seen = set()
    for r in range(world):
        z = np.load(tmp_path / f"shard{r}.npz")
        for key in z.files:
            b, hk = map(int, key.split("_"))
            assert key not in seen
            seen.add(key)
            assert np.abs(z[key] - wo[b:b + 1, hk * grp:(hk + 1) * grp]).max() < 1e-6
    assert len(seen) == B * Hkv
