"""GPU test of the backward entry point that brings its own scratch memory, for callers that cannot allocate.

Some users of this library run where a device allocation is not possible: inside another component's stream
capture, in a loop whose owner forbids cudaMalloc, or from a binding that owns no allocator.  For them
``sntl_attn_bwd_static_scratch`` keeps its scratch in a fixed 32 MiB array inside the library.  This test calls it
through the C ABI twice in a row -- with different problems, so that what the first call left in the shared array
would show up as an error in the second -- and compares every gradient with the ordinary ``sntl_attn_bwd`` that was
given a caller-owned workspace.  It also checks that a problem beyond the built-in capacity is refused with its own
status code.  The file name makes pytest collect it last.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

BF16_ABS, BF16_REL = 2e-2, 5e-3   # the bounds the tensor-core parity tests use


def _desc(lib_mod, q, k, causal=True):
    B, Hq, Sq, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    dtype = lib_mod.DTYPE_BF16 if q.dtype == torch.bfloat16 else lib_mod.DTYPE_F32
    return lib_mod.Desc(dtype, lib_mod.LAYOUT_BHSD, B, Hq, Hkv, Sq, Skv, D, float(D ** -0.5), int(causal), 0, 0, 0)


def _both_backwards(sb, q, k, v, do):
    """Returns (gradients from sntl_attn_bwd with a caller workspace, gradients from the static-scratch call)."""
    lib = sb._lib.load()
    o, lse = sb.attention_forward(q, k, v)
    d = _desc(sb._lib, q, k)
    stream = torch.cuda.current_stream().cuda_stream
    need = lib.sntl_attn_bwd_workspace_bytes(C.byref(d))
    assert 0 < need <= lib.sntl_attn_static_scratch_capacity()
    ws = torch.empty(need, dtype=torch.uint8, device=q.device)
    ref = [torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)]
    rc = lib.sntl_attn_bwd(C.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), do.data_ptr(),
                           ref[0].data_ptr(), ref[1].data_ptr(), ref[2].data_ptr(), ws.data_ptr(), need, stream)
    assert rc == sb._lib.OK
    got = [torch.full_like(q, 7.0), torch.full_like(k, 7.0), torch.full_like(v, 7.0)]
    rc = lib.sntl_attn_bwd_static_scratch(C.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                          do.data_ptr(), got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(), stream)
    assert rc == sb._lib.OK, lib.sntl_status_string(rc)
    torch.cuda.synchronize()
    assert sb.poll_device_status() == 0
    return ref, got


def _close(got, want, what):
    g, w = got.float().cpu().numpy(), want.float().cpu().numpy()
    assert np.isfinite(g).all(), what
    assert float(np.abs(g - w).max()) <= BF16_ABS, what
    assert float(np.linalg.norm(g - w) / max(np.linalg.norm(w), 1e-30)) <= BF16_REL, what


def test_static_scratch_backward_matches_workspace_backward_twice_in_a_row():
    import sentinel_b200 as sb
    w = sb.WORKLOADS["gqa7b_d128"]
    # first call: tensor-core route, 3 query tiles, grouped-query heads
    q, k, v, do = (t.cuda() for t in sb.make_inputs(w, batch=1, q_heads=4, kv_heads=2, seq=384))
    ref, got = _both_backwards(sb, q, k, v, do)
    assert sb.last_path() == "tcgen05"
    for g, r, name in zip(got, ref, ("dQ", "dK", "dV")):
        _close(g, r, "first call " + name)
    assert torch.equal(got[1], ref[1]) and torch.equal(got[2], ref[2])   # dK/dV have one owner each: bit-identical
    # second call straight after, a different and smaller problem: stale scratch contents must not leak in
    q, k, v, do = (t.cuda() for t in sb.make_inputs(w, batch=2, q_heads=2, kv_heads=1, seq=200, seed_offset=3))
    ref, got = _both_backwards(sb, q, k, v, do)
    for g, r, name in zip(got, ref, ("dQ", "dK", "dV")):
        _close(g, r, "second call " + name)
    assert torch.equal(got[1], ref[1]) and torch.equal(got[2], ref[2])
    # and once more on the exact-fp32 route, which keeps only delta in the array
    w1 = sb.WORKLOADS["toy_f32"]
    q, k, v, do = (t.cuda() for t in sb.make_inputs(w1))
    ref, got = _both_backwards(sb, q, k, v, do)
    assert sb.last_path() == "simt_f32"
    for g, r in zip(got, ref):
        assert torch.equal(g, r)


def test_static_scratch_refuses_problems_beyond_its_capacity():
    import sentinel_b200 as sb
    lib = sb._lib.load()
    cap = lib.sntl_attn_static_scratch_capacity()
    assert cap == 32 << 20
    # B=2, Hq=28, S=8192, D=128 needs ~235 MB of scratch: refused before anything is launched or dereferenced
    d = sb._lib.Desc(sb._lib.DTYPE_BF16, sb._lib.LAYOUT_BHSD, 2, 28, 4, 8192, 8192, 128, 0.088, 1, 0, 0, 0)
    assert lib.sntl_attn_bwd_workspace_bytes(C.byref(d)) > cap
    before = lib.sntl_attn_launch_count()
    dummy = C.c_void_p(256)
    rc = lib.sntl_attn_bwd_static_scratch(C.byref(d), dummy, dummy, dummy, dummy, dummy, dummy, dummy, dummy, dummy, None)
    assert rc == sb._lib.ERR_SCRATCH_LIMIT
    assert b"32 MiB" in lib.sntl_status_string(rc)
    assert lib.sntl_attn_launch_count() == before
    # an invalid descriptor is reported as such, not as a capacity problem
    bad = sb._lib.Desc(sb._lib.DTYPE_BF16, sb._lib.LAYOUT_BHSD, 1, 7, 2, 128, 128, 128, 0.088, 1, 0, 0, 0)
    rc = lib.sntl_attn_bwd_static_scratch(C.byref(bad), dummy, dummy, dummy, dummy, dummy, dummy, dummy, dummy, dummy, None)
    assert rc == sb._lib.ERR_BAD_ARGUMENT
