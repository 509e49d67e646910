"""GPU tests of the boundary contract: the host-buffer call (transfers overlapped with the kernels) returns the same
results as the device-resident calls, and the C-ABI calls can be captured into a CUDA graph and replayed, which is how
the reference's trainer drives its attention (CudaLanguageModel.cu:2176-2209: two eager warm-ups, then capture/replay)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sb():
    import sentinel_b200
    sentinel_b200._lib.load()
    return sentinel_b200


def test_host_buffer_call_matches_device_calls(sb):
    w = sb.WORKLOADS["gqa7b_d128"]
    q, k, v, do = (t.pin_memory() for t in sb.make_inputs(w, batch=3, q_heads=4, kv_heads=2, seq=640))
    qd, kd, vd, dod = (t.cuda() for t in (q, k, v, do))
    o, lse = sb.attention_forward(qd, kd, vd)
    dq, dk, dv = sb.attention_backward(qd, kd, vd, o, lse, dod)
    for chunks in (None, 1, 2, 6):      # KV-group chunks, whole problem, batch chunks, one chunk per unit
        from sentinel_b200.host_pipeline import forward_backward_host
        ho, hl, hdq, hdk, hdv = forward_backward_host(q, k, v, do, chunks=chunks)
        assert torch.equal(ho, o.cpu()) and torch.equal(hl, lse.cpu())
        assert torch.equal(hdk, dk.cpu()) and torch.equal(hdv, dv.cpu())          # one owner each: bit-identical
        assert float((hdq.float() - dq.cpu().float()).abs().max()) <= 1e-3 * float(dq.float().abs().max())  # reduction order varies
    assert sb.poll_device_status() == 0


def test_c_abi_calls_are_graph_capturable(sb):
    w = sb.WORKLOADS["gqa7b_d128"]
    q, k, v, do = (t.cuda() for t in sb.make_inputs(w, batch=1, q_heads=4, kv_heads=1, seq=512))
    o, lse = torch.empty_like(q), torch.empty(q.shape[:3], dtype=torch.float32, device="cuda")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)

    def step():
        sb.attention_forward(q, k, v, out=o, lse=lse)
        sb.attention_backward(q, k, v, o, lse, do, dq=dq, dk=dk, dv=dv)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):               # eager warm-ups: kernel attributes set, scratch grown
            step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    want = [t.clone() for t in (o, lse, dk, dv)]
    want_dq = dq.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for t in (o, lse, dq, dk, dv):
        t.zero_()
    graph.replay()
    graph.replay()
    torch.cuda.synchronize()
    for got, ref in zip((o, lse, dk, dv), want):
        assert torch.equal(got, ref)
    assert float((dq.float() - want_dq.float()).abs().max()) <= 1e-3 * float(want_dq.float().abs().max())
    assert sb.poll_device_status() == 0


def test_calls_on_two_streams_keep_their_scratch_apart(sb):
    """Backward calls that overlap on the GPU (two streams, as in the host-buffer pipeline's two compute streams) must
    not share scratch: each stream's results equal those of the same call run alone."""
    w = sb.WORKLOADS["gqa7b_d128"]
    cases = []
    for seed in (0, 1):
        q, k, v, do = (t.cuda() for t in sb.make_inputs(w, batch=1, q_heads=7, kv_heads=1, seq=1024, seed_offset=seed))
        o, lse = sb.attention_forward(q, k, v)
        dq, dk, dv = sb.attention_backward(q, k, v, o, lse, do)
        cases.append((q, k, v, do, o, lse, dq.clone(), dk.clone(), dv.clone()))
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    for _ in range(5):
        outs = []
        for st, (q, k, v, do, o, lse, *_ref) in zip(streams, cases):
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                outs.append(sb.attention_backward(q, k, v, o, lse, do))
        torch.cuda.synchronize()
        for (dq, dk, dv), case in zip(outs, cases):
            assert torch.equal(dk, case[7]) and torch.equal(dv, case[8])
            assert float((dq.float() - case[6].float()).abs().max()) <= 1e-3 * float(case[6].float().abs().max())
    assert sb.poll_device_status() == 0


def test_bounded_wait_runs_out_reports_and_leaves_the_context_usable(sb):
    """Failure detection without a fault: a one-warp kernel waits, with a 2 ms limit, on a barrier that by construction
    never receives its arrival.  The wait runs out exactly as a stuck production wait would after its one second: the
    kernel returns normally, the poll reports SNTL_ERR_DEVICE_TIMEOUT with the self-test's site code, the report is
    cleared by that poll, and the next real call (made after the short give-up window has passed) is clean and exact."""
    import ctypes as C
    import time
    from sentinel_b200 import _lib
    lib = _lib.load()
    assert sb.poll_device_status() == 0
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.sntl_attn_selftest_wait_timeout(2000, stream) == _lib.OK
    fwd, bwd = C.c_uint32(0), C.c_uint32(0)
    rc = lib.sntl_attn_poll_device_status_words(stream, C.byref(fwd), C.byref(bwd))
    assert rc == _lib.ERR_DEVICE_TIMEOUT
    assert fwd.value >> 24 == 0x7e and bwd.value == 0
    assert lib.sntl_attn_poll_device_status_words(stream, C.byref(fwd), C.byref(bwd)) == _lib.OK   # cleared by the poll
    with pytest.raises(RuntimeError):      # the python mirror raises at its synchronisation point
        assert lib.sntl_attn_selftest_wait_timeout(1000, stream) == _lib.OK
        sb.raise_if_device_wait_timed_out()
    time.sleep(0.05)                       # well past the 1-2 ms during which other waits would give up early
    w = sb.WORKLOADS["gqa7b_d128"]
    q, k, v, do = (t.cuda() for t in sb.make_inputs(w, batch=1, q_heads=4, kv_heads=2, seq=512))
    o1, lse1 = sb.attention_forward(q, k, v)
    dq1, dk1, dv1 = sb.attention_backward(q, k, v, o1, lse1, do)
    assert sb.poll_device_status() == 0
    o2, lse2 = sb.attention_forward(q, k, v)
    assert torch.equal(o1, o2) and torch.equal(lse1, lse2)
    assert lib.sntl_attn_selftest_wait_timeout(0, stream) == _lib.ERR_BAD_ARGUMENT
    assert lib.sntl_attn_selftest_wait_timeout(200000, stream) == _lib.ERR_BAD_ARGUMENT


def test_deterministic_flag_makes_dq_bit_reproducible(sb):
    """SNTL_FLAG_DETERMINISTIC: dQ is summed in 64-bit fixed point, so it is bit-identical from run to run, between the
    one-stream and two-stream variants and through the chunked host-buffer pipeline -- and it meets the same oracle
    bounds as the default path (it is the exact sum of the same fp32 contributions, rounded once)."""
    import numpy as np
    from oracle import cpu
    from sentinel_b200 import _lib
    from sentinel_b200.host_pipeline import forward_backward_host
    det = _lib.FLAG_DETERMINISTIC
    for name, kw in (("gqa7b_d128", dict(batch=2, q_heads=8, kv_heads=2, seq=1152)), ("llama1b_gqa", dict(batch=1, q_heads=8, kv_heads=4, seq=777))):
        w = sb.WORKLOADS[name]
        q, k, v, do = (t.pin_memory() for t in sb.make_inputs(w, **kw))
        qd, kd, vd, dod = (t.cuda() for t in (q, k, v, do))
        o, lse = sb.attention_forward(qd, kd, vd)
        dq1, dk1, dv1 = sb.attention_backward(qd, kd, vd, o, lse, dod, flags=det)
        runs = [sb.attention_backward(qd, kd, vd, o, lse, dod, flags=det) for _ in range(4)]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            runs.append(sb.attention_backward(qd, kd, vd, o, lse, dod, flags=det))
        runs.append(sb.attention_backward(qd, kd, vd, o, lse, dod, flags=det))     # overlaps the side stream's call
        torch.cuda.synchronize()
        for dq, dk, dv in runs:
            assert torch.equal(dq, dq1) and torch.equal(dk, dk1) and torch.equal(dv, dv1)
        for chunks in (None, 1, 2):
            _, _, hdq, hdk, hdv = forward_backward_host(q, k, v, do, chunks=chunks, flags=det)
            assert torch.equal(hdq, dq1.cpu()) and torch.equal(hdk, dk1.cpu()) and torch.equal(hdv, dv1.cpu())
        # the default path differs from it only in the last bits, and both sit inside the oracle bounds
        dq0, _, _ = sb.attention_backward(qd, kd, vd, o, lse, dod)
        assert float((dq0.float() - dq1.float()).abs().max()) <= 1e-2 * float(dq1.float().abs().max())
        wdq, wdk, wdv, _ = cpu.attn_bwd(*(t.float().numpy() for t in (q, k, v, do)))
        got = dq1.float().cpu().numpy()
        assert float(np.abs(got - wdq).max()) <= 2e-2
        assert float(np.linalg.norm(got - wdq) / np.linalg.norm(wdq)) <= 5e-3
    assert sb.poll_device_status() == 0
