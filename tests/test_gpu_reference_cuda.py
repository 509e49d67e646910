"""The reference's own CUDA flash kernels (compiled for sm_100a from the reference sources, oracle/_ref) held to the same
oracle and tolerances as the product's tensor-core kernels, and timed beside them.  Skipped where that library was not
built.  head_dim <= 64 only: the reference's kernels stop there (CudaFlashAttention.hpp:16)."""
import numpy as np
import pytest
import torch

from conftest import load_golden, max_abs, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(oracle):
    if not oracle.ref_cuda_available():
        pytest.skip("oracle/_ref/libsentinel_ref_cuda.so not built")
    return oracle


def test_reference_cuda_flash_on_the_toy_fp32_workload(ref):
    """Config 1 (B=4, H=4, S=64, D=16): the reference CUDA kernel against the reference CPU layer's frozen outputs.
    Its operands are rounded to fp16 inside the kernel, so it is held to the reduced-precision bound, not to 1e-4."""
    g = load_golden("toy_f32_b4_h4_s64_d16")
    o, lse, dq, dk, dv, _ = ref.ref_cuda_flash(g["q"], g["k"], g["v"], g["dout"])
    for got, key in ((o, "o"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert rel_l2(got, g[key]) <= 5e-3, (key, rel_l2(got, g[key]))
    assert max_abs(lse, g["lse"]) <= 2e-2


@pytest.mark.parametrize("shape", [(2, 12, 12, 256, 64), (1, 8, 2, 128, 64)])
def test_reference_cuda_flash_and_product_kernels_against_the_same_oracle(ref, shape):
    import sentinel_b200 as sb
    B, Hq, Hkv, S, D = shape
    w = sb.WORKLOADS["gpt2_small"]
    q, k, v, do = sb.make_inputs(w, batch=B, q_heads=Hq, kv_heads=Hkv, seq=S)
    qf, kf, vf, dof = (t.float().numpy() for t in (q, k, v, do))
    wo, wl = ref.attn_fwd(qf, kf, vf)
    wdq, wdk, wdv, _ = ref.attn_bwd(qf, kf, vf, dof)
    ro, rl, rdq, rdk, rdv, _ = ref.ref_cuda_flash(qf, kf, vf, dof)
    qd, kd, vd, dod = (t.cuda() for t in (q, k, v, do))
    o, lse = sb.attention_forward(qd, kd, vd)
    dq, dk, dv = sb.attention_backward(qd, kd, vd, o, lse, dod)
    ours = [t.float().cpu().numpy() for t in (o, dq, dk, dv)]
    for got_ref, got_ours, want, name in zip((ro, rdq, rdk, rdv), ours, (wo, wdq, wdk, wdv), ("O", "dQ", "dK", "dV")):
        assert max_abs(got_ref, want) <= 2e-2 and rel_l2(got_ref, want) <= 5e-3, ("reference CUDA", name, rel_l2(got_ref, want))
        assert max_abs(got_ours, want) <= 2e-2 and rel_l2(got_ours, want) <= 5e-3, ("tensor-core", name, rel_l2(got_ours, want))
