"""GPU tests of the boundary conversions fused with the rotary embedding (fp32 feature-major <-> bf16 token-major).
Integer-exact parity: the kernels round products and sums separately, as the reference's RotaryEmbedding does on the
host (RotaryEmbedding.cpp:38-81), so the bf16 output is the rounding of exactly the reference's fp32 value."""
import numpy as np
import pytest
import torch

from conftest import ROPE_GOLDEN_CASES, ROPE_LAYER_GOLDEN, load_golden, max_abs, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sb():
    import sentinel_b200
    sentinel_b200._lib.load()
    assert torch.cuda.is_available()
    return sentinel_b200


def _fm_to_bhsd(m, B, H, S, D, col0):
    """feature-major (H*D) x stride -> [B,H,S,D] of the pack window starting at col0"""
    return np.ascontiguousarray(m[:, col0:col0 + B * S].reshape(H, D, B, S).transpose(2, 0, 3, 1))


def _bits(t):
    return t.view(torch.int16).cpu().numpy()


@pytest.mark.parametrize("name", ROPE_GOLDEN_CASES)
def test_pack_matches_reference_rotation_bit_for_bit(sb, oracle, name):
    g = load_golden(name)
    H, D = int(g["heads"]), int(g["head_dim"])
    cols = g["matrix"].shape[1]
    m = torch.from_numpy(g["matrix"]).cuda()
    cos_t, sin_t = torch.from_numpy(g["cos"]).cuda(), torch.from_numpy(g["sin"]).cuda()
    got = sb.pack_heads(m, 1, H, cols, D, cos_table=cos_t, sin_table=sin_t)
    want = torch.from_numpy(_fm_to_bhsd(oracle.round_bf16(g["rotated"]), 1, H, cols, D, 0)).to(torch.bfloat16)
    assert np.array_equal(_bits(got), _bits(want))
    # no tables: relayout + cast only
    got = sb.pack_heads(m, 1, H, cols, D)
    want = torch.from_numpy(_fm_to_bhsd(oracle.round_bf16(g["matrix"]), 1, H, cols, D, 0)).to(torch.bfloat16)
    assert np.array_equal(_bits(got), _bits(want))
    # unpack with the inverse rotation: exact fp32 values of the reference's rotateInverseInPlace on bf16-representable input
    src = oracle.round_bf16(g["matrix"])
    want_inv = oracle.rope_rotate(src, H, D, g["cos"], g["sin"], inverse=True)
    want_fwd = oracle.rope_rotate(src, H, D, g["cos"], g["sin"])
    t = torch.from_numpy(_fm_to_bhsd(src, 1, H, cols, D, 0)).to(torch.bfloat16).cuda()
    out = torch.full_like(m, -777.0)
    sb.unpack_heads(t, out, cos_table=cos_t, sin_table=sin_t, inverse=True)
    assert np.array_equal(out.cpu().numpy(), want_inv)
    sb.unpack_heads(t, out, cos_table=cos_t, sin_table=sin_t)
    assert np.array_equal(out.cpu().numpy(), want_fwd)
    sb.unpack_heads(t, out)
    assert np.array_equal(out.cpu().numpy(), src)


@pytest.mark.parametrize("B,H,S,D,col0,extra,offset", [(3, 2, 50, 64, 8, 5, 0), (1, 4, 129, 128, 0, 0, 37), (2, 1, 7, 2, 4, 4, 0),
                                                       (1, 2, 300, 16, 16, 0, 0)])
def test_pack_windows_offsets_and_ragged_shapes_vs_oracle(sb, oracle, B, H, S, D, col0, extra, offset):
    """Pack windows (column_start, several packs whose positions restart at 0), a position offset (continued sequence),
    lengths that are not a multiple of the 32-wide tiles, the smallest head size; columns outside the window untouched."""
    rng = np.random.default_rng(B * 1000 + S)
    stride = col0 + B * S + extra
    m = rng.standard_normal((H * D, stride)).astype(np.float32)
    positions = offset + S + 3
    cos_np, sin_np = oracle.rope_tables(D, positions, 1.0e4)
    cos_t, sin_t = torch.from_numpy(cos_np).cuda(), torch.from_numpy(sin_np).cuda()
    got = sb.pack_heads(torch.from_numpy(m).cuda(), B, H, S, D, column_start=col0, cos_table=cos_t, sin_table=sin_t,
                        position_offset=offset)
    window = np.ascontiguousarray(m[:, col0:col0 + B * S])
    rot = oracle.rope_rotate(window, H, D, cos_np, sin_np, position_offset=offset, segment=S if B > 1 else 0)
    want = torch.from_numpy(_fm_to_bhsd(oracle.round_bf16(rot), B, H, S, D, 0)).to(torch.bfloat16)
    assert np.array_equal(_bits(got), _bits(want))
    # and back: inverse rotation of the packed values into a wider matrix
    out = torch.full((H * D, stride), -777.0, device="cuda")
    sb.unpack_heads(got, out, column_start=col0, cos_table=cos_t, sin_table=sin_t, position_offset=offset, inverse=True)
    back = oracle.rope_rotate(np.ascontiguousarray(oracle.round_bf16(rot)), H, D, cos_np, sin_np, position_offset=offset,
                              segment=S if B > 1 else 0, inverse=True)
    o = out.cpu().numpy()
    assert np.array_equal(o[:, col0:col0 + B * S], back)
    assert (o[:, :col0] == -777.0).all() and (o[:, col0 + B * S:] == -777.0).all()
    # the rotation is orthogonal: un-rotating the rotated values returns the input up to the bf16 rounding in between
    assert max_abs(o[:, col0:col0 + B * S], window) <= 2.0 ** -7 * float(np.abs(window).max())


def test_rotary_layer_path_matches_reference_layer(sb):
    """The whole neighbourhood of the hot path as the reference layer runs it (CudaCausalSelfAttention.cu:181-253, :392-509):
    un-rotated fp32 feature-major Q/K/V -> rotate + pack -> attention forward/backward on the tensor cores -> unpack with the
    inverse rotation; against the reference CPU layer with its rotary embedding active."""
    g = load_golden(ROPE_LAYER_GOLDEN)
    B, Hq, S, D = g["q"].shape
    Hkv = g["k"].shape[1]
    from oracle import cpu
    cos_np, sin_np = cpu.rope_tables(D, S, float(g["base"]))
    cos_t, sin_t = torch.from_numpy(cos_np).cuda(), torch.from_numpy(sin_np).cuda()
    fm = lambda x: torch.from_numpy(np.ascontiguousarray(x.transpose(1, 3, 0, 2).reshape(x.shape[1] * D, B * S))).cuda()
    q = sb.pack_heads(fm(g["q"]), B, Hq, S, D, cos_table=cos_t, sin_table=sin_t)
    k = sb.pack_heads(fm(g["k"]), B, Hkv, S, D, cos_table=cos_t, sin_table=sin_t)
    v = sb.pack_heads(fm(g["v"]), B, Hkv, S, D)
    do = sb.pack_heads(fm(g["dout"] * 1e-2), B, Hq, S, D)
    o, lse = sb.attention_forward(q, k, v)
    assert sb.last_path() == "tcgen05"
    dq, dk, dv = sb.attention_backward(q, k, v, o, lse, do)
    mo, mdq = torch.empty(Hq * D, B * S, device="cuda"), torch.empty(Hq * D, B * S, device="cuda")
    mdk, mdv = torch.empty(Hkv * D, B * S, device="cuda"), torch.empty(Hkv * D, B * S, device="cuda")
    sb.unpack_heads(o, mo)
    sb.unpack_heads(dq, mdq, cos_table=cos_t, sin_table=sin_t, inverse=True)
    sb.unpack_heads(dk, mdk, cos_table=cos_t, sin_table=sin_t, inverse=True)
    sb.unpack_heads(dv, mdv)
    for got, H, key, scale in ((mo, Hq, "o", 1.0), (mdq, Hq, "dq", 1e-2), (mdk, Hkv, "dk", 1e-2), (mdv, Hkv, "dv", 1e-2)):
        got_b = _fm_to_bhsd(got.cpu().numpy(), B, H, S, D, 0)
        want = g[key] * scale
        assert max_abs(got_b, want) <= 2e-2, key
        assert rel_l2(got_b, want) <= 1e-2, (key, rel_l2(got_b, want))     # bf16 rounding of the rotated Q/K on top of the kernels' own
    assert sb.poll_device_status() == 0


def test_pack_argument_errors(sb):
    m = torch.zeros(2 * 16, 40, device="cuda")
    cos_t = torch.ones(32, 8, device="cuda")
    with pytest.raises(ValueError):
        sb.pack_heads(m, 1, 2, 40, 16, cos_table=cos_t, sin_table=cos_t)        # sequence longer than the table (RotaryEmbedding.cpp:42)
    with pytest.raises(ValueError):
        sb.pack_heads(m, 2, 2, 30, 16)                                         # pack window exceeds the matrix
    with pytest.raises(ValueError):
        sb.pack_heads(m, 1, 2, 40, 16, cos_table=cos_t)                         # tables come together
