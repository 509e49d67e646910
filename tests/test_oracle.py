"""CPU tests of the checker itself: the fp64 restatement against the reference's frozen outputs (golden
fixtures), against the live reference where it is built, and against the invariants the reference's own
smokes assert (GQA == MHA with repeated K/V, finite differences)."""
import numpy as np
import pytest

from conftest import GOLDEN_CASES, ROPE_GOLDEN_CASES, ROPE_LAYER_GOLDEN, WINDOW_GOLDEN_CASES, load_golden, max_abs


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_oracle_matches_reference_golden(oracle, name):
    g = load_golden(name)
    o, lse = oracle.attn_fwd(g["q"], g["k"], g["v"])
    dq, dk, dv, _ = oracle.attn_bwd(g["q"], g["k"], g["v"], g["dout"])
    # the reference computes in fp32 (blocked GEMM, S-long sums); the oracle in fp64
    assert max_abs(o, g["o"]) < 5e-6
    assert max_abs(lse, g["lse"]) < 5e-6
    assert max_abs(dq, g["dq"]) < 2e-5
    assert max_abs(dk, g["dk"]) < 2e-5
    assert max_abs(dv, g["dv"]) < 2e-5


@pytest.mark.parametrize("name", WINDOW_GOLDEN_CASES)
def test_oracle_sliding_window_matches_reference_golden(oracle, name):
    """Sliding window + global tokens (CausalSelfAttention::allowsKey): the reference layer's frozen outputs."""
    g = load_golden(name)
    kw = dict(window=int(g["window"]), global_tokens=int(g["global_tokens"]))
    o, lse = oracle.attn_fwd(g["q"], g["k"], g["v"], **kw)
    dq, dk, dv, _ = oracle.attn_bwd(g["q"], g["k"], g["v"], g["dout"], **kw)
    assert max_abs(o, g["o"]) < 5e-6
    assert max_abs(lse, g["lse"]) < 5e-6
    assert max_abs(dq, g["dq"]) < 2e-5
    assert max_abs(dk, g["dk"]) < 2e-5
    assert max_abs(dv, g["dv"]) < 2e-5
    # the mask really bites: plain causal attention on the same inputs differs
    o_plain, _ = oracle.attn_fwd(g["q"], g["k"], g["v"])
    assert max_abs(o_plain, g["o"]) > 1e-3


def test_oracle_window_mask_is_allows_key(oracle):
    """With V = one-hot rows, O[i] is the probability vector of query i: it must be zero exactly where the
    reference's allowsKey (CausalSelfAttention.cpp:95-100) says false, and a window >= S is plain causal."""
    S, W, G = 24, 5, 3
    rng = np.random.default_rng(3)
    q = rng.standard_normal((1, 1, S, S), dtype=np.float32)
    k = rng.standard_normal((1, 1, S, S), dtype=np.float32)
    v = np.eye(S, dtype=np.float32)[None, None]
    o, _ = oracle.attn_fwd(q, k, v, window=W, global_tokens=G)
    for i in range(S):
        for j in range(S):
            allowed = j <= i and (j < G or j >= i - W + 1)
            assert (o[0, 0, i, j] > 0) == allowed, (i, j)
    o_wide, _ = oracle.attn_fwd(q, k, v, window=S, global_tokens=0)
    o_plain, _ = oracle.attn_fwd(q, k, v)
    assert np.array_equal(o_wide, o_plain)


@pytest.mark.parametrize("name", ["mha_h4_s48_d16", "win64_g5_h4_s200_d32", "win100_g3_h4_kv1_s300_d64_bf16in"])
def test_oracle_cached_queries_equal_reference_full_sequence_rows(oracle, name):
    """New tokens against a KV cache (Sq < Skv, query i at position Skv - Sq + i, window measured from there) are the
    last rows of full causal attention: the reference CPU layer's frozen outputs pin the offset rule."""
    g = load_golden(name)
    kw = dict(window=int(g["window"]), global_tokens=int(g["global_tokens"])) if "window" in g else {}
    S = g["q"].shape[2]
    for T in (1, 5):
        o, lse = oracle.attn_fwd(g["q"][:, :, S - T:], g["k"], g["v"], **kw)
        assert max_abs(o, g["o"][:, :, S - T:]) < 5e-6
        assert max_abs(lse, g["lse"][:, :, S - T:]) < 5e-6


@pytest.mark.parametrize("name", ROPE_GOLDEN_CASES)
def test_oracle_rotary_embedding_matches_reference_bit_for_bit(oracle, name):
    """Angle tables and both rotations against the frozen outputs of the reference's RotaryEmbedding: exact equality."""
    g = load_golden(name)
    H, D = int(g["heads"]), int(g["head_dim"])
    cos_t, sin_t = oracle.rope_tables(D, g["cos"].shape[0], float(g["base"]))
    assert np.array_equal(cos_t, g["cos"]) and np.array_equal(sin_t, g["sin"])
    assert np.array_equal(oracle.rope_rotate(g["matrix"], H, D, cos_t, sin_t), g["rotated"])
    assert np.array_equal(oracle.rope_rotate(g["matrix"], H, D, cos_t, sin_t, inverse=True), g["inverse_rotated"])
    # packs restart positions; an offset continues a sequence
    cols = g["matrix"].shape[1]
    seg = oracle.rope_rotate(g["matrix"], H, D, cos_t, sin_t, segment=cols // 2)
    assert np.array_equal(seg[:, :cols // 2], g["rotated"][:, :cols // 2])
    assert np.array_equal(seg[:, cols // 2:2 * (cols // 2)],
                          oracle.rope_rotate(np.ascontiguousarray(g["matrix"][:, cols // 2:2 * (cols // 2)]), H, D, cos_t, sin_t))
    off = oracle.rope_rotate(np.ascontiguousarray(g["matrix"][:, 5:]), H, D, cos_t, sin_t, position_offset=5)
    assert np.array_equal(off, g["rotated"][:, 5:])


def test_oracle_composed_with_rotation_matches_reference_layer_with_rope(oracle):
    """rotate -> attention -> inverse-rotate the gradients, restated piecewise, against the reference layer run with its
    rotary embedding active (frozen outputs)."""
    g = load_golden(ROPE_LAYER_GOLDEN)
    B, Hq, S, D = g["q"].shape
    Hkv = g["k"].shape[1]
    cos_t, sin_t = oracle.rope_tables(D, S, float(g["base"]))
    fm = lambda x: np.ascontiguousarray(x[0].transpose(0, 2, 1).reshape(-1, S))
    un = lambda m, H: np.ascontiguousarray(m.reshape(H, D, S).transpose(0, 2, 1))[None]
    qr, kr = un(oracle.rope_rotate(fm(g["q"]), Hq, D, cos_t, sin_t), Hq), un(oracle.rope_rotate(fm(g["k"]), Hkv, D, cos_t, sin_t), Hkv)
    o, _ = oracle.attn_fwd(qr, kr, g["v"])
    dq, dk, dv, _ = oracle.attn_bwd(qr, kr, g["v"], g["dout"])
    dq = un(oracle.rope_rotate(fm(dq), Hq, D, cos_t, sin_t, inverse=True), Hq)
    dk = un(oracle.rope_rotate(fm(dk), Hkv, D, cos_t, sin_t, inverse=True), Hkv)
    assert max_abs(o, g["o"]) < 5e-6 and max_abs(dq, g["dq"]) < 2e-5 and max_abs(dk, g["dk"]) < 2e-5 and max_abs(dv, g["dv"]) < 2e-5


def test_reference_live_matches_golden_and_core_route(oracle):
    """Where the reference CPU path is built: it reproduces its own fixtures bit for bit, and the primitive
    route used for timing is bit-identical to the public layer route."""
    if not oracle.ref_available():
        pytest.skip("oracle/_ref not built (reference sources absent)")
    g = load_golden("mha_h4_s48_d16")
    o, lse, dq, dk, dv = oracle.ref_layer_fwd_bwd(g["q"], g["k"], g["v"], g["dout"])
    for got, key in ((o, "o"), (lse, "lse"), (dq, "dq"), (dk, "dk"), (dv, "dv")):
        assert np.array_equal(got, g[key]), key
    co, cdq, cdk, cdv, secs = oracle.ref_core_fwd_bwd(g["q"], g["k"], g["v"], g["dout"])
    assert np.array_equal(co, o) and np.array_equal(cdq, dq) and np.array_equal(cdk, dk) and np.array_equal(cdv, dv)
    assert secs[0] > 0 and secs[1] > 0


def test_gqa_equals_mha_with_repeated_kv(oracle):
    """The reference's runGqaHostSmokeDemo invariant (CausalSelfAttention.cpp:549-684): GQA == MHA with K/V
    repeated per group, and K/V grads are the sums over the group."""
    rng = np.random.default_rng(7)
    B, Hq, Hkv, S, D = 1, 8, 2, 16, 8
    q = rng.standard_normal((B, Hq, S, D), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, S, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, S, D), dtype=np.float32)
    do = rng.standard_normal((B, Hq, S, D), dtype=np.float32)
    g = Hq // Hkv
    kr, vr = np.repeat(k, g, axis=1), np.repeat(v, g, axis=1)
    o1, l1 = oracle.attn_fwd(q, k, v)
    o2, l2 = oracle.attn_fwd(q, kr, vr)
    assert max_abs(o1, o2) < 1e-6 and max_abs(l1, l2) < 1e-6
    dq1, dk1, dv1, _ = oracle.attn_bwd(q, k, v, do)
    dq2, dk2, dv2, _ = oracle.attn_bwd(q, kr, vr, do)
    assert max_abs(dq1, dq2) < 1e-5
    assert max_abs(dk1, dk2.reshape(B, Hkv, g, S, D).sum(2)) < 1e-5
    assert max_abs(dv1, dv2.reshape(B, Hkv, g, S, D).sum(2)) < 1e-5


def test_backward_finite_difference(oracle):
    """Finite-difference check of dQ, dK, dV as in the reference's sparse-backward smoke
    (CausalSelfAttention.cpp:420-500, eps = 1e-3)."""
    rng = np.random.default_rng(11)
    B, Hq, Hkv, S, D = 1, 2, 1, 12, 8
    q = rng.standard_normal((B, Hq, S, D), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, S, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, S, D), dtype=np.float32)
    do = rng.standard_normal((B, Hq, S, D), dtype=np.float32)
    dq, dk, dv, _ = oracle.attn_bwd(q, k, v, do)

    def loss(q_, k_, v_):
        o, _ = oracle.attn_fwd(q_, k_, v_)
        return float((o.astype(np.float64) * do).sum())

    eps = 1e-3
    for arr, grad, idx in ((q, dq, (0, 1, 7, 3)), (k, dk, (0, 0, 2, 5)), (v, dv, (0, 0, 4, 1))):
        hi, lo = arr.copy(), arr.copy()
        hi[idx] += eps
        lo[idx] -= eps
        args_hi = [hi if a is arr else a for a in (q, k, v)]
        args_lo = [lo if a is arr else a for a in (q, k, v)]
        fd = (loss(*args_hi) - loss(*args_lo)) / (2 * eps)
        assert abs(fd - float(grad[idx])) < 5e-3 * max(1.0, abs(fd))


def test_sampled_rows_and_cols_equal_full(oracle):
    rng = np.random.default_rng(3)
    B, Hq, Hkv, S, D = 2, 4, 2, 70, 16
    q = rng.standard_normal((B, Hq, S, D), dtype=np.float32)
    k = rng.standard_normal((B, Hkv, S, D), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, S, D), dtype=np.float32)
    do = rng.standard_normal((B, Hq, S, D), dtype=np.float32)
    o, lse = oracle.attn_fwd(q, k, v)
    dq, dk, dv, _ = oracle.attn_bwd(q, k, v, do)
    rows = np.array([0, 1, 33, 69])
    orow, lrow, dqrow = oracle.attn_rows(q, k, v, do, 1, 3, rows)
    assert np.array_equal(orow, o[1, 3, rows]) and np.array_equal(lrow, lse[1, 3, rows])
    assert max_abs(dqrow, dq[1, 3, rows]) < 1e-6
    cols = np.array([0, 31, 69])
    dkc, dvc = oracle.attn_cols(q, k, v, do, 1, 1, cols)
    assert max_abs(dkc, dk[1, 1, cols]) < 1e-6 and max_abs(dvc, dv[1, 1, cols]) < 1e-6


def test_noncausal_rectangular_and_empty_rows(oracle):
    """Off-diagonal ring blocks are non-causal with Sq != Skv; LSE merge of two key halves equals the full result."""
    rng = np.random.default_rng(5)
    B, H, Sq, Skv, D = 1, 2, 9, 20, 8
    q = rng.standard_normal((B, H, Sq, D), dtype=np.float32)
    k = rng.standard_normal((B, H, Skv, D), dtype=np.float32)
    v = rng.standard_normal((B, H, Skv, D), dtype=np.float32)
    o, lse = oracle.attn_fwd(q, k, v, causal=False)
    oa, la = oracle.attn_fwd(q, k[:, :, :8], v[:, :, :8], causal=False)
    ob, lb = oracle.attn_fwd(q, k[:, :, 8:], v[:, :, 8:], causal=False)
    m = np.maximum(la, lb)
    wa, wb = np.exp(la - m), np.exp(lb - m)
    merged = (oa * wa[..., None] + ob * wb[..., None]) / (wa + wb)[..., None]
    assert max_abs(merged, o) < 1e-6
    assert max_abs(m + np.log(wa + wb), lse) < 1e-6


def test_bf16_rounding_matches_torch(oracle):
    torch = pytest.importorskip("torch")
    x = np.random.default_rng(1).standard_normal(4096).astype(np.float32) * 3
    want = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(oracle.round_bf16(x), want)
