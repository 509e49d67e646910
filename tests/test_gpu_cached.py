"""GPU tests of the KV-cache forward (new tokens against cached keys; the reference's attendCachedQuery / decode,
CudaCausalSelfAttention.cu:318-341, :557-571).  The reference has no CPU twin of its cache path; what pins it is
that a cached query equals the matching row of full causal attention, so the checks are the reference CPU layer's
frozen full-sequence outputs (tests/golden) and the fp64 oracle, whose key-offset rule is pinned to the same fixtures."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import load_golden, max_abs, rel_l2

pytestmark = pytest.mark.gpu

F32_TOL = 1e-4
BF16_ABS, BF16_REL = 2e-2, 5e-3


@pytest.fixture(scope="module")
def sb():
    import sentinel_b200
    sentinel_b200._lib.load()
    assert torch.cuda.is_available()
    return sentinel_b200


def _np(t):
    return t.detach().to(torch.float32).cpu().numpy()


def _cache(x, capacity, dtype):
    """[B,H,S,D] numpy -> device cache [B,H,capacity,D]; rows past S hold NaN (they must never be read)."""
    B, H, S, D = x.shape
    c = torch.full((B, H, capacity, D), float("nan"), dtype=dtype, device="cuda")
    c[:, :, :S] = torch.from_numpy(x).to("cuda").to(dtype)
    return c


@pytest.mark.parametrize("name", ["mha_h4_s48_d16", "gqa_h8_kv2_s16_d8", "win64_g5_h4_s200_d32", "win17_g0_h4_kv2_s96_d16"])
@pytest.mark.parametrize("T", [1, 5])
def test_exact_cached_forward_matches_reference_rows(sb, name, T):
    g = load_golden(name)
    kw = dict(window=int(g["window"]), global_tokens=int(g["global_tokens"])) if "window" in g else {}
    S = g["q"].shape[2]
    q = torch.from_numpy(np.ascontiguousarray(g["q"][:, :, S - T:])).cuda()
    kc, vc = _cache(g["k"], S + 13, torch.float32), _cache(g["v"], S + 13, torch.float32)
    o, lse = sb.attention_cached_forward(q, kc, vc, S, **kw)
    assert sb.last_path() == "simt_f32"
    assert max_abs(_np(o), g["o"][:, :, S - T:]) <= F32_TOL
    assert max_abs(_np(lse), g["lse"][:, :, S - T:]) <= F32_TOL
    # an earlier state of the same cache: only the first L keys in use
    L = S // 2
    q = torch.from_numpy(np.ascontiguousarray(g["q"][:, :, L - T:L])).cuda()
    o, lse = sb.attention_cached_forward(q, kc, vc, L, **kw)
    # rows L-T..L-1 of full causal attention never look past key L-1, so the full-sequence fixture still applies
    assert max_abs(_np(o), g["o"][:, :, L - T:L]) <= F32_TOL
    assert max_abs(_np(lse), g["lse"][:, :, L - T:L]) <= F32_TOL


def test_exact_cached_forward_reference_matrix_layout(sb):
    """The reference's own shapes: query (Hq*D) x 1, caches (Hkv*D) x maximumPositionCount feature-major (CudaKvCache)."""
    lib = sb._lib.load()
    g = load_golden("gqa_h8_kv2_s16_d8")
    _, Hq, S, D = g["q"].shape
    Hkv, cap = g["k"].shape[1], 32
    fm = lambda x, cols: np.ascontiguousarray(np.pad(x[0].transpose(0, 2, 1).reshape(-1, x.shape[2]), ((0, 0), (0, cols - x.shape[2])),
                                                     constant_values=np.nan).astype(np.float32))
    for L in (S, 7, 1):
        q = torch.from_numpy(fm(g["q"][:, :, L - 1:L], 1)).cuda()
        kc, vc = torch.from_numpy(fm(g["k"], cap)).cuda(), torch.from_numpy(fm(g["v"], cap)).cuda()
        o = torch.empty_like(q)
        lse = torch.empty(Hq, 1, device="cuda")
        d = sb._lib.Desc(sb._lib.DTYPE_F32, sb._lib.LAYOUT_SENTINEL, 1, Hq, Hkv, 1, L, D, D ** -0.5, 1, 1, 0, 0, 0, 0)
        rc = lib.sntl_attn_cached_fwd(C.byref(d), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), cap, o.data_ptr(), lse.data_ptr(),
                                      None, 0, None)
        assert rc == 0
        torch.cuda.synchronize()
        want_o = g["o"][0, :, L - 1].reshape(-1)            # row h*D + d
        assert max_abs(_np(o).reshape(-1), want_o) <= F32_TOL
        assert max_abs(_np(lse).reshape(-1), g["lse"][0, :, L - 1]) <= F32_TOL


@pytest.mark.parametrize("wname,B,Hq,Hkv,L,T,window,global_tokens", [
    ("gqa7b_d128", 2, 28, 4, 8192, 1, 0, 0),        # the headline shape decoding its 8192nd token
    ("gqa7b_d128", 2, 28, 4, 8191, 1, 0, 0),        # ragged cache length
    ("gqa7b_d128", 1, 28, 4, 5000, 4, 0, 0),        # four new tokens (28 rows per KV head)
    ("gqa7b_d128", 1, 14, 2, 3000, 40, 0, 0),       # 280 rows per KV head: two query blocks
    ("gqa7b_d128", 2, 28, 4, 8192, 1, 1024, 64),    # sliding window + global tokens
    ("gqa7b_d128", 1, 8, 2, 2500, 3, 300, 200),     # global tokens spill into a second tile
    ("llama1b_gqa", 4, 32, 8, 4096, 1, 0, 0),
    ("llama1b_gqa", 1, 32, 8, 100, 2, 0, 0),        # cache shorter than one tile
    ("gpt2_small", 2, 12, 12, 1024, 1, 0, 0),       # no grouping: one row per KV head
])
def test_bf16_cached_forward_vs_oracle(sb, oracle, wname, B, Hq, Hkv, L, T, window, global_tokens):
    w = sb.WORKLOADS[wname]
    q, k, v, _ = sb.make_inputs(w, batch=B, q_heads=Hq, kv_heads=Hkv, seq=L)
    qn = q[:, :, L - T:].contiguous()
    kw = dict(window=window, global_tokens=global_tokens)
    wo, wl = oracle.attn_fwd(qn.float().numpy(), k.float().numpy(), v.float().numpy(), **kw)
    kc, vc = _cache(k.float().numpy(), L + 77, torch.bfloat16), _cache(v.float().numpy(), L + 77, torch.bfloat16)
    o, lse = sb.attention_cached_forward(qn.cuda(), kc, vc, L, **kw)
    assert sb.last_path() == "tcgen05_cache", sb.last_path()
    assert sb.poll_device_status() == 0
    got = _np(o)
    assert np.isfinite(got).all()
    assert max_abs(got, wo) <= BF16_ABS and rel_l2(got, wo) <= BF16_REL, (max_abs(got, wo), rel_l2(got, wo))
    assert max_abs(_np(lse), wl) <= 1e-3
    # the exact kernel on the same cache
    o32, lse32 = sb.attention_cached_forward(qn.cuda().float(), kc.float(), vc.float(), L, **kw)
    assert sb.last_path() == "simt_f32"
    assert max_abs(_np(o32), wo) <= F32_TOL and max_abs(_np(lse32), wl) <= F32_TOL


def test_cached_forward_equals_rows_of_full_attention(sb):
    """Decoding token L-1 from a cache is row L-1 of causal attention over the first L tokens."""
    w = sb.WORKLOADS["gqa7b_d128"]
    L = 2048
    q, k, v, _ = (t.cuda() for t in sb.make_inputs(w, batch=1, q_heads=28, kv_heads=4, seq=L))
    o_full, lse_full = sb.attention_forward(q, k, v)
    for T in (1, 9):
        o, lse = sb.attention_cached_forward(q[:, :, L - T:].contiguous(), k, v, L)
        assert float((o.float() - o_full[:, :, L - T:].float()).abs().max()) <= 4e-3
        assert float((lse - lse_full[:, :, L - T:]).abs().max()) <= 1e-4


def test_cached_forward_argument_errors(sb):
    q = torch.zeros(1, 4, 1, 64, dtype=torch.bfloat16, device="cuda")
    kc = torch.zeros(1, 2, 256, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        sb.attention_cached_forward(q, kc, kc, 257)        # more keys in use than the cache holds
    with pytest.raises(ValueError):
        sb.attention_cached_forward(q, kc, kc, 0)          # an empty cache has no key for the new token
    q5 = torch.zeros(1, 4, 5, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        sb.attention_cached_forward(q5, kc, kc, 3)         # more new tokens than cached keys
