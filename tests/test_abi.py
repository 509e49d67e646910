"""CPU tests of the boundary: the C-ABI library loads, exports every symbol the header declares, validates
arguments like the reference's host code, and the Python/C++ mirrors raise the reference's error kinds.
No compute entry point runs a kernel here (there is no GPU in this suite)."""
import ctypes as C
import os
import re

import pytest

from sentinel_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(_lib.LIB_PATH):
        from sentinel_b200 import build
        build.build()
    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "sntl_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sntl_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_symbols()
    assert set(names) == set(_lib.EXPORTS), "header and loader disagree on the ABI surface"
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/sntl_attn.h but not exported"


def test_version_and_status_strings(lib):
    assert lib.sntl_attn_version() >= 100
    seen = {lib.sntl_status_string(i).decode() for i in range(7)}
    assert len(seen) == 7 and lib.sntl_status_string(99).decode() == "unknown status"


def _desc(**kw):
    base = dict(dtype=_lib.DTYPE_BF16, layout=_lib.LAYOUT_BHSD, batch=2, q_heads=8, kv_heads=2, seq_q=256, seq_kv=256,
                head_dim=128, scale=0.088, causal=1, stride_columns=0, column_start=0, flags=0)
    base.update(kw)
    return _lib.Desc(**base)


def test_workspace_sizes(lib):
    d = _desc()
    assert lib.sntl_attn_fwd_workspace_bytes(C.byref(d)) == 0          # native bf16 needs no forward scratch
    bwd = lib.sntl_attn_bwd_workspace_bytes(C.byref(d))
    assert bwd >= 4 * 2 * 8 * 256                                      # at least delta
    f32 = _desc(dtype=_lib.DTYPE_F32, head_dim=16)
    assert lib.sntl_attn_fwd_workspace_bytes(C.byref(f32)) == 0        # exact fp32 path: no staging
    assert lib.sntl_attn_bwd_workspace_bytes(C.byref(f32)) >= 4 * 2 * 8 * 256
    staged = _desc(dtype=_lib.DTYPE_F32, flags=_lib.FLAG_ALLOW_BF16_COMPUTE)
    assert lib.sntl_attn_fwd_workspace_bytes(C.byref(staged)) >= 2 * (2 * 2 * 8 * 256 * 128)
    assert lib.sntl_attn_bwd_workspace_bytes(C.byref(_desc(batch=0))) == 0


@pytest.mark.parametrize("kw,status", [
    (dict(batch=0), _lib.ERR_BAD_ARGUMENT),
    (dict(q_heads=7), _lib.ERR_BAD_ARGUMENT),                 # not divisible by kv_heads
    (dict(seq_kv=128), _lib.ERR_BAD_ARGUMENT),                # causal needs seq_q == seq_kv
    (dict(scale=0.0), _lib.ERR_BAD_ARGUMENT),
    (dict(dtype=5), _lib.ERR_BAD_ARGUMENT),
    (dict(head_dim=512), _lib.ERR_UNSUPPORTED),
    (dict(layout=_lib.LAYOUT_SENTINEL), _lib.ERR_UNSUPPORTED),            # feature-major is fp32 only
    (dict(layout=_lib.LAYOUT_SENTINEL, dtype=_lib.DTYPE_F32, stride_columns=500, column_start=0), _lib.ERR_BAD_ARGUMENT),  # 2*256 > 500
    (dict(layout=_lib.LAYOUT_SENTINEL, dtype=_lib.DTYPE_F32, stride_columns=600, column_start=-1), _lib.ERR_BAD_ARGUMENT),
])
def test_argument_validation_status_codes(lib, kw, status):
    d = _desc(**kw)
    dummy = C.c_void_p(16)   # never dereferenced: validation fails first
    assert lib.sntl_attn_fwd(C.byref(d), dummy, dummy, dummy, dummy, dummy, None, 0, None) == status
    assert lib.sntl_attn_bwd(C.byref(d), dummy, dummy, dummy, dummy, dummy, dummy, dummy, dummy, dummy, dummy, 1 << 30,
                             None) == status


def test_null_pointers_and_missing_device(lib):
    d = _desc()
    dummy = C.c_void_p(16)
    assert lib.sntl_attn_fwd(C.byref(d), None, dummy, dummy, dummy, dummy, None, 0, None) == _lib.ERR_BAD_ARGUMENT
    assert lib.sntl_attn_fwd(None, dummy, dummy, dummy, dummy, dummy, None, 0, None) == _lib.ERR_BAD_ARGUMENT
    import torch
    if not torch.cuda.is_available():
        # no fallback of any kind: without an sm_100 device the call reports it and does nothing
        assert lib.sntl_attn_fwd(C.byref(d), dummy, dummy, dummy, dummy, dummy, None, 0, None) == _lib.ERR_NO_DEVICE
    assert lib.sntl_attn_merge(0, 0, -1, 64, dummy, dummy, dummy, dummy, None) == _lib.ERR_BAD_ARGUMENT


def test_status_to_exception_mapping():
    with pytest.raises(ValueError):
        _lib.check(_lib.ERR_BAD_ARGUMENT, "x")
    with pytest.raises(ValueError):
        _lib.check(_lib.ERR_UNSUPPORTED, "x")
    with pytest.raises(RuntimeError):
        _lib.check(_lib.ERR_CUDA, "x")
    _lib.check(_lib.OK, "x")


@pytest.mark.parametrize("args,ok", [
    ((64, 64, 96, 4, 16, 0, 48, 2), True),      # two packs of 48 fill the matrix
    ((64, 32, 96, 4, 16, 0, 48, 2), True),      # grouped-query: 2 KV heads
    ((64, 64, 96, 4, 16, 0, 0, 1), True),       # columnCount <= 0 means "to the end"
    ((64, 64, 96, 4, 16, 8, 48, 2), False),     # pack window exceeds columns
    ((64, 64, 96, 4, 16, -1, 48, 1), False),    # invalid column window
    ((64, 64, 96, 3, 16, 0, 48, 1), False),     # rows != headCount*headDim
    ((64, 48, 96, 4, 16, 0, 48, 1), False),     # 3 KV heads do not divide 4
])
def test_compat_class_argument_checks(lib, args, ok):
    """The C++ operator class validates like validateMultiHeadShape/resolveColumnWindow
    (CudaFlashAttention.cu:1458-1471, :1533-1539) and reports std::invalid_argument."""
    err = C.create_string_buffer(256)
    rc = lib.sntl_compat_validate(*args, err, 256)
    assert (rc == 0) == ok, err.value
    if not ok:
        assert err.value.startswith(b"CudaFlashAttention")


def test_python_mirror_raises_reference_error_kinds():
    import torch
    from sentinel_b200 import CudaFlashAttention as FA
    q = torch.zeros(64, 96)
    k = torch.zeros(64, 96)
    with pytest.raises(ValueError, match="query rows mismatch"):
        FA.forwardMultiHead(q, k, k, None, None, 3, 16, 0.25)
    with pytest.raises(ValueError, match="pack window exceeds columns"):
        FA.forwardMultiHead(q, k, k, None, None, 4, 16, 0.25, True, 8, 48, 2)
    with pytest.raises(ValueError, match="invalid column window"):
        FA.forwardMultiHead(q, k, k, None, None, 4, 16, 0.25, True, 90, 48, 1)
    with pytest.raises(ValueError, match="CUDA tensor"):   # host tensors are refused: there is no CPU path
        FA.forwardMultiHead(q, k, k, None, None, 4, 16, 0.25)
    with pytest.raises(ValueError, match="logSumExp shape mismatch"):
        FA.backwardMultiHead(q, k, k, q, torch.zeros(3, 96), q, None, None, None, None, 4, 16, 0.25)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(_lib.LibraryMissing, match="no CPU or PyTorch fallback"):
        _lib.load()


@pytest.mark.parametrize("B,Hq,Hkv,chunks", [(2, 28, 4, None), (2, 28, 4, 1), (2, 28, 4, 2), (2, 28, 4, 3), (3, 4, 2, 4),
                                              (1, 32, 8, None), (8, 12, 12, None), (4, 4, 4, 100)])
def test_host_pipeline_chunks_cover_every_unit_once(B, Hq, Hkv, chunks):
    """The host-buffer call cuts the problem into (batch, KV group) chunks: every unit exactly once, query heads
    matching their KV groups, each chunk contiguous in a [B,H,S,D] tensor."""
    from sentinel_b200.host_pipeline import _chunk_slices
    g = Hq // Hkv
    seen_q, seen_k = set(), set()
    for sb, sq, sk in _chunk_slices(B, Hq, Hkv, chunks):
        bs, qs, ks = range(*sb.indices(B)), range(*sq.indices(Hq)), range(*sk.indices(Hkv))
        assert len(bs) and len(qs) and len(ks)
        assert qs.start == ks.start * g and qs.stop == ks.stop * g
        assert len(bs) == 1 or (len(qs) == Hq and len(ks) == Hkv)      # contiguous: several batch elements only whole
        for b in bs:
            for h in qs:
                assert (b, h) not in seen_q
                seen_q.add((b, h))
            for h in ks:
                assert (b, h) not in seen_k
                seen_k.add((b, h))
    assert len(seen_q) == B * Hq and len(seen_k) == B * Hkv


def test_dropin_smoke_binaries_resolve_their_libraries():
    """The reference's attention layer linked with this library's compat translation unit in place of the reference's
    CudaFlashAttention.cu (oracle/Makefile, target dropin): both executables load, i.e. every symbol the reference's
    call sites need is defined by that translation unit and libsntl_attn.so.  Without a GPU they stop at "no CUDA device"."""
    import subprocess
    from oracle import cpu
    for exe, want in ((cpu.DROPIN_SMOKE, "64"), (cpu.DROPIN_SMOKE_D128, "128")):
        if not os.path.exists(exe):
            pytest.skip("drop-in smokes not built (reference sources absent at build time)")
        r = subprocess.run([exe, "gqa"], capture_output=True, text=True, timeout=120)
        assert f"maxHeadDimension={want}" in r.stdout, (r.stdout, r.stderr)
        assert r.returncode in (0, 4), (r.returncode, r.stdout, r.stderr)


def test_pieces_ring_and_selftest_entry_points_validate_without_a_gpu(lib):
    """The entry points added for the ring schedule and for failure detection refuse bad input before touching a device."""
    d = _desc()
    need = lib.sntl_attn_bwd_pieces_workspace_bytes(C.byref(d))
    assert need >= 4 * 2 * 8 * 256 * 128                                     # at least the fp32 dQ accumulator
    assert lib.sntl_attn_bwd_pieces_workspace_bytes(C.byref(_desc(dtype=_lib.DTYPE_F32))) == 0
    assert lib.sntl_attn_bwd_pieces_workspace_bytes(C.byref(_desc(window_size=64))) == 0
    assert lib.sntl_attn_bwd_pieces_workspace_bytes(C.byref(_desc(flags=_lib.FLAG_DETERMINISTIC))) == 0
    dummy = C.c_void_p(16)
    assert lib.sntl_attn_bwd_begin(C.byref(_desc(dtype=_lib.DTYPE_F32)), dummy, dummy, dummy, dummy, 1 << 30, None) == _lib.ERR_UNSUPPORTED
    assert lib.sntl_attn_bwd_begin(C.byref(d), dummy, dummy, dummy, dummy, 16, None) == _lib.ERR_WORKSPACE
    assert lib.sntl_attn_bwd_block(C.byref(d), dummy, dummy, dummy, dummy, None, dummy, dummy, need, None) == _lib.ERR_BAD_ARGUMENT
    assert lib.sntl_attn_bwd_end(C.byref(d), None, dummy, need, None) == _lib.ERR_BAD_ARGUMENT
    # deterministic flag: the backward scratch doubles its dQ accumulator
    # (kv_heads == q_heads: no key tiles cut by query head, whose partials the default form would add to its scratch)
    plain = lib.sntl_attn_bwd_workspace_bytes(C.byref(_desc(kv_heads=8)))
    det = lib.sntl_attn_bwd_workspace_bytes(C.byref(_desc(kv_heads=8, flags=_lib.FLAG_DETERMINISTIC)))
    assert det - plain == 4 * 2 * 8 * 256 * 128
    # ring: no handle, no work
    assert lib.sntl_ring_unique_id(None) == _lib.ERR_BAD_ARGUMENT
    assert lib.sntl_ring_attn_workspace_bytes(None, C.byref(d)) == 0
    assert lib.sntl_ring_attn_fwd(None, C.byref(d), dummy, dummy, dummy, dummy, dummy, dummy, 1 << 30, None) == _lib.ERR_BAD_ARGUMENT
    assert lib.sntl_ring_comm_create(None, 0, 1, None) == _lib.ERR_BAD_ARGUMENT
    assert lib.sntl_ring_comm_destroy(None) == _lib.OK
    # self-test hook: limits are checked first
    assert lib.sntl_attn_selftest_wait_timeout(0, None) == _lib.ERR_BAD_ARGUMENT
    assert lib.sntl_attn_selftest_wait_timeout(10 ** 6, None) == _lib.ERR_BAD_ARGUMENT
    assert lib.sntl_status_string(_lib.ERR_COMM).decode().startswith("NCCL")


def test_python_mirror_refuses_result_tensors_of_the_wrong_shape_or_dtype(lib, monkeypatch):
    """The kernels write caller-supplied result tensors through raw pointers, so the Python mirror checks them before any
    call.  Host tensors stand in for device tensors here (the device check is switched off); nothing is launched."""
    import torch
    from sentinel_b200 import flash_attention as fa
    monkeypatch.setattr(fa, "_require", lambda t, name: None)
    q = torch.zeros(1, 4, 128, 64, dtype=torch.bfloat16)
    k = torch.zeros(1, 2, 128, 64, dtype=torch.bfloat16)
    lse = torch.zeros(1, 4, 128)
    with pytest.raises(ValueError, match="out must be"):
        fa.attention_forward(q, k, k, out=torch.zeros(1, 4, 64, 64, dtype=torch.bfloat16))
    with pytest.raises(ValueError, match="out must be"):
        fa.attention_forward(q, k, k, out=torch.zeros(1, 4, 128, 64))                     # fp32 where bf16 is written
    with pytest.raises(ValueError, match="lse must be"):
        fa.attention_forward(q, k, k, lse=torch.zeros(1, 4, 127))
    with pytest.raises(ValueError, match="share dtype"):
        fa.attention_backward(q, k, k, q.float(), lse, q)                                  # o in another dtype
    with pytest.raises(ValueError, match="dk must be"):
        fa.attention_backward(q, k, k, q, lse, q, dk=torch.zeros_like(q))                  # query-head shaped dK
    with pytest.raises(ValueError, match="dq must be"):
        fa.attention_backward(q, k, k, q, lse, q, dq=torch.zeros(1, 4, 128, 64))
    with pytest.raises(ValueError, match="o_part must match"):
        fa.merge_partials(q.float(), lse, torch.zeros(1, 4, 64, 64), lse)
    FA = fa.CudaFlashAttention
    m = torch.zeros(64, 96)
    with pytest.raises(ValueError, match="expects fp32"):
        FA.forwardMultiHead(m.bfloat16(), m.bfloat16(), m.bfloat16(), None, None, 4, 16, 0.25)
    with pytest.raises(ValueError, match="out must be"):
        FA.forwardMultiHead(m, m, m, torch.zeros(64, 48), None, 4, 16, 0.25)
    with pytest.raises(ValueError, match="logSumExp must be"):
        FA.forwardMultiHead(m, m, m, None, torch.zeros(2, 96), 4, 16, 0.25)
    with pytest.raises(ValueError, match="keyGradient must be"):
        FA.backwardMultiHead(m, m, m, m, torch.zeros(4, 96), m, None, torch.zeros(32, 96), None, None, 4, 16, 0.25)


def test_header_is_plain_c_and_a_c_program_links_and_calls_the_library(lib, tmp_path):
    """include/sntl_attn.h compiles as C99 and as C++11 without warnings, and a C program linked against the shared library
    (no Python, no torch in between) reaches the entry points that need no GPU."""
    import shutil
    import subprocess
    gcc, gxx = shutil.which("gcc"), shutil.which("g++")
    if gcc is None or gxx is None:
        pytest.skip("no host compiler")
    header = os.path.join(ROOT, "include", "sntl_attn.h")
    for cmd in ([gcc, "-std=c99", "-x", "c"], [gxx, "-std=c++11", "-x", "c++"]):
        r = subprocess.run(cmd + ["-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only", header], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
    src = tmp_path / "caller.c"
    src.write_text(r'''
#include <stdio.h>
#include <string.h>
#include "sntl_attn.h"
int main(void)
{
    sntl_attn_desc d;
    memset(&d, 0, sizeof d);
    d.dtype = SNTL_DTYPE_BF16; d.layout = SNTL_LAYOUT_BHSD; d.batch = 2; d.q_heads = 28; d.kv_heads = 4;
    d.seq_q = d.seq_kv = 8192; d.head_dim = 128; d.scale = 0.088388f; d.causal = 1;
    printf("%d|%s|%zu|%zu\n", sntl_attn_version(), sntl_status_string(SNTL_ERR_UNSUPPORTED),
           sntl_attn_fwd_workspace_bytes(&d), sntl_attn_bwd_workspace_bytes(&d));
    d.head_dim = 0;                       /* an invalid descriptor is refused before anything touches a device */
    return sntl_attn_fwd(&d, 0, 0, 0, 0, 0, 0, 0, 0) == SNTL_ERR_BAD_ARGUMENT ? 0 : 1;
}
''')
    exe = tmp_path / "caller"
    libdir = os.path.dirname(_lib.LIB_PATH)
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
                        "-L", libdir, "-lsntl_attn", f"-Wl,-rpath,{libdir}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, (r.stdout, r.stderr)
    version, text, fwd_bytes, bwd_bytes = r.stdout.strip().split("|")
    assert int(version) == lib.sntl_attn_version()
    assert text == lib.sntl_status_string(_lib.ERR_UNSUPPORTED).decode()
    d = _lib.Desc(_lib.DTYPE_BF16, _lib.LAYOUT_BHSD, 2, 28, 4, 8192, 8192, 128, 0.088388, 1, 0, 0, 0, 0, 0)
    assert int(fwd_bytes) == lib.sntl_attn_fwd_workspace_bytes(C.byref(d))
    assert int(bwd_bytes) == lib.sntl_attn_bwd_workspace_bytes(C.byref(d)) > 0


def test_native_ring_binding_refuses_tensors_it_cannot_hand_to_the_library():
    import torch
    from sentinel_b200.ring import NativeRing
    q = torch.zeros(1, 4, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA tensor"):      # host memory: there is no CPU path
        NativeRing._check(q, q[:, :2], q[:, :2])
