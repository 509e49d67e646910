"""ctypes bindings for the two CPU checkers (TEST INFRASTRUCTURE, never on the product path).

* ``liboracle_attn.so``  -- fp64 restatement of the reference algorithm (``attn_oracle.c``).
* ``_ref/libsentinel_ref_attn.so`` -- the reference project's own CPU attention compiled from its
  sources (``ref_harness.cpp`` + ``Makefile``); present only where it was built.

Only tests, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py`` may
import this module.  All tensors are numpy fp32, token-major ``[B, H, S, D]``.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "liboracle_attn.so")
_REF_SO = os.path.join(_HERE, "_ref", "libsentinel_ref_attn.so")


class _Shape(C.Structure):
    _fields_ = [("batch", C.c_int), ("q_heads", C.c_int), ("kv_heads", C.c_int), ("seq_q", C.c_int),
                ("seq_kv", C.c_int), ("head_dim", C.c_int), ("causal", C.c_int), ("scale", C.c_float),
                ("window", C.c_int), ("global_tokens", C.c_int)]


def build(force: bool = False, everything: bool = False) -> None:
    """Compile the checkers (make); the reference builds are skipped when its sources are absent.

    ``everything`` also runs the targets that depend on the product library (the drop-in smokes), whatever the age
    of the fp64 checker."""
    if force or everything or not os.path.exists(_ORACLE_SO) or \
            os.path.getmtime(_ORACLE_SO) < os.path.getmtime(os.path.join(_HERE, "attn_oracle.c")):
        subprocess.run(["make", "-C", _HERE, "-B"] if force else ["make", "-C", _HERE], check=True,
                       stdout=subprocess.DEVNULL)


DROPIN_SMOKE = os.path.join(_HERE, "_ref", "dropin_smoke")
DROPIN_SMOKE_D128 = os.path.join(_HERE, "_ref", "dropin_smoke_d128")
DROPIN_SMOKE_REFERENCE = os.path.join(_HERE, "_ref", "dropin_smoke_reference")


_oracle = None
_ref = None


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None


def _ip(a):
    return a.ctypes.data_as(C.POINTER(C.c_int)) if a is not None else None


def oracle_lib():
    global _oracle
    if _oracle is None:
        if not os.path.exists(_ORACLE_SO):
            build()
        _oracle = C.CDLL(_ORACLE_SO)
    return _oracle


def ref_available() -> bool:
    return os.path.exists(_REF_SO)


def ref_lib():
    global _ref
    if _ref is None:
        if not ref_available():
            raise FileNotFoundError(f"{_REF_SO} not built (reference sources absent at build time)")
        _ref = C.CDLL(_REF_SO)
        _ref.ref_threads.restype = C.c_int
    return _ref


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _shape(q, k, causal, scale, window=0, global_tokens=0):
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    return _Shape(B, Hq, Hkv, Sq, Skv, D, int(bool(causal)), float(scale), int(window), int(global_tokens))


def attn_fwd(q, k, v, causal=True, scale=None, window=0, global_tokens=0):
    """fp64 oracle forward -> (O [B,Hq,Sq,D], LSE [B,Hq,Sq]) as fp32 arrays."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    s = _shape(q, k, causal, scale, window, global_tokens)
    o = np.empty_like(q)
    lse = np.empty(q.shape[:3], np.float32)
    rc = oracle_lib().oracle_attn_fwd(C.byref(s), _fp(q), _fp(k), _fp(v), _fp(o), _fp(lse))
    assert rc == 0, rc
    return o, lse


def attn_bwd(q, k, v, dout, causal=True, scale=None, window=0, global_tokens=0):
    """fp64 oracle backward -> (dQ, dK, dV, delta)."""
    q, k, v, dout = _f32(q), _f32(k), _f32(v), _f32(dout)
    s = _shape(q, k, causal, scale, window, global_tokens)
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    delta = np.empty(q.shape[:3], np.float32)
    rc = oracle_lib().oracle_attn_bwd(C.byref(s), _fp(q), _fp(k), _fp(v), _fp(dout), _fp(dq), _fp(dk), _fp(dv),
                                      _fp(delta))
    assert rc == 0, rc
    return dq, dk, dv, delta


def attn_rows(q, k, v, dout, b, h, rows, causal=True, scale=None, window=0, global_tokens=0):
    """Sampled oracle: (O rows, LSE rows, dQ rows) for query indices ``rows`` of (b, h)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    dout = _f32(dout) if dout is not None else None
    s = _shape(q, k, causal, scale, window, global_tokens)
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    D = q.shape[-1]
    o = np.empty((len(rows), D), np.float32)
    lse = np.empty((len(rows),), np.float32)
    dq = np.empty((len(rows), D), np.float32) if dout is not None else None
    rc = oracle_lib().oracle_attn_rows(C.byref(s), int(b), int(h), _fp(q), _fp(k), _fp(v), _fp(dout), _ip(rows),
                                       len(rows), _fp(o), _fp(lse), _fp(dq))
    assert rc == 0, rc
    return o, lse, dq


def attn_cols(q, k, v, dout, b, hk, cols, causal=True, scale=None, window=0, global_tokens=0):
    """Sampled oracle: (dK rows, dV rows) for key indices ``cols`` of (b, kv head hk)."""
    q, k, v, dout = _f32(q), _f32(k), _f32(v), _f32(dout)
    s = _shape(q, k, causal, scale, window, global_tokens)
    cols = np.ascontiguousarray(cols, dtype=np.int32)
    D = q.shape[-1]
    dk = np.empty((len(cols), D), np.float32)
    dv = np.empty((len(cols), D), np.float32)
    rc = oracle_lib().oracle_attn_cols(C.byref(s), int(b), int(hk), _fp(q), _fp(k), _fp(v), _fp(dout), _ip(cols),
                                       len(cols), _fp(dk), _fp(dv))
    assert rc == 0, rc
    return dk, dv


def round_bf16(x):
    """fp32 -> bf16 (round to nearest even) -> fp32, done in C so it does not depend on torch."""
    y = _f32(x).copy()
    oracle_lib().oracle_round_bf16(_fp(y), C.c_size_t(y.size))
    return y


def rope_tables(head_dim, positions, base=10000.0):
    """cos/sin tables [positions][head_dim/2] as RotaryEmbedding.cpp:19-27 builds them (fp32 pow/cos/sin)."""
    cos_t = np.empty((positions, head_dim // 2), np.float32)
    sin_t = np.empty_like(cos_t)
    oracle_lib().oracle_rope_tables(int(head_dim), int(positions), C.c_float(base), _fp(cos_t), _fp(sin_t))
    return cos_t, sin_t


def rope_rotate(matrix, heads, head_dim, cos_t, sin_t, position_offset=0, segment=0, inverse=False):
    """Rotates a feature-major (heads*head_dim) x cols fp32 matrix; returns a new array."""
    m = _f32(matrix).copy()
    assert m.shape[0] == heads * head_dim
    oracle_lib().oracle_rope_rotate(_fp(m), int(heads), int(head_dim), int(m.shape[1]), _fp(_f32(cos_t)), _fp(_f32(sin_t)),
                                    int(position_offset), int(segment), int(bool(inverse)))
    return m


def ref_rope(matrix, heads, head_dim, positions, base=10000.0, inverse=False):
    """The reference's RotaryEmbedding::rotateInPlace / rotateInverseInPlace -> (rotated matrix, cos table, sin table)."""
    m = _f32(matrix).copy()
    cos_t = np.empty((positions, head_dim // 2), np.float32)
    sin_t = np.empty_like(cos_t)
    rc = ref_lib().ref_rope(int(head_dim), int(positions), C.c_float(base), int(heads), int(m.shape[1]), _fp(m),
                            int(bool(inverse)), _fp(cos_t), _fp(sin_t))
    assert rc == 0, "reference RotaryEmbedding threw"
    return m, cos_t, sin_t


def ref_layer_fwd_bwd_rope(q, k, v, dout, rope_base=10000.0, window=0, global_tokens=0):
    """The reference layer with its own rotary embedding active: q, k are un-rotated; returns (O, dQ, dK, dV) with the
    gradients taken with respect to the un-rotated inputs."""
    q, k, v, dout = _f32(q), _f32(k), _f32(v), _f32(dout)
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    o, dq, dk, dv = np.empty_like(q), np.empty_like(q), np.empty_like(k), np.empty_like(v)
    rc = ref_lib().ref_layer_fwd_bwd_rope(B, Hq, Hkv, S, D, C.c_float(rope_base), int(window), int(global_tokens), _fp(q),
                                          _fp(k), _fp(v), _fp(dout), _fp(o), _fp(dq), _fp(dk), _fp(dv))
    assert rc == 0, "reference layer threw"
    return o, dq, dk, dv


def oracle_threads() -> int:
    lib = oracle_lib()
    lib.oracle_threads.restype = C.c_int
    return lib.oracle_threads()


def ref_layer_fwd_bwd(q, k, v, dout=None, window=0, global_tokens=0):
    """The reference's public CausalSelfAttention layer on [Q;K;V] -> (O, LSE, dQ, dK, dV) (grads None without dout).

    Causal, Sq == Skv, scale 1/sqrt(D): the only mode the reference layer has; ``window`` / ``global_tokens`` are its
    windowSize / globalTokenCount constructor arguments (0 = whole sequence)."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    o = np.empty_like(q)
    lse = np.empty((B, Hq, S), np.float32)
    dq = dk = dv = None
    if dout is not None:
        dout = _f32(dout)
        dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    rc = ref_lib().ref_layer_fwd_bwd_windowed(B, Hq, Hkv, S, D, int(window), int(global_tokens), _fp(q), _fp(k), _fp(v),
                                              _fp(dout), _fp(o), _fp(lse), _fp(dq), _fp(dk), _fp(dv))
    assert rc == 0, "reference layer threw"
    return o, lse, dq, dk, dv


def ref_core_fwd_bwd(q, k, v, dout=None, head_limit=0, want_outputs=True):
    """The reference's primitives (Matrix::gemm, Softmax::applyInto) in the layer's dense order, attention core only.

    Returns (O, dQ, dK, dV, (fwd_seconds, bwd_seconds))."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    o = np.zeros_like(q) if want_outputs else None
    dq = dk = dv = None
    if dout is not None:
        dout = _f32(dout)
        if want_outputs:
            dq, dk, dv = np.zeros_like(q), np.zeros_like(k), np.zeros_like(v)
    secs = (C.c_double * 2)()
    rc = ref_lib().ref_core_fwd_bwd(B, Hq, Hkv, S, D, int(head_limit), _fp(q), _fp(k), _fp(v), _fp(dout), _fp(o),
                                    _fp(dq), _fp(dk), _fp(dv), secs)
    assert rc == 0, "reference primitives threw"
    return o, dq, dk, dv, (secs[0], secs[1])


def ref_threads() -> int:
    return ref_lib().ref_threads()


# ---------------------------------------------------------------------------------------------------------------
# The reference's own CUDA flash kernels (GPU baseline / second parity subject), built into _ref/ by the Makefile
# ---------------------------------------------------------------------------------------------------------------
_REF_CUDA_SO = os.path.join(_HERE, "_ref", "libsentinel_ref_cuda.so")
_ref_cuda = None


def ref_cuda_available() -> bool:
    return os.path.exists(_REF_CUDA_SO)


def ref_cuda_flash(q, k, v, dout=None, reps=0):
    """Runs the reference CUDA flash attention (its forwardMultiHead/backwardMultiHead) on [B,H,S,D] fp32 arrays.

    Grouped-query inputs are expanded to the query head count first (the reference's call site does the same with
    expandKvHeadsInto) and the expanded dK/dV are summed back per group.  head_dim <= 64 only (its maxHeadDimension).
    Returns (O, LSE, dQ, dK, dV, (fwd_ms, bwd_ms))."""
    global _ref_cuda
    if _ref_cuda is None:
        _ref_cuda = C.CDLL(_REF_CUDA_SO)
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    ke, ve = np.repeat(k, g, axis=1), np.repeat(v, g, axis=1)

    def fm(x):   # [B,H,S,D] -> (H*D) x (B*S), sequences side by side
        return np.ascontiguousarray(x.transpose(1, 3, 0, 2).reshape(x.shape[1] * D, B * S))

    def unfm(m, H):
        return np.ascontiguousarray(m.reshape(H, D, B, S).transpose(2, 0, 3, 1))

    cols = B * S
    out = np.empty((Hq * D, cols), np.float32)
    lse = np.empty((Hq, cols), np.float32)
    have_grad = dout is not None
    dq = np.empty_like(out) if have_grad else None
    dk = np.empty_like(out) if have_grad else None
    dv = np.empty_like(out) if have_grad else None
    ms = (C.c_float * 2)()
    err = C.create_string_buffer(256)
    rc = _ref_cuda.ref_cuda_flash_fwd_bwd(Hq, D, cols, S, B, _fp(fm(q)), _fp(fm(ke)), _fp(fm(ve)),
                                          _fp(fm(_f32(dout))) if have_grad else None, _fp(out), _fp(lse), _fp(dq), _fp(dk),
                                          _fp(dv), int(reps), ms, err, 256)
    if rc != 0:
        raise RuntimeError("reference CUDA flash attention threw: " + err.value.decode())
    o = unfm(out, Hq)
    lse_b = np.ascontiguousarray(lse.reshape(Hq, B, S).transpose(1, 0, 2))
    if not have_grad:
        return o, lse_b, None, None, None, (ms[0], ms[1])
    dq_b = unfm(dq, Hq)
    dk_b = unfm(dk, Hq).reshape(B, Hkv, g, S, D).sum(2)
    dv_b = unfm(dv, Hq).reshape(B, Hkv, g, S, D).sum(2)
    return o, lse_b, dq_b, dk_b, dv_b, (ms[0], ms[1])
