"""Python host side of the attention path: ctypes calls into the C ABI on torch-owned device memory.

Two levels:

* ``attention_forward`` / ``attention_backward`` -- the native interface: bf16 (or fp32) token-major
  ``[B, H, S, D]`` CUDA tensors, grouped-query heads native.
* ``CudaFlashAttention`` -- the reference's operator interface (same method names, argument order, defaults
  and error behaviour as ``sentinel/NeuralNet/Cuda/CudaFlashAttention.hpp:10-41``) on fp32 feature-major
  ``(H*D) x strideColumns`` CUDA tensors, so the reference's parity procedures can be replayed against it.

Nothing here computes attention: every result comes from ``lib/libsntl_attn.so``.  torch supplies memory and
the current stream.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_ws_cache: dict = {}


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _workspace(nbytes: int, device) -> torch.Tensor | None:
    """Grow-only scratch per (device, stream) (the reference grows its buffers the same way, CudaMatmul.cu:119-136).
    Calls on different streams may overlap on the GPU, so each stream gets scratch of its own."""
    if nbytes == 0:
        return None
    key = (device.type, device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _ws_cache.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
        _ws_cache[key] = buf
    return buf


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.DTYPE_BF16
    if t.dtype == torch.float32:
        return _lib.DTYPE_F32
    raise ValueError(f"unsupported dtype {t.dtype}: bf16 or fp32 expected")


def _require(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _check_out(t: torch.Tensor, shape, dtype, like: torch.Tensor, name: str) -> torch.Tensor:
    """A caller-supplied result tensor is written by the kernels through its raw pointer: it must be exactly what the
    call would have allocated itself."""
    _require(t, name)
    if tuple(t.shape) != tuple(shape) or t.dtype != dtype or t.device != like.device:
        raise ValueError(f"{name} must be a {dtype} tensor of shape {tuple(shape)} on {like.device}")
    return t


def _same_device(ref: torch.Tensor, *named) -> None:
    for t, n in named:
        if t.device != ref.device:
            raise ValueError(f"{n} is on {t.device}, q on {ref.device}")


def _bhsd_desc(q, k, causal, scale, flags, window=0, global_tokens=0) -> _lib.Desc:
    if q.dim() != 4 or k.dim() != 4:
        raise ValueError("expected [B, H, S, D] tensors")
    B, Hq, Sq, D = q.shape
    Bk, Hkv, Skv, Dk = k.shape
    if Bk != B or Dk != D:
        raise ValueError("q and k disagree on batch or head_dim")
    if scale is None:
        scale = D ** -0.5
    return _lib.Desc(_dtype_code(q), _lib.LAYOUT_BHSD, B, Hq, Hkv, Sq, Skv, D, float(scale), int(bool(causal)), 0, 0,
                     int(flags), int(window), int(global_tokens))


def attention_forward(q, k, v, *, causal=True, scale=None, flags=0, out=None, lse=None, window=0, global_tokens=0):
    """O, LSE = attention(Q, K, V).  q: [B,Hq,Sq,D]; k, v: [B,Hkv,Skv,D]; LSE: [B,Hq,Sq] fp32 (natural log).

    ``window`` / ``global_tokens``: the reference layer's sliding window and always-visible first keys
    (CausalSelfAttention.cpp:95-100); key j is visible to query i iff j <= i and (j < global_tokens or window <= 0 or
    j >= i - window + 1)."""
    lib = _lib.load()
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _require(t, n)
    if k.shape != v.shape or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("k and v must share shape; q, k, v must share dtype")
    _same_device(q, (k, "k"), (v, "v"))
    d = _bhsd_desc(q, k, causal, scale, flags, window, global_tokens)
    o = torch.empty_like(q) if out is None else _check_out(out, q.shape, q.dtype, q, "out")
    lse = (torch.empty(q.shape[:3], dtype=torch.float32, device=q.device) if lse is None
           else _check_out(lse, q.shape[:3], torch.float32, q, "lse"))
    nbytes = lib.sntl_attn_fwd_workspace_bytes(C.byref(d))
    ws = _workspace(nbytes, q.device)
    rc = lib.sntl_attn_fwd(C.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                           ws.data_ptr() if ws is not None else None, nbytes, _stream_ptr())
    _lib.check(rc, "sntl_attn_fwd")
    return o, lse


def attention_cached_forward(q, k_cache, v_cache, cache_length, *, scale=None, flags=0, out=None, lse=None, window=0,
                             global_tokens=0):
    """New tokens against a KV cache (the reference's attendCachedQuery / decode, CudaCausalSelfAttention.cu:318-341).

    q: [B,Hq,T,D], the T newest tokens; k_cache, v_cache: [B,Hkv,capacity,D] with the first ``cache_length`` rows in use,
    the new tokens' keys already appended at the end.  Query i sits at position cache_length - T + i.  Returns
    (O [B,Hq,T,D], LSE [B,Hq,T])."""
    lib = _lib.load()
    for t, n in ((q, "q"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        _require(t, n)
    if k_cache.shape != v_cache.shape or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise ValueError("k_cache and v_cache must share shape; q and the caches must share dtype")
    if q.dim() != 4 or k_cache.dim() != 4 or k_cache.shape[0] != q.shape[0] or k_cache.shape[3] != q.shape[3]:
        raise ValueError("expected q [B,Hq,T,D] and caches [B,Hkv,capacity,D]")
    B, Hq, T, D = q.shape
    Hkv, capacity = k_cache.shape[1], k_cache.shape[2]
    if scale is None:
        scale = D ** -0.5
    d = _lib.Desc(_dtype_code(q), _lib.LAYOUT_BHSD, B, Hq, Hkv, T, int(cache_length), D, float(scale), 1, 0, 0, int(flags),
                  int(window), int(global_tokens))
    _same_device(q, (k_cache, "k_cache"), (v_cache, "v_cache"))
    o = torch.empty_like(q) if out is None else _check_out(out, q.shape, q.dtype, q, "out")
    lse = (torch.empty(q.shape[:3], dtype=torch.float32, device=q.device) if lse is None
           else _check_out(lse, q.shape[:3], torch.float32, q, "lse"))
    nbytes = lib.sntl_attn_cached_fwd_workspace_bytes(C.byref(d), capacity)
    ws = _workspace(nbytes, q.device)
    rc = lib.sntl_attn_cached_fwd(C.byref(d), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), capacity, o.data_ptr(),
                                  lse.data_ptr(), ws.data_ptr() if ws is not None else None, nbytes, _stream_ptr())
    _lib.check(rc, "sntl_attn_cached_fwd")
    return o, lse


def _tables(cos_table, sin_table, head_dim, device):
    if (cos_table is None) != (sin_table is None):
        raise ValueError("cos_table and sin_table come together")
    if cos_table is None:
        return None, None, 0
    for t, n in ((cos_table, "cos_table"), (sin_table, "sin_table")):
        _require(t, n)
        if t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != head_dim // 2:
            raise ValueError(f"{n} must be fp32 [positions, head_dim/2]")
    if cos_table.shape != sin_table.shape:
        raise ValueError("cos_table and sin_table must share shape")
    return cos_table.data_ptr(), sin_table.data_ptr(), cos_table.shape[0]


def pack_heads(matrix, batch, heads, seq, head_dim, *, column_start=0, cos_table=None, sin_table=None, position_offset=0,
               out=None):
    """fp32 feature-major ``(heads*head_dim) x stride`` matrix -> bf16 ``[batch, heads, seq, head_dim]``, rotated by the
    angle tables on the way (``None``: no rotation).  One kernel in place of the reference's rotaryRotateInPlace
    (CudaOps.cu:362-381) plus a relayout and a cast."""
    lib = _lib.load()
    _require(matrix, "matrix")
    if matrix.dtype != torch.float32 or matrix.dim() != 2 or matrix.shape[0] != heads * head_dim:
        raise ValueError("matrix must be fp32 (heads*head_dim) x stride")
    cp, sp, positions = _tables(cos_table, sin_table, head_dim, matrix.device)
    dst = (torch.empty(batch, heads, seq, head_dim, dtype=torch.bfloat16, device=matrix.device) if out is None
           else _check_out(out, (batch, heads, seq, head_dim), torch.bfloat16, matrix, "out"))
    rc = lib.sntl_attn_pack_heads(matrix.data_ptr(), dst.data_ptr(), batch, heads, seq, head_dim, matrix.shape[1], column_start,
                                  cp, sp, position_offset, positions, _stream_ptr())
    _lib.check(rc, "sntl_attn_pack_heads")
    return dst


def unpack_heads(tensor, matrix, *, column_start=0, cos_table=None, sin_table=None, position_offset=0, inverse=False):
    """bf16 ``[batch, heads, seq, head_dim]`` -> columns of an fp32 feature-major matrix (written in place), with the
    forward or (``inverse=True``, for dQ and dK) inverse rotation on the way."""
    lib = _lib.load()
    _require(tensor, "tensor")
    _require(matrix, "matrix")
    if tensor.dtype != torch.bfloat16 or tensor.dim() != 4:
        raise ValueError("tensor must be bf16 [batch, heads, seq, head_dim]")
    batch, heads, seq, head_dim = tensor.shape
    if matrix.dtype != torch.float32 or matrix.dim() != 2 or matrix.shape[0] != heads * head_dim:
        raise ValueError("matrix must be fp32 (heads*head_dim) x stride")
    cp, sp, positions = _tables(cos_table, sin_table, head_dim, tensor.device)
    rc = lib.sntl_attn_unpack_heads(tensor.data_ptr(), matrix.data_ptr(), batch, heads, seq, head_dim, matrix.shape[1],
                                    column_start, cp, sp, position_offset, positions, int(bool(inverse)), _stream_ptr())
    _lib.check(rc, "sntl_attn_unpack_heads")
    return matrix


def attention_backward(q, k, v, o, lse, dout, *, causal=True, scale=None, flags=0, dq=None, dk=None, dv=None, window=0,
                       global_tokens=0):
    """dQ, dK, dV from dO (P recomputed from LSE).  Shapes as in attention_forward."""
    lib = _lib.load()
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (o, "o"), (lse, "lse"), (dout, "dout")):
        _require(t, n)
    if o.shape != q.shape or dout.shape != q.shape or lse.shape != q.shape[:3] or lse.dtype != torch.float32:
        raise ValueError("o/dout must match q; lse must be fp32 [B,Hq,Sq]")
    if k.shape != v.shape or any(t.dtype != q.dtype for t in (k, v, o, dout)):
        raise ValueError("k and v must share shape; q, k, v, o, dout must share dtype")
    _same_device(q, (k, "k"), (v, "v"), (o, "o"), (lse, "lse"), (dout, "dout"))
    d = _bhsd_desc(q, k, causal, scale, flags, window, global_tokens)
    dq = torch.empty_like(q) if dq is None else _check_out(dq, q.shape, q.dtype, q, "dq")
    dk = torch.empty_like(k) if dk is None else _check_out(dk, k.shape, k.dtype, q, "dk")
    dv = torch.empty_like(v) if dv is None else _check_out(dv, v.shape, v.dtype, q, "dv")
    nbytes = lib.sntl_attn_bwd_workspace_bytes(C.byref(d))
    ws = _workspace(nbytes, q.device)
    rc = lib.sntl_attn_bwd(C.byref(d), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                           dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                           ws.data_ptr() if ws is not None else None, nbytes, _stream_ptr())
    _lib.check(rc, "sntl_attn_bwd")
    return dq, dk, dv


class BackwardPieces:
    """Backward of ONE block of queries against several blocks of keys in turn (sntl_attn_bwd_begin / _block / _end):
    the work that depends only on the query block -- delta, the rescaled LSE, zeroing and converting the fp32 dQ
    accumulator -- runs once, and each ``block`` call adds its dQ into that accumulator and its dK, dV into the
    caller's fp32 accumulators.  ``lse`` must be the FINAL log-sum-exp of the query rows over all keys."""

    def __init__(self, q, o, lse, dout, *, scale=None, workspace=None):
        lib = _lib.load()
        for t, n in ((q, "q"), (o, "o"), (lse, "lse"), (dout, "dout")):
            _require(t, n)
        if o.shape != q.shape or dout.shape != q.shape or lse.shape != q.shape[:3] or lse.dtype != torch.float32:
            raise ValueError("o/dout must match q; lse must be fp32 [B,Hq,Sq]")
        if o.dtype != q.dtype or dout.dtype != q.dtype:
            raise ValueError("q, o, dout must share dtype")
        _same_device(q, (o, "o"), (lse, "lse"), (dout, "dout"))
        self.q, self.dout = q, dout
        self.scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
        d = self._desc(q.shape[1], q.shape[2], False)
        self.nbytes = lib.sntl_attn_bwd_pieces_workspace_bytes(C.byref(d))
        if self.nbytes == 0:
            _lib.check(_lib.ERR_UNSUPPORTED, "sntl_attn_bwd_begin")
        if workspace is None:
            workspace = torch.empty(self.nbytes, dtype=torch.uint8, device=q.device)
        if workspace.numel() < self.nbytes:
            raise ValueError("workspace too small")
        self.ws = workspace
        rc = lib.sntl_attn_bwd_begin(C.byref(d), o.data_ptr(), lse.data_ptr(), dout.data_ptr(), self.ws.data_ptr(), self.nbytes,
                                     _stream_ptr())
        _lib.check(rc, "sntl_attn_bwd_begin")

    def _desc(self, kv_heads, seq_kv, causal):
        B, Hq, Sq, D = self.q.shape
        return _lib.Desc(_dtype_code(self.q), _lib.LAYOUT_BHSD, B, Hq, kv_heads, Sq, seq_kv, D, self.scale, int(bool(causal)), 0, 0,
                         0, 0, 0)

    def block(self, k, v, dk_acc, dv_acc, *, causal):
        """Adds the (query block, this key block) pair: dQ into the accumulator, dK*scale / dV into fp32 dk_acc / dv_acc."""
        for t, n in ((k, "k"), (v, "v"), (dk_acc, "dk_acc"), (dv_acc, "dv_acc")):
            _require(t, n)
        if k.shape != v.shape or dk_acc.shape != k.shape or dv_acc.shape != k.shape:
            raise ValueError("k, v, dk_acc, dv_acc must share shape")
        if dk_acc.dtype != torch.float32 or dv_acc.dtype != torch.float32:
            raise ValueError("dk_acc / dv_acc must be fp32")
        if k.dtype != self.q.dtype or v.dtype != self.q.dtype or k.dim() != 4 or k.shape[0] != self.q.shape[0] or k.shape[3] != self.q.shape[3]:
            raise ValueError("k, v must be [B, Hkv, Skv, D] tensors of q's dtype, batch and head_dim")
        _same_device(self.q, (k, "k"), (v, "v"), (dk_acc, "dk_acc"), (dv_acc, "dv_acc"))
        d = self._desc(k.shape[1], k.shape[2], causal)
        rc = _lib.load().sntl_attn_bwd_block(C.byref(d), self.q.data_ptr(), k.data_ptr(), v.data_ptr(), self.dout.data_ptr(),
                                             dk_acc.data_ptr(), dv_acc.data_ptr(), self.ws.data_ptr(), self.nbytes, _stream_ptr())
        _lib.check(rc, "sntl_attn_bwd_block")

    def end(self, dq=None):
        dq = torch.empty_like(self.q) if dq is None else _check_out(dq, self.q.shape, self.q.dtype, self.q, "dq")
        d = self._desc(self.q.shape[1], self.q.shape[2], False)
        rc = _lib.load().sntl_attn_bwd_end(C.byref(d), dq.data_ptr(), self.ws.data_ptr(), self.nbytes, _stream_ptr())
        _lib.check(rc, "sntl_attn_bwd_end")
        return dq


def attention_forward_backward_host(q, k, v, dout, *, causal=True, scale=None, flags=0, device="cuda", chunks=None,
                                    window=0, global_tokens=0, out=None):
    """End-to-end call on HOST tensors (pinned memory recommended): uploads Q, K, V, dO, runs forward and
    backward on the device, downloads O, LSE, dQ, dK, dV.  This is the path the benchmark's ``e2e`` times.
    The returned tensors are reused by the next call unless ``out`` = (O, LSE, dQ, dK, dV) supplies the caller's own."""
    from .host_pipeline import forward_backward_host   # transfers overlapped with the kernels, chunked over (batch, KV group)
    return forward_backward_host(q, k, v, dout, causal=causal, scale=scale, flags=flags, device=device, chunks=chunks,
                                 window=window, global_tokens=global_tokens, out=out)


def merge_partials(o_acc, lse_acc, o_part, lse_part):
    """In-place log-sum-exp merge of two partial results over disjoint key sets (ring combine step)."""
    lib = _lib.load()
    for t, n in ((o_acc, "o_acc"), (lse_acc, "lse_acc"), (o_part, "o_part"), (lse_part, "lse_part")):
        _require(t, n)
    D = o_acc.shape[-1]
    rows = o_acc.numel() // D
    if o_part.shape != o_acc.shape or lse_acc.numel() != rows or lse_part.numel() != rows:
        raise ValueError("o_part must match o_acc; lse_acc / lse_part hold one value per row")
    if lse_acc.dtype != torch.float32 or lse_part.dtype != torch.float32:
        raise ValueError("lse_acc / lse_part must be fp32")
    _same_device(o_acc, (lse_acc, "lse_acc"), (o_part, "o_part"), (lse_part, "lse_part"))
    rc = lib.sntl_attn_merge(_dtype_code(o_acc), _dtype_code(o_part), rows, D, o_acc.data_ptr(), lse_acc.data_ptr(),
                             o_part.data_ptr(), lse_part.data_ptr(), _stream_ptr())
    _lib.check(rc, "sntl_attn_merge")
    return o_acc, lse_acc


def accumulate(acc, part):
    """acc (fp32) += part (bf16 or fp32), in place, on the library's kernel."""
    lib = _lib.load()
    _require(acc, "acc")
    _require(part, "part")
    if acc.dtype != torch.float32 or acc.numel() != part.numel():
        raise ValueError("acc must be fp32 and match part in size")
    rc = lib.sntl_attn_accumulate(_dtype_code(part), acc.numel(), acc.data_ptr(), part.data_ptr(), _stream_ptr())
    _lib.check(rc, "sntl_attn_accumulate")
    return acc


def last_path() -> str:
    return _lib.load().sntl_attn_last_path().decode()


def launch_count() -> int:
    return int(_lib.load().sntl_attn_launch_count())


def poll_device_status() -> int:
    """Synchronises the current stream and returns the device status word (0 = no bounded wait ran out)."""
    word = C.c_uint32(0)
    rc = _lib.load().sntl_attn_poll_device_status(_stream_ptr(), C.byref(word))
    if rc not in (_lib.OK, _lib.ERR_DEVICE_TIMEOUT):
        _lib.check(rc, "sntl_attn_poll_device_status")
    return int(word.value)


def raise_if_device_wait_timed_out() -> None:
    """Synchronises the current stream and raises ``_lib.SntlError`` (a RuntimeError) when a bounded device-side wait
    ran out since the last poll: the results of the calls made since then are not to be trusted.  The asynchronous
    entry points cannot report this themselves; the host-buffer call and the ring schedule call this at the point
    where they synchronise anyway."""
    fwd, bwd = C.c_uint32(0), C.c_uint32(0)
    rc = _lib.load().sntl_attn_poll_device_status_words(_stream_ptr(), C.byref(fwd), C.byref(bwd))
    if rc == _lib.ERR_DEVICE_TIMEOUT:
        raise _lib.SntlError(rc, f"device status (forward 0x{fwd.value:08x}, backward 0x{bwd.value:08x})")
    _lib.check(rc, "sntl_attn_poll_device_status_words")


class CudaFlashAttention:
    """The reference's operator interface (CudaFlashAttention.hpp:10-41) over fp32 feature-major CUDA tensors.

    ``query`` is ``(headCount*headDimension) x strideColumns``; ``key``/``value`` are
    ``(kvHeads*headDimension) x strideColumns`` (kvHeads == headCount reproduces the reference call, fewer
    heads = grouped-query attention without repeating K/V); ``logSumExp`` is ``headCount x strideColumns``.
    Outputs are allocated by the callee when not passed, as the reference's ensureSize does.
    """
    queryTileSize = 128
    keyTileSize = 128
    maxHeadDimension = 128
    allow_reduced_precision = False

    @staticmethod
    def _desc(query, key, headCount, headDimension, scale, causal, columnStart, columnCount, packCount, windowSize=0,
              globalTokenCount=0):
        op = "CudaFlashAttention"
        if query.numel() == 0 or key.numel() == 0:
            raise ValueError(f"{op} empty input")
        if query.dim() != 2 or key.dim() != 2 or query.dtype != torch.float32 or key.dtype != torch.float32:
            raise ValueError(f"{op} expects fp32 matrices")
        if headCount <= 0 or headDimension <= 0:
            raise ValueError(f"{op} invalid head geometry")
        if query.shape[0] != headCount * headDimension:
            raise ValueError(f"{op} query rows mismatch headCount*headDim")
        if key.shape[0] % headDimension != 0 or headCount % (key.shape[0] // headDimension) != 0:
            raise ValueError(f"{op} key/value rows mismatch")
        if query.shape[1] != key.shape[1]:
            raise ValueError(f"{op} sequenceLength mismatch")
        if packCount <= 0:
            packCount = 1
        stride = query.shape[1]
        if columnCount <= 0:                      # resolveColumnWindow, CudaFlashAttention.cu:1533-1539
            columnCount = stride - columnStart
        if columnStart < 0 or columnCount <= 0 or columnStart + columnCount > stride:
            raise ValueError(f"{op} invalid column window")
        if columnStart + packCount * columnCount > stride:
            raise ValueError(f"{op} pack window exceeds columns")
        flags = _lib.FLAG_ALLOW_BF16_COMPUTE if CudaFlashAttention.allow_reduced_precision else 0
        return _lib.Desc(_lib.DTYPE_F32, _lib.LAYOUT_SENTINEL, packCount, headCount, key.shape[0] // headDimension,
                         columnCount, columnCount, headDimension, float(scale), int(bool(causal)), stride, columnStart,
                         flags, int(windowSize), int(globalTokenCount))

    @staticmethod
    def forwardMultiHead(query, key, value, out, logSumExp, headCount, headDimension, scale, causal=True, columnStart=0,
                         columnCount=0, packCount=1, windowSize=0, globalTokenCount=0):
        lib = _lib.load()
        if key.shape != value.shape:
            raise ValueError("CudaFlashAttention key/value rows mismatch")
        d = CudaFlashAttention._desc(query, key, headCount, headDimension, scale, causal, columnStart, columnCount, packCount,
                                     windowSize, globalTokenCount)
        for t, n in ((query, "query"), (key, "key"), (value, "value")):
            _require(t, n)
        if value.dtype != torch.float32:
            raise ValueError("CudaFlashAttention expects fp32 matrices")
        _same_device(query, (key, "key"), (value, "value"))
        # the reference resizes its outputs (ensureSize); a torch tensor handed in must already have the size
        out = torch.zeros_like(query) if out is None else _check_out(out, query.shape, torch.float32, query, "out")
        logSumExp = (torch.zeros(headCount, query.shape[1], dtype=torch.float32, device=query.device) if logSumExp is None
                     else _check_out(logSumExp, (headCount, query.shape[1]), torch.float32, query, "logSumExp"))
        nbytes = lib.sntl_attn_fwd_workspace_bytes(C.byref(d))
        ws = _workspace(nbytes, query.device)
        rc = lib.sntl_attn_fwd(C.byref(d), query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(),
                               logSumExp.data_ptr(), ws.data_ptr() if ws is not None else None, nbytes, _stream_ptr())
        _lib.check(rc, "CudaFlashAttention::forwardMultiHead")
        return out, logSumExp

    @staticmethod
    def forward(query, key, value, out, logSumExp, scale, causal=True):
        return CudaFlashAttention.forwardMultiHead(query, key, value, out, logSumExp, 1, query.shape[0], scale, causal, 0,
                                                   query.shape[1])

    @staticmethod
    def backwardMultiHead(query, key, value, out, logSumExp, outGradient, queryGradient, keyGradient, valueGradient,
                          deltaWorkspace, headCount, headDimension, scale, causal=True, columnStart=0, columnCount=0,
                          packCount=1, windowSize=0, globalTokenCount=0):
        lib = _lib.load()
        d = CudaFlashAttention._desc(query, key, headCount, headDimension, scale, causal, columnStart, columnCount, packCount,
                                     windowSize, globalTokenCount)
        if out.shape != query.shape:
            raise ValueError("CudaFlashAttention::backwardMultiHead out shape mismatch")
        if outGradient.shape != query.shape:
            raise ValueError("CudaFlashAttention::backwardMultiHead outGradient shape mismatch")
        if tuple(logSumExp.shape) != (headCount, query.shape[1]):
            raise ValueError("CudaFlashAttention::backwardMultiHead logSumExp shape mismatch")
        for t, n in ((query, "query"), (key, "key"), (value, "value"), (out, "out"), (logSumExp, "logSumExp"),
                     (outGradient, "outGradient")):
            _require(t, n)
        if key.shape != value.shape:
            raise ValueError("CudaFlashAttention key/value rows mismatch")
        if any(t.dtype != torch.float32 for t in (value, out, logSumExp, outGradient)):
            raise ValueError("CudaFlashAttention expects fp32 matrices")
        _same_device(query, (key, "key"), (value, "value"), (out, "out"), (logSumExp, "logSumExp"), (outGradient, "outGradient"))
        queryGradient = (torch.zeros_like(query) if queryGradient is None
                         else _check_out(queryGradient, query.shape, torch.float32, query, "queryGradient"))
        keyGradient = (torch.zeros_like(key) if keyGradient is None
                       else _check_out(keyGradient, key.shape, torch.float32, query, "keyGradient"))
        valueGradient = (torch.zeros_like(value) if valueGradient is None
                         else _check_out(valueGradient, value.shape, torch.float32, query, "valueGradient"))
        nbytes = lib.sntl_attn_bwd_workspace_bytes(C.byref(d))
        ws = _workspace(nbytes, query.device)
        rc = lib.sntl_attn_bwd(C.byref(d), query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(),
                               logSumExp.data_ptr(), outGradient.data_ptr(), queryGradient.data_ptr(),
                               keyGradient.data_ptr(), valueGradient.data_ptr(),
                               ws.data_ptr() if ws is not None else None, nbytes, _stream_ptr())
        _lib.check(rc, "CudaFlashAttention::backwardMultiHead")
        return queryGradient, keyGradient, valueGradient

    @staticmethod
    def backward(query, key, value, out, logSumExp, outGradient, queryGradient, keyGradient, valueGradient, scale,
                 causal=True):
        return CudaFlashAttention.backwardMultiHead(query, key, value, out, logSumExp, outGradient, queryGradient,
                                                    keyGradient, valueGradient, None, 1, query.shape[0], scale, causal, 0,
                                                    query.shape[1])
