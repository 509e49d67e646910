"""Loader for the C-ABI CUDA library.  There is no fallback: if the library is missing the import of any
compute entry point fails loudly, and the library itself refuses to run on anything but an sm_100 device."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("SNTL_ATTN_LIB") or os.path.join(HERE, "lib", "libsntl_attn.so")   # env: another build of the same ABI

OK, ERR_BAD_ARGUMENT, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_NO_DEVICE, ERR_DEVICE_TIMEOUT = range(7)
DTYPE_BF16, DTYPE_F32 = 0, 1
LAYOUT_BHSD, LAYOUT_SENTINEL = 0, 1
FLAG_ALLOW_BF16_COMPUTE, FLAG_FORCE_SIMT, FLAG_DETERMINISTIC, FLAG_RING_ZIGZAG = 1, 2, 4, 8

# every symbol include/sntl_attn.h declares
EXPORTS = ["sntl_attn_version", "sntl_status_string", "sntl_attn_fwd_workspace_bytes", "sntl_attn_bwd_workspace_bytes",
           "sntl_attn_fwd", "sntl_attn_bwd", "sntl_attn_merge", "sntl_attn_last_path", "sntl_attn_launch_count",
           "sntl_attn_poll_device_status", "sntl_attn_bwd_static_scratch", "sntl_attn_static_scratch_capacity", "sntl_attn_accumulate",
           "sntl_attn_cached_fwd", "sntl_attn_cached_fwd_workspace_bytes", "sntl_attn_pack_heads", "sntl_attn_unpack_heads",
           "sntl_attn_poll_device_status_words", "sntl_attn_selftest_wait_timeout",
           "sntl_attn_bwd_pieces_workspace_bytes", "sntl_attn_bwd_begin", "sntl_attn_bwd_block", "sntl_attn_bwd_end",
           "sntl_ring_unique_id", "sntl_ring_comm_create", "sntl_ring_comm_adopt", "sntl_ring_comm_destroy",
           "sntl_ring_attn_workspace_bytes", "sntl_ring_attn_fwd", "sntl_ring_attn_bwd"]
ERR_SCRATCH_LIMIT = 7
ERR_COMM = 8


class Desc(C.Structure):
    """``sntl_attn_desc`` of include/sntl_attn.h."""
    _fields_ = [("dtype", C.c_int32), ("layout", C.c_int32), ("batch", C.c_int32), ("q_heads", C.c_int32),
                ("kv_heads", C.c_int32), ("seq_q", C.c_int32), ("seq_kv", C.c_int32), ("head_dim", C.c_int32),
                ("scale", C.c_float), ("causal", C.c_int32), ("stride_columns", C.c_int32),
                ("column_start", C.c_int32), ("flags", C.c_int32), ("window_size", C.c_int32), ("global_tokens", C.c_int32)]


class LibraryMissing(RuntimeError):
    pass


_lib = None


def load():
    """dlopen the library and declare the prototypes; raises LibraryMissing when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(f"{LIB_PATH} is missing: run `python -m sentinel_b200.build` (needs nvcc). "
                             "There is no CPU or PyTorch fallback for this path.")
    lib = C.CDLL(LIB_PATH)
    vp, sz, dp = C.c_void_p, C.c_size_t, C.POINTER(Desc)
    lib.sntl_attn_version.restype = C.c_int
    lib.sntl_status_string.restype = C.c_char_p
    lib.sntl_status_string.argtypes = [C.c_int]
    lib.sntl_attn_fwd_workspace_bytes.restype = sz
    lib.sntl_attn_fwd_workspace_bytes.argtypes = [dp]
    lib.sntl_attn_bwd_workspace_bytes.restype = sz
    lib.sntl_attn_bwd_workspace_bytes.argtypes = [dp]
    lib.sntl_attn_fwd.restype = C.c_int
    lib.sntl_attn_fwd.argtypes = [dp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.sntl_attn_cached_fwd_workspace_bytes.restype = sz
    lib.sntl_attn_cached_fwd_workspace_bytes.argtypes = [dp, C.c_int32]
    lib.sntl_attn_cached_fwd.restype = C.c_int
    lib.sntl_attn_cached_fwd.argtypes = [dp, vp, vp, vp, C.c_int32, vp, vp, vp, sz, vp]
    lib.sntl_attn_bwd.restype = C.c_int
    lib.sntl_attn_bwd.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.sntl_attn_bwd_static_scratch.restype = C.c_int
    lib.sntl_attn_bwd_static_scratch.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.sntl_attn_static_scratch_capacity.restype = sz
    lib.sntl_attn_accumulate.restype = C.c_int
    lib.sntl_attn_accumulate.argtypes = [C.c_int32, C.c_int64, vp, vp, vp]
    lib.sntl_attn_pack_heads.restype = C.c_int
    lib.sntl_attn_pack_heads.argtypes = [vp, vp] + [C.c_int32] * 6 + [vp, vp, C.c_int32, C.c_int32, vp]
    lib.sntl_attn_unpack_heads.restype = C.c_int
    lib.sntl_attn_unpack_heads.argtypes = [vp, vp] + [C.c_int32] * 6 + [vp, vp, C.c_int32, C.c_int32, C.c_int32, vp]
    lib.sntl_attn_merge.restype = C.c_int
    lib.sntl_attn_merge.argtypes = [C.c_int32, C.c_int32, C.c_int64, C.c_int32, vp, vp, vp, vp, vp]
    lib.sntl_attn_last_path.restype = C.c_char_p
    lib.sntl_attn_launch_count.restype = C.c_uint64
    lib.sntl_attn_poll_device_status.restype = C.c_int
    lib.sntl_attn_poll_device_status.argtypes = [vp, C.POINTER(C.c_uint32)]
    lib.sntl_attn_bwd_pieces_workspace_bytes.restype = sz
    lib.sntl_attn_bwd_pieces_workspace_bytes.argtypes = [dp]
    lib.sntl_attn_bwd_begin.restype = C.c_int
    lib.sntl_attn_bwd_begin.argtypes = [dp, vp, vp, vp, vp, sz, vp]
    lib.sntl_attn_bwd_block.restype = C.c_int
    lib.sntl_attn_bwd_block.argtypes = [dp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.sntl_attn_bwd_end.restype = C.c_int
    lib.sntl_attn_bwd_end.argtypes = [dp, vp, vp, sz, vp]
    lib.sntl_ring_unique_id.restype = C.c_int
    lib.sntl_ring_unique_id.argtypes = [vp]
    lib.sntl_ring_comm_create.restype = C.c_int
    lib.sntl_ring_comm_create.argtypes = [vp, C.c_int, C.c_int, C.POINTER(vp)]
    lib.sntl_ring_comm_adopt.restype = C.c_int
    lib.sntl_ring_comm_adopt.argtypes = [vp, C.c_int, C.c_int, C.POINTER(vp)]
    lib.sntl_ring_comm_destroy.restype = C.c_int
    lib.sntl_ring_comm_destroy.argtypes = [vp]
    lib.sntl_ring_attn_workspace_bytes.restype = sz
    lib.sntl_ring_attn_workspace_bytes.argtypes = [vp, dp]
    lib.sntl_ring_attn_fwd.restype = C.c_int
    lib.sntl_ring_attn_fwd.argtypes = [vp, dp, vp, vp, vp, vp, vp, vp, sz, vp]
    lib.sntl_ring_attn_bwd.restype = C.c_int
    lib.sntl_ring_attn_bwd.argtypes = [vp, dp, vp, vp, vp, vp, vp, vp, vp, vp, vp, C.c_int, vp, sz, vp]
    lib.sntl_attn_poll_device_status_words.restype = C.c_int
    lib.sntl_attn_poll_device_status_words.argtypes = [vp, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
    lib.sntl_attn_selftest_wait_timeout.restype = C.c_int
    lib.sntl_attn_selftest_wait_timeout.argtypes = [C.c_uint32, vp]
    # test hooks of the C++ operator class (sentinel_compat.cu)
    fp = C.POINTER(C.c_float)
    lib.sntl_compat_forward_backward.restype = C.c_int
    lib.sntl_compat_forward_backward.argtypes = [fp, fp, fp, fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int,
                                                 C.c_int, C.c_int, C.c_int, C.c_int, fp, fp, fp, fp, fp, C.c_char_p, sz,
                                                 C.c_char_p, sz]
    lib.sntl_compat_forward_backward_windowed.restype = C.c_int
    lib.sntl_compat_forward_backward_windowed.argtypes = [fp, fp, fp, fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float] + \
        [C.c_int] * 7 + [fp, fp, fp, fp, fp, C.c_char_p, sz, C.c_char_p, sz]
    lib.sntl_compat_validate.restype = C.c_int
    lib.sntl_compat_validate.argtypes = [C.c_int] * 8 + [C.c_char_p, sz]
    _lib = lib
    return lib


class SntlError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {load().sntl_status_string(status).decode()} (status {status})")


def check(status: int, where: str) -> None:
    """Maps status codes the way the reference maps its failures: argument errors -> ValueError (the
    reference throws std::invalid_argument), the rest -> RuntimeError."""
    if status == OK:
        return
    if status in (ERR_BAD_ARGUMENT, ERR_UNSUPPORTED):
        raise ValueError(f"{where}: {load().sntl_status_string(status).decode()}")
    raise SntlError(status, where)
