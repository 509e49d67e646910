"""sentinel_b200 -- causal self-attention forward/backward for NVIDIA B200 (sm_100a), a drop-in for the
flash-attention launch sites of ToldByNun/sentinel.

The product is the C-ABI library ``lib/libsntl_attn.so`` (``include/sntl_attn.h``); this package is the
Python host side: it binds that ABI with ctypes and mirrors the reference's operator interface
(``CudaFlashAttention``).  PyTorch is used for device memory, streams and process groups only.
"""
from . import _lib
from .flash_attention import (BackwardPieces, CudaFlashAttention, accumulate, attention_backward, attention_cached_forward, attention_forward,
                              attention_forward_backward_host,
                              last_path, launch_count, merge_partials, pack_heads, poll_device_status,
                              raise_if_device_wait_timed_out, unpack_heads)
from .workloads import WORKLOADS, Workload, make_inputs

__all__ = ["BackwardPieces", "CudaFlashAttention", "attention_forward", "attention_backward", "attention_cached_forward",
           "attention_forward_backward_host",
           "merge_partials", "accumulate", "pack_heads", "unpack_heads", "last_path", "launch_count", "poll_device_status", "raise_if_device_wait_timed_out", "WORKLOADS", "Workload", "make_inputs",
           "_lib"]
