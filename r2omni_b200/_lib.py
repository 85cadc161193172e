"""ctypes binding of the C ABI declared in ``include/r2k_b200.h``."""
from __future__ import annotations

import ctypes as C
import os

from .build import LIB

OK, ERR_NULL, ERR_GEOMETRY, ERR_ALIGNMENT, ERR_CAPACITY, ERR_WORKSPACE, ERR_CUDA, ERR_DEVICE_TIMEOUT, ERR_EMPTY = range(9)
DTYPE_BF16, DTYPE_FP16 = 0, 1
FLAG_OUTPUT_HADAMARD, FLAG_OUT_F32, FLAG_OUT_STATE = 1, 2, 4

EXPORTS = (
    "r2k_status_string", "r2k_launch_count", "r2k_decode_workspace_bytes", "r2k_decode_workspace_init", "r2k_decode",
    "r2k_decode_static", "r2k_decode_static_status", "r2k_decode_static_reset", "r2k_decode_device_status", "r2k_merge_states", "r2k_pack_k_int4", "r2k_pack_v_int4", "r2k_pack_v_int2",
    "r2k_gather_rows", "r2k_fwht128", "r2k_qk_mrope", "r2k_qkv_prologue", "r2k_append_recent", "r2k_flush_recent",
    "r2k_exchange_bytes", "r2k_exchange_create", "r2k_exchange_open", "r2k_exchange_close", "r2k_decode_exchange",
    "r2k_decode_host_staging_bytes", "r2k_decode_host",
)


class Geom(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "batch", "num_q_heads", "num_kv_heads", "head_dim", "dtype", "page_size", "k_block", "v2_group",
        "n_fp", "n_i4", "n_i2", "k_capacity", "k_off_fp", "k_off_i4", "k_off_i2",
        "fp_capacity", "i4_capacity", "i2_capacity", "recent_capacity")] + [("sm_scale", C.c_float)]


_PTRS = ("k_packed", "k_scale", "k_zero", "fp_v", "i4_packed", "i4_scale", "i2_packed", "i2_scale", "i2_zero",
         "recent_k", "recent_v", "recent_len", "recent_global", "recent_logical", "recent_page_lengths")


class CacheView(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in _PTRS] + [(n + "_bstride", C.c_int64) for n in _PTRS]


class Append(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("indices", C.c_void_p),
                ("global_index", C.c_int64), ("logical_position", C.c_int64)]


MAX_RANKS = 8


class Exchange(C.Structure):
    """include/r2k_b200.h: R2KExchange."""
    _fields_ = [("buffers", C.c_void_p * MAX_RANKS), ("rank", C.c_int32), ("world", C.c_int32), ("seq", C.c_uint32),
                ("wait_us", C.c_uint32)]


_lib = None


def lib():
    """The loaded shared library.  There is no fallback: a missing library is an error."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            raise RuntimeError(
                f"{LIB} is missing: build it with `python -m r2omni_b200.build` (needs nvcc); "
                "this package has no CPU or Triton fallback")
        handle = C.CDLL(LIB)
        handle.r2k_status_string.restype = C.c_char_p
        handle.r2k_launch_count.restype = C.c_uint64
        for name in EXPORTS[2:]:
            getattr(handle, name).restype = C.c_int
        # the per-step call: declared argument types let plain ints and byref() objects through without
        # building a ctypes wrapper per argument
        handle.r2k_decode.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                      C.c_uint32, C.c_void_p]
        handle.r2k_decode_exchange.argtypes = handle.r2k_decode.argtypes[:8] + [C.c_void_p, C.c_void_p]
        handle.r2k_decode_host.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                           C.c_size_t, C.c_void_p, C.c_uint32, C.c_void_p]
        _lib = handle
    return _lib


def check(status: int, what: str = "") -> None:
    """Map a status code onto the exception types the reference raises."""
    if status == OK:
        return
    msg = f"{what}: {lib().r2k_status_string(status).decode()}" if what else lib().r2k_status_string(status).decode()
    if status in (ERR_GEOMETRY, ERR_ALIGNMENT, ERR_NULL, ERR_EMPTY):
        raise ValueError(msg)
    raise RuntimeError(msg)
