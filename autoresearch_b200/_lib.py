"""ctypes binding of libarattn.so (the declarations of include/arattn.h)."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "csrc", "libarattn.so")
_lib = None

AR_OK = 0
AR_ERR_BAD_ARG = -1
AR_ERR_UNSUPPORTED = -2
AR_ERR_CUDA = -3
AR_ERR_WORKSPACE = -4
AR_ERR_TIMEOUT = -5
AR_F32 = 0
AR_BF16 = 1
AR_FLAG_SYNC = 1
AR_FLAG_ROPE_PREPASS = 2
AR_FLAG_BWD_SKIP_D = 4
AR_FLAG_BWD_SKIP_DQ = 8
AR_FLAG_BWD_SKIP_DKV = 16

_i64 = ctypes.c_int64
_vp = ctypes.c_void_p


class ArattnError(RuntimeError):
    """A libarattn call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"libarattn status {status}: {message}")
        self.status = status


class ArAttnParams(ctypes.Structure):
    """struct ar_attn_params (include/arattn.h)."""
    _fields_ = [
        ("struct_size", ctypes.c_uint32), ("flags", ctypes.c_uint32),
        ("io_dtype", ctypes.c_int32), ("grad_dtype", ctypes.c_int32),
        ("B", _i64), ("T", _i64), ("H", _i64), ("D", _i64),
        ("window", _i64),
        ("rope_mode", ctypes.c_int32), ("reserved", ctypes.c_int32),
        ("cos_buf", _vp), ("sin_buf", _vp), ("rope_rows", _i64),
        ("workspace", _vp), ("workspace_bytes", ctypes.c_uint64),
        ("stream", _vp),
        ("q_rot", _vp), ("k_rot", _vp),
        ("stride_b", _i64), ("stride_t", _i64), ("stride_h", _i64),
    ]


# name -> (restype, argtypes); every symbol include/arattn.h declares.
SIGNATURES = {
    "ar_version": (ctypes.c_int32, []),
    "ar_last_error": (ctypes.c_char_p, []),
    "ar_device_status": (ctypes.c_int32, []),
    "ar_selftest_wait_timeout": (ctypes.c_int32, [ctypes.c_int32, _vp]),
    "ar_rope_fwd": (ctypes.c_int32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "ar_rope_bwd": (ctypes.c_int32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "ar_qk_norm_rope_cast": (ctypes.c_int32, [_vp] * 8 + [ctypes.c_int32, _vp, _vp] + [_i64] * 4 + [ctypes.c_float, _vp]),
    "ar_flash_attn_fwd": (ctypes.c_int32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    "ar_flash_attn_fwd_noalloc": (ctypes.c_int32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp]),
    "ar_noalloc_status": (ctypes.c_int32, []),
    "ar_flash_attn_bwd_precompute_d": (ctypes.c_int32, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "ar_flash_attn_bwd_dq": (ctypes.c_int32, [_vp] * 7 + [_i64] * 5 + [_vp]),
    "ar_flash_attn_bwd_dkv": (ctypes.c_int32, [_vp] * 8 + [_i64] * 5 + [_vp]),
    "ar_linear_fwd": (ctypes.c_int32, [_vp, _vp, _vp, _i64, _i64, _i64, ctypes.c_int32, ctypes.c_int32, _vp]),
    "ar_linear_bwd_dx": (ctypes.c_int32, [_vp, _vp, _vp, _i64, _i64, _i64, ctypes.c_int32, ctypes.c_int32, _vp]),
    "ar_linear_bwd_dw": (ctypes.c_int32, [_vp, _vp, _vp, _i64, _i64, _i64, ctypes.c_int32, _vp]),
    "ar_attn_workspace_bytes": (ctypes.c_uint64, [ctypes.POINTER(ArAttnParams), ctypes.c_int32]),
    "ar_attn_fwd": (ctypes.c_int32, [ctypes.POINTER(ArAttnParams)] + [_vp] * 5),
    "ar_attn_bwd": (ctypes.c_int32, [ctypes.POINTER(ArAttnParams)] + [_vp] * 10),
}


def lib_path() -> str:
    return _SO


def lib() -> ctypes.CDLL:
    """Load libarattn.so.  Raises if the library has not been built: there is no
    fallback implementation."""
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            raise ArattnError(AR_ERR_CUDA, f"{_SO} is missing; build it with `make -C "
                              f"{os.path.dirname(_SO)}` (or __graft_entry__.build())")
        handle = ctypes.CDLL(_SO)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != AR_OK:
        raise ArattnError(status, lib().ar_last_error().decode("utf-8", "replace"))
