"""ctypes binding of libb200fa.so (the C-ABI declared in include/b200fa.h).

The library is the only compute path: when it is missing or fails to load the
operators raise, they never fall back to another implementation.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libb200fa.so"

OK = 0
ERR_INVALID_ARG = -1
ERR_UNSUPPORTED = -2
ERR_WORKSPACE = -3
ERR_CUDA = -4
ERR_DEVICE = -5

F16, BF16, F32, I8, E4M3 = 0, 1, 2, 3, 4
FLAG_FORCE_MMA_SYNC = 1
FLAG_PACKED_F32 = 4
FLAG_FWD_PERSISTENT = 8
FLAG_FWD_ONE_ITEM = 16


class Desc(C.Structure):
    """Mirror of ``b200fa_desc``."""

    _fields_ = [
        ("dtype", C.c_int32),
        ("kv_dtype", C.c_int32),
        ("B", C.c_int32),
        ("Hq", C.c_int32),
        ("Hkv", C.c_int32),
        ("N", C.c_int32),
        ("S", C.c_int32),
        ("D", C.c_int32),
        ("q_strides", C.c_int64 * 3),
        ("k_strides", C.c_int64 * 3),
        ("v_strides", C.c_int64 * 3),
        ("o_strides", C.c_int64 * 3),
        ("scale", C.c_float),
        ("softcap", C.c_float),
        ("causal", C.c_int32),
        ("window_left", C.c_int32),
        ("num_splits", C.c_int32),
        ("flags", C.c_int32),
        ("alibi_slopes", C.c_void_p),
        ("block_mask", C.c_void_p),
        ("mask_bq", C.c_int32),
        ("mask_bk", C.c_int32),
        ("mask_nk", C.c_int32),
        ("kv_lens", C.c_void_p),
    ]


class DeviceInfo(C.Structure):
    """Mirror of ``b200fa_device_info_t``."""

    _fields_ = [
        ("cc_major", C.c_int32),
        ("cc_minor", C.c_int32),
        ("sm_count", C.c_int32),
        ("smem_per_block_optin", C.c_int32),
        ("total_mem", C.c_int64),
        ("has_tcgen05", C.c_int32),
        ("name", C.c_char * 128),
    ]


_P = C.c_void_p
_DP = C.POINTER(Desc)
_I = C.c_int32
_Z = C.c_size_t

# name -> (restype, argtypes); one entry per symbol declared in include/b200fa.h
SIGNATURES = {
    "b200fa_device_info": (_I, [_I, C.POINTER(DeviceInfo)]),
    "b200fa_last_error": (C.c_char_p, []),
    "b200fa_version": (C.c_char_p, []),
    "b200fa_fwd_workspace_bytes": (_Z, [_DP]),
    "b200fa_fwd": (_I, [_DP, _P, _P, _P, _P, _P, _P, _Z, _P]),
    "b200fa_fwd_varlen_workspace_bytes": (_Z, [_DP, _I, _I, _I]),
    "b200fa_fwd_varlen": (_I, [_DP, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _Z, _P]),
    "b200fa_bwd_workspace_bytes": (_Z, [_DP]),
    "b200fa_bwd": (_I, [_DP, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _Z, _P]),
    "b200fa_bwd_varlen_workspace_bytes": (_Z, [_DP, _I, _I, _I]),
    "b200fa_bwd_varlen": (_I, [_DP, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P, _P, _P, _P, _Z, _P]),
    "b200fa_decode_paged_workspace_bytes": (_Z, [_DP, _I]),
    "b200fa_decode_paged": (_I, [_DP, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _Z, _P]),
    "b200fa_decode_paged_static": (_I, [_DP, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P]),
    "b200fa_combine_partials": (_I, [_P, _I, C.c_int64, _I, _I, _P, _P, _P]),
    "b200fa_fwd_paged": (_I, [_DP, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P]),
    "b200fa_paged_kv_gather_dequant": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _P]),
    "b200fa_decode_paged_static_status": (_I, [_P, C.POINTER(C.c_int32)]),
    "b200fa_paged_kv_scatter_add": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P]),
    "b200fa_kv_append": (_I, [_I, _I, _I, _I, _I, _I, C.c_int64, _P, _P, C.c_int64, C.c_int64, _P, _P, _P, _P, _P, _P]),
    "b200fa_rope": (_I, [_I, _I, _I, _I, _I, _I, _I, _I, _P, C.POINTER(C.c_int64), _P, C.POINTER(C.c_int64), _P, _P, _I, _P, _I, _P]),
    "b200fa_kernel_status": (_I, [_P, C.POINTER(C.c_int32)]),
    "b200fa_workspace_status": (_I, [_P, _P, C.POINTER(C.c_int32)]),
    "b200fa_paged_kv_gather": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _P]),
}

_lib = None


def load() -> C.CDLL:
    """Loads the library once and declares every prototype."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is not built. Run: python -m mlx_flashattention_steel_b200.build "
            "(needs nvcc). There is no fallback implementation."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def is_built() -> bool:
    return LIB_PATH.exists()


def last_error() -> str:
    return load().b200fa_last_error().decode("utf-8", "replace")


def check(status: int, what: str) -> None:
    """Maps a C-ABI status to the exception class the reference raises at the
    same condition (ValueError for bad arguments, NotImplementedError for an
    unsupported configuration, RuntimeError otherwise)."""
    if status == OK:
        return
    msg = f"{what}: {last_error()}"
    if status == ERR_INVALID_ARG:
        raise ValueError(msg)
    if status == ERR_UNSUPPORTED:
        raise NotImplementedError(msg)
    raise RuntimeError(f"{msg} (status {status})")
