"""ctypes binding of libfa_b200.so (the C ABI declared in include/fa_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfa_b200.so")

FA_BF16, FA_FP16, FA_FP32 = 0, 1, 2
FA_ID_NONE, FA_ID_INT32, FA_ID_INT64 = 0, 1, 2
FA_GROUP_MAX_ROWS = 16384

EXPORTS = (
    "fa_version", "fa_error_string", "fa_padded_rows", "fa_plan_bytes", "fa_plan_build", "fa_fwd",
    "fa_bwd_delta", "fa_bwd_dkdv", "fa_bwd_dq", "fa_debug_mask", "fa_classify_tile", "fa_fwd_static_plan",
    "fa_debug_wait_timeout", "fa_group_rows", "fa_permute_rows",
)


class Problem(ctypes.Structure):
    _fields_ = [
        ("B", ctypes.c_int32), ("H", ctypes.c_int32), ("Hk", ctypes.c_int32),
        ("M", ctypes.c_int32), ("N", ctypes.c_int32), ("D", ctypes.c_int32),
        ("dtype", ctypes.c_int32), ("causal", ctypes.c_int32), ("mode", ctypes.c_int32),
        ("id_heads", ctypes.c_int32), ("sm_scale", ctypes.c_float),
    ]


class Tensor(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride", ctypes.c_int64 * 4)]


class Ids(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride", ctypes.c_int64 * 3), ("dtype", ctypes.c_int32)]


_lib = None


def load():
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python build.py` in the package directory "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(LIB_PATH)
    P, T, I = ctypes.POINTER(Problem), ctypes.POINTER(Tensor), ctypes.POINTER(Ids)
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    lib.fa_version.restype = i32
    lib.fa_error_string.restype = ctypes.c_char_p
    lib.fa_error_string.argtypes = [i32]
    lib.fa_padded_rows.restype = ctypes.c_int64
    lib.fa_padded_rows.argtypes = [ctypes.c_int32]
    lib.fa_plan_bytes.restype = i32
    lib.fa_plan_bytes.argtypes = [P, ctypes.POINTER(ctypes.c_size_t)]
    lib.fa_plan_build.restype = i32
    lib.fa_plan_build.argtypes = [P, I, I, vp, ctypes.c_size_t, vp, vp]
    lib.fa_fwd.restype = i32
    lib.fa_fwd.argtypes = [P, T, T, T, T, vp, vp, vp, vp]
    lib.fa_bwd_delta.restype = i32
    lib.fa_bwd_delta.argtypes = [P, T, T, vp, vp]
    lib.fa_bwd_dkdv.restype = i32
    lib.fa_bwd_dkdv.argtypes = [P, T, T, T, T, vp, vp, T, T, vp, vp, vp]
    lib.fa_bwd_dq.restype = i32
    lib.fa_bwd_dq.argtypes = [P, T, T, T, T, vp, vp, T, vp, vp, vp]
    lib.fa_debug_mask.restype = i32
    lib.fa_debug_mask.argtypes = [P, vp, vp, vp, vp]
    lib.fa_fwd_static_plan.restype = i32
    lib.fa_fwd_static_plan.argtypes = [P, T, T, T, T, vp, I, I, vp, vp]
    lib.fa_debug_wait_timeout.restype = i32
    lib.fa_debug_wait_timeout.argtypes = [vp, ctypes.c_int64, ctypes.c_int32, vp]
    lib.fa_group_rows.restype = i32
    lib.fa_group_rows.argtypes = [P, I, vp, vp, vp, vp, vp]
    lib.fa_permute_rows.restype = i32
    lib.fa_permute_rows.argtypes = [P, T, T, vp, vp]
    lib.fa_classify_tile.restype = ctypes.c_uint32
    lib.fa_classify_tile.argtypes = [ctypes.c_int32] * 10
    _lib = lib
    return lib


def check(rc, what):
    if rc != 0:
        msg = load().fa_error_string(rc).decode()
        raise RuntimeError(f"{what} failed with code {rc}: {msg}")
