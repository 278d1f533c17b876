"""ctypes binding of libflashlazy.so (the C ABI declared in include/fla.h).

The library is the product: there is no fallback.  If the shared object is missing
or a call fails, a RuntimeError is raised with the library's own message.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libflashlazy.so")

FLA_F32, FLA_F16, FLA_BF16 = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TCGEN05 = 0, 1, 2
PATH_NAMES = {PATH_AUTO: "auto", PATH_SIMT: "simt", PATH_TCGEN05: "tcgen05"}
FLAG_NO_CANDIDATE_LIST, FLAG_PLAIN_FIRST_STEP, FLAG_CANDIDATE_LIST, FLAG_ONE_TILE_CTAS = 1, 2, 4, 8


class Tensor4(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride", C.c_int64 * 4)]


class AttnGeom(C.Structure):
    _fields_ = [("B", C.c_int32), ("H", C.c_int32), ("L", C.c_int32), ("D", C.c_int32),
                ("dtype", C.c_int32), ("causal", C.c_int32), ("varlen", C.c_void_p),
                ("path", C.c_int32), ("status", C.c_void_p), ("flags", C.c_int32), ("Hkv", C.c_int32)]


_P4 = C.POINTER(Tensor4)
_PG = C.POINTER(AttnGeom)
_vp, _i32, _i64, _f32, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes): exactly the declarations of include/fla.h
SIGNATURES = {
    "fla_version": (C.c_int, []),
    "fla_last_error": (C.c_char_p, []),
    "fla_device_supported": (C.c_int, [C.c_int]),
    "fla_last_path": (C.c_int, []),
    "fla_attn_uses_tensor_cores": (C.c_int, [_PG, _P4, _P4, _P4]),
    "fla_entmax_fwd": (C.c_int, [_vp, _vp, _i64, _i64, _f32, C.c_int, C.c_int, C.c_int, _vp]),
    "fla_entmax_bwd": (C.c_int, [_vp, _vp, _vp, _i64, _i64, _f32, C.c_int, _vp]),
    "fla_rope_qk": (C.c_int, [_P4, _P4, C.c_int32, _P4, _P4, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _f32,
                              C.c_int32, C.c_int32, _vp]),
    "fla_block_mask_words": (_i64, [_i32]),
    "fla_check_status": (C.c_int, [_vp, _vp]),
    "fla_entmax_attn_fwd": (C.c_int, [_PG, _P4, _P4, _P4, _P4, _f32, C.c_int, _vp, _vp, _vp, _vp, _vp]),
    "fla_entmax_attn_bwd_workspace": (_sz, [_PG]),
    "fla_entmax_attn_bwd": (C.c_int, [_PG, _P4, _P4, _P4, _P4, _f32, _vp, _vp, _vp, _vp, _P4, _P4, _P4,
                                      _vp, _sz, _vp]),
    "fla_entmax_attn_bwd_static_max_rows": (_i64, []),
    "fla_entmax_attn_bwd_static": (C.c_int, [_PG, _P4, _P4, _P4, _P4, _f32, _vp, _vp, _vp, _vp, _P4, _P4, _P4, _vp]),
    "fla_lazy_attn_fwd": (C.c_int, [_PG, _P4, _P4, _P4, _P4, _vp, _i64, _vp, _i32, _vp, _vp, _vp]),
    "fla_lazy_attn_bwd_workspace": (_sz, [_PG]),
    "fla_lazy_attn_bwd": (C.c_int, [_PG, _P4, _P4, _P4, _P4, _P4, _vp, _i64, _vp, _i32, _vp, _vp,
                                    _P4, _P4, _P4, _vp, _i64, _vp, _vp, _sz, _vp]),
    "fla_selftest_umma": (C.c_int, [_vp, _vp, _vp, C.c_int, _vp, _vp]),
}

_lib = None
_lock = threading.Lock()


def load() -> C.CDLL:
    """Load libflashlazy.so once and attach the signatures."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            path = LIB_PATH
            if not os.path.exists(path):
                raise RuntimeError(
                    f"{path} is missing: build it with `python -m flash_lazy_attention_b200.build` "
                    "(needs nvcc).  There is no fallback implementation.")
            lib = C.CDLL(path)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def last_error() -> str:
    return load().fla_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        kinds = {1: "invalid argument", 2: "unsupported", 3: "CUDA error", 4: "device wait expired"}
        raise RuntimeError(f"{what}: {kinds.get(rc, rc)}: {last_error()}")
