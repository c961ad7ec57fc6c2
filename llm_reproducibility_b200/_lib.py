"""ctypes binding of libtbik_b200.so.

There is no CPU fallback: if the library is missing or a call fails, a `RuntimeError`
is raised with the library's own message.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libtbik_b200.so")

TBIK_OK = 0
DTYPE_BF16, DTYPE_FP16, DTYPE_FP32 = 0, 1, 2
NODE_INPUT, NODE_FP32, NODE_FP32_OUT_FP32 = 0, 1, 2

_lib: Optional[ctypes.CDLL] = None

_i32, _i64, _vp, _sz = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t

_PROTOTYPES = {
    "tbik_last_error": (ctypes.c_char_p, []),
    "tbik_version": (_i32, []),
    "tbik_tree_shape": (_i32, [_i64, _i32, ctypes.POINTER(_i32), ctypes.POINTER(_i32), ctypes.POINTER(_i32)]),
    "tbik_gemm": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _vp]),
    "tbik_gemm_workspace_bytes": (_sz, [_i32, _i32, _i64, _i32]),
    "tbik_gemm_ws": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _vp, _sz, _vp]),
    "tbik_gemm_plan": (_i32, [_i32, _i32, _i64, _i32, _i32, _sz, ctypes.POINTER(_i32)]),
    "tbik_gemm_ex": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "tbik_gemm_slabs_workspace_bytes": (_sz, [_i32, _i32, _i64, _i32, _i32, _i32]),
    "tbik_gemm_slabs": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _vp, _sz, _vp]),
    "tbik_gemm_static": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _i64, _i64, _i64, _i32, _i32, _i32, _vp]),
    "tbik_gemm_static_scratch_bytes": (_sz, []),
    "tbik_gemm_static_accepts": (_i32, [_i32, _i32, _i64, _i32]),
    "tbik_gemm_status": (_i32, [ctypes.POINTER(ctypes.c_uint32)]),
    "tbik_ar_meta_size": (_sz, []),
    "tbik_ar_create": (_i32, [ctypes.POINTER(_vp), _i32, _i32, _vp, _sz, _i32, ctypes.POINTER(_vp)]),
    "tbik_ar_destroy": (_i32, [_vp]),
    "tbik_ar_configure": (_i32, [_vp, _i32, _i64]),
    "tbik_ar_register_buffer": (_i32, [_vp, ctypes.POINTER(_vp)]),
    "tbik_ar_tree_allreduce": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp, _sz, _vp]),
    "tbik_ar_allreduce": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp, _sz, _vp]),
    "tbik_ar_tree_allreduce_within": (_i32, [_vp, _vp, _sz, _vp, _i64, _i32, _vp]),
    "tbik_ar_tree_allreduce_rounding": (_i32, [_vp, _vp, _sz, _vp, _i64, _i32, _vp]),
    "tbik_ar_row_split_layer": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i64, _i64, _i32, _i32, _vp, _sz, _vp, _sz,
                                        ctypes.POINTER(_i32), _i32, _i32, _vp, _vp]),
    "tbik_ar_trace": (_i32, [_vp, ctypes.POINTER(ctypes.c_uint64), _i32, ctypes.POINTER(_i32)]),
    "tbik_ar_graph_meta_count": (_i32, [_vp, ctypes.POINTER(_i32)]),
    "tbik_ar_graph_meta": (_i32, [_vp, _vp, ctypes.POINTER(_i64)]),
    "tbik_ar_register_graph_buffers": (_i32, [_vp, ctypes.POINTER(_vp), ctypes.POINTER(ctypes.POINTER(_i64))]),
    "tbik_ar_status": (_i32, [_vp, ctypes.POINTER(ctypes.c_uint32)]),
}

AR_CFG_SCRATCH_BYTES, AR_CFG_ONESHOT_MAX_BYTES, AR_CFG_MAX_BLOCKS, AR_CFG_WAIT_LIMIT_NS = 1, 2, 3, 4


def exported_symbols():
    """Names this binding expects the library to export (kept equal to include/tbik.h)."""
    return sorted(_PROTOTYPES)


def lib() -> ctypes.CDLL:
    """Load the library once.  torch must be imported first so that its libcudart is the one in use."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m llm_reproducibility_b200._build` "
                "(there is no fallback implementation)")
        import torch  # noqa: F401  (loads libcudart.so.12 into the process)
        handle = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error() -> str:
    return lib().tbik_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc != TBIK_OK:
        raise RuntimeError(f"{what} failed ({rc}): {last_error()}")
