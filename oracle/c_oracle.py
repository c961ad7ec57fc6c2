"""ctypes loader for the C restatement of the oracle (TEST INFRASTRUCTURE ONLY; see oracle/tbik_ref.c)."""
import ctypes
from typing import Sequence

import torch

from . import build_c

_DT = {torch.bfloat16: 0, torch.float16: 1}
_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = ctypes.CDLL(build_c.build())
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
        L.tbik_oracle_matmul.restype = i32
        L.tbik_oracle_matmul.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32]
        L.tbik_oracle_matmul_fp32_nodes.restype = i32
        L.tbik_oracle_matmul_fp32_nodes.argtypes = [vp, vp, vp, i32, i32, i32, i32, i32]
        L.tbik_oracle_tree_allreduce.restype = i32
        L.tbik_oracle_tree_allreduce.argtypes = [ctypes.POINTER(vp), i32, vp, i64, i32]
        L.tbik_oracle_tree_shape.restype = i32
        L.tbik_oracle_tree_shape.argtypes = [i64, i32, ctypes.POINTER(i32), ctypes.POINTER(i32), ctypes.POINTER(i32)]
        L.tbik_oracle_up.restype = None
        L.tbik_oracle_up.argtypes = [vp, vp, i64, i32]
        L.tbik_oracle_down.restype = None
        L.tbik_oracle_down.argtypes = [vp, vp, i64, i32]
        _lib = L
    return _lib


def matmul(A: torch.Tensor, B: torch.Tensor, leaf: int = 256) -> torch.Tensor:
    """C = A @ B in the reference's tree order; A [M,K], B [K,N], bf16 or fp16 CPU tensors."""
    assert A.device.type == "cpu" and A.dtype in _DT and B.dtype == A.dtype
    A, B = A.contiguous(), B.contiguous()
    M, K = A.shape
    N = B.shape[1]
    C = torch.empty(M, N, dtype=A.dtype)
    rc = lib().tbik_oracle_matmul(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, leaf, _DT[A.dtype])
    if rc != 0:
        raise ValueError(f"tbik_oracle_matmul failed with {rc}")
    return C


def matmul_fp32_nodes(A: torch.Tensor, B: torch.Tensor, leaf: int) -> torch.Tensor:
    """The same tree with fp32 nodes and nothing rounded: the fp32 root, [M, N] float32."""
    assert A.device.type == "cpu" and A.dtype in _DT and B.dtype == A.dtype
    A, B = A.contiguous(), B.contiguous()
    M, K = A.shape
    N = B.shape[1]
    C = torch.empty(M, N, dtype=torch.float32)
    rc = lib().tbik_oracle_matmul_fp32_nodes(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, leaf, _DT[A.dtype])
    if rc != 0:
        raise ValueError(f"tbik_oracle_matmul_fp32_nodes failed with {rc}")
    return C


def tree_allreduce(parts: Sequence[torch.Tensor]) -> torch.Tensor:
    parts = [p.contiguous() for p in parts]
    dt = parts[0].dtype
    assert dt in _DT
    out = torch.empty_like(parts[0])
    arr = (ctypes.c_void_p * len(parts))(*[p.data_ptr() for p in parts])
    rc = lib().tbik_oracle_tree_allreduce(arr, len(parts), out.data_ptr(), out.numel(), _DT[dt])
    if rc != 0:
        raise ValueError(f"tbik_oracle_tree_allreduce failed with {rc}")
    return out


def up(x: torch.Tensor) -> torch.Tensor:
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=torch.float32)
    lib().tbik_oracle_up(x.data_ptr(), out.data_ptr(), x.numel(), _DT[x.dtype])
    return out


def down(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    x = x.contiguous().float()
    out = torch.empty(x.shape, dtype=dtype)
    lib().tbik_oracle_down(x.data_ptr(), out.data_ptr(), x.numel(), _DT[dtype])
    return out
