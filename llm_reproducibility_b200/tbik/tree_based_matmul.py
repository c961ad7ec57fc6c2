"""`matmul_tp_persistent`: tree-ordered, batch- and TP-invariant matmul on B200.

Drop-in for the reference's `src/tbik/tree_based_matmul.py:190-276` (same name, arguments,
return value and assertions); the Triton kernel behind it is replaced by the hand-written
tcgen05/TMA kernel in `csrc/tree_gemm_sm100a.cu`, reached through the C ABI (`tbik_gemm`).
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .. import _lib

# Leaf (K-chunk) width per dtype: the reference's BLOCK_SIZE_K (tree_based_matmul.py:206-231).
_LEAF = {torch.bfloat16: 256, torch.float16: 256}
_DTYPE_CODE = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16}


def tree_shape(K: int, leaf: int):
    """(T, F, L) exactly as the reference derives them (tree_based_matmul.py:240-249)."""
    import ctypes
    T, F, L = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    _lib.check(_lib.lib().tbik_tree_shape(K, leaf, ctypes.byref(T), ctypes.byref(F), ctypes.byref(L)), "tbik_tree_shape")
    return T.value, F.value, L.value


def leaf_for(K_total: int, max_tp: int = 8, dtype: torch.dtype = torch.bfloat16) -> int:
    """Leaf width for a row-split layer whose FULL reduction length is `K_total`, such that every tensor-parallel
    degree up to `max_tp` (a power of two) sees a whole, aligned subtree per rank -- and therefore every degree,
    TP = 1 included, produces the same bits.

    The reference fixes the leaf at 256 (src/tbik/tree_based_matmul.py:206-231) and asserts K % 256 == 0 per rank
    (:240-243), which a Qwen3-32B down_proj (K = 25600) fails at TP = 8 (3200 columns per rank).  Here the leaf is
    the widest of 256, 128, 64 that divides K_total / max_tp and whose tree has at least max_tp subtrees at one
    level; all ranks and all TP degrees must call with the same K_total and max_tp."""
    if max_tp < 1 or max_tp & (max_tp - 1):
        raise ValueError("max_tp must be a power of two")
    for leaf in ((_LEAF.get(dtype, 256)), 128, 64):
        if K_total % (leaf * max_tp) != 0:
            continue
        _, _, L = tree_shape(K_total, leaf)
        if (1 << (L - 1)) % max_tp == 0:
            return leaf
    raise ValueError(f"no leaf width of 256, 128 or 64 splits K = {K_total} into {max_tp} aligned subtrees")


def leaf_for_fp32_nodes(K_total: int, max_tp: int = 8) -> int:
    """Leaf width for the fp32-node mode: K_total / max_tp, so that the tree has exactly `max_tp` leaves, every
    level is binary, every tensor-parallel degree up to `max_tp` holds a whole subtree per rank, and the stack of
    the fastest tilings (three levels) suffices.  Long leaves cost no accuracy here: a leaf is one fp32 tensor-core
    accumulation that is not rounded afterwards."""
    if max_tp < 1 or max_tp & (max_tp - 1):
        raise ValueError("max_tp must be a power of two")
    if K_total % (64 * max_tp) != 0:
        raise ValueError(f"K = {K_total} does not split into {max_tp} leaves that are multiples of 64")
    return K_total // max_tp


def _node_code(A: torch.Tensor, node_dtype, out_dtype) -> int:
    """C-ABI node mode for (node_dtype, out_dtype); None / the operand type = the reference's arithmetic."""
    if node_dtype is None and os.environ.get("TBIK_NODE_FP32") == "1":
        node_dtype = torch.float32
    if node_dtype is None or node_dtype == A.dtype:
        if out_dtype not in (None, A.dtype):
            raise ValueError("out_dtype other than the operand type needs node_dtype=torch.float32")
        return _lib.NODE_INPUT
    if node_dtype != torch.float32:
        raise ValueError("node_dtype is the operand type or torch.float32")
    if out_dtype in (None, A.dtype):
        return _lib.NODE_FP32
    if out_dtype != torch.float32:
        raise ValueError("out_dtype is the operand type or torch.float32")
    return _lib.NODE_FP32_OUT_FP32


def _k_major_weight(B: torch.Tensor) -> torch.Tensor:
    """Return W[N,K] (K contiguous) holding B[K,N]'s values.

    `weight.t()` -- what the row-parallel layer passes -- is already such a view, so this is
    free on the hot path; any other layout is copied once.
    """
    Wt = B.t()
    if Wt.stride(1) == 1 and Wt.stride(0) % 8 == 0 and Wt.data_ptr() % 16 == 0 and Wt.stride(0) >= Wt.shape[1]:
        return Wt
    return Wt.contiguous()


_WORKSPACES = {}  # (device index, stream) -> uint8 tensor; scratch for the upper levels of the tree stack


def _workspace(device: torch.device, stream: int, nbytes: int) -> Optional[torch.Tensor]:
    """Scratch buffer for one (device, stream); grown on demand, never shared between streams.  Allocated
    zero-filled: the arrival counters at its head must start at zero, and every call leaves them zero."""
    if nbytes == 0:
        return None
    key = (device.index, stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


_WS_NEED = {}  # (device index, M, N, K, leaf) -> bytes of scratch the automatic schedule wants

# raw handle of the current stream of a device: the private fast getter when this torch has it (a fraction of a
# microsecond), the public API otherwise (several microseconds per call, which is felt at decode sizes)
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or (lambda index: torch.cuda.current_stream(index).cuda_stream)


def _launch(A, W, C, M, N, K, leaf, dev, max_ctas=0, node=_lib.NODE_INPUT) -> int:
    """Enqueue the GEMM on the current stream of `dev` (which must be the current device)."""
    L = _lib.lib()
    if node != _lib.NODE_INPUT:
        # fp32 nodes: the stack lives in tensor memory, no workspace
        return L.tbik_gemm_ex(A.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K,
                              max(A.stride(0), K), max(W.stride(0), K), max(C.stride(0), N),
                              _DTYPE_CODE[A.dtype], leaf, node, max_ctas, 0, None, 0, _raw_stream(dev.index))
    key = (dev.index, M, N, K, leaf)
    need = _WS_NEED.get(key)
    if need is None:
        need = _WS_NEED[key] = int(L.tbik_gemm_workspace_bytes(M, N, K, leaf))
    stream = _raw_stream(dev.index)
    ws = _workspace(dev, stream, need)
    if max_ctas > 0:
        return L.tbik_gemm_ex(A.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K,
                              max(A.stride(0), K), max(W.stride(0), K), max(C.stride(0), N),
                              _DTYPE_CODE[A.dtype], leaf, _lib.NODE_INPUT, max_ctas, 0,
                              ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, stream)
    return L.tbik_gemm_ws(A.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K,
                          max(A.stride(0), K), max(W.stride(0), K), max(C.stride(0), N),
                          _DTYPE_CODE[A.dtype], leaf, _lib.NODE_INPUT,
                          ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0, stream)


def prepare_operands(A: torch.Tensor, B: torch.Tensor):
    """(A', W) in the layout the kernels take: A' row-major with aligned rows, W = B^T with K contiguous."""
    M, K = A.shape
    if A.stride(1) != 1 or A.stride(0) % 8 != 0 or A.data_ptr() % 16 != 0 or (M > 1 and A.stride(0) < K):
        A = A.contiguous()
    return A, _k_major_weight(B)


def matmul_tp_persistent(A: torch.Tensor, B: torch.Tensor, bias: Optional[torch.Tensor] = None,
                         *, leaf: Optional[int] = None, out: Optional[torch.Tensor] = None,
                         max_ctas: int = 0, node_dtype: Optional[torch.dtype] = None,
                         out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """C = A @ B with the K reduction in the fixed tree order; returns a new [M, N] tensor of A's dtype.

    A: [M, K]; B: [K, N] (any strides; a K-contiguous view such as `weight.t()` is used in place).
    `leaf` (keyword, extension) overrides the leaf width; the default is the reference's 256.
    `max_ctas` (keyword, extension) bounds the CTAs of the launch (0 = one per SM); the bits do not depend on it.
    `node_dtype=torch.float32` (keyword, extension; also TBIK_NODE_FP32=1): leaves and nodes stay fp32 and only the
    root is rounded -- the same tree, so the invariances hold, but not the reference's bits; the default leaf is
    then K / 8 (`leaf_for_fp32_nodes`).  `out_dtype=torch.float32` with it returns the unrounded root (what a
    tensor-parallel rank contributes to the cross-rank levels).
    """
    assert A.shape[-1] == B.shape[-2], "Dim doesn't match"
    assert A.dim() == 2 and B.dim() == 2
    if not A.is_cuda:
        raise RuntimeError("matmul_tp_persistent needs CUDA tensors (there is no CPU fallback)")
    if A.dtype not in _LEAF:
        raise NotImplementedError(f"matmul_tp_persistent: dtype {A.dtype} is not supported by the sm_100a kernel")
    assert B.dtype == A.dtype
    M, K = A.shape
    _, N = B.shape
    node = _node_code(A, node_dtype, out_dtype)
    if node == _lib.NODE_INPUT:
        leaf = leaf or int(os.environ.get("TBIK_LEAF", _LEAF[A.dtype]))
    else:
        leaf = leaf or leaf_for_fp32_nodes(K, 8)
    assert K % leaf == 0
    if A.stride(1) != 1 or A.stride(0) % 8 != 0 or A.data_ptr() % 16 != 0 or (M > 1 and A.stride(0) < K):
        A = A.contiguous()
    W = _k_major_weight(B)
    c_dtype = torch.float32 if node == _lib.NODE_FP32_OUT_FP32 else A.dtype
    C = out if out is not None else torch.empty((M, N), device=A.device, dtype=c_dtype)
    assert C.shape == (M, N) and C.stride(1) == 1 and C.dtype == c_dtype
    dev = A.device
    if torch.cuda.current_device() == dev.index:
        rc = _launch(A, W, C, M, N, K, leaf, dev, max_ctas, node)
    else:
        with torch.cuda.device(dev):
            rc = _launch(A, W, C, M, N, K, leaf, dev, max_ctas, node)
    if rc != 0:
        _lib.check(rc, "tbik_gemm_ws")
    if bias is not None:
        C += bias
    return C


def gemm_device_status():
    """(code, block, role, _) of the GEMM kernels' bounded-wait watchdog; code 0 = healthy."""
    import ctypes
    out = (ctypes.c_uint32 * 4)()
    _lib.check(_lib.lib().tbik_gemm_status(out), "tbik_gemm_status")
    return tuple(out)
