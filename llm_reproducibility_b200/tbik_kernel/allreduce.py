"""Registration of `torch.ops.tbik_kernel.*` and thin forwarding functions.

Op names and schemas are those of the reference (mini_allreduce/csrc/common_ops_allreduce.cc:37-58,
mini_allreduce/tbik_kernel/allreduce.py:15-44).  The implementations are calls into the C ABI
(`include/tbik.h`); there is no Python or CPU arithmetic behind them.
"""
from __future__ import annotations

import ctypes
from typing import List, Tuple

import torch

from .. import _lib

_HANDLE_BYTES = 64  # sizeof(cudaIpcMemHandle_t)
_DTYPE_CODE = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_FP16, torch.float32: _lib.DTYPE_FP32}

try:
    _lib.lib()
except Exception as exc:  # the reference raises ImportError when its extension is missing
    raise ImportError(
        "libtbik_b200.so failed to load. Build it with:\n  python -m llm_reproducibility_b200._build\n"
    ) from exc


def _ptr_array(values):
    arr = (ctypes.c_void_p * len(values))()
    for i, v in enumerate(values):
        arr[i] = v
    return arr


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_of(t: torch.Tensor) -> int:
    if _raw_stream is not None and t.device.index is not None:
        return _raw_stream(t.device.index)
    return torch.cuda.current_stream(t.device).cuda_stream


def _is_weak_contiguous(t: torch.Tensor) -> bool:
    return t.is_contiguous() or (
        t.untyped_storage().nbytes() - t.storage_offset() * t.element_size() == t.numel() * t.element_size())


# ------------------------------------------------------------------ implementations
def _init_custom_ar(ipc_tensors: List[int], rank_data: torch.Tensor, rank: int, full_nvlink: bool) -> int:
    world = len(ipc_tensors)
    if world > 8:
        raise ValueError("world size > 8 is not supported")
    if world != 1 and world % 2 != 0:
        raise ValueError("Odd num gpus is not supported for now")
    if rank < 0 or rank >= world:
        raise ValueError("invalid rank passed in")
    out = ctypes.c_void_p()
    with torch.cuda.device(rank_data.device):
        rc = _lib.lib().tbik_ar_create(_ptr_array(ipc_tensors), world, rank, rank_data.data_ptr(),
                                       rank_data.numel() * rank_data.element_size(), int(bool(full_nvlink)),
                                       ctypes.byref(out))
    _lib.check(rc, "tbik_ar_create")
    return int(out.value)


def _run(fa: int, inp: torch.Tensor, out: torch.Tensor, reg_buffer: int, reg_buffer_sz_bytes: int, tree: bool) -> None:
    if inp.dtype != out.dtype:
        raise RuntimeError("inp and out must have the same dtype")
    if inp.numel() != out.numel():
        raise RuntimeError("inp and out must have the same number of elements")
    if not _is_weak_contiguous(out) or not _is_weak_contiguous(inp):
        raise RuntimeError("inp and out must be (weakly) contiguous")
    code = _DTYPE_CODE.get(inp.dtype)
    if code is None:
        raise RuntimeError("custom allreduce only supports float32, float16 and bfloat16")
    fn = _lib.lib().tbik_ar_tree_allreduce if tree else _lib.lib().tbik_ar_allreduce
    with torch.cuda.device(inp.device):
        rc = fn(fa, inp.data_ptr(), out.data_ptr(), inp.numel(), code, reg_buffer or None, reg_buffer_sz_bytes,
                _stream_of(inp))
    _lib.check(rc, "tbik_ar_tree_allreduce" if tree else "tbik_ar_allreduce")


def _all_reduce(fa: int, inp: torch.Tensor, out: torch.Tensor, reg_buffer: int, reg_buffer_sz_bytes: int) -> None:
    _run(fa, inp, out, reg_buffer, reg_buffer_sz_bytes, tree=False)


def _tree_all_reduce(fa: int, inp: torch.Tensor, out: torch.Tensor, reg_buffer: int, reg_buffer_sz_bytes: int) -> None:
    _run(fa, inp, out, reg_buffer, reg_buffer_sz_bytes, tree=True)


def _dispose(fa: int) -> None:
    _lib.check(_lib.lib().tbik_ar_destroy(fa), "tbik_ar_destroy")


def _meta_size() -> int:
    return int(_lib.lib().tbik_ar_meta_size())


def _register_buffer(fa: int, ipc_tensors: List[int]) -> None:
    _lib.check(_lib.lib().tbik_ar_register_buffer(fa, _ptr_array(ipc_tensors)), "tbik_ar_register_buffer")


def _get_graph_buffer_ipc_meta(fa: int) -> Tuple[List[int], List[int]]:
    n = ctypes.c_int()
    _lib.check(_lib.lib().tbik_ar_graph_meta_count(fa, ctypes.byref(n)), "tbik_ar_graph_meta_count")
    handles = (ctypes.c_ubyte * (max(n.value, 1) * _HANDLE_BYTES))()
    offsets = (ctypes.c_int64 * max(n.value, 1))()
    _lib.check(_lib.lib().tbik_ar_graph_meta(fa, ctypes.cast(handles, ctypes.c_void_p), offsets), "tbik_ar_graph_meta")
    return list(handles[: n.value * _HANDLE_BYTES]), list(offsets[: n.value])


def _register_graph_buffers(fa: int, handles: List[List[int]], offsets: List[List[int]]) -> None:
    world = len(handles)
    keep = []
    hptrs = (ctypes.c_void_p * world)()
    optrs = (ctypes.POINTER(ctypes.c_int64) * world)()
    for r in range(world):
        hb = (ctypes.c_ubyte * max(len(handles[r]), 1))(*[int(b) & 0xFF for b in handles[r]])
        ob = (ctypes.c_int64 * max(len(offsets[r]), 1))(*offsets[r])
        keep += [hb, ob]
        hptrs[r] = ctypes.cast(hb, ctypes.c_void_p)
        optrs[r] = ctypes.cast(ob, ctypes.POINTER(ctypes.c_int64))
    _lib.check(_lib.lib().tbik_ar_register_graph_buffers(fa, hptrs, optrs), "tbik_ar_register_graph_buffers")


def _configure(fa: int, key: int, value: int) -> None:
    _lib.check(_lib.lib().tbik_ar_configure(fa, key, value), "tbik_ar_configure")


def _status(fa: int) -> List[int]:
    out = (ctypes.c_uint32 * 8)()
    _lib.check(_lib.lib().tbik_ar_status(fa, out), "tbik_ar_status")
    return list(out)


def _tree_all_reduce_within(fa: int, reg_base: int, byte_offset: int, out: torch.Tensor) -> None:
    """Tree all-reduce of `out.numel()` elements that lie `byte_offset` bytes into the registered buffer at
    `reg_base` (written there in place by a producer kernel); the result goes to `out`."""
    code = _DTYPE_CODE.get(out.dtype)
    if code is None:
        raise RuntimeError("custom allreduce only supports float32, float16 and bfloat16")
    if not _is_weak_contiguous(out):
        raise RuntimeError("out must be (weakly) contiguous")
    with torch.cuda.device(out.device):
        rc = _lib.lib().tbik_ar_tree_allreduce_within(fa, reg_base, byte_offset, out.data_ptr(), out.numel(), code,
                                                      _stream_of(out))
    _lib.check(rc, "tbik_ar_tree_allreduce_within")


def _tree_all_reduce_rounding(fa: int, reg_base: int, byte_offset: int, out: torch.Tensor) -> None:
    """Tree all-reduce of `out.numel()` fp32 contributions that lie `byte_offset` bytes into the registered buffer
    at `reg_base`, summed in fp32 and rounded once to `out`'s 16-bit type (tbik_ar_tree_allreduce_rounding)."""
    if out.dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError("the rounded result is bfloat16 or float16")
    if not _is_weak_contiguous(out):
        raise RuntimeError("out must be (weakly) contiguous")
    with torch.cuda.device(out.device):
        rc = _lib.lib().tbik_ar_tree_allreduce_rounding(fa, reg_base, byte_offset, out.data_ptr(), out.numel(),
                                                        _DTYPE_CODE[out.dtype], _stream_of(out))
    _lib.check(rc, "tbik_ar_tree_allreduce_rounding")


def _row_split_layer(fa: int, A: torch.Tensor, B: torch.Tensor, reg_base: int, reg_bytes: int, block_rows: List[int],
                     comm_ctas: int, side_stream: int, leaf: int = 0) -> torch.Tensor:
    """out = tree all-reduce over ranks of (A @ B), pipelined over blocks of rows (tbik_ar_row_split_layer).
    `side_stream` is the raw handle of the stream the all-reduces run on."""
    from ..tbik.tree_based_matmul import _DTYPE_CODE as GEMM_DTYPES, _LEAF, _workspace, prepare_operands
    if A.dtype not in GEMM_DTYPES or B.dtype != A.dtype:
        raise RuntimeError("row_split_layer supports bfloat16 and float16")
    M, K = A.shape
    N = B.shape[1]
    leaf = leaf or _LEAF[A.dtype]
    A2, W = prepare_operands(A, B)
    out = torch.empty((M, N), device=A.device, dtype=A.dtype)
    with torch.cuda.device(A.device):
        stream = _stream_of(A)
        L = _lib.lib()
        ws = _workspace(A.device, stream, max(int(L.tbik_gemm_workspace_bytes(r, N, K, leaf)) for r in set(block_rows)))
        rows_arr = (ctypes.c_int * len(block_rows))(*block_rows)
        rc = L.tbik_ar_row_split_layer(fa, A2.data_ptr(), W.data_ptr(), out.data_ptr(), M, N, K, max(A2.stride(0), K),
                                       max(W.stride(0), K), GEMM_DTYPES[A.dtype], leaf, reg_base, reg_bytes,
                                       ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                       rows_arr, len(block_rows), comm_ctas, stream, side_stream)
    _lib.check(rc, "tbik_ar_row_split_layer")
    return out


def _trace(fa: int) -> List[int]:
    """Phase time stamps (ns) of the last launch, 8 per CTA, flattened (see tbik_ar_trace)."""
    cap = 320
    buf = (ctypes.c_uint64 * (8 * cap))()
    n = ctypes.c_int()
    _lib.check(_lib.lib().tbik_ar_trace(fa, buf, cap, ctypes.byref(n)), "tbik_ar_trace")
    return [int(v) for v in buf[: 8 * n.value]]


def _tree_matmul(A: torch.Tensor, B: torch.Tensor, bias=None) -> torch.Tensor:
    from ..tbik.tree_based_matmul import matmul_tp_persistent
    return matmul_tp_persistent(A, B, bias)


# ------------------------------------------------------------------ registration (once per process)
_REGISTERED = False


def _register() -> None:
    global _REGISTERED, _LIBRARY
    if _REGISTERED:
        return
    lib = torch.library.Library("tbik_kernel", "FRAGMENT")
    any_key = "CompositeExplicitAutograd"
    lib.define("get_graph_buffer_ipc_meta(int fa) -> (int[], int[])")
    lib.impl("get_graph_buffer_ipc_meta", _get_graph_buffer_ipc_meta, any_key)
    lib.define("register_graph_buffers(int fa, int[][] handles, int[][] offsets) -> ()")
    lib.impl("register_graph_buffers", _register_graph_buffers, any_key)
    lib.define("dispose(int fa) -> ()")
    lib.impl("dispose", _dispose, any_key)
    lib.define("meta_size() -> int")
    lib.impl("meta_size", _meta_size, any_key)
    lib.define("register_buffer(int fa, int[] ipc_tensors) -> ()")
    lib.impl("register_buffer", _register_buffer, any_key)
    lib.define("init_custom_ar(int[] ipc_tensors, Tensor rank_data, int rank, bool full_nvlink) -> int")
    lib.impl("init_custom_ar", _init_custom_ar, "CUDA")
    lib.define("all_reduce(int fa, Tensor inp, Tensor! out, int reg_buffer, int reg_buffer_sz_bytes) -> ()")
    lib.impl("all_reduce", _all_reduce, "CUDA")
    lib.define("tree_all_reduce(int fa, Tensor inp, Tensor! out, int reg_buffer, int reg_buffer_sz_bytes) -> ()")
    lib.impl("tree_all_reduce", _tree_all_reduce, "CUDA")
    # additions of this implementation
    lib.define("configure(int fa, int key, int value) -> ()")
    lib.impl("configure", _configure, any_key)
    lib.define("status(int fa) -> int[]")
    lib.impl("status", _status, any_key)
    lib.define("tree_all_reduce_within(int fa, int reg_base, int byte_offset, Tensor! out) -> ()")
    lib.impl("tree_all_reduce_within", _tree_all_reduce_within, "CUDA")
    lib.define("tree_all_reduce_rounding(int fa, int reg_base, int byte_offset, Tensor! out) -> ()")
    lib.impl("tree_all_reduce_rounding", _tree_all_reduce_rounding, "CUDA")
    lib.define("row_split_layer(int fa, Tensor A, Tensor B, int reg_base, int reg_bytes, int[] block_rows, "
               "int comm_ctas, int side_stream, int leaf=0) -> Tensor")
    lib.impl("row_split_layer", _row_split_layer, "CUDA")
    lib.define("trace(int fa) -> int[]")
    lib.impl("trace", _trace, any_key)
    lib.define("tree_matmul(Tensor A, Tensor B, Tensor? bias=None) -> Tensor")
    lib.impl("tree_matmul", _tree_matmul, "CUDA")
    _LIBRARY = lib  # keep alive
    _REGISTERED = True


_register()


def init_custom_ar(*args, **kwargs):
    return torch.ops.tbik_kernel.init_custom_ar.default(*args, **kwargs)


def dispose(*args, **kwargs):
    return torch.ops.tbik_kernel.dispose.default(*args, **kwargs)


def all_reduce(*args, **kwargs):
    return torch.ops.tbik_kernel.all_reduce.default(*args, **kwargs)


def tree_all_reduce(*args, **kwargs):
    return torch.ops.tbik_kernel.tree_all_reduce.default(*args, **kwargs)


def get_graph_buffer_ipc_meta(*args, **kwargs):
    return torch.ops.tbik_kernel.get_graph_buffer_ipc_meta.default(*args, **kwargs)


def register_buffer(*args, **kwargs):
    return torch.ops.tbik_kernel.register_buffer.default(*args, **kwargs)


def register_graph_buffers(*args, **kwargs):
    return torch.ops.tbik_kernel.register_graph_buffers.default(*args, **kwargs)


def meta_size(*args, **kwargs):
    return torch.ops.tbik_kernel.meta_size.default(*args, **kwargs)


def tree_all_reduce_within(*args, **kwargs):
    return torch.ops.tbik_kernel.tree_all_reduce_within.default(*args, **kwargs)


def tree_all_reduce_rounding(*args, **kwargs):
    return torch.ops.tbik_kernel.tree_all_reduce_rounding.default(*args, **kwargs)


def row_split_layer(*args, **kwargs):
    return torch.ops.tbik_kernel.row_split_layer.default(*args, **kwargs)


def trace(*args, **kwargs):
    return torch.ops.tbik_kernel.trace.default(*args, **kwargs)


def configure(*args, **kwargs):
    return torch.ops.tbik_kernel.configure.default(*args, **kwargs)


def status(*args, **kwargs):
    return torch.ops.tbik_kernel.status.default(*args, **kwargs)
