"""Function-level API of the native all-reduce ops (reference: mini_allreduce/custom_all_reduce_ops.py:46-87).

The eight reference functions keep their names and signatures; `configure` and `status` are
additions.  `IS_CUSTOM_AR_AVAILABLE` is False when CUDA or the native library is absent.
"""
import logging
from typing import List, Tuple

import torch

from .utils import is_cuda

logger = logging.getLogger(__name__)

IS_CUSTOM_AR_AVAILABLE = is_cuda()
_custom_ar = None

try:
    from ..tbik_kernel import allreduce as _custom_ar
except ImportError as exc:
    if IS_CUSTOM_AR_AVAILABLE:
        logger.warning("Failed to import tbik_kernel.allreduce: %r", exc)
    IS_CUSTOM_AR_AVAILABLE = False


def init_custom_ar(ipc_tensors: List[int], rank_data: torch.Tensor, rank: int, full_nvlink: bool) -> int:
    return _custom_ar.init_custom_ar(ipc_tensors, rank_data, rank, full_nvlink)


def all_reduce(fa: int, inp: torch.Tensor, out: torch.Tensor, reg_buffer: int, reg_buffer_sz_bytes: int) -> None:
    _custom_ar.all_reduce(fa, inp, out, reg_buffer, reg_buffer_sz_bytes)


def tree_all_reduce(fa: int, inp: torch.Tensor, out: torch.Tensor, reg_buffer: int, reg_buffer_sz_bytes: int) -> None:
    _custom_ar.tree_all_reduce(fa, inp, out, reg_buffer, reg_buffer_sz_bytes)


def dispose(fa: int) -> None:
    _custom_ar.dispose(fa)


def meta_size() -> int:
    return _custom_ar.meta_size()


def register_buffer(fa: int, ipc_tensors: List[int]) -> None:
    _custom_ar.register_buffer(fa, ipc_tensors)


def get_graph_buffer_ipc_meta(fa: int) -> Tuple[List[int], List[int]]:
    return _custom_ar.get_graph_buffer_ipc_meta(fa)


def register_graph_buffers(fa: int, handles: List[List[int]], offsets: List[List[int]]) -> None:
    _custom_ar.register_graph_buffers(fa, handles, offsets)


def tree_all_reduce_within(fa: int, reg_base: int, byte_offset: int, out: torch.Tensor) -> None:
    """Tree all-reduce of a message a producer wrote in place inside a registered buffer (addition)."""
    _custom_ar.tree_all_reduce_within(fa, reg_base, byte_offset, out)


def tree_all_reduce_rounding(fa: int, reg_base: int, byte_offset: int, out: torch.Tensor) -> None:
    """Tree all-reduce of fp32 contributions inside a registered buffer, rounded once to `out`'s 16-bit type
    (addition: the cross-rank levels of a tree whose nodes stay fp32)."""
    _custom_ar.tree_all_reduce_rounding(fa, reg_base, byte_offset, out)


def row_split_layer(fa: int, A: torch.Tensor, B: torch.Tensor, reg_base: int, reg_bytes: int, block_rows: List[int],
                    comm_ctas: int, side_stream: int, leaf: int = 0) -> torch.Tensor:
    """Row-split GEMM + tree all-reduce pipelined over blocks of rows on two streams (addition)."""
    return _custom_ar.row_split_layer(fa, A, B, reg_base, reg_bytes, block_rows, comm_ctas, side_stream, leaf)


def trace(fa: int) -> List[int]:
    """Per-CTA phase time stamps of the last launch; needs configure(CFG_TRACE, 1) (addition)."""
    return _custom_ar.trace(fa)


# keys of `configure`
CFG_SCRATCH_BYTES, CFG_ONESHOT_MAX_BYTES, CFG_MAX_BLOCKS, CFG_WAIT_LIMIT_NS, CFG_THREADS = 1, 2, 3, 4, 5
CFG_PUSH_MIN_BYTES, CFG_PUSH_CHUNKS, CFG_VEC_PACKS, CFG_LOADS_IN_FLIGHT, CFG_TRACE, CFG_CLUSTER_PAIRS = 6, 7, 8, 9, 10, 11


def configure(fa: int, key: int, value: int) -> None:
    _custom_ar.configure(fa, key, value)


def status(fa: int) -> List[int]:
    return _custom_ar.status(fa)
