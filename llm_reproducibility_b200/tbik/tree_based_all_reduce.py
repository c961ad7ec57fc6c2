"""`tree_all_reduce_sum`: cross-rank sum in the fixed rank-pair tree order.

Drop-in for the reference's `src/tbik/tree_based_all_reduce.py:4-37`.  Differences:
  * the peer-to-peer kernel serves every size up to the communicator's `max_size` (the
    reference hands everything above 2**16 elements to NCCL all_gather + adds); the cut-off
    stays available through $TBIK_AR_NATIVE_CUTOFF (elements; 0 = none);
  * only "communicator disabled" or "tensor not eligible" fall back to the native path; real
    errors are raised instead of being swallowed by a bare `except`.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

custom_ar = None  # per-process singleton, bound to the first group it is used with


def _max_size() -> int:
    return int(os.environ.get("TBIK_AR_MAX_SIZE", 128 * 1024 * 1024))


def tree_all_reduce_sum(x: torch.Tensor, device_group=None) -> torch.Tensor:
    global custom_ar
    cutoff = int(os.environ.get("TBIK_AR_NATIVE_CUTOFF", "0"))
    if cutoff and x.numel() > cutoff:
        return tree_all_reduce_sum_native(x, device_group)
    if custom_ar is None:
        from ..mini_allreduce import CustomTreeAllreduce
        custom_ar = CustomTreeAllreduce(group=device_group, device=x.device, max_size=_max_size())
    if custom_ar.disabled:
        return tree_all_reduce_sum_native(x, device_group)
    y = custom_ar.custom_tree_all_reduce(x)
    if y is None:  # not eligible (size, alignment, layout)
        return tree_all_reduce_sum_native(x, device_group)
    return y


def tree_matmul_all_reduce(A: torch.Tensor, B: torch.Tensor, device_group=None) -> torch.Tensor:
    """Row-split layer in one call: this rank's tree matmul, then the tree all-reduce.

    Same bits as `tree_all_reduce_sum(matmul_tp_persistent(A, B), group)`.  Default: the GEMM writes its
    partial result directly into the IPC-registered buffer the peers read from (no staging copy), then the
    tree all-reduce kernel runs.  With $TBIK_FUSED=1 the single fused kernel is used instead
    (`CustomTreeAllreduce.matmul_tree_all_reduce`): same bits; on the measured B200s one SM pulls only
    about 12-15 GB/s over NVLink, so the communication CTAs it takes from the GEMM cost more than the
    overlap returns, which is why it is not the default."""
    global custom_ar
    from .tree_based_matmul import matmul_tp_persistent
    if custom_ar is None:
        from ..mini_allreduce import CustomTreeAllreduce
        custom_ar = CustomTreeAllreduce(group=device_group, device=A.device, max_size=_max_size())
    if not custom_ar.disabled and os.environ.get("TBIK_FUSED", "0") == "1":
        y = custom_ar.matmul_tree_all_reduce(A, B)  # GEMM and all-reduce overlapped in one kernel
        if y is not None:
            return y
    view = None
    capturing = A.is_cuda and torch.cuda.is_current_stream_capturing()
    if not custom_ar.disabled and not custom_ar._IS_CAPTURING and not capturing:
        view = custom_ar.registered_view((A.shape[0], B.shape[1]), A.dtype)
    if view is None:
        return tree_all_reduce_sum(matmul_tp_persistent(A, B), device_group)
    matmul_tp_persistent(A, B, out=view)
    return custom_ar.all_reduce(view, registered=True)


def tree_all_reduce_sum_native(x: torch.Tensor, device_group=None) -> torch.Tensor:
    """all_gather, then pairwise in-place adds in tree order (library collective; the comparator)."""
    world_size = dist.get_world_size(device_group)
    if world_size & (world_size - 1) != 0:
        raise ValueError("world_size must be the pow of 2 in order to use all_reduce_sum。")
    result = [torch.zeros_like(x) for _ in range(world_size)]
    dist.all_gather(result, x, group=device_group)
    for level in range(1, world_size.bit_length()):
        for left in range(0, world_size, 1 << level):
            right = left + (1 << (level - 1))
            result[left] += result[right]
    return result[0]


def reset_communicator() -> None:
    """Close and forget the singleton (tests, or after the process group changed)."""
    global custom_ar
    if custom_ar is not None:
        custom_ar.close()
        custom_ar = None
