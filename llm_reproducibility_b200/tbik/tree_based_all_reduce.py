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


_COMM_STREAMS = {}  # device index -> side stream the row blocks are reduced on

# Row-block pipeline of `tree_matmul_all_reduce`: rows per block (a multiple of the 256-row GEMM tile: 2048 rows
# x 4096 columns are exactly four waves of 256x128 tiles on 64 CTA pairs) and the CTAs left to the all-reduce
# while a GEMM runs beside it.
_PIPE_ROWS = int(os.environ.get("TBIK_PIPELINE_ROWS", "2048"))
_PIPE_COMM_CTAS = int(os.environ.get("TBIK_PIPELINE_COMM_CTAS", "20"))


def _pipeline_blocks(M: int, N: int, K_local: int, world: int) -> int:
    """How many row blocks to cut the layer into (1 = no pipelining).

    Batch invariance makes the cut free of numerical consequences: a row of C does not depend on which other
    rows are computed with it.  Pipelining pays when the GEMM of a block takes about as long as its all-reduce,
    so that one hides the other; when the all-reduce dominates (short K per rank, many ranks) one large message
    is cheaper than several small ones.  Estimates: 1.2 PFLOP/s for the GEMM, 500 GB/s of bus bandwidth."""
    mode = os.environ.get("TBIK_PIPELINE", "auto")
    if mode == "0" or world < 2 or M < 2 * _PIPE_ROWS:
        return 1
    if mode != "1":
        t_gemm = 2.0 * M * N * K_local / 1.2e15
        t_ar = 2.0 * (world - 1) / world * M * N * 2 / 500e9
        if t_gemm < 0.5 * t_ar:
            return 1
    return -(-M // _PIPE_ROWS)


def tree_matmul_all_reduce(A: torch.Tensor, B: torch.Tensor, device_group=None) -> torch.Tensor:
    """Row-split layer in one call: this rank's tree matmul, then the tree all-reduce.

    Same bits as `tree_all_reduce_sum(matmul_tp_persistent(A, B), group)`.  The GEMM writes its partial
    result directly into the IPC-registered buffer the peers read from (no staging copy), then the tree
    all-reduce kernel runs.  Large calls are cut into blocks of rows: block i is reduced on a side stream by a
    few CTAs while the remaining CTAs multiply block i + 1, so most of the NVLink time hides behind the
    tensor-core time (the partial sums of different rows never meet, so the cut cannot change a bit)."""
    global custom_ar
    from .tree_based_matmul import matmul_tp_persistent
    if custom_ar is None:
        from ..mini_allreduce import CustomTreeAllreduce
        custom_ar = CustomTreeAllreduce(group=device_group, device=A.device, max_size=_max_size())
    view = None
    M, N = A.shape[0], B.shape[1]
    if not custom_ar.disabled:
        # under stream capture the buffer is usable as well: it was registered when the communicator was built
        view = custom_ar.registered_view((M, N), A.dtype)
    if view is None:
        return tree_all_reduce_sum(matmul_tp_persistent(A, B), device_group)
    capturing = A.is_cuda and torch.cuda.is_current_stream_capturing()
    nblk = 1 if (capturing or custom_ar._IS_CAPTURING) else _pipeline_blocks(M, N, A.shape[1], custom_ar.world_size)
    if nblk == 1:
        matmul_tp_persistent(A, B, out=view)
        if custom_ar._IS_CAPTURING and not capturing:
            return torch.zeros_like(view)  # warm-up run before a capture: only the shape matters
        return custom_ar.all_reduce(view, registered=True)
    dev = A.device
    main = torch.cuda.current_stream(dev)
    comm = _COMM_STREAMS.get(dev.index)
    if comm is None:
        comm = _COMM_STREAMS[dev.index] = torch.cuda.Stream(device=dev, priority=-1)
    out = torch.empty((M, N), device=dev, dtype=A.dtype)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    gemm_ctas = max(2, sms - _PIPE_COMM_CTAS)
    rows = -(-M // nblk)
    rows = -(-rows // 256) * 256
    r0 = 0
    while r0 < M:
        r1 = min(M, r0 + rows)
        last = r1 == M
        # the first block has the GPU to itself; the later ones leave SMs to the all-reduce of their predecessor
        matmul_tp_persistent(A[r0:r1], B, out=view[r0:r1], max_ctas=0 if r0 == 0 else gemm_ctas)
        ready = main.record_event()
        with torch.cuda.stream(comm):
            comm.wait_event(ready)
            custom_ar.tree_all_reduce_rows(view[r0:r1], out[r0:r1], max_blocks=0 if last else _PIPE_COMM_CTAS)
        r0 = r1
    main.wait_stream(comm)
    return out


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
