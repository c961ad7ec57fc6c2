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

# Row-block pipeline of `tree_matmul_all_reduce`.  Measured on two B200s (M = 8192, N = 4096, K per rank 2048 and
# 6144): an all-reduce launch costs about 25 us of barriers and launch latency whatever its size, a GEMM cut into
# blocks loses a few per cent per cut, and an all-reduce that runs beside a GEMM moves its bytes 35 - 80 % slower
# than alone (both kernels' traffic meets in the peers' memory systems).  What survives: two equal blocks, 32 CTAs
# for the all-reduce beside the second GEMM (fewer CTAs lose link rate, more starve the GEMM), and only where GEMM
# and all-reduce take about equally long (o_proj at TP = 2: 243 -> 222 us; down_proj at TP = 2, three times more
# GEMM than all-reduce: no cut beat GEMM-then-all-reduce, 417 us; down_proj at TP = 8, half as much GEMM as
# all-reduce: 284 us either way).
_PIPE_MIN_ROWS = 1024      # shortest block worth a launch of its own
_PIPE_COMM_CTAS = 32
_PIPE_FORCE = None         # tests: (block_rows, comm_ctas) to use instead of the plan below


def _estimates(M: int, N: int, K_local: int, world: int):
    """(GEMM, all-reduce) seconds for one layer on one rank: 1.15 PFLOP/s plus 5 us for the GEMM; 25 us plus the
    bytes that cross NVLink at 700 GB/s for the all-reduce (S at two ranks, 2 (n-1)/n S beyond)."""
    t_gemm = 2.0 * M * N * K_local / 1.15e15 + 5e-6
    S = M * N * 2
    t_ar = 25e-6 + (S if world == 2 else 2.0 * (world - 1) / world * S) / 700e9
    return t_gemm, t_ar


def _pipeline_plan(M: int, N: int, K_local: int, world: int):
    """(rows of each block, CTAs for the all-reduce beside a GEMM), or None for "GEMM, then one all-reduce".

    Two blocks: while the second block's GEMM runs on most of the SMs, the first block's all-reduce runs on the
    rest; the second block's all-reduce then has the GPU to itself.  Batch invariance makes the cut free of
    numerical consequences: a row of C does not depend on which other rows are computed with it."""
    mode = os.environ.get("TBIK_PIPELINE", "auto")
    if mode == "0" or world < 2 or M < 2 * _PIPE_MIN_ROWS or N % 8:
        return None
    if _PIPE_FORCE is not None:
        return _PIPE_FORCE
    if mode != "1":
        t_gemm, t_ar = _estimates(M, N, K_local, world)
        if not (0.7 * t_ar <= t_gemm <= 1.5 * t_ar):
            return None
    first = -(-(M // 2) // 256) * 256
    return [first, M - first], _PIPE_COMM_CTAS


def tree_matmul_all_reduce(A: torch.Tensor, B: torch.Tensor, device_group=None, leaf=None,
                           node_dtype=None) -> torch.Tensor:
    """Row-split layer in one call: this rank's tree matmul, then the tree all-reduce.

    Same bits as `tree_all_reduce_sum(matmul_tp_persistent(A, B), group)`.  The GEMM writes its partial
    result directly into the IPC-registered buffer the peers read from (no staging copy), then the tree
    all-reduce kernel runs.  Large calls are cut into blocks of rows: block i is reduced on a side stream by a
    few CTAs while the remaining CTAs multiply block i + 1, so most of the NVLink time hides behind the
    tensor-core time (the partial sums of different rows never meet, so the cut cannot change a bit).
    `leaf` (extension): leaf width, the same on every rank and at every TP degree (see `leaf_for`).
    `node_dtype=torch.float32` (extension; also TBIK_NODE_FP32=1): the fp32-node mode.  Each rank writes the
    unrounded fp32 root of its subtree into the registered buffer, the cross-rank levels add in fp32, and the result
    is rounded once -- bit-identical to `matmul_tp_persistent(A_full, B_full, node_dtype=torch.float32, leaf=leaf)`
    on one GPU.  `leaf` is then required (`leaf_for_fp32_nodes(K_total, max_tp)`), since only the caller knows the
    unsharded K."""
    global custom_ar
    from .tree_based_matmul import matmul_tp_persistent
    if custom_ar is None:
        from ..mini_allreduce import CustomTreeAllreduce
        custom_ar = CustomTreeAllreduce(group=device_group, device=A.device, max_size=_max_size())
    if node_dtype is None and os.environ.get("TBIK_NODE_FP32") == "1":
        node_dtype = torch.float32
    if node_dtype == torch.float32:
        if leaf is None:
            raise ValueError("fp32 nodes: pass the layer's leaf width (leaf_for_fp32_nodes(K_total, max_tp))")
        if custom_ar.disabled:
            raise RuntimeError("fp32 nodes across ranks need the peer-to-peer all-reduce (it is disabled here)")
        view32 = custom_ar.registered_view((A.shape[0], B.shape[1]), torch.float32)
        if view32 is None:
            raise RuntimeError("fp32 nodes: the partial result does not fit the registered buffer (raise TBIK_AR_MAX_SIZE)")
        matmul_tp_persistent(A, B, out=view32, leaf=leaf, node_dtype=torch.float32, out_dtype=torch.float32)
        return custom_ar.all_reduce_rounding(view32, A.dtype)
    view = None
    M, N = A.shape[0], B.shape[1]
    if not custom_ar.disabled:
        # under stream capture the buffer is usable as well: it was registered when the communicator was built
        view = custom_ar.registered_view((M, N), A.dtype)
    if view is None:
        return tree_all_reduce_sum(matmul_tp_persistent(A, B, leaf=leaf), device_group)
    capturing = A.is_cuda and torch.cuda.is_current_stream_capturing()
    plan = None if (capturing or custom_ar._IS_CAPTURING) else _pipeline_plan(M, N, A.shape[1], custom_ar.world_size)
    if plan is None:
        matmul_tp_persistent(A, B, out=view, leaf=leaf)
        if custom_ar._IS_CAPTURING and not capturing:
            return torch.zeros_like(view)  # warm-up run before a capture: only the shape matters
        return custom_ar.all_reduce(view, registered=True)
    dev = A.device
    comm = _COMM_STREAMS.get(dev.index)
    if comm is None:
        comm = _COMM_STREAMS[dev.index] = torch.cuda.Stream(device=dev, priority=-1)
    from ..mini_allreduce import custom_all_reduce_ops as ops
    # one native call enqueues all blocks: GEMMs on the current stream, all-reduces on the side stream, the
    # events between them, and the final join (the current stream waits for the last all-reduce)
    block_rows, comm_ctas = plan
    return ops.row_split_layer(custom_ar._ptr, A, B, custom_ar.buffer_ptrs[custom_ar.rank], custom_ar.max_size,
                               block_rows, comm_ctas, comm.cuda_stream, leaf or 0)


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
