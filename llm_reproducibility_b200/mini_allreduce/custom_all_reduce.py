"""`CustomAllreduce` / `CustomTreeAllreduce`: the per-process communicator objects.

Same constructor, attributes, methods and return conventions as the reference classes
(mini_allreduce/custom_all_reduce.py:45-257): the object disables itself (never raises) when
the environment is not eligible; `custom_all_reduce` / `custom_tree_all_reduce` return `None`
for ineligible tensors so that the caller can fall back.

Differences, all on the safe side:
  * the flag area of the meta buffer is zero-filled before its handle is published (the
    reference relies on fresh allocations being zero);
  * the scratch capacity behind the flags is handed to the native object, and large messages
    use the two-shot schedule, so `max_size` may be raised well beyond the reference's 8 MiB;
  * `check_status()` reads the kernels' host-visible watchdog word.
"""
from __future__ import annotations

import ctypes
import logging
import os
import socket
from contextlib import contextmanager
from typing import List, Optional, Union

import torch
import torch.distributed as dist
from torch.distributed import ProcessGroup

from . import custom_all_reduce_ops as ops
from .cuda_wrapper import CudaRTLibrary
from .custom_all_reduce_utils import gpu_p2p_access_check, is_full_nvlink, is_weak_contiguous
from .utils import is_cuda, log_info_on_rank0

logger = logging.getLogger(__name__)


def _can_p2p(rank: int, world_size: int) -> bool:
    return all(gpu_p2p_access_check(rank, i) for i in range(world_size) if i != rank)


def in_the_same_node_as(pg: ProcessGroup, source_rank: int = 0) -> List[bool]:
    """Per rank: does it run on the same host as `source_rank`?  (Collective over `pg`.)"""
    world_size = dist.get_world_size(group=pg)
    hostnames: List[Optional[str]] = [None] * world_size
    dist.all_gather_object(hostnames, socket.gethostname(), group=pg)
    return [h == hostnames[source_rank] for h in hostnames]


def _physical_device_id(device: torch.device) -> int:
    if device.type != "cuda":
        return 0
    visible = os.environ.get("CUDA_VISIBLE_DEVICES", None)
    ids = list(map(int, visible.split(","))) if visible else list(range(torch.cuda.device_count()))
    return ids[device.index]


class CustomAllreduce:
    _SUPPORTED_WORLD_SIZES = [2, 4, 6, 8]
    _MAX_CAR_SIZE = 8192 * 1024

    def __init__(self, group: ProcessGroup, device: Union[int, str, torch.device],
                 max_size: int = _MAX_CAR_SIZE) -> None:
        self._IS_CAPTURING = False
        self.disabled = True
        self._ptr = 0

        if not is_cuda() or not ops.IS_CUSTOM_AR_AVAILABLE:
            return
        self.group = group
        if not all(in_the_same_node_as(group, source_rank=0)):
            logger.warning("Custom all-reduce disabled: multi-node group detected.")
            return

        rank = dist.get_rank(group=self.group)
        world_size = dist.get_world_size(group=self.group)
        if world_size == 1 and 1 not in self._SUPPORTED_WORLD_SIZES:
            return
        if world_size not in self._SUPPORTED_WORLD_SIZES:
            logger.warning("Custom all-reduce disabled: unsupported world size %d.", world_size)
            return

        if isinstance(device, int):
            device = torch.device(f"cuda:{device}")
        elif isinstance(device, str):
            device = torch.device(device)
        assert isinstance(device, torch.device)
        if device.type == "cuda" and device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = device

        physical_ids: List[Optional[int]] = [None] * world_size
        dist.all_gather_object(physical_ids, _physical_device_id(device), group=self.group)
        full_nvlink = is_full_nvlink(physical_ids, world_size)
        if world_size > 2 and not full_nvlink:
            logger.warning("Custom all-reduce disabled: no full NVLink for world_size > 2.")
            return
        if not _can_p2p(rank, world_size):
            logger.warning("Custom all-reduce disabled: P2P test failed.")
            return

        self.max_size = max_size
        self.rank = rank
        self.world_size = world_size
        self.full_nvlink = full_nvlink

        # meta buffer = flag area + scratch for the two-shot schedule; data buffer = staging area
        self.meta_ptrs = self.create_shared_buffer(ops.meta_size() + max_size, group=group, zero_bytes=ops.meta_size())
        self.buffer_ptrs = self.create_shared_buffer(max_size, group=group)
        self.rank_data = torch.empty(8 * 1024 * 1024, dtype=torch.uint8, device=self.device)
        self._ptr = ops.init_custom_ar(self.meta_ptrs, self.rank_data, rank, self.full_nvlink)
        ops.configure(self._ptr, ops.CFG_SCRATCH_BYTES, max_size)
        # optional: messages from this many bytes on use the push schedule (see tbik.h, TBIK_AR_CFG_PUSH_MIN_BYTES)
        push_min = int(os.environ.get("TBIK_AR_PUSH_MIN_BYTES", "0"))
        if push_min > 0:
            ops.configure(self._ptr, ops.CFG_PUSH_MIN_BYTES, push_min)
        self._max_blocks_default = int(os.environ.get("TBIK_AR_MAX_BLOCKS", "0"))
        if self._max_blocks_default > 0:
            ops.configure(self._ptr, ops.CFG_MAX_BLOCKS, self._max_blocks_default)
        for env, key in (("TBIK_AR_VEC_PACKS", ops.CFG_VEC_PACKS), ("TBIK_AR_LOADS_IN_FLIGHT", ops.CFG_LOADS_IN_FLIGHT),
                         ("TBIK_AR_THREADS", ops.CFG_THREADS), ("TBIK_AR_ONESHOT_MAX_BYTES", ops.CFG_ONESHOT_MAX_BYTES),
                         ("TBIK_AR_CLUSTER_PAIRS", ops.CFG_CLUSTER_PAIRS)):
            if os.environ.get(env):
                ops.configure(self._ptr, key, int(os.environ[env]))
        ops.register_buffer(self._ptr, self.buffer_ptrs)
        self.disabled = False

    @staticmethod
    def create_shared_buffer(size_in_bytes: int, group: Optional[ProcessGroup] = None,
                             zero_bytes: int = 0) -> List[int]:
        """cudaMalloc on every rank, exchange IPC handles, return the n addresses valid in this process."""
        lib = CudaRTLibrary()
        pointer = lib.cudaMalloc(size_in_bytes)
        if zero_bytes:
            lib.cudaMemset(pointer, 0, min(zero_bytes, size_in_bytes))
            lib.cudaDeviceSynchronize()
        handle = lib.cudaIpcGetMemHandle(pointer)
        world_size = dist.get_world_size(group=group)
        rank = dist.get_rank(group=group)
        handles = [None] * world_size
        dist.all_gather_object(handles, handle, group=group)
        pointers: List[int] = []
        for i, h in enumerate(handles):
            pointers.append(pointer.value if i == rank else lib.cudaIpcOpenMemHandle(h).value)
        return pointers

    @staticmethod
    def free_shared_buffer(pointers: List[int], group: Optional[ProcessGroup] = None) -> None:
        """Unmap the peers' copies, then free this rank's own allocation."""
        if not dist.is_available() or not dist.is_initialized():
            return
        rank = dist.get_rank(group=group)
        lib = CudaRTLibrary()
        for i, p in enumerate(pointers):
            if i != rank:
                try:
                    lib.cudaIpcCloseMemHandle(ctypes.c_void_p(p))
                except RuntimeError as exc:  # the owner is gone already: nothing left to unmap
                    logger.debug("cudaIpcCloseMemHandle: %s", exc)
        lib.cudaFree(ctypes.c_void_p(pointers[rank]))

    @contextmanager
    def capture(self):
        """Wrap CUDA-graph capture: inputs seen while capturing are registered when the block ends."""
        try:
            self._IS_CAPTURING = True
            yield
        finally:
            self._IS_CAPTURING = False
            if not self.disabled:
                self.register_graph_buffers()

    def register_graph_buffers(self) -> None:
        handle, offset = ops.get_graph_buffer_ipc_meta(self._ptr)
        log_info_on_rank0(logger, f"Registering {len(offset)} cuda graph addresses")
        all_data = [None] * dist.get_world_size(group=self.group)
        dist.all_gather_object(all_data, (handle, offset), group=self.group)
        ops.register_graph_buffers(self._ptr, [d[0] for d in all_data], [d[1] for d in all_data])

    def should_custom_ar(self, inp: torch.Tensor) -> bool:
        if self.disabled:
            return False
        inp_size = inp.numel() * inp.element_size()
        if inp_size % 16 != 0:
            return False
        if not is_weak_contiguous(inp):
            return False
        if self.world_size == 2 or self.full_nvlink:
            return inp_size < self.max_size
        return False

    def _native_all_reduce(self, *args):
        ops.all_reduce(*args)

    def all_reduce(self, inp: torch.Tensor, *, out: torch.Tensor = None, registered: bool = False) -> torch.Tensor:
        """Out-of-place all-reduce.  registered=True: `inp` is itself an IPC-registered buffer;
        otherwise it is staged through this object's registered buffer first."""
        if out is None:
            out = torch.empty_like(inp)
        if registered:
            self._native_all_reduce(self._ptr, inp, out, 0, 0)
        else:
            self._native_all_reduce(self._ptr, inp, out, self.buffer_ptrs[self.rank], self.max_size)
        return out

    def all_reduce_rounding(self, view: torch.Tensor, out_dtype: torch.dtype, *, out: torch.Tensor = None) -> torch.Tensor:
        """Tree all-reduce of fp32 contributions, summed in fp32 and rounded once to `out_dtype` (bf16 / fp16).
        `view` is a float32 `registered_view` of this object that a producer has filled (addition: the cross-rank
        levels of a tree whose nodes stay fp32)."""
        assert view.dtype == torch.float32 and view.is_contiguous()
        if out is None:
            out = torch.empty(view.shape, dtype=out_dtype, device=view.device)
        base = self.buffer_ptrs[self.rank]
        ops.tree_all_reduce_rounding(self._ptr, base, view.data_ptr() - base, out)
        return out

    def registered_view(self, shape, dtype: torch.dtype) -> Optional[torch.Tensor]:
        """A tensor that aliases the start of this rank's IPC-registered data buffer, or None if it
        does not fit.  A producer (the row-split GEMM) can write its partial result straight into it
        and call `all_reduce(view, registered=True)`: the staging copy of the reference
        (custom_all_reduce.cu:112-114) disappears.  The view is only valid until the next all-reduce
        through this object has been enqueued."""
        if self.disabled or self.device.type != "cuda":
            return None
        numel = 1
        for d in shape:
            numel *= int(d)
        nbytes = numel * torch.empty(0, dtype=dtype).element_size()
        if nbytes == 0 or nbytes % 16 != 0 or nbytes >= self.max_size:
            return None

        class _Raw:
            __cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "version": 2,
                                        "data": (self.buffer_ptrs[self.rank], False)}

        flat = torch.as_tensor(_Raw(), device=self.device)
        return flat.view(dtype).view(*shape)

    def _dispatch(self, input: torch.Tensor) -> Optional[torch.Tensor]:
        if self.disabled or not self.should_custom_ar(input):
            return None
        if self._IS_CAPTURING:
            if torch.cuda.is_current_stream_capturing():
                return self.all_reduce(input, registered=False)
            # warm-up run before capture: only the shape of the result matters
            return torch.zeros_like(input)
        return self.all_reduce(input, registered=False)

    def custom_all_reduce(self, input: torch.Tensor) -> Optional[torch.Tensor]:
        return self._dispatch(input)

    def check_status(self) -> None:
        """Raise if one of this communicator's kernels gave up waiting for a peer."""
        if self.disabled or not self._ptr:
            return
        st = ops.status(self._ptr)
        if st[0] != 0:
            raise RuntimeError(
                f"all-reduce kernel timed out: rank {st[1]} block {st[2]} waited for rank {st[3]} "
                f"(expected epoch {st[4]}, saw {st[5]}, barrier {st[6]})")

    def close(self) -> None:
        if not self.disabled and getattr(self, "_ptr", 0):
            ops.dispose(self._ptr)
            if dist.is_available() and dist.is_initialized():
                self.free_shared_buffer(self.meta_ptrs, group=self.group)
                self.free_shared_buffer(self.buffer_ptrs, group=self.group)
            self._ptr = 0
            self.disabled = True

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CustomTreeAllreduce(CustomAllreduce):
    """All-reduce whose sum is the fixed rank-pair tree ((0+1)+(2+3))+((4+5)+(6+7))."""

    _SUPPORTED_WORLD_SIZES = [1, 2, 4, 8]

    def _native_all_reduce(self, *args):
        ops.tree_all_reduce(*args)

    def custom_tree_all_reduce(self, input: torch.Tensor) -> Optional[torch.Tensor]:
        return self._dispatch(input)
