"""A CPU stand-in for the CUDA runtime and the native all-reduce ops, for host-logic tests only.

"Device memory" is POSIX shared memory, an "IPC handle" is the segment's name, and the fake
`tree_all_reduce` does what the kernels do (stage the input, barrier, read every rank's buffer,
reduce in tree order, barrier) with the CPU oracle as its arithmetic.  It lets the constructor,
handle exchange, eligibility rules, dispatcher and close() of the host classes run on gloo ranks.
Nothing in the product imports this file.
"""
import ctypes
from multiprocessing import shared_memory

import torch
import torch.distributed as dist

from oracle.tbik_ref import tree_allreduce_ref


class FakeHandle:
    def __init__(self, name, size):
        self.name, self.size = name, size


class FakeCudaRT:
    """Replaces mini_allreduce.cuda_wrapper.CudaRTLibrary."""
    segments = {}   # fake address -> SharedMemory
    owned = set()
    next_addr = [0x10000000]

    def _new_addr(self, shm):
        addr = self.next_addr[0]
        self.next_addr[0] += (shm.size + 0xFFFF) & ~0xFFFF
        self.segments[addr] = shm
        return addr

    def cudaMalloc(self, size):
        shm = shared_memory.SharedMemory(create=True, size=max(size, 1))
        addr = self._new_addr(shm)
        self.owned.add(addr)
        shm.buf[:size] = b"\xAB" * size  # fresh memory is NOT zero: the host code must clear the flags
        return ctypes.c_void_p(addr)

    def cudaMemset(self, ptr, value, count):
        self.segments[ptr.value].buf[:count] = bytes([value]) * count

    def cudaDeviceSynchronize(self):
        pass

    def cudaIpcGetMemHandle(self, ptr):
        shm = self.segments[ptr.value]
        return FakeHandle(shm.name, shm.size)

    def cudaIpcOpenMemHandle(self, handle):
        if not isinstance(handle, FakeHandle) or not handle.name:
            raise RuntimeError("CUDART error: invalid resource handle")
        shm = shared_memory.SharedMemory(name=handle.name)
        return ctypes.c_void_p(self._new_addr(shm))

    def cudaIpcCloseMemHandle(self, ptr):
        self.cudaFree(ptr)

    def cudaFree(self, ptr):
        shm = self.segments.pop(ptr.value)
        shm.close()
        if ptr.value in self.owned:
            self.owned.discard(ptr.value)
            shm.unlink()

    @classmethod
    def view(cls, addr, nbytes):
        return cls.segments[addr].buf[:nbytes]

    @classmethod
    def cleanup(cls):
        for addr, shm in list(cls.segments.items()):
            try:
                shm.close()
                if addr in cls.owned:
                    shm.unlink()
            except Exception:
                pass
        cls.segments.clear()
        cls.owned.clear()


class FakeOps:
    """Replaces mini_allreduce.custom_all_reduce_ops (the 8 reference functions + configure/status)."""
    IS_CUSTOM_AR_AVAILABLE = True
    CFG_SCRATCH_BYTES, CFG_ONESHOT_MAX_BYTES, CFG_MAX_BLOCKS, CFG_WAIT_LIMIT_NS, CFG_THREADS = 1, 2, 3, 4, 5
    CFG_PUSH_MIN_BYTES, CFG_PUSH_CHUNKS, CFG_VEC_PACKS, CFG_LOADS_IN_FLIGHT, CFG_TRACE, CFG_CLUSTER_PAIRS = 6, 7, 8, 9, 10, 11

    def __init__(self, group):
        self.group = group
        self.comms = {}
        self.calls = []

    def meta_size(self):
        return 256

    def init_custom_ar(self, ipc_tensors, rank_data, rank, full_nvlink):
        world = len(ipc_tensors)
        if world > 8:
            raise ValueError("world size > 8 is not supported")
        if world != 1 and world % 2:
            raise ValueError("Odd num gpus is not supported for now")
        if not 0 <= rank < world:
            raise ValueError("invalid rank passed in")
        # the flag area must have been cleared by its owner before the handles were exchanged
        for p in ipc_tensors:
            assert bytes(FakeCudaRT.view(p, 256)) == b"\x00" * 256, "flag area not zero-filled"
        fa = len(self.comms) + 1
        self.comms[fa] = {"rank": rank, "world": world, "buffers": {}, "cfg": {}}
        return fa

    def register_buffer(self, fa, ipc_tensors):
        c = self.comms[fa]
        assert len(ipc_tensors) == c["world"]
        c["buffers"][ipc_tensors[c["rank"]]] = list(ipc_tensors)

    def configure(self, fa, key, value):
        self.comms[fa]["cfg"][key] = value

    def status(self, fa):
        return [0] * 8

    def _reduce(self, fa, inp, out, reg_buffer, reg_sz, tree):
        c = self.comms[fa]
        if reg_buffer not in c["buffers"]:
            raise RuntimeError(f"buffer address {reg_buffer} is not registered!")
        nbytes = inp.numel() * inp.element_size()
        if nbytes > reg_sz:
            raise RuntimeError("input larger than the registered staging buffer")
        raw = inp.contiguous().view(torch.uint8).numpy().tobytes()
        FakeCudaRT.view(reg_buffer, nbytes)[:] = raw
        dist.barrier(group=self.group)
        parts = []
        for p in c["buffers"][reg_buffer]:
            b = bytes(FakeCudaRT.view(p, nbytes))
            parts.append(torch.frombuffer(bytearray(b), dtype=inp.dtype).clone())
        if tree:
            res = tree_allreduce_ref(parts)
        else:
            acc = parts[0].float()
            for q in parts[1:]:
                acc = acc + q.float()
            res = acc.to(inp.dtype)
        out.view(-1).copy_(res)
        dist.barrier(group=self.group)
        self.calls.append(("tree" if tree else "linear", inp.numel()))

    def tree_all_reduce(self, fa, inp, out, reg_buffer, reg_sz):
        self._reduce(fa, inp, out, reg_buffer, reg_sz, True)

    def all_reduce(self, fa, inp, out, reg_buffer, reg_sz):
        self._reduce(fa, inp, out, reg_buffer, reg_sz, False)

    def dispose(self, fa):
        self.comms.pop(fa)

    def get_graph_buffer_ipc_meta(self, fa):
        return [], []

    def register_graph_buffers(self, fa, handles, offsets):
        pass


def install(monkey_target, group, *, full_nvlink=True, can_p2p=True, hostname=None):
    """Patch module `monkey_target` (mini_allreduce.custom_all_reduce) to run on the fakes; returns the FakeOps."""
    ops = FakeOps(group)
    monkey_target.ops = ops
    monkey_target.CudaRTLibrary = FakeCudaRT
    monkey_target.is_cuda = lambda: True
    monkey_target.is_full_nvlink = lambda ids, world: full_nvlink
    monkey_target._can_p2p = lambda rank, world: can_p2p
    if hostname is not None:
        monkey_target.socket.gethostname = lambda: hostname
    return ops
