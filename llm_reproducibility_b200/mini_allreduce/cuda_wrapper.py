"""ctypes access to the CUDA runtime already loaded in the process
(reference: mini_allreduce/cuda_wrapper.py:16-146).

Used for the raw allocations whose IPC handles are exchanged between the TP worker
processes: torch's caching allocator sub-allocates, and an IPC handle always names a whole
allocation.
"""
import ctypes
from typing import Dict, Optional

import torch  # noqa: F401  (makes sure libcudart is mapped)

cudaError_t = ctypes.c_int


class cudaIpcMemHandle_t(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


def find_loaded_library(lib_name: str) -> Optional[str]:
    """Path of a shared object mapped into this process whose file name starts with `lib_name`."""
    with open("/proc/self/maps") as f:
        for line in f:
            if lib_name in line and "/" in line:
                path = line[line.index("/"):].strip()
                fname = path.rsplit("/", 1)[-1]
                if fname.rpartition(".so")[0].startswith(lib_name):
                    return path
    return None


_SIGNATURES = {
    "cudaSetDevice": (cudaError_t, [ctypes.c_int]),
    "cudaDeviceSynchronize": (cudaError_t, []),
    "cudaDeviceReset": (cudaError_t, []),
    "cudaGetErrorString": (ctypes.c_char_p, [cudaError_t]),
    "cudaMalloc": (cudaError_t, [ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t]),
    "cudaFree": (cudaError_t, [ctypes.c_void_p]),
    "cudaMemset": (cudaError_t, [ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t]),
    "cudaMemcpy": (cudaError_t, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]),
    "cudaIpcGetMemHandle": (cudaError_t, [ctypes.POINTER(cudaIpcMemHandle_t), ctypes.c_void_p]),
    "cudaIpcOpenMemHandle": (cudaError_t, [ctypes.POINTER(ctypes.c_void_p), cudaIpcMemHandle_t, ctypes.c_uint]),
    "cudaIpcCloseMemHandle": (cudaError_t, [ctypes.c_void_p]),
}


class CudaRTLibrary:
    _libs: Dict[str, ctypes.CDLL] = {}

    def __init__(self, so_file: Optional[str] = None):
        if so_file is None:
            so_file = find_loaded_library("libcudart")
            assert so_file is not None, "libcudart is not loaded in the current process"
        if so_file not in CudaRTLibrary._libs:
            handle = ctypes.CDLL(so_file)
            for name, (res, args) in _SIGNATURES.items():
                fn = getattr(handle, name)
                fn.restype, fn.argtypes = res, args
            CudaRTLibrary._libs[so_file] = handle
        self.lib = CudaRTLibrary._libs[so_file]

    def CUDART_CHECK(self, result: int) -> None:
        if result != 0:
            raise RuntimeError(f"CUDART error: {self.cudaGetErrorString(result)}")

    def cudaGetErrorString(self, error: int) -> str:
        return self.lib.cudaGetErrorString(error).decode("utf-8")

    def cudaSetDevice(self, device: int) -> None:
        self.CUDART_CHECK(self.lib.cudaSetDevice(device))

    def cudaDeviceSynchronize(self) -> None:
        self.CUDART_CHECK(self.lib.cudaDeviceSynchronize())

    def cudaDeviceReset(self) -> None:
        self.CUDART_CHECK(self.lib.cudaDeviceReset())

    def cudaMalloc(self, size: int) -> ctypes.c_void_p:
        ptr = ctypes.c_void_p()
        self.CUDART_CHECK(self.lib.cudaMalloc(ctypes.byref(ptr), size))
        return ptr

    def cudaFree(self, dev_ptr: ctypes.c_void_p) -> None:
        self.CUDART_CHECK(self.lib.cudaFree(dev_ptr))

    def cudaMemset(self, dev_ptr: ctypes.c_void_p, value: int, count: int) -> None:
        self.CUDART_CHECK(self.lib.cudaMemset(dev_ptr, value, count))

    def cudaMemcpy(self, dst: ctypes.c_void_p, src: ctypes.c_void_p, count: int) -> None:
        self.CUDART_CHECK(self.lib.cudaMemcpy(dst, src, count, 4))  # cudaMemcpyDefault

    def cudaIpcGetMemHandle(self, dev_ptr: ctypes.c_void_p) -> cudaIpcMemHandle_t:
        handle = cudaIpcMemHandle_t()
        self.CUDART_CHECK(self.lib.cudaIpcGetMemHandle(ctypes.byref(handle), dev_ptr))
        return handle

    def cudaIpcOpenMemHandle(self, handle: cudaIpcMemHandle_t) -> ctypes.c_void_p:
        ptr = ctypes.c_void_p()
        self.CUDART_CHECK(self.lib.cudaIpcOpenMemHandle(ctypes.byref(ptr), handle, 1))  # lazy peer access
        return ptr

    def cudaIpcCloseMemHandle(self, dev_ptr: ctypes.c_void_p) -> None:
        self.CUDART_CHECK(self.lib.cudaIpcCloseMemHandle(dev_ptr))
