"""Peer-to-peer all-reduce over CUDA-IPC buffers (reference package: mini_allreduce)."""
from .custom_all_reduce import CustomAllreduce, CustomTreeAllreduce

__all__ = ["CustomAllreduce", "CustomTreeAllreduce"]
