"""`tbik_kernel`: the native op namespace (`torch.ops.tbik_kernel.*`).

The reference builds a torch C++ extension `tbik_kernel.common_ops`
(mini_allreduce/csrc/common_ops_allreduce.cc:37-58).  Here the ops are registered with
`torch.library` and forward to the C-ABI library `libtbik_b200.so`; importing
`tbik_kernel.allreduce` performs the registration as a side effect, as in the reference
(mini_allreduce/tbik_kernel/allreduce.py:6-12).
"""
__all__ = ["allreduce"]
