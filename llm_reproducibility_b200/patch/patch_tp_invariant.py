"""Replace `RowParallelLinear.forward` (o_proj, down_proj) by the tree matmul + tree all-reduce
(reference: src/patch/patch_tp_invariant.py:10-52).

`row_parallel_forward` holds the logic and needs nothing from vLLM, so it can be exercised
with any object that has the layer's attributes; `patch_row_linear` binds it to vLLM's class.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from ..tbik.tree_based_all_reduce import tree_matmul_all_reduce
from ..tbik.tree_based_matmul import matmul_tp_persistent


def row_parallel_forward(self, input_, *, device_group_fn: Optional[Callable] = None,
                         split_fn: Optional[Callable] = None):
    """Forward of a row-parallel linear layer with K split over `self.tp_size` ranks.

    Attributes used (those of vLLM's layer): input_is_parallel, tp_size, tp_rank, weight [N, K/tp],
    bias, skip_bias_add, reduce_results, return_bias, quant_method.
    """
    if self.input_is_parallel:
        input_parallel = input_
    else:
        if split_fn is None:
            chunk = input_.shape[-1] // self.tp_size
            input_parallel = input_[..., self.tp_rank * chunk:(self.tp_rank + 1) * chunk].contiguous()
        else:
            input_parallel = split_fn(input_, num_partitions=self.tp_size)[self.tp_rank].contiguous()

    assert self.quant_method is not None
    # the bias is added once, after the reduction, and only where it is not skipped
    lead = input_parallel.shape[:-1]
    x2d = input_parallel.reshape(-1, input_parallel.shape[-1])
    if self.reduce_results and self.tp_size > 1:
        group = device_group_fn() if device_group_fn is not None else None
        output = tree_matmul_all_reduce(x2d, self.weight.t(), group)
    else:
        output = matmul_tp_persistent(x2d, self.weight.t())
    output = output.reshape(*lead, output.shape[-1])

    if (not self.skip_bias_add) and self.bias is not None:
        output += self.bias

    output_bias = self.bias if self.skip_bias_add else None
    if not self.return_bias:
        return output
    return output, output_bias


def patch_row_linear():
    from vllm.distributed import split_tensor_along_last_dim
    from vllm.distributed.parallel_state import get_tp_group
    from vllm.model_executor.layers.linear import RowParallelLinear

    def _forward(self, input_):
        return row_parallel_forward(self, input_, device_group_fn=lambda: get_tp_group().device_group,
                                    split_fn=split_tensor_along_last_dim)

    RowParallelLinear.forward = _forward


def patch_tp_invariant():
    patch_row_linear()
    print("Successfully patched vLLM to use custom tp_invariant implementation")
