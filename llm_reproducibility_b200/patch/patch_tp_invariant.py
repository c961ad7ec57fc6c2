"""Replace `RowParallelLinear.forward` (o_proj, down_proj) by the tree matmul + tree all-reduce
(reference: src/patch/patch_tp_invariant.py:10-52).

`row_parallel_forward` holds the logic and needs nothing from vLLM, so it can be exercised
with any object that has the layer's attributes; `patch_row_linear` binds it to vLLM's class.
"""
from __future__ import annotations

import logging
import os
from typing import Callable, Optional

import torch

from ..tbik.tree_based_all_reduce import tree_matmul_all_reduce
from ..tbik.tree_based_matmul import leaf_for, matmul_tp_persistent

logger = logging.getLogger(__name__)

# Largest tensor-parallel degree whose results must agree bit for bit with every smaller one (TP = 1 included).
# It fixes the leaf width of every row-split layer from the layer's FULL K, so that engines started with
# different TP degrees walk the same reduction tree.  Set through `patch_tp_invariant(max_tp=...)`.
MAX_TP = 8
CALLS = 0  # forwards served by `row_parallel_forward` in this process (lets an end-to-end run prove the patch is live)


def layer_leaf(K_total: int, tp_size: int, dtype: torch.dtype) -> int:
    """Leaf width of a layer with unsharded reduction length K_total: sized for MAX_TP ranks; a layer too short
    for that many aligned subtrees is sized for the largest degree below it that still covers `tp_size`."""
    max_tp = max(MAX_TP, tp_size)
    while True:
        try:
            return leaf_for(K_total, max_tp, dtype)
        except ValueError:
            if max_tp // 2 < max(tp_size, 1):
                raise
            max_tp //= 2


def row_parallel_forward(self, input_, *, device_group_fn: Optional[Callable] = None,
                         split_fn: Optional[Callable] = None):
    """Forward of a row-parallel linear layer with K split over `self.tp_size` ranks.

    Attributes used (those of vLLM's layer): input_is_parallel, tp_size, tp_rank, weight [N, K/tp],
    bias, skip_bias_add, reduce_results, return_bias, quant_method.
    """
    global CALLS
    CALLS += 1
    if CALLS == 1:
        logger.info("tree row-parallel forward active in process %d (tp rank %d of %d)", os.getpid(), self.tp_rank,
                    self.tp_size)
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
    # one leaf width per layer, derived from the unsharded K: the same at every TP degree
    leaf = layer_leaf(x2d.shape[-1] * self.tp_size, self.tp_size, x2d.dtype)
    if self.reduce_results and self.tp_size > 1:
        group = device_group_fn() if device_group_fn is not None else None
        output = tree_matmul_all_reduce(x2d, self.weight.t(), group, leaf=leaf)
        if os.environ.get("TBIK_VERIFY") == "1":
            # debugging aid: the same layer through the library collective (all_gather + ordered adds)
            from ..tbik.tree_based_all_reduce import tree_all_reduce_sum_native
            want = tree_all_reduce_sum_native(matmul_tp_persistent(x2d, self.weight.t(), leaf=leaf), group)
            bad = int((want.view(torch.int16) != output.view(torch.int16)).sum())
            if bad or CALLS <= 8:
                print(f"[tbik verify] pid {os.getpid()} rank {self.tp_rank} call {CALLS} x {tuple(x2d.shape)} "
                      f"strides {tuple(x2d.stride())} w {tuple(self.weight.shape)} leaf {leaf}: {bad} mismatching elements",
                      flush=True)
    else:
        output = matmul_tp_persistent(x2d, self.weight.t(), leaf=leaf)
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


def patch_tp_invariant(max_tp: int = 8):
    """`max_tp` (extension): the largest TP degree that must reproduce the bits of all smaller ones."""
    global MAX_TP
    if max_tp < 1 or max_tp & (max_tp - 1):
        raise ValueError("max_tp must be a power of two")
    MAX_TP = max_tp
    patch_row_linear()
    print("Successfully patched vLLM to use custom tp_invariant implementation")
