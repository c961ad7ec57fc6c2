"""Training-side use of the tree matmul: forward AND backward through the same fixed-order kernel.

The reference adds gradient support to its invariant matmul by registering backward implementations for the
overridden aten ops (src/patch/patch_batch_invariant.py:38-73, `enable_batch_invariant_backward_mode`), so that a
trainer's logprobs can be compared bit for bit with the rollout engine's.  Here the same role is played by an
autograd function: `tree_matmul(A, B)` and `tree_linear(x, weight, bias)` compute their forward with
`matmul_tp_persistent`, and both gradients with it too,

    dA = dC @ B^T        (reduction over N: batch-invariant like the forward -- row i of dA depends on row i of dC only)
    dB = A^T @ dC        (reduction over the M rows of the batch, padded with zero rows to a multiple of the leaf)

so every number of a training step comes out of the one reduction order, run after run and whatever else shares
the batch.  There is no CPU path.
"""
from __future__ import annotations

from typing import Optional

import torch

from .tree_based_matmul import _LEAF, matmul_tp_persistent


def _pad_rows(t: torch.Tensor, multiple: int) -> torch.Tensor:
    pad = (-t.shape[0]) % multiple
    if pad == 0:
        return t
    return torch.cat([t, t.new_zeros((pad,) + tuple(t.shape[1:]))], dim=0)


class _TreeMatmul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
        ctx.save_for_backward(A, B)
        return matmul_tp_persistent(A, B)

    @staticmethod
    def backward(ctx, dC: torch.Tensor):
        A, B = ctx.saved_tensors
        dC = dC.contiguous()
        dA = dB = None
        leaf = _LEAF[A.dtype]
        if ctx.needs_input_grad[0]:
            # [M, N] x [N, K]: the reduction runs over N
            if B.shape[1] % leaf:
                raise RuntimeError(f"tree_matmul backward: N = {B.shape[1]} must be a multiple of {leaf}")
            dA = matmul_tp_persistent(dC, B.t())
        if ctx.needs_input_grad[1]:
            # [K, M] x [M, N]: the reduction runs over the rows of the batch; zero rows fill the last leaf
            At = _pad_rows(A, leaf).t().contiguous()
            dB = matmul_tp_persistent(At, _pad_rows(dC, leaf))
        return dA, dB


def tree_matmul(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """Differentiable `matmul_tp_persistent(A, B)` for 2-D bf16 / fp16 CUDA tensors."""
    return _TreeMatmul.apply(A, B)


def tree_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differentiable y = x @ weight^T (+ bias) with weight [N, K] as torch.nn.Linear stores it; leading
    dimensions of x are flattened for the matmul and restored."""
    lead = x.shape[:-1]
    y = tree_matmul(x.reshape(-1, x.shape[-1]), weight.t())
    if bias is not None:
        y = y + bias
    return y.reshape(*lead, weight.shape[0])
