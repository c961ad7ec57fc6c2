"""CPU oracle for the TP-invariant row-split path (TEST INFRASTRUCTURE ONLY).

This module restates, on the CPU with torch, the reduction order of the reference's
tree-based matmul and tree all-reduce.  It is the checker for the CUDA path: only the
test-suite, the smoke entry and the benchmark's CPU-baseline leg may import it.  The
product package never imports anything from here.

Parity pin: `tests/golden/*.pt` hold outputs of the reference's own Triton kernel
(`src/tbik/tree_based_matmul.py`, run under the Triton CPU interpreter in fp16/fp32)
and of the reference's `tree_all_reduce_sum_native` (run on gloo ranks); the
functions below reproduce those files bit for bit (tests/test_oracle_golden.py).

Reference lines restated:
  * `tree_shape`           <- src/tbik/tree_based_matmul.py:240-249   (T, FIRST_LEVEL_BLOCK, LEVEL_K)
  * `default_leaf`         <- src/tbik/tree_based_matmul.py:206-231   (BLOCK_SIZE_K per dtype)
  * `tbik_matmul_ref`      <- src/tbik/tree_based_matmul.py:121-174   (leaf dot, rounding, carry chain)
  * `tree_allreduce_ref`   <- src/tbik/tree_based_all_reduce.py:32-35 and
                              mini_allreduce/tbik_kernel/csrc/allreduce/custom_all_reduce.cuh:203-234
  * `sharded_matmul_ref`   <- simple_matmul.py:23-43                  (K shards + simulated tree)
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch


def default_leaf(dtype: torch.dtype) -> int:
    """K-chunk ("leaf") width the reference uses for a dtype (BLOCK_SIZE_K)."""
    return 128 if dtype == torch.float32 else 256


def tree_shape(K: int, leaf: int) -> Tuple[int, int, int]:
    """Return (T, F, L): number of leaves, radix of level 0, number of levels.

    T = F * 2**(L-1).  F is T with its factors of two removed, except that a last
    factor 2 stays in F (so F is 1, 2 or an odd number >= 3).
    """
    if K <= 0 or K % leaf != 0:
        raise ValueError(f"K={K} is not a positive multiple of the leaf width {leaf}")
    T = K // leaf
    F, L = T, 1
    while F > 2 and F % 2 == 0:
        F //= 2
        L += 1
    return T, F, L


def _pairwise(nodes: List[torch.Tensor]) -> torch.Tensor:
    """Perfect binary tree over `nodes` (len = power of two); left operand = lower index."""
    while len(nodes) > 1:
        assert len(nodes) % 2 == 0
        nodes = [nodes[i] + nodes[i + 1] for i in range(0, len(nodes), 2)]
    return nodes[0]


def tbik_matmul_ref(
    A: torch.Tensor,
    B: torch.Tensor,
    leaf: Optional[int] = None,
    node_dtype: Optional[torch.dtype] = None,
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """Tree-ordered C = A @ B on the CPU.

    leaf_i  = round_to_node_dtype( fp32 dot over the i-th `leaf`-wide K chunk )
    group_j = ((leaf_{jF} + leaf_{jF+1}) + ...) + leaf_{jF+F-1}   (each + rounded to node_dtype)
    C       = perfect binary tree over the groups, node = left + right in node_dtype.

    With `node_dtype=None` nodes are kept in A's dtype, which is what the reference does
    (its accumulators have the input dtype).  `node_dtype=torch.float32` describes the
    fp32-node variant of the CUDA kernel: leaves stay fp32, one final rounding to
    `out_dtype`.
    """
    assert A.dim() == 2 and B.dim() == 2 and A.shape[1] == B.shape[0]
    dt = A.dtype
    node_dtype = node_dtype or dt
    out_dtype = out_dtype or dt
    leaf = leaf or default_leaf(dt)
    M, K = A.shape
    T, F, L = tree_shape(K, leaf)
    Af, Bf = A.float(), B.float()
    leaves = [
        (Af[:, i * leaf:(i + 1) * leaf] @ Bf[i * leaf:(i + 1) * leaf, :]).to(node_dtype)
        for i in range(T)
    ]
    groups = []
    for j in range(T // F):
        g = leaves[j * F]
        for i in range(1, F):
            g = g + leaves[j * F + i]
        groups.append(g)
    return _pairwise(groups).to(out_dtype)


def tree_allreduce_ref(parts: Sequence[torch.Tensor]) -> torch.Tensor:
    """Rank-pair tree sum ((0+1)+(2+3))+((4+5)+(6+7)) with adds in the tensors' dtype."""
    n = len(parts)
    if n & (n - 1) != 0 or n == 0:
        raise ValueError("world size must be a power of two")
    res = [p.clone() for p in parts]
    level = 1
    while (1 << level) <= n:
        for left in range(0, n, 1 << level):
            right = left + (1 << (level - 1))
            res[left] = res[left] + res[right]
        level += 1
    return res[0]


def sharded_matmul_ref(
    A: torch.Tensor,
    B: torch.Tensor,
    tp: int,
    leaf: Optional[int] = None,
    node_dtype: Optional[torch.dtype] = None,
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """K split into `tp` contiguous shards, one tree matmul per shard, tree all-reduce."""
    K = A.shape[1]
    assert K % tp == 0
    ks = K // tp
    node_dtype = node_dtype or A.dtype
    parts = [
        tbik_matmul_ref(A[:, r * ks:(r + 1) * ks], B[r * ks:(r + 1) * ks, :], leaf, node_dtype, node_dtype)
        for r in range(tp)
    ]
    return tree_allreduce_ref(parts).to(out_dtype or A.dtype)


def matmul_fp64(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """Exact-ish reference for tolerance checks."""
    return A.double() @ B.double()


def exact_int_inputs(M: int, K: int, N: int, dtype: torch.dtype, seed: int, amax: int = 15):
    """Integer-valued operands in [-amax, amax].

    Every product and every 256-term leaf sum is exact in fp32 whatever the summation
    order inside the leaf, so any conforming implementation must agree bit for bit; the
    leaf sums exceed the 8-bit (bf16) / 11-bit (fp16) significand, so every rounding
    step of the tree is exercised.
    """
    g = torch.Generator().manual_seed(seed)
    A = torch.randint(-amax, amax + 1, (M, K), generator=g).to(dtype)
    B = torch.randint(-amax, amax + 1, (K, N), generator=g).to(dtype)
    return A, B


def normal_inputs(M: int, K: int, N: int, dtype: torch.dtype, seed: int, w_std: float = 0.02):
    """Activations ~N(0,1), weights ~N(0, w_std): the distribution of the benchmark configs."""
    g = torch.Generator().manual_seed(seed)
    A = torch.randn((M, K), generator=g).to(dtype)
    B = (torch.randn((K, N), generator=g) * w_std).to(dtype)
    return A, B
