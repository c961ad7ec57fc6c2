"""The CPU oracle must reproduce, bit for bit, what the reference's own code produced.

The fixtures were written by tests/golden/make_golden.py from the reference Triton kernel
(CPU interpreter, fp16/fp32) and the reference native tree all-reduce (gloo ranks).
"""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

from make_golden import AR_CASES, MATMUL_CASES, ar_input, make_inputs  # noqa: E402
from oracle.tbik_ref import (  # noqa: E402
    sharded_matmul_ref,
    tbik_matmul_ref,
    tree_allreduce_ref,
    tree_shape,
)

GOLD_MM = torch.load(os.path.join(HERE, "golden", "matmul_reference_interpreter.pt"))
GOLD_AR = torch.load(os.path.join(HERE, "golden", "allreduce_reference_native.pt"))


def bits(t):
    return t.contiguous().view(torch.int16 if t.element_size() == 2 else torch.int32)


@pytest.mark.parametrize("case", MATMUL_CASES, ids=[c[0] for c in MATMUL_CASES])
def test_matmul_oracle_matches_reference_kernel(case):
    name, dt, M, K, N, gen, seed = case
    A, B = make_inputs(dt, M, K, N, gen, seed)
    C = tbik_matmul_ref(A, B)
    assert C.dtype == dt
    assert torch.equal(bits(C), bits(GOLD_MM[name]))


@pytest.mark.parametrize("case", AR_CASES, ids=[c[0] for c in AR_CASES])
def test_allreduce_oracle_matches_reference_native(case):
    name, dt, world, numel, seed = case
    parts = [ar_input(dt, r, numel, seed) for r in range(world)]
    y = tree_allreduce_ref(parts)
    assert torch.equal(bits(y), bits(GOLD_AR[name]))


@pytest.mark.parametrize("K,leaf,expect", [
    (4096, 256, (16, 2, 4)), (12288, 256, (48, 3, 5)), (8192, 256, (32, 2, 5)),
    (25600, 256, (100, 25, 3)), (6144, 256, (24, 3, 4)), (256, 256, (1, 1, 1)),
    (512, 256, (2, 2, 1)), (768, 256, (3, 3, 1)), (1536, 128, (12, 3, 3)),
])
def test_tree_shape(K, leaf, expect):
    assert tree_shape(K, leaf) == expect


def test_tree_shape_rejects_ragged_k():
    with pytest.raises(ValueError):
        tree_shape(3200, 256)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("K,tps", [(4096, (1, 2, 4, 8)), (12288, (1, 2, 4, 8)), (6144, (1, 2, 4))])
def test_shard_invariance_of_oracle(dt, K, tps):
    """Property the reference checks in simple_matmul.py:23-43: K shards + tree == unsharded."""
    from oracle.tbik_ref import normal_inputs
    A, B = normal_inputs(16, K, 64, dt, seed=K)
    full = tbik_matmul_ref(A, B)
    for tp in tps:
        assert torch.equal(bits(sharded_matmul_ref(A, B, tp)), bits(full)), tp


def test_config1_plain_matmul_is_not_invariant():
    """Sanity of the property test: plain bf16 matmul split 4-way does differ."""
    from oracle.tbik_ref import normal_inputs
    A, B = normal_inputs(64, 4096, 1024, torch.bfloat16, seed=0)
    full = A @ B
    parts = [A[:, i * 1024:(i + 1) * 1024] @ B[i * 1024:(i + 1) * 1024] for i in range(4)]
    split = (parts[0] + parts[1]) + (parts[2] + parts[3])
    assert not torch.equal(bits(full), bits(split))
    assert torch.equal(bits(sharded_matmul_ref(A, B, 4)), bits(tbik_matmul_ref(A, B)))


def test_batch_invariance_of_oracle():
    """simple_matmul.py:16-20: f(A,B)[:m] == f(A[:m],B)."""
    from oracle.tbik_ref import exact_int_inputs
    A, B = exact_int_inputs(32, 1536, 64, torch.bfloat16, seed=3)
    full = tbik_matmul_ref(A, B)
    assert torch.equal(bits(full[:7]), bits(tbik_matmul_ref(A[:7], B)))
