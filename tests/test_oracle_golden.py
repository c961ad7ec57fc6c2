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
    exact_int_inputs,
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


# ---------------------------------------------------------------- the C restatement (oracle/tbik_ref.c)
INT_CASES = [c for c in MATMUL_CASES if c[5] == "int" and c[1] in (torch.float16, torch.bfloat16)]
AR16_CASES = [c for c in AR_CASES if c[1] in (torch.float16, torch.bfloat16)]


@pytest.mark.parametrize("case", INT_CASES, ids=[c[0] for c in INT_CASES])
def test_c_oracle_matches_reference_kernel(case):
    """Scalar C loops against the stored outputs of the reference's own kernel, every tree shape."""
    from oracle import c_oracle
    name, dt, M, K, N, gen, seed = case
    A, B = make_inputs(dt, M, K, N, gen, seed)
    assert torch.equal(bits(c_oracle.matmul(A, B)), bits(GOLD_MM[name]))


@pytest.mark.parametrize("case", AR16_CASES, ids=[c[0] for c in AR16_CASES])
def test_c_oracle_allreduce_matches_reference_native(case):
    from oracle import c_oracle
    name, dt, world, numel, seed = case
    parts = [ar_input(dt, r, numel, seed) for r in range(world)]
    assert torch.equal(bits(c_oracle.tree_allreduce(parts)), bits(GOLD_AR[name]))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_c_oracle_conversions_are_round_to_nearest_even(dt):
    """Its own 16-bit conversions against torch's: every bit pattern upwards; random values, every midpoint between
    neighbouring representable values, overflow and underflow edges downwards."""
    from oracle import c_oracle
    allp = torch.arange(65536, dtype=torch.int32).to(torch.int16).view(dt)
    a, b = c_oracle.up(allp), allp.float()
    assert bool(((a.view(torch.int32) == b.view(torch.int32)) | (a.isnan() & b.isnan())).all())
    g = torch.Generator().manual_seed(0)
    x = torch.cat([torch.randn(200_000, generator=g) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 300.0, 7e4)])
    mid = (b[:-1] + b[1:]) / 2
    edges = torch.tensor([0.0, -0.0, float("inf"), -float("inf"), 65504.0, 65519.9, 65520.0, 65536.0,
                          5.96e-8, 2.98e-8, 2.9802322e-8, 2.99e-8, 3.4e38, -3.4e38])
    x = torch.cat([x, mid[torch.isfinite(mid)], edges])
    assert torch.equal(bits(c_oracle.down(x, dt)), bits(x.to(dt)))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,N", [(5, 256, 8), (7, 1536, 24), (3, 4096, 16), (4, 12288, 8), (2, 25600, 8), (9, 768, 40)])
def test_c_and_python_oracles_agree(dt, M, K, N):
    from oracle import c_oracle
    A, B = exact_int_inputs(M, K, N, dt, seed=K + M, amax=7)
    assert torch.equal(bits(c_oracle.matmul(A, B)), bits(tbik_matmul_ref(A, B)))
    parts = [torch.randn(777, generator=torch.Generator().manual_seed(r)).to(dt) for r in range(8)]
    for w in (1, 2, 4, 8):
        assert torch.equal(bits(c_oracle.tree_allreduce(parts[:w])), bits(tree_allreduce_ref(parts[:w])))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("K,tps", [(4096, (2, 4, 8)), (12288, (2, 4, 8)), (6144, (2, 4, 8)), (25600, (2, 4))])
def test_c_oracle_is_shard_invariant(dt, K, tps):
    """The property the whole path exists for, stated on the C restatement alone: K-shards reduced separately and
    combined by the rank-pair tree give the bits of the unsplit reduction (random operands, not integer ones)."""
    from oracle import c_oracle
    g = torch.Generator().manual_seed(K)
    A = torch.randn(6, K, generator=g).to(dt)
    B = (torch.randn(K, 24, generator=g) * 0.02).to(dt)
    full = c_oracle.matmul(A, B)
    for tp in tps:
        ks = K // tp
        parts = [c_oracle.matmul(A[:, r * ks:(r + 1) * ks], B[r * ks:(r + 1) * ks]) for r in range(tp)]
        assert torch.equal(bits(c_oracle.tree_allreduce(parts)), bits(full)), tp
    # batch invariance: a row computed alone has the bits it has inside the batch
    assert torch.equal(bits(c_oracle.matmul(A[2:3], B)), bits(full[2:3]))


def _graded(M, K, N, leaf, dt, seed):
    """Small integers, one power-of-two scale per leaf: leaves exact in fp32 whatever the order inside them, sums of
    leaves not (the scales spread them over more than 24 bits)."""
    g = torch.Generator().manual_seed(seed)
    A = torch.randint(-15, 16, (M, K), generator=g).float()
    B = torch.randint(-15, 16, (K, N), generator=g).float()
    step = 5 if dt == torch.bfloat16 else 2
    for i in range(K // leaf):
        A[:, i * leaf:(i + 1) * leaf] *= 2.0 ** (-step * (i % 8))
    return A.to(dt), B.to(dt)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,N,leaf", [(6, 4096, 24, 512), (5, 12288, 16, 1536), (4, 1536, 8, 256), (3, 2048, 8, 64),
                                        (7, 512, 40, 512)])
def test_fp32_node_oracles_agree_and_are_shard_invariant(dt, M, K, N, leaf):
    """The fp32-node mode of the CUDA library (same tree, nothing rounded below the root; no such mode in the
    reference) is checked against `tbik_matmul_ref(node_dtype=float32)`: here the C restatement, written
    independently, gives the same bits, and K-shards combined by the rank-pair tree in fp32 give the unsplit root."""
    from oracle import c_oracle
    A, B = _graded(M, K, N, leaf, dt, seed=K + M)
    py32 = tbik_matmul_ref(A, B, leaf, torch.float32, torch.float32)
    c32 = c_oracle.matmul_fp32_nodes(A, B, leaf)
    assert torch.equal(c32.view(torch.int32), py32.view(torch.int32))
    assert torch.equal(bits(c_oracle.down(c32, dt)), bits(tbik_matmul_ref(A, B, leaf, torch.float32, dt)))
    # the operands tell this mode from the reference's (rounded nodes) wherever there is more than one leaf
    if K > leaf:
        assert (bits(c_oracle.down(c32, dt)) != bits(c_oracle.matmul(A, B, leaf))).any()
    T = K // leaf
    for tp in (2, 4, 8):
        if T % tp or (T & (T - 1)):
            continue   # whole, aligned subtrees per rank need a power-of-two number of leaves
        ks = K // tp
        parts = [c_oracle.matmul_fp32_nodes(A[:, r * ks:(r + 1) * ks], B[r * ks:(r + 1) * ks], leaf) for r in range(tp)]
        stride = 1
        while stride < tp:
            for i in range(0, tp, 2 * stride):
                parts[i] = parts[i] + parts[i + stride]
            stride *= 2
        assert torch.equal(parts[0].view(torch.int32), c32.view(torch.int32)), tp
