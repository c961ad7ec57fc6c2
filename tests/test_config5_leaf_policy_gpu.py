"""Qwen3-32B-shaped row-split layers (o_proj K = 8192, down_proj K = 25600, N = 5120) at TP = 1/2/4/8.

The reference cannot run down_proj at TP = 8 (K / 8 = 3200 is not a multiple of its fixed leaf of 256:
src/tbik/tree_based_matmul.py:240-243).  Here the leaf width of a layer is derived from its unsharded K and the
largest TP degree to support (`leaf_for`), every TP degree uses that same leaf, and the K-shard results combined
in the rank-pair tree must equal the TP = 1 result bit for bit.  Parity with the reference at leaf 128 is
"tolerance against fp64" by necessity; against the CPU oracle (which takes any leaf) it is bit-exact on
integer-valued operands.
"""
import pytest
import torch

from oracle.tbik_ref import exact_int_inputs, matmul_fp64, sharded_matmul_ref, tbik_matmul_ref

pytestmark = pytest.mark.gpu

LAYERS = {"o_proj": (8192, 5120), "down_proj": (25600, 5120)}  # K, N


def bits(t):
    return t.contiguous().view(torch.int16)


def pair_tree(parts):
    while len(parts) > 1:
        parts = [parts[i] + parts[i + 1] for i in range(0, len(parts), 2)]
    return parts[0]


def test_leaf_policy_table():
    from llm_reproducibility_b200.patch.patch_tp_invariant import layer_leaf
    from llm_reproducibility_b200.tbik.tree_based_matmul import leaf_for
    assert leaf_for(8192, 8) == 256 and leaf_for(25600, 8) == 128 and leaf_for(25600, 4) == 256
    assert leaf_for(4096, 8) == 256 and leaf_for(12288, 8) == 256
    for tp in (1, 2, 4, 8):  # the same leaf whatever degree the engine runs at
        assert layer_leaf(25600, tp, torch.bfloat16) == 128 and layer_leaf(8192, tp, torch.bfloat16) == 256
    with pytest.raises(ValueError):
        leaf_for(25600 + 64, 8)


@pytest.mark.parametrize("layer", ["o_proj", "down_proj"])
@pytest.mark.parametrize("M", [16, 8192])
def test_shards_at_every_tp_degree_equal_tp1_bitwise(layer, M):
    from llm_reproducibility_b200.tbik.tree_based_matmul import gemm_device_status, leaf_for, matmul_tp_persistent
    K, N = LAYERS[layer]
    leaf = leaf_for(K, 8)
    g = torch.Generator(device="cuda").manual_seed(K + M)
    A = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    full = matmul_tp_persistent(A, W.t(), leaf=leaf)
    for tp in (2, 4, 8):
        ks = K // tp
        parts = [matmul_tp_persistent(A[:, r * ks:(r + 1) * ks], W[:, r * ks:(r + 1) * ks].t(), leaf=leaf) for r in range(tp)]
        assert torch.equal(bits(pair_tree(parts)), bits(full)), (layer, M, tp)
        del parts
    # batch invariance at this leaf
    assert torch.equal(bits(matmul_tp_persistent(A[:5], W.t(), leaf=leaf)), bits(full[:5]))
    torch.cuda.synchronize()
    assert gemm_device_status()[0] == 0
    if M == 16:  # accuracy against fp64 (the only parity statement possible with the reference at leaf 128)
        f64 = matmul_fp64(A.cpu(), W.cpu().t())
        assert ((full.cpu().double() - f64).abs().max() / f64.abs().max()).item() < 1.0e-2


@pytest.mark.parametrize("tp", [1, 8])
def test_leaf_128_matches_the_oracle_on_integer_operands(tp):
    """down_proj of config 5 with the leaf the policy picks (128): a 512-column slice against the CPU oracle."""
    from llm_reproducibility_b200.tbik.tree_based_matmul import leaf_for, matmul_tp_persistent
    K, M, N = 25600, 16, 512
    leaf = leaf_for(K, 8)
    A, B = exact_int_inputs(M, K, N, torch.bfloat16, seed=5 + tp, amax=7)
    Ad, Wd = A.cuda(), B.cuda().t().contiguous()
    ks = K // tp
    parts = [matmul_tp_persistent(Ad[:, r * ks:(r + 1) * ks], Wd[:, r * ks:(r + 1) * ks].t(), leaf=leaf) for r in range(tp)]
    got = pair_tree(parts).cpu()
    assert torch.equal(bits(got), bits(tbik_matmul_ref(A, B, leaf=leaf)))
    assert torch.equal(bits(got), bits(sharded_matmul_ref(A, B, 8, leaf=leaf)))
