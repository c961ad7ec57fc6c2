"""The fp32-node mode of the tree GEMM: leaves and nodes stay fp32, one rounding at the root.

The reference rounds every node to the operand type (src/tbik/tree_based_matmul.py:109-170: its accumulators
have the input dtype); this mode keeps the reference's TREE (shape and order) and only moves the roundings, so the
properties the reference exists for -- batch invariance and TP invariance -- are tested here exactly as for the
default mode, and the arithmetic is checked bit for bit against the CPU oracle's `node_dtype=torch.float32`.

Operands for the bit-exact cases have leaves that are exact in fp32 whatever order the tensor core adds them in
(small integers, one power-of-two scale per leaf) while the sums of leaves are NOT exact (the scales spread the
leaves over more than 24 bits): any change of the tree's order or of where it rounds shows.
"""
import pytest
import torch

from oracle.tbik_ref import matmul_fp64, normal_inputs, tbik_matmul_ref, tree_shape

pytestmark = pytest.mark.gpu


def bits(t):
    return t.view(torch.int32) if t.dtype == torch.float32 else t.view(torch.int16)


def graded_inputs(M, K, N, leaf, dtype, seed):
    """Integers in [-15, 15]; the i-th leaf's columns of A carry the scale 2^-(step * (i mod 8))."""
    g = torch.Generator().manual_seed(seed)
    A = torch.randint(-15, 16, (M, K), generator=g).float()
    B = torch.randint(-15, 16, (K, N), generator=g).float()
    step = 5 if dtype == torch.bfloat16 else 2
    for i in range(K // leaf):
        A[:, i * leaf:(i + 1) * leaf] *= 2.0 ** (-step * (i % 8))
    A16, B16 = A.to(dtype), B.to(dtype)
    assert torch.equal(A16.float(), A) and torch.equal(B16.float(), B)
    return A16, B16


def run(A, B, **kw):
    from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent
    out = matmul_tp_persistent(A.cuda(), B.cuda(), **kw)
    torch.cuda.synchronize()
    return out.cpu()


def gemm_ex(A, B, leaf, node, tiling, out_dtype):
    """Through the C ABI with an explicit tiling."""
    from llm_reproducibility_b200 import _lib
    from llm_reproducibility_b200.tbik.tree_based_matmul import _DTYPE_CODE, _raw_stream
    Ad, Wd = A.cuda().contiguous(), B.t().contiguous().cuda()
    M, K = A.shape
    N = B.shape[1]
    C = torch.empty(M, N, dtype=out_dtype, device="cuda")
    rc = _lib.lib().tbik_gemm_ex(Ad.data_ptr(), Wd.data_ptr(), C.data_ptr(), M, N, K, K, K, N, _DTYPE_CODE[A.dtype], leaf,
                                 node, 0, tiling, None, 0, _raw_stream(0))
    torch.cuda.synchronize()
    return rc, C.cpu()


def test_the_graded_operands_tell_orders_and_roundings_apart():
    A, B = graded_inputs(64, 4096, 128, 512, torch.bfloat16, 1)
    tree32 = tbik_matmul_ref(A, B, 512, torch.float32, torch.float32)
    leaves = [A[:, i * 512:(i + 1) * 512].float() @ B[i * 512:(i + 1) * 512].float() for i in range(8)]
    seq = leaves[0].clone()
    for x in leaves[1:]:
        seq = seq + x
    rev = leaves[7].clone()
    for x in reversed(leaves[:7]):
        rev = rev + x
    assert (bits(seq) != bits(rev)).any(), "node sums are exact: the operands test nothing"
    assert (bits(tree32) != bits(rev)).any()
    assert (bits(tbik_matmul_ref(A, B, 512)) != bits(tree32.to(torch.bfloat16))).any()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,N,leaf", [
    (256, 4096, 256, 512),     # T = 8, L = 3: the benchmark layer's tree (o_proj)
    (300, 12288, 384, 1536),   # T = 8, leaf of 24 k-blocks (down_proj), ragged M
    (77, 1024, 136, 256),      # T = 4, L = 2, ragged M and N
    (128, 512, 128, 512),      # a single leaf: no node at all
    (64, 1536, 64, 256),       # T = 6: F = 3, L = 2 (a radix-3 level 0)
    (16, 2048, 512, 64),       # T = 32, L = 5: only the 64- and 32-column tilings hold it
])
def test_bit_exact_against_the_oracle(dtype, M, K, N, leaf):
    A, B = graded_inputs(M, K, N, leaf, dtype, 7 + M)
    want32 = tbik_matmul_ref(A, B, leaf, torch.float32, torch.float32)
    got32 = run(A, B, leaf=leaf, node_dtype=torch.float32, out_dtype=torch.float32)
    assert got32.dtype == torch.float32
    assert torch.equal(bits(got32), bits(want32))
    got16 = run(A, B, leaf=leaf, node_dtype=torch.float32)
    assert got16.dtype == dtype
    assert torch.equal(bits(got16), bits(want32.to(dtype)))


@pytest.mark.parametrize("tiling", [1, 2, 5, 6])
def test_every_tiling_gives_the_same_bits(tiling):
    from llm_reproducibility_b200 import _lib
    A, B = graded_inputs(520, 4096, 392, 512, torch.bfloat16, 3)
    want = tbik_matmul_ref(A, B, 512, torch.float32, torch.float32)
    rc, got = gemm_ex(A, B, 512, _lib.NODE_FP32_OUT_FP32, tiling, torch.float32)
    assert rc == 0
    assert torch.equal(bits(got), bits(want))
    rc, got = gemm_ex(A, B, 512, _lib.NODE_FP32, tiling, torch.bfloat16)
    assert rc == 0
    assert torch.equal(bits(got), bits(want.to(torch.bfloat16)))
    # unstructured operands: the tilings agree with each other
    A, B = normal_inputs(520, 4096, 392, torch.bfloat16, 5)
    _, ref = gemm_ex(A, B, 512, _lib.NODE_FP32_OUT_FP32, 1, torch.float32)
    _, got = gemm_ex(A, B, 512, _lib.NODE_FP32_OUT_FP32, tiling, torch.float32)
    assert torch.equal(bits(got), bits(ref))


def test_a_tree_too_deep_for_tensor_memory_is_refused_not_approximated():
    from llm_reproducibility_b200 import _lib
    A, B = graded_inputs(128, 4096, 128, 256, torch.bfloat16, 9)   # T = 16: L = 4
    assert tree_shape(4096, 256)[2] == 4
    for tiling in (1, 2):
        rc, _ = gemm_ex(A, B, 256, _lib.NODE_FP32, tiling, torch.bfloat16)
        assert rc != 0
        assert "tensor memory" in _lib.last_error()
    for tiling in (3, 4):
        rc, _ = gemm_ex(A, B, 256, _lib.NODE_FP32, tiling, torch.bfloat16)
        assert rc != 0
    # the automatic choice falls back to a tiling that holds it
    want = tbik_matmul_ref(A, B, 256, torch.float32, torch.float32)
    got = run(A, B, leaf=256, node_dtype=torch.float32, out_dtype=torch.float32)
    assert torch.equal(bits(got), bits(want))
    A, B = graded_inputs(32, 4096, 64, 64, torch.bfloat16, 10)     # T = 64: L = 6
    want = tbik_matmul_ref(A, B, 64, torch.float32, torch.float32)
    got = run(A, B, leaf=64, node_dtype=torch.float32, out_dtype=torch.float32)
    assert torch.equal(bits(got), bits(want))


def test_batch_invariance():
    A, B = normal_inputs(1024, 4096, 512, torch.bfloat16, 21)
    full = run(A, B, leaf=512, node_dtype=torch.float32)
    for rows in (1, 7, 16, 129, 300):
        part = run(A[:rows], B, leaf=512, node_dtype=torch.float32)
        assert torch.equal(bits(part), bits(full[:rows])), rows
    few = run(A, B, leaf=512, node_dtype=torch.float32, max_ctas=24)
    assert torch.equal(bits(few), bits(full))


@pytest.mark.parametrize("K,N", [(4096, 512), (12288, 256)])
def test_tp_invariance_through_fp32_subtree_roots(K, N):
    """K sharded over 2, 4, 8 ranks: every rank's unrounded subtree root, the rank-pair tree in fp32, one rounding:
    the bits of the unsharded call."""
    from llm_reproducibility_b200.tbik.tree_based_matmul import leaf_for_fp32_nodes
    leaf = leaf_for_fp32_nodes(K, 8)
    A, B = normal_inputs(384, K, N, torch.bfloat16, 33)
    want = run(A, B, leaf=leaf, node_dtype=torch.float32)
    for tp in (2, 4, 8):
        ks = K // tp
        parts = [run(A[:, r * ks:(r + 1) * ks], B[r * ks:(r + 1) * ks], leaf=leaf, node_dtype=torch.float32,
                     out_dtype=torch.float32) for r in range(tp)]
        stride = 1
        while stride < tp:
            for i in range(0, tp, 2 * stride):
                parts[i] = parts[i] + parts[i + stride]
            stride *= 2
        assert torch.equal(bits(parts[0].to(torch.bfloat16)), bits(want)), tp


def test_fp32_nodes_are_closer_to_fp64_than_rounded_nodes():
    A, B = normal_inputs(512, 12288, 512, torch.bfloat16, 44)
    exact = matmul_fp64(A, B)
    err16 = (run(A, B).double() - exact).abs().mean().item()
    err32 = (run(A, B, leaf=1536, node_dtype=torch.float32).double() - exact).abs().mean().item()
    once = (exact.to(torch.bfloat16).double() - exact).abs().mean().item()   # one rounding of the exact result
    assert err32 < 0.5 * err16
    assert err32 < 1.05 * once


def test_environment_switch_and_argument_errors(monkeypatch):
    A, B = normal_inputs(64, 4096, 128, torch.bfloat16, 55)
    want = run(A, B, node_dtype=torch.float32)          # default leaf: K / 8
    assert torch.equal(bits(want), bits(run(A, B, leaf=512, node_dtype=torch.float32)))
    monkeypatch.setenv("TBIK_NODE_FP32", "1")
    assert torch.equal(bits(run(A, B)), bits(want))
    monkeypatch.delenv("TBIK_NODE_FP32")
    with pytest.raises(ValueError):
        run(A, B, out_dtype=torch.float32)
    with pytest.raises(ValueError):
        run(A, B, node_dtype=torch.float64)
