"""The CUDA tree GEMM against the reference's own Triton kernel, both on the same GPU, same operands.

The reference kernel is staged under oracle/_ref/ by oracle/build_ref.py (a build output, never committed);
without it these tests skip.  What they pin: the one thing no CPU oracle can -- the bits of a leaf, i.e. the
order in which the matrix unit adds the 256 fp32 products of a K chunk (decided by Triton's `tl.dot` lowering
in the reference, src/tbik/tree_based_matmul.py:136, and by tcgen05.mma here).

Bars: integer-valued operands (leaf sums exact in any order) must agree bit for bit; on the benchmark's
N(0,1) x N(0,0.02) operands at most MAX_MISMATCH_FRACTION of the elements may differ, each by at most one
bf16 unit in the last place of the largest output value (a leaf that rounds the other way moves the result by
one unit of that LEAF; an output near zero is then many of its own, smaller, units away).
"""
import importlib.util
import math
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

REF_PATH = os.path.join(ROOT, "oracle", "_ref", "tree_based_matmul.py")
MAX_MISMATCH_FRACTION = 5e-4
MAX_ULP = 1

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not os.path.isfile(REF_PATH), reason="reference kernel not staged (oracle/build_ref.py)")]

_ref_mod = None


def reference_matmul():
    global _ref_mod
    if _ref_mod is None:
        # triton picks its CPU interpreter when it decorates a kernel with this switch set; its bf16 arithmetic
        # there is invalid, so a GPU comparison must never run under it
        assert os.environ.get("TRITON_INTERPRET", "0") in ("", "0"), "TRITON_INTERPRET is set: the reference would not run on the GPU"
        spec = importlib.util.spec_from_file_location("tbik_reference_triton", REF_PATH)
        _ref_mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_ref_mod)
    return _ref_mod.matmul_tp_persistent


def compare(ours, ref):
    """(number of elements whose bits differ, largest |difference| in units of the last place of max|ref|)"""
    mism = int((ours.view(torch.int16) != ref.view(torch.int16)).sum())
    amax = ref.float().abs().max().item()
    unit = 2.0 ** (math.floor(math.log2(amax)) - 7) if amax > 0 else 1.0
    return mism, (ours.float() - ref.float()).abs().max().item() / unit


def operands(M, K, N, dtype, seed, integer):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if integer:
        A = torch.randint(-15, 16, (M, K), generator=g, device="cuda").to(dtype)
        W = torch.randint(-15, 16, (N, K), generator=g, device="cuda").to(dtype)
    else:
        A = torch.randn(M, K, generator=g, device="cuda").to(dtype)
        W = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(dtype)
    return A, W


SHAPES = [(64, 4096, 1024)] + [(M, K, 4096) for K in (4096, 12288) for M in (1, 16, 256, 2048)]


@pytest.mark.parametrize("M,K,N", SHAPES)
def test_integer_operands_bit_equal_to_reference_kernel(M, K, N):
    from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent
    ref = reference_matmul()
    A, W = operands(M, K, N, torch.bfloat16, 1000 + M + K, integer=True)
    ours = matmul_tp_persistent(A, W.t())
    theirs = ref(A, W.t())
    torch.cuda.synchronize()
    assert torch.equal(ours.view(torch.int16), theirs.view(torch.int16))


@pytest.mark.parametrize("M,K,N", SHAPES)
def test_normal_operands_within_one_ulp_of_reference_kernel(M, K, N, record_property):
    from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent
    ref = reference_matmul()
    A, W = operands(M, K, N, torch.bfloat16, 2000 + M + K, integer=False)
    ours = matmul_tp_persistent(A, W.t())
    theirs = ref(A, W.t())
    torch.cuda.synchronize()
    mism, max_ulp = compare(ours, theirs)
    record_property("mismatching_elements", mism)
    record_property("max_ulp", max_ulp)
    print(f"reference-kernel parity M={M} K={K} N={N}: {mism} of {M * N} elements differ, max {max_ulp:.3f} units")
    assert mism <= max(1, int(MAX_MISMATCH_FRACTION * M * N)), (mism, M * N)
    assert max_ulp <= MAX_ULP


@pytest.mark.parametrize("M,K,N", [(192, 3072, 384), (200, 3072, 256), (100, 6144, 128)])
def test_fp16_integer_operands_bit_equal_to_reference_kernel(M, K, N):
    """fp16, radix-3 trees, ragged M.  N stays a multiple of the reference's 128-column tile: at other N the
    GPU-compiled reference kernel (triton 3.6.0, sm_100) was observed to differ from its own CPU-interpreter run --
    and from the oracle, which this repository's kernel matches there -- in a few hundred elements of columns 1..7,
    so such shapes cannot serve as a comparison."""
    from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent
    ref = reference_matmul()
    A, W = operands(M, K, N, torch.float16, 7, integer=True)
    assert torch.equal(matmul_tp_persistent(A, W.t()).view(torch.int16), ref(A, W.t()).view(torch.int16))
