"""Parity of the sm_100a tree GEMM (called through the C ABI) against the CPU oracle, the golden
outputs of the reference kernel, and the invariance properties the reference checks.

Bit-exact cases use integer-valued operands: every leaf dot product is then exact in fp32 in any
summation order, so the only freedom left is the rounding/tree order under test.  With N(0,1) x
N(0,0.02) operands the order of the 256 fp32 additions inside a leaf (fixed by the tensor core, not
by this code or the reference's) can move a leaf by one rounding step; those cases are held to a
mismatch budget and to the oracle's own error against fp64.
"""
import ctypes
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

from make_golden import MATMUL_CASES, make_inputs  # noqa: E402
from oracle.tbik_ref import exact_int_inputs, matmul_fp64, normal_inputs, sharded_matmul_ref, tbik_matmul_ref  # noqa: E402

pytestmark = pytest.mark.gpu

# budget for operands whose leaf sums are not exact in fp32
MAX_MISMATCH_FRACTION = 5e-4   # measured: 1.7e-4 and 3.1e-4
MAX_MISMATCH_ULP = 1           # in units of the last place of the largest output value
MAX_REL_ERR_VS_FP64 = 1.0e-2  # of max|C|; the oracle itself sits at ~6.5e-3 for bf16 nodes


def bits(t):
    return t.contiguous().view(torch.int16)


def kmajor(B):
    """[K,N] view whose memory is K-contiguous, like weight.t() of a row-parallel layer."""
    return B.cuda().t().contiguous().t()


@pytest.fixture(scope="module")
def mm():
    from llm_reproducibility_b200.tbik.tree_based_matmul import gemm_device_status, matmul_tp_persistent

    def run(A, B, *args, **kw):
        C = matmul_tp_persistent(A, B, *args, **kw)
        torch.cuda.synchronize()
        assert gemm_device_status()[0] == 0
        return C
    return run


GOLD = torch.load(os.path.join(HERE, "golden", "matmul_reference_interpreter.pt"))
FP16_INT_CASES = [c for c in MATMUL_CASES if c[1] == torch.float16 and c[5] == "int"]


@pytest.mark.parametrize("case", FP16_INT_CASES, ids=[c[0] for c in FP16_INT_CASES])
def test_matches_reference_kernel_golden_outputs(mm, case):
    """CUDA kernel vs the stored outputs of the reference's own Triton kernel (every tree shape)."""
    name, dt, M, K, N, gen, seed = case
    A, B = make_inputs(dt, M, K, N, gen, seed)
    C = mm(A.cuda(), kmajor(B))
    assert torch.equal(bits(C.cpu()), bits(GOLD[name]))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,N", [
    (1, 256, 8), (1, 4096, 4096), (16, 12288, 256), (37, 1536, 200), (128, 512, 128), (129, 768, 136),
    (130, 12800, 128), (256, 4096, 512), (300, 6144, 384), (64, 25600, 128),
])
def test_bit_exact_vs_oracle_integer_operands(mm, dt, M, K, N):
    amax = 15 if dt == torch.bfloat16 else 7
    A, B = exact_int_inputs(M, K, N, dt, seed=M * 7 + K, amax=amax)
    C = mm(A.cuda(), kmajor(B))
    assert torch.equal(bits(C.cpu()), bits(tbik_matmul_ref(A, B)))


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,N", [(1, 4096, 64), (37, 1536, 200), (130, 12288, 136), (16, 25600, 128)])
def test_bit_exact_vs_c_oracle_integer_operands(mm, dt, M, K, N):
    """The CUDA path against the plain-C restatement (scalar loops, own conversions), decode- and prefill-sized."""
    from oracle import c_oracle
    A, B = exact_int_inputs(M, K, N, dt, seed=M + K + N, amax=7)
    C = mm(A.cuda(), kmajor(B))
    assert torch.equal(bits(C.cpu()), bits(c_oracle.matmul(A, B)))


@pytest.mark.parametrize("K", [16384, 32768])
def test_deep_trees_use_the_shared_memory_levels(mm, K):
    """L = 6 and 7: levels above the TMEM stack are kept in shared memory."""
    A, B = exact_int_inputs(130, K, 136, torch.bfloat16, seed=K, amax=7)
    C = mm(A.cuda(), kmajor(B))
    assert torch.equal(bits(C.cpu()), bits(tbik_matmul_ref(A, B)))


def test_very_deep_tree_scratch_rules():
    """L = 8 (K = 65536).  The 256-wide tilings keep only one level above the registers on chip and need
    scratch for the rest: without it they are refused with a message naming the need.  The entry point
    without scratch still works (it picks a tiling whose whole stack fits tensor memory)."""
    from llm_reproducibility_b200 import _lib
    A, B = exact_int_inputs(130, 65536, 136, torch.bfloat16, seed=8, amax=3)
    Ad, W = A.cuda(), B.cuda().t().contiguous()
    ref = tbik_matmul_ref(A, B)
    C = torch.empty(130, 136, dtype=torch.bfloat16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    L = _lib.lib()
    assert L.tbik_gemm(Ad.data_ptr(), W.data_ptr(), C.data_ptr(), 130, 136, 65536, 65536, 65536, 136, 0, 256, 0, s) == 0
    torch.cuda.synchronize()
    assert torch.equal(bits(C.cpu()), bits(ref))
    rc = L.tbik_gemm_ex(Ad.data_ptr(), W.data_ptr(), C.data_ptr(), 130, 136, 65536, 65536, 65536, 136, 0, 256, 0,
                        0, 3, None, 0, s)
    assert rc == -2 and "scratch" in _lib.last_error()
    for tiling in TILINGS:
        assert torch.equal(bits(_gemm_ex(Ad, W, 130, 136, 65536, 0, tiling).cpu()), bits(ref)), tiling


def test_entry_point_without_scratch_matches_the_ones_with_scratch():
    """tbik_gemm (no scratch: it picks the 256x128 pair tiling, whose stack fits on chip), the schedule the automatic
    choice prefers when it is given scratch (256x256 pair tiles), the 128x256 tiling (needs scratch for a 5-level tree)
    and tbik_gemm_ws at a decode-sized M (K-slabs, roots in the workspace) agree bitwise."""
    from llm_reproducibility_b200 import _lib
    from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent
    L = _lib.lib()
    M, K, N = 1000, 12288, 4096
    assert L.tbik_gemm_workspace_bytes(M, N, K, 256) > 0          # 256x256 pair tiles: upper stack levels in scratch
    assert L.tbik_gemm_slabs_workspace_bytes(M, N, K, 256, 2, 1) == 0   # 256x128 pair tiles: the whole stack in tensor memory
    assert L.tbik_gemm_slabs_workspace_bytes(M, N, K, 256, 3, 1) > 0   # 128x256 tiles, 5-level tree: 3 levels go to scratch
    assert L.tbik_gemm_workspace_bytes(64, N, K, 256) > 0         # small M: room for the K-slab roots
    assert L.tbik_gemm_workspace_bytes(64, N, 256, 256) == 0      # one leaf: nothing to cut, no scratch
    g = torch.Generator(device="cuda").manual_seed(1)
    A = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    C0 = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert L.tbik_gemm(A.data_ptr(), W.data_ptr(), C0.data_ptr(), M, N, K, K, K, N, 0, 256, 0, s) == 0
    C1 = matmul_tp_persistent(A, W.t())
    C3 = _gemm_ex(A, W, M, N, K, 0, 3)
    torch.cuda.synchronize()
    assert torch.equal(bits(C0), bits(C1)) and torch.equal(bits(C0), bits(C3))
    # decode-sized M: no scratch -> one CTA per tile, with scratch -> K-slabs; same bits
    C4 = torch.empty(64, N, dtype=torch.bfloat16, device="cuda")
    assert L.tbik_gemm(A.data_ptr(), W.data_ptr(), C4.data_ptr(), 64, N, K, K, K, N, 0, 256, 0, s) == 0
    C5 = matmul_tp_persistent(A[:64], W.t())
    torch.cuda.synchronize()
    assert torch.equal(bits(C4), bits(C5)) and torch.equal(bits(C4), bits(C0[:64]))


@pytest.mark.parametrize("leaf,K", [(128, 3200), (64, 1600), (640, 3200), (512, 4096)])
def test_other_leaf_widths(mm, leaf, K):
    """Leaf widths other than 256, e.g. 128 for a K/8 = 3200 shard (Qwen3-32B down_proj at TP=8)."""
    A, B = exact_int_inputs(40, K, 72, torch.bfloat16, seed=leaf, amax=7)
    C = mm(A.cuda(), kmajor(B), leaf=leaf)
    assert torch.equal(bits(C.cpu()), bits(tbik_matmul_ref(A, B, leaf=leaf)))


@pytest.mark.parametrize("M,K,N", [(64, 4096, 1024), (256, 12288, 512), (2048, 4096, 4096)])
def test_normal_operands_within_budget(mm, M, K, N):
    A, B = normal_inputs(M, K, N, torch.bfloat16, seed=0)
    C = mm(A.cuda(), kmajor(B)).cpu()
    ref = tbik_matmul_ref(A, B)
    mismatch = (bits(C) != bits(ref)).float().mean().item()
    # A leaf whose fp32 sum lands on the other side of a rounding boundary moves the result by one unit in the
    # last place OF THAT LEAF; leaves are no larger than the largest output, so no element may be off by more
    # than MAX_MISMATCH_ULP such units (an element near zero is then many of its own, much smaller, units away).
    import math
    unit = 2.0 ** (math.floor(math.log2(ref.float().abs().max().item())) - 7)
    assert (C.float() - ref.float()).abs().max().item() <= MAX_MISMATCH_ULP * unit
    f64 = matmul_fp64(A, B)
    scale = f64.abs().max().item()
    err = (C.double() - f64).abs().max().item() / scale
    err_ref = (ref.double() - f64).abs().max().item() / scale
    assert mismatch <= MAX_MISMATCH_FRACTION, mismatch
    assert err <= MAX_REL_ERR_VS_FP64 and err <= 1.5 * err_ref + 1e-6, (err, err_ref)


@pytest.mark.parametrize("K,N", [(4096, 4096), (12288, 4096)])
@pytest.mark.parametrize("M", [1, 16, 256])
def test_config2_shard_invariance_vs_oracle(mm, M, K, N):
    """Qwen3-8B o_proj / down_proj: K shards at tp=1/2/4/8 + rank-pair tree == unsharded, bitwise,
    and (integer operands) == the oracle's sharded result."""
    Nn = 512  # a 512-column slice of the layer keeps the CPU oracle fast; tiles are independent in N
    A, B = exact_int_inputs(M, K, Nn, torch.bfloat16, seed=M + K, amax=7)
    Ad, Bd = A.cuda(), kmajor(B)
    full = mm(Ad, Bd)
    assert torch.equal(bits(full.cpu()), bits(tbik_matmul_ref(A, B)))
    for tp in (2, 4, 8):
        ks = K // tp
        parts = [mm(Ad[:, r * ks:(r + 1) * ks], Bd[r * ks:(r + 1) * ks]) for r in range(tp)]
        while len(parts) > 1:
            parts = [parts[i] + parts[i + 1] for i in range(0, len(parts), 2)]
        assert torch.equal(bits(parts[0]), bits(full)), tp
        assert torch.equal(bits(parts[0].cpu()), bits(sharded_matmul_ref(A, B, tp))), tp


@pytest.mark.parametrize("K,N", [(4096, 4096), (12288, 4096)])
def test_full_size_invariance_properties(mm, K, N):
    """M = 8192 (too big for the CPU oracle): batch invariance and shard invariance, bitwise."""
    g = torch.Generator(device="cuda").manual_seed(K)
    A = torch.randn(8192, K, generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    full = mm(A, W.t())
    for m in (1, 16, 256, 2048):
        assert torch.equal(bits(mm(A[:m], W.t())), bits(full[:m])), m
    off = 4096 + 77  # a row window that starts inside a tile
    assert torch.equal(bits(mm(A[off:off + 300], W.t())), bits(full[off:off + 300]))
    for tp in (2, 4, 8):
        ks = K // tp
        parts = [mm(A[:, r * ks:(r + 1) * ks], W.t()[r * ks:(r + 1) * ks]) for r in range(tp)]
        while len(parts) > 1:
            parts = [parts[i] + parts[i + 1] for i in range(0, len(parts), 2)]
        assert torch.equal(bits(parts[0]), bits(full)), tp
    # agreement with an fp32-accumulated product, as a sanity bound on the whole tile grid
    ref = (A[:512].float() @ W.float().t())
    rel = ((full[:512].float() - ref).abs().max() / ref.abs().max()).item()
    assert rel < MAX_REL_ERR_VS_FP64


_WS = {}


def _gemm_ex(Ad, W, M, N, K, ctas, tiling, dtype_code=0, leaf=256, workspace=True):
    from llm_reproducibility_b200 import _lib
    C = torch.empty(M, N, dtype=Ad.dtype, device="cuda")
    if workspace:
        if "ws" not in _WS:
            _WS["ws"] = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
        wp, wn = _WS["ws"].data_ptr(), _WS["ws"].numel()
    else:
        wp, wn = None, 0
    rc = _lib.lib().tbik_gemm_ex(Ad.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, K, K, N,
                                 dtype_code, leaf, _lib.NODE_INPUT, ctas, tiling, wp, wn,
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    return C


TILINGS = [1, 2, 3, 4, 5, 6]


@pytest.mark.parametrize("tiling", TILINGS)
def test_result_does_not_depend_on_cta_count(tiling):
    A, B = normal_inputs(700, 1536, 520, torch.bfloat16, seed=5)
    Ad, W = A.cuda(), B.cuda().t().contiguous()
    outs = [_gemm_ex(Ad, W, 700, 520, 1536, ctas, tiling) for ctas in (0, 1, 2, 3, 7, 148)]
    for C in outs[1:]:
        assert torch.equal(bits(C), bits(outs[0]))


@pytest.mark.parametrize("K", [512, 1024, 1536])
def test_short_k_many_tiles_every_tiling_repeatedly(K):
    """Tensor-parallel shard shapes: few leaves per tile, many tiles per CTA, so tile hand-overs (accumulator buffers,
    stack slot, staged stores of C) happen every few microseconds.  Every tiling, three times, same bits."""
    M, N = 2048, 4096
    g = torch.Generator(device="cuda").manual_seed(K)
    A = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    one = _gemm_ex(A, W, M, N, K, 0, 1)
    for tiling in TILINGS:
        for rep in range(3):
            assert torch.equal(bits(one), bits(_gemm_ex(A, W, M, N, K, 0, tiling))), (tiling, rep)
    auto = _gemm_ex(A, W, M, N, K, 0, 0)
    assert torch.equal(bits(one), bits(auto))


def _gemm_slabs(Ad, W, M, N, K, tiling, slabs, dtype_code=0, leaf=256, ldc=None):
    from llm_reproducibility_b200 import _lib
    L = _lib.lib()
    ldc = ldc or N
    C = torch.zeros(M, ldc, dtype=Ad.dtype, device="cuda")
    need = L.tbik_gemm_slabs_workspace_bytes(M, N, K, leaf, tiling, slabs)
    assert need > 0 or slabs == 1
    ws = torch.zeros(max(need, 16), dtype=torch.uint8, device="cuda")
    rc = L.tbik_gemm_slabs(Ad.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, K, K, ldc, dtype_code, leaf, _lib.NODE_INPUT,
                           tiling, slabs, ws.data_ptr(), need, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _lib.last_error()
    torch.cuda.synchronize()
    from llm_reproducibility_b200.tbik.tree_based_matmul import gemm_device_status
    assert gemm_device_status()[0] == 0
    return C[:, :N]


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (16, 12288, 4096), (128, 12288, 520), (200, 2048, 1000),
                                   (64, 1536, 4096), (300, 8192, 264), (7, 6144, 99)])
def test_k_slabs_give_the_same_bits(M, K, N):
    """Cutting K into 2..16 subtrees that separate CTAs compute, then adding the roots pairwise, is the reduction tree
    itself: every (tiling, slabs) combination equals the unsplit kernel bit for bit (random operands) and the oracle
    (integer operands).  N not a multiple of 8 and a padded C exercise the scalar stores of the in-kernel combine."""
    from llm_reproducibility_b200 import _lib
    T, F, _ = (ctypes.c_int(), ctypes.c_int(), ctypes.c_int())
    assert _lib.lib().tbik_tree_shape(K, 256, ctypes.byref(T), ctypes.byref(F), ctypes.byref(_)) == 0
    groups = T.value // F.value
    g = torch.Generator(device="cuda").manual_seed(M * 3 + K + N)
    A = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    one = _gemm_ex(A, W, M, N, K, 0, 1)
    Ai, Bi = exact_int_inputs(M, K, N, torch.bfloat16, seed=K + N, amax=7)
    ref_i = tbik_matmul_ref(Ai, Bi)
    Aid, Wi = Ai.cuda(), Bi.cuda().t().contiguous()
    tested = 0
    for tiling in TILINGS:
        for slabs in (2, 4, 8, 16):
            if slabs > groups:
                assert _lib.lib().tbik_gemm_slabs_workspace_bytes(M, N, K, 256, tiling, slabs) == 0
                continue
            assert torch.equal(bits(_gemm_slabs(A, W, M, N, K, tiling, slabs)), bits(one)), (tiling, slabs)
            assert torch.equal(bits(_gemm_slabs(Aid, Wi, M, N, K, tiling, slabs, ldc=N + 24).cpu()), bits(ref_i)), (tiling, slabs)
            tested += 1
    assert tested >= 6
    h, Wh = A.to(torch.float16), W.to(torch.float16)
    one = _gemm_ex(h, Wh, M, N, K, 0, 1, dtype_code=1)
    assert torch.equal(bits(_gemm_slabs(h, Wh, M, N, K, 3, 2, dtype_code=1)), bits(one))


def test_stack_scratch_and_k_slabs_share_one_workspace():
    """A launch that keeps tree levels in the workspace (256-column tilings) followed, on the SAME workspace, by a
    decode-sized launch that counts K-slab arrivals at its head: the first must not leave the counters non-zero.
    (Found under a serving engine: the profile run of 4096 rows used the scratch, the decode steps after it
    returned garbage.)"""
    from llm_reproducibility_b200 import _lib
    L = _lib.lib()
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(11)
    K, N = 1536, 1024
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    s = torch.cuda.current_stream().cuda_stream

    def ws_call(A, leaf, tiling=None):
        M = A.shape[0]
        C = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
        if tiling is None:
            rc = L.tbik_gemm_ws(A.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, K, K, N, 0, leaf, 0, ws.data_ptr(), ws.numel(), s)
        else:
            rc = L.tbik_gemm_ex(A.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, K, K, N, 0, leaf, 0, 0, tiling, ws.data_ptr(), ws.numel(), s)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        return C

    for leaf in (128, 256):
        big = torch.randn(4096, K, generator=g, device="cuda").to(torch.bfloat16)
        small = torch.randn(4, K, generator=g, device="cuda").to(torch.bfloat16)
        want = _gemm_ex(small, W, 4, N, K, 0, 1, leaf=leaf)       # 128x128 tiling, its own workspace
        for tiling in (None, 3, 4):                                # automatic, 128x256, 256x256: stack levels in scratch
            ws_call(big, leaf, tiling)
            for _ in range(2):
                assert torch.equal(bits(ws_call(small, leaf)), bits(want)), (leaf, tiling)
    from llm_reproducibility_b200.tbik.tree_based_matmul import gemm_device_status
    assert gemm_device_status()[0] == 0


def test_k_slab_argument_errors():
    from llm_reproducibility_b200 import _lib
    L = _lib.lib()
    A = torch.zeros(16, 1024, dtype=torch.bfloat16, device="cuda")
    W = torch.zeros(64, 1024, dtype=torch.bfloat16, device="cuda")
    C = torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda")
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    call = lambda tiling, slabs, wsb: L.tbik_gemm_slabs(A.data_ptr(), W.data_ptr(), C.data_ptr(), 16, 64, 1024, 1024, 1024, 64,
                                                        0, 256, 0, tiling, slabs, ws.data_ptr(), wsb, s)
    assert call(0, 2, ws.numel()) == -1                       # automatic tiling is not accepted here
    assert call(1, 3, ws.numel()) == -1                       # not a power of two
    assert call(1, 32, ws.numel()) == -1                      # more than 16
    assert call(1, 4, ws.numel()) == -2 and "subtrees" in _lib.last_error()   # T = 4, F = 2: only 2 whole subtrees
    assert call(1, 2, 64) == -2 and "scratch" in _lib.last_error()            # workspace too small for the roots
    assert call(1, 2, ws.numel()) == 0
    torch.cuda.synchronize()


@pytest.mark.parametrize("M,K,N", [(1, 4096, 512), (100, 4096, 512), (128, 12288, 256), (129, 4096, 384),
                                   (700, 1536, 520), (2048, 4096, 4096), (4096, 12288, 1024)])
def test_all_tilings_agree_bitwise(M, K, N):
    """Random (not exactly representable) operands: the 128x128, 256x128 (CTA pair), 128x256 and
    256x256 (CTA pair) schedules must give the same bits, otherwise results would change with the
    batch size (the automatic choice depends on M)."""
    g = torch.Generator(device="cuda").manual_seed(M + K + N)
    A = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    one = _gemm_ex(A, W, M, N, K, 0, 1)
    for tiling in TILINGS[1:]:
        assert torch.equal(bits(one), bits(_gemm_ex(A, W, M, N, K, 0, tiling))), tiling
    h = torch.randn(M, K, generator=g, device="cuda").to(torch.float16)
    Wh = W.to(torch.float16)
    one = _gemm_ex(h, Wh, M, N, K, 0, 1, dtype_code=1)
    for tiling in TILINGS[1:]:
        assert torch.equal(bits(one), bits(_gemm_ex(h, Wh, M, N, K, 0, tiling, dtype_code=1))), tiling


@pytest.mark.parametrize("tiling", TILINGS)
@pytest.mark.parametrize("M,K,N", [(300, 12288, 384), (130, 12800, 128), (130, 16384, 136), (257, 768, 136)])
def test_both_tilings_bit_exact_vs_oracle(tiling, M, K, N):
    A, B = exact_int_inputs(M, K, N, torch.bfloat16, seed=M + K, amax=7)
    C = _gemm_ex(A.cuda(), B.cuda().t().contiguous(), M, N, K, 0, tiling)
    assert torch.equal(bits(C.cpu()), bits(tbik_matmul_ref(A, B)))


def test_strided_operands_and_output_and_bias(mm):
    A, B = exact_int_inputs(50, 512, 96, torch.bfloat16, seed=11, amax=7)
    big = torch.zeros(50, 1024, dtype=torch.bfloat16, device="cuda")
    big[:, 256:768] = A.cuda()
    Av = big[:, 256:768]                      # row stride 1024, 16-byte aligned start
    Bn = B.cuda()                             # N-contiguous [K,N]: copied to K-major once
    ref = tbik_matmul_ref(A, B)
    assert torch.equal(bits(mm(Av, Bn).cpu()), bits(ref))
    odd = big[:, 1:513]                       # misaligned start: wrapper makes it contiguous
    assert torch.equal(bits(mm(odd, Bn).cpu()), bits(tbik_matmul_ref(odd.cpu(), B)))
    outbuf = torch.zeros(50, 200, dtype=torch.bfloat16, device="cuda")
    mm(Av, Bn, out=outbuf[:, 8:104])          # C with a row stride larger than N
    assert torch.equal(bits(outbuf[:, 8:104].cpu()), bits(ref))
    assert float(outbuf[:, :8].abs().sum()) == 0 and float(outbuf[:, 104:].abs().sum()) == 0
    bias = torch.arange(96, dtype=torch.bfloat16, device="cuda")
    assert torch.equal(bits(mm(Av, Bn, bias).cpu()), bits(ref + bias.cpu()))


def test_empty_and_error_paths(mm):
    from llm_reproducibility_b200 import _lib
    A = torch.zeros(0, 256, dtype=torch.bfloat16, device="cuda")
    B = torch.zeros(256, 16, dtype=torch.bfloat16, device="cuda")
    assert mm(A, kmajor(B.cpu())).shape == (0, 16)
    with pytest.raises(AssertionError):       # K % 256 != 0, as the reference asserts
        mm(torch.zeros(4, 320, dtype=torch.bfloat16, device="cuda"), torch.zeros(320, 8, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(NotImplementedError):
        mm(torch.zeros(4, 256, device="cuda"), torch.zeros(256, 8, device="cuda"))
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent
        matmul_tp_persistent(torch.zeros(4, 256, dtype=torch.bfloat16), torch.zeros(256, 8, dtype=torch.bfloat16))
    # C ABI level: bad leaf, bad alignment, null pointer
    L = _lib.lib()
    x = torch.zeros(256 * 8 + 8, dtype=torch.bfloat16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert L.tbik_gemm(x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, 8, 256, 256, 256, 8, 0, 100, 0, s) == -2
    assert "leaf" in _lib.last_error()
    assert L.tbik_gemm(x.data_ptr() + 2, x.data_ptr(), x.data_ptr(), 1, 8, 256, 256, 256, 8, 0, 256, 0, s) == -4
    assert L.tbik_gemm(None, x.data_ptr(), x.data_ptr(), 1, 8, 256, 256, 256, 8, 0, 256, 0, s) == -1
    assert L.tbik_gemm(x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, 8, 256, 256, 256, 8, 2, 256, 0, s) == -3


def test_simple_matmul_demo_shape(mm):
    """The reference's self-check (simple_matmul.py): M,K,N = 1024,6144,2048, 4 shards."""
    g = torch.Generator(device="cuda").manual_seed(0)
    A = torch.randn(1024, 6144, generator=g, device="cuda").to(torch.bfloat16)
    B = torch.randn(6144, 2048, generator=g, device="cuda").to(torch.bfloat16)
    full = mm(A, B)
    assert torch.equal(bits(mm(A[:512], B)), bits(full[:512]))
    parts = [mm(A[:, i * 1536:(i + 1) * 1536], B[i * 1536:(i + 1) * 1536]) for i in range(4)]
    assert torch.equal(bits((parts[0] + parts[1]) + (parts[2] + parts[3])), bits(full))
