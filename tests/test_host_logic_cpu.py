"""CPU tests: the C ABI's export list, the env switches, and the all-reduce host logic on gloo ranks
(with tests/fake_backend.py standing in for the CUDA runtime and the native ops)."""
import ctypes
import os
import re
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, HERE)

from _dist_utils import run_ranks  # noqa: E402
import _host_workers as hw  # noqa: E402


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "tbik.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tbik_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from llm_reproducibility_b200 import _lib
    names = _declared_functions()
    assert len(names) >= 15
    handle = _lib.lib()
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in include/tbik.h but not exported"
    assert sorted(_lib.exported_symbols()) == names, "ctypes prototypes and include/tbik.h disagree"


def test_cabi_calls_that_need_no_gpu():
    from llm_reproducibility_b200 import _lib
    L = _lib.lib()
    assert L.tbik_version() >= 1000
    T, F, Lv = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    for K, leaf, want in ((4096, 256, (16, 2, 4)), (12288, 256, (48, 3, 5)), (25600, 256, (100, 25, 3)),
                          (3200, 128, (25, 25, 1)), (256, 256, (1, 1, 1))):
        assert L.tbik_tree_shape(K, leaf, ctypes.byref(T), ctypes.byref(F), ctypes.byref(Lv)) == 0
        assert (T.value, F.value, Lv.value) == want
    assert L.tbik_tree_shape(3200, 256, ctypes.byref(T), ctypes.byref(F), ctypes.byref(Lv)) == -2
    assert "multiple" in _lib.last_error()
    assert L.tbik_ar_meta_size() % 128 == 0 and L.tbik_ar_meta_size() > 0
    out = ctypes.c_void_p()
    assert L.tbik_ar_create(None, 2, 0, None, 0, 1, ctypes.byref(out)) == -1
    sig = (ctypes.c_void_p * 9)(*([1] * 9))
    assert L.tbik_ar_create(sig, 9, 0, 1, 1 << 20, 1, ctypes.byref(out)) == -2 and "world size > 8" in _lib.last_error()
    assert L.tbik_ar_create(sig, 3, 0, 1, 1 << 20, 1, ctypes.byref(out)) == -2 and "Odd num gpus" in _lib.last_error()
    assert L.tbik_ar_create(sig, 2, 5, 1, 1 << 20, 1, ctypes.byref(out)) == -1 and "invalid rank" in _lib.last_error()


def test_product_never_touches_the_oracle_or_a_cpu_fallback():
    """The oracle is test infrastructure: nothing under the package may import, read or run it."""
    pkg = os.path.join(ROOT, "llm_reproducibility_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f), encoding="utf-8").read()
                assert "oracle" not in text, os.path.join(base, f)
                assert "_work/" not in text, os.path.join(base, f)


def test_k_slab_plan_queries_need_no_gpu():
    """Which (tiling, slabs) combinations exist and what scratch they need is host arithmetic."""
    from llm_reproducibility_b200 import _lib
    L = _lib.lib()
    need = L.tbik_gemm_slabs_workspace_bytes
    M, N, K = 16, 4096, 12288                       # T = 48, F = 3: 16 level-0 groups
    for tiling in range(1, 7):
        sizes = [need(M, N, K, 256, tiling, s) for s in (2, 4, 8, 16)]
        assert all(b >= s * M * N * 2 for b, s in zip(sizes, (2, 4, 8, 16))), (tiling, sizes)   # room for every root
        assert all(b % 16 == 0 for b in sizes)
        assert need(M, N, K, 256, tiling, 32) == 0   # more than 16 slabs
        assert need(M, N, K, 256, tiling, 3) == 0    # not a power of two
    assert need(M, N, 1536, 256, 1, 4) == 0          # T = 6, F = 3: only two whole subtrees
    assert need(M, N, 1536, 256, 1, 2) >= 2 * M * N * 2
    assert need(M, N, K, 256, 0, 2) == 0 and need(M, N, K, 256, 7, 2) == 0   # tiling out of range
    assert need(M, N, 1000, 256, 1, 2) == 0          # K not a multiple of the leaf
    assert need(M, 4090, K, 256, 1, 2) >= 2 * M * 4096 * 2                   # rows of the roots padded to 8 columns


def test_automatic_plan_weighs_the_two_pair_tilings_by_whole_waves():
    """With scratch the 256x256 CTA-pair tile (code 4) is taken unless the last partial wave makes 256x128 (code 2)
    cheaper; without scratch only 256x128 can hold a tree of leaves of 256.  Host arithmetic (148 SMs assumed when
    there is no device)."""
    import ctypes
    from llm_reproducibility_b200 import _lib
    L = _lib.lib()
    out = (ctypes.c_int * 4)()

    def plan(M, N, K, ctas=0, ws=1 << 30):
        assert L.tbik_gemm_plan(M, N, K, 256, ctas, ctypes.c_size_t(ws), out) == 0
        return out[0], out[1], out[2]

    assert plan(8192, 4096, 4096) == (4, 1, 148) and plan(8192, 4096, 12288) == (4, 1, 148)   # the benchmark step
    assert plan(8192, 4096, 4096, ws=0)[0] == 2 and plan(8192, 4096, 12288, ws=0)[0] == 2     # no scratch
    assert plan(8192, 4096, 512)[0] == 4                       # short K: fewer tiles to refill the pipeline for
    assert plan(4096, 4096, 2048, ctas=116)[0] == 2            # 58 pairs: 9 waves of 256x128 against 5 of 256x256
    t, s, _ = plan(16, 4096, 4096)                             # decode: a narrow tile and K-slabs
    assert t in (5, 6) and s >= 2
    assert L.tbik_gemm_workspace_bytes(8192, 4096, 4096, 256) > 0


def test_fp32_node_leaf_rule_and_argument_checks():
    """K_total / max_tp: exactly max_tp leaves, every level binary, a whole subtree per rank at every TP degree."""
    import torch
    from llm_reproducibility_b200 import _lib
    from llm_reproducibility_b200.tbik.tree_based_matmul import _node_code, leaf_for_fp32_nodes, tree_shape
    assert leaf_for_fp32_nodes(4096, 8) == 512 and leaf_for_fp32_nodes(12288, 8) == 1536
    assert leaf_for_fp32_nodes(25600, 8) == 3200 and leaf_for_fp32_nodes(4096, 2) == 2048
    for K, tp in ((4096, 8), (12288, 8), (25600, 8), (8192, 4)):
        leaf = leaf_for_fp32_nodes(K, tp)
        T, F, L = tree_shape(K, leaf)
        assert T == tp and F <= 2 and L <= 3                       # fits the tensor-memory stack of the fast tilings
        for deg in (1, 2, 4, 8):
            if deg <= tp:
                assert (K // deg) % leaf == 0                       # whole leaves per rank
    with pytest.raises(ValueError):
        leaf_for_fp32_nodes(4096, 3)
    with pytest.raises(ValueError):
        leaf_for_fp32_nodes(1000, 8)
    a = torch.empty(1, dtype=torch.bfloat16)
    assert _node_code(a, None, None) == _lib.NODE_INPUT and _node_code(a, torch.bfloat16, None) == _lib.NODE_INPUT
    assert _node_code(a, torch.float32, None) == _lib.NODE_FP32
    assert _node_code(a, torch.float32, torch.float32) == _lib.NODE_FP32_OUT_FP32
    for bad in ((None, torch.float32), (torch.float64, None), (torch.float32, torch.float16)):
        with pytest.raises(ValueError):
            _node_code(a, *bad)


def test_oracle_tree_shape_agrees_with_library():
    from llm_reproducibility_b200.tbik.tree_based_matmul import tree_shape as lib_shape
    from oracle.tbik_ref import tree_shape
    for K in range(256, 256 * 130, 256):
        assert lib_shape(K, 256) == tree_shape(K, 256)


def test_env_switches(monkeypatch):
    from llm_reproducibility_b200 import utils
    for k in ("VLLM_BATCH_INVARIANT", "VLLM_TP_INVARIANT", "ALIGN_TRAIN_INFERENCE", "TP_INVARIANT_MATMUL"):
        monkeypatch.delenv(k, raising=False)
    assert not utils.batch_invariant_is_enabled() and not utils.tp_invariant_is_enabled()
    assert not utils.compatible_mode_is_enabled() and not utils.check_invariant_compat()
    monkeypatch.setenv("VLLM_TP_INVARIANT", "1")
    with pytest.raises(AssertionError):   # TP invariance needs batch invariance
        utils.tp_invariant_is_enabled()
    monkeypatch.setenv("VLLM_BATCH_INVARIANT", "1")
    assert utils.tp_invariant_is_enabled() and utils.check_invariant_compat()
    monkeypatch.setenv("VLLM_BATCH_INVARIANT", "yes")   # not an integer -> off
    assert not utils.batch_invariant_is_enabled()
    monkeypatch.setenv("TP_INVARIANT_MATMUL", "1")
    assert utils.tp_invariant_matmul_is_enabled()


def test_apply_patches_without_flags_is_a_noop(monkeypatch, capsys):
    from llm_reproducibility_b200.patch import apply_patches
    for k in ("VLLM_BATCH_INVARIANT", "VLLM_TP_INVARIANT", "ALIGN_TRAIN_INFERENCE"):
        monkeypatch.delenv(k, raising=False)
    apply_patches()
    assert "No patches applied" in capsys.readouterr().out


def test_matmul_wrapper_refuses_cpu_tensors():
    from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        matmul_tp_persistent(torch.zeros(2, 256, dtype=torch.bfloat16), torch.zeros(256, 8, dtype=torch.bfloat16))
    with pytest.raises(AssertionError):
        matmul_tp_persistent(torch.zeros(2, 256), torch.zeros(128, 8))


def test_weak_contiguity_rule():
    from llm_reproducibility_b200.mini_allreduce.custom_all_reduce_utils import is_weak_contiguous
    A = torch.zeros(3, 3, 3)
    assert is_weak_contiguous(A) and is_weak_contiguous(A[1:]) and is_weak_contiguous(A.permute(2, 0, 1))
    assert is_weak_contiguous(A[1:].permute(2, 0, 1))
    assert not is_weak_contiguous(A[None].expand(2, -1, -1, -1)) and not is_weak_contiguous(A[:, 1:, 1:])


def test_full_nvlink_probe_with_fake_nvml():
    from llm_reproducibility_b200.mini_allreduce.custom_all_reduce_utils import is_full_nvlink

    class FakeNvml:
        NVML_P2P_CAPS_INDEX_NVLINK, NVML_P2P_STATUS_OK = 2, 0

        class NVMLError(Exception):
            pass

        def __init__(self, broken=(), raises=False):
            self.broken, self.raises, self.inits = broken, raises, 0

        def nvmlInit(self):
            self.inits += 1

        def nvmlShutdown(self):
            self.inits -= 1

        def nvmlDeviceGetHandleByIndex(self, i):
            return i

        def nvmlDeviceGetP2PStatus(self, a, b, idx):
            if self.raises:
                raise self.NVMLError()
            return 1 if (a, b) in self.broken else 0

    ok = FakeNvml()
    assert is_full_nvlink([0, 1, 2, 3], 4, nvml=ok) and ok.inits == 0
    assert not is_full_nvlink([0, 1, 2, 3], 4, nvml=FakeNvml(broken={(1, 3)}))
    assert not is_full_nvlink([0, 1], 2, nvml=FakeNvml(raises=True))


@pytest.mark.parametrize("world", [1, 2, 4])
def test_communicator_lifecycle_on_gloo_ranks(world):
    assert all(run_ranks(hw.communicator_lifecycle, world, backend="gloo"))


@pytest.mark.parametrize("world", [2, 4])
def test_communicator_disables_itself(world):
    assert all(run_ranks(hw.disabled_paths, world, backend="gloo"))


def test_dispatcher_paths_on_gloo_ranks():
    assert all(run_ranks(hw.dispatcher_paths, 2, backend="gloo"))


def test_native_tree_sum_rejects_non_power_of_two_world():
    assert all(run_ranks(hw.native_rejects_non_power_of_two, 3, backend="gloo"))


@pytest.mark.parametrize("world", [2, 4])
def test_row_parallel_forward_on_gloo_ranks(world):
    assert all(run_ranks(hw.row_parallel_layer, world, backend="gloo"))


def test_install_aliases_gives_the_reference_import_names():
    import subprocess
    code = ("import sys; sys.path.insert(0, %r); import llm_reproducibility_b200 as p; p.install_aliases();"
            "from src.tbik.tree_based_matmul import matmul_tp_persistent;"
            "from tbik.tree_based_all_reduce import tree_all_reduce_sum, tree_all_reduce_sum_native;"
            "from mini_allreduce import CustomAllreduce, CustomTreeAllreduce;"
            "import mini_allreduce.custom_all_reduce_ops as ops; import tbik_kernel.allreduce;"
            "from src.patch import apply_patches; from src.utils import tp_invariant_is_enabled;"
            "assert ops.meta_size() > 0; print('ok')") % ROOT
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr


def test_patch_binds_to_installed_vllm():
    """The row-parallel patch must import against the vLLM in this image (0.22) and replace forward."""
    import subprocess
    code = ("import sys; sys.path.insert(0, %r);"
            "from llm_reproducibility_b200.patch.patch_tp_invariant import patch_row_linear;"
            "from vllm.model_executor.layers.linear import RowParallelLinear as R; old = R.forward;"
            "patch_row_linear(); assert R.forward is not old; print('ok')") % ROOT
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    if "No module named 'vllm'" in out.stderr:
        pytest.skip("vllm not installed")
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-2000:]
