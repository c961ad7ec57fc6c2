"""Tree GEMM at the benchmark shapes, tiling by tiling and leaf width by leaf width, and -- with --wait-profile n --
where block 0's UMMA issuer and first epilogue warp spend their cycles.

    python tests/bench_gemm_tilings.py                      # TFLOP/s per (leaf, tiling), shipped library
    python tests/bench_gemm_tilings.py --wait-profile 2     # builds a development library with -DTBIK_WAIT_PROFILE=2
                                                            # (nvcc, about two minutes) and prints its counters

M = 8192, bf16, nodes of the operand type; o_proj (K = 4096) and down_proj (K = 12288), N = 4096.  Only leaf 256
reproduces the reference's bits (src/tbik/tree_based_matmul.py:206-231); the wider leaves show what each tiling's
main loop gives when the epilogue has little to do.  Operand sets rotate through more than L2; CUDA events.
--wait-profile: 1 = issuer (wait for a drained accumulator / for a landed stage); 2 = epilogue (wait for a leaf /
leaf ready to accumulator released); 3 = converting the last chunk / loads and adds of the climb; 4 = group-closing
leaves up to the store / stack stores; 5 = staged root stores / root stores from registers.
"""
import argparse
import ctypes
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

vp, i32, i64, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t


def load(path):
    L = ctypes.CDLL(path)
    L.tbik_gemm_ex.restype = i32
    L.tbik_gemm_ex.argtypes = [vp, vp, vp, i32, i32, i32, i64, i64, i64, i32, i32, i32, i32, i32, vp, sz, vp]
    L.tbik_last_error.restype = ctypes.c_char_p
    L.tbik_gemm_status.restype = i32
    return L


def build_profile_library(mode):
    src = os.path.join(ROOT, "llm_reproducibility_b200", "csrc")
    out_dir = os.path.join(ROOT, "llm_reproducibility_b200", "build")
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, f"libtbik_wait_profile{mode}.so")
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-cudart", "shared",
           f"-DTBIK_WAIT_PROFILE={mode}", "-I", os.path.join(ROOT, "include"), "-shared", "-o", out] + \
          [os.path.join(src, f) for f in ("capi.cu", "tree_gemm_sm100a.cu", "tree_allreduce.cu")]
    subprocess.run(cmd, check=True)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--wait-profile", type=int, default=0)
    ap.add_argument("--tilings", default="2,3,4")
    ap.add_argument("--m", type=int, default=8192)
    args = ap.parse_args()
    tilings = [int(t) for t in args.tilings.split(",")]
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    ws = torch.zeros(512 << 20, dtype=torch.uint8, device=dev)
    M = args.m
    if args.wait_profile:
        L = load(build_profile_library(args.wait_profile))
    else:
        L = load(os.path.join(ROOT, "llm_reproducibility_b200", "libtbik_b200.so"))
    labels = {1: ("accumulator_wait", "stage_wait"), 2: ("leaf_wait", "ready_to_release"), 3: ("convert_after_release", "climb"),
              4: ("group_leaf_to_store", "stack_store"), 5: ("staged_root", "register_root")}
    for name, K, N in (("o_proj", 4096, 4096), ("down_proj", 12288, 4096)):
        nset = max(2, -(-2 * (126 << 20) // (2 * (M * K + N * K + M * N))))
        sets = [(torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16),
                 (torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16),
                 torch.empty(M, N, dtype=torch.bfloat16, device=dev)) for _ in range(nset)]
        leaves = (256, 512) if args.wait_profile else (256, K // 8, K // 4, K // 2, K)
        for leaf in leaves:
            out = []
            for t in tilings:
                def run(i):
                    X, W, C = sets[i % nset]
                    rc = L.tbik_gemm_ex(X.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, K, K, N, 0, leaf, 0, 0, t,
                                        ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
                    assert rc == 0, L.tbik_last_error()
                for i in range(4):
                    run(i)
                torch.cuda.synchronize()
                if args.wait_profile:
                    st = (ctypes.c_uint32 * 4)()
                    L.tbik_gemm_status(st)
                    a, b = labels[args.wait_profile]
                    out.append(f"tiling {t}: block 0 {st[3]} cycles, {a} {100.0 * st[1] / st[3]:.1f} %, {b} {100.0 * st[2] / st[3]:.1f} %")
                    continue
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                n = 20
                e0.record()
                for i in range(n):
                    run(i)
                e1.record()
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / n
                out.append(f"tiling {t}: {us:.1f} us = {2.0 * M * N * K / us / 1e6:.0f} TFLOP/s")
            print(name, "leaf", leaf, "|", " | ".join(out), flush=True)
        del sets


if __name__ == "__main__":
    main()
