"""Decode-sized calls of the tree GEMM (M = 1 .. 256 rows): microseconds per call under a CUDA graph with the weight
streaming from HBM (weights rotate through more than L2), for the automatic schedule, for every explicit
(tiling, K-slabs) combination, and for cuBLAS (torch.matmul, not invariant) beside them.

    python tests/bench_decode.py            [MS=1,16,64,128,256]

This is the measurement the schedule's cost model (plan_cost_us in csrc/tree_gemm_sm100a.cu) was fitted to.
"""
import ctypes
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from llm_reproducibility_b200 import _lib  # noqa: E402

L2 = 126 << 20


def timed_graph(fns, reps=20):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        for f in fns:
            f()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=side):
            for f in fns:
                f()
    torch.cuda.current_stream().wait_stream(side)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(fns))


def main():
    L = _lib.lib()
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(1)
    Ms = [int(x) for x in os.environ.get("MS", "1,16,64,128,256").split(",")]
    plan = (ctypes.c_int * 4)()
    for name, K, N in (("o_proj", 4096, 4096), ("down_proj", 12288, 4096)):
        copies = max(2, -(-2 * L2 // (N * K * 2)))
        Ws = [(torch.randn(N, K, generator=gen, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        for M in Ms:
            X = torch.randn(M, K, generator=gen, device=dev).to(torch.bfloat16)
            C = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            ws = torch.zeros(64 << 20, dtype=torch.uint8, device=dev)
            res = {"cublas": timed_graph([(lambda W=W: torch.matmul(X, W.t(), out=C)) for W in Ws])}

            def auto(W):
                rc = L.tbik_gemm_ws(X.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, K, K, N, 0, 256, 0, ws.data_ptr(),
                                    ws.numel(), torch.cuda.current_stream().cuda_stream)
                assert rc == 0, _lib.last_error()
            res["auto"] = timed_graph([(lambda W=W: auto(W)) for W in Ws])
            L.tbik_gemm_plan(M, N, K, 256, 0, ws.numel(), plan)
            for tiling in range(1, 7):
                for slabs in (1, 2, 4, 8, 16):
                    if slabs > 1 and L.tbik_gemm_slabs_workspace_bytes(M, N, K, 256, tiling, slabs) == 0:
                        continue

                    def call(W, tiling=tiling, slabs=slabs):
                        rc = L.tbik_gemm_slabs(X.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, K, K, N, 0, 256, 0, tiling,
                                               slabs, ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
                        assert rc == 0, _lib.last_error()
                    res[f"t{tiling}s{slabs}"] = timed_graph([(lambda W=W: call(W)) for W in Ws])
            best = sorted((v, k) for k, v in res.items())[:6]
            ideal = N * K * 2 / 6555.2e9 * 1e6
            print(f"{name} M={M}: weight stream at the measured HBM rate {ideal:.1f} us; cuBLAS {res['cublas']:.1f}; automatic "
                  f"(tiling {plan[0]}, {plan[1]} slabs) {res['auto']:.1f}; fastest " + ", ".join(f"{k}={v:.1f}" for v, k in best),
                  flush=True)
            print("   all: " + " ".join(f"{k}={v:.1f}" for k, v in res.items()), flush=True)
        del Ws
    st = (ctypes.c_uint32 * 4)()
    L.tbik_gemm_status(st)
    assert st[0] == 0, list(st)


if __name__ == "__main__":
    main()
