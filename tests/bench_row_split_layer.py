"""One row-split layer (tree GEMM + tree all-reduce) at TP = N: GEMM alone, GEMM then all-reduce, and the row-block
pipeline with several cuts and CTA budgets -- the measurement the pipeline's plan (`_pipeline_plan`) rests on.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        tests/bench_row_split_layer.py

Qwen3-8B o_proj and down_proj shards at M = 8192, bf16; CUDA events, maximum over ranks; rank 0 prints one line per
layer, microseconds per call.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from llm_reproducibility_b200.tbik import tree_based_all_reduce as tar
    from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent
    M = 8192

    def timed(fn, iters=10, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e3

    g = torch.Generator(device=dev).manual_seed(1 + rank)
    for name, K, N in (("o_proj", 4096, 4096), ("down_proj", 12288, 4096)):
        ks = K // world
        Xs = [torch.randn(M, ks, generator=g, device=dev).to(torch.bfloat16) for _ in range(3)]
        Ws = [(torch.randn(N, ks, generator=g, device=dev) * 0.02).to(torch.bfloat16) for _ in range(3)]
        C = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        cnt = [0]

        def nxt():
            cnt[0] += 1
            return Xs[cnt[0] % 3], Ws[cnt[0] % 3]

        def gemm_full():
            X, W = nxt()
            matmul_tp_persistent(X, W.t(), out=C)

        def gemm_blocks(ctas):
            X, W = nxt()
            for r0 in range(0, M, 2048):
                matmul_tp_persistent(X[r0:r0 + 2048], W.t(), out=C[r0:r0 + 2048], max_ctas=ctas)

        def layer():
            X, W = nxt()
            return tar.tree_matmul_all_reduce(X, W.t(), None)

        res = {"gemm": timed(gemm_full)}
        for ctas in (148, 128, 116):
            res[f"gemm_4x2048_rows_{ctas}_ctas"] = timed(lambda: gemm_blocks(ctas))
        os.environ["TBIK_PIPELINE"] = "0"
        res["gemm_then_allreduce"] = timed(layer)
        os.environ["TBIK_PIPELINE"] = "1"
        for blocks in ([4096, 4096], [6144, 2048], [5120, 3072], [4096, 2048, 2048], [2048] * 4):
            for ctas in (20, 32):
                tar._PIPE_FORCE = (blocks, ctas)
                res["pipeline_" + "+".join(str(b) for b in blocks) + f"_{ctas}_ctas"] = timed(layer)
        tar._PIPE_FORCE = None
        os.environ["TBIK_PIPELINE"] = "auto"
        res["automatic"] = timed(layer)
        tar.custom_ar.check_status()
        if rank == 0:
            print(name, "TP", world, "plan", tar._pipeline_plan(M, N, ks, world), " ".join(f"{k}={v:.0f}" for k, v in res.items()),
                  flush=True)
    dist.barrier()
    tar.reset_communicator()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
