"""fp32-node mode across ranks: the row-split layer against the default mode, and the rounding tree all-reduce
(fp32 contributions, fp32 tree, one rounding to bf16) under both of its schedules against the bf16 all-reduce of
as many elements.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        tests/bench_fp32_nodes.py

Qwen3-8B o_proj and down_proj shards at M = 8192, bf16 operands; CUDA events, maximum over ranks, microseconds per
call; rank 0 prints.  The registered buffer is sized for the fp32 partial result (128 MiB) unless TBIK_AR_MAX_SIZE says
otherwise.
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ.setdefault("TBIK_AR_MAX_SIZE", str(192 << 20))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce_ops as ops
    from llm_reproducibility_b200.tbik import tree_based_all_reduce as tar
    g = torch.Generator(device=dev).manual_seed(1 + rank)

    def timed(fn, n=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t) * 1e3

    M = 8192
    for name, K, N in (("o_proj", 4096, 4096), ("down_proj", 12288, 4096)):
        ks = K // world
        X = torch.randn(M, ks, generator=g, device=dev).to(torch.bfloat16)
        W = (torch.randn(N, ks, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        t16 = timed(lambda: tar.tree_matmul_all_reduce(X, W.t(), None))
        t32 = timed(lambda: tar.tree_matmul_all_reduce(X, W.t(), None, leaf=K // 8, node_dtype=torch.float32))
        if rank == 0:
            print(name, "world", world, f"default {t16:.1f} us, fp32 nodes {t32:.1f} us", flush=True)
    ar = tar.custom_ar
    for mb in (1, 4, 16, 32, 64, 128):
        numel = (mb << 20) // 4
        view = ar.registered_view((numel,), torch.float32)
        view.normal_()
        out = torch.empty(numel, dtype=torch.bfloat16, device=dev)
        res = {}
        for label, one_max in (("oneshot", 1 << 30), ("twoshot", 1024)):
            ops.configure(ar._ptr, ops.CFG_ONESHOT_MAX_BYTES, one_max)
            res[label] = round(timed(lambda: ar.all_reduce_rounding(view, torch.bfloat16, out=out)), 1)
        ops.configure(ar._ptr, ops.CFG_ONESHOT_MAX_BYTES, 0)
        v16 = ar.registered_view((numel,), torch.bfloat16)
        res["bf16_same_numel"] = round(timed(lambda: ar.all_reduce(v16, out=out, registered=True)), 1)
        if rank == 0:
            print("rounding all-reduce, fp32 MiB", mb, res, flush=True)
    ar.check_status()
    dist.barrier()
    tar.reset_communicator()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
