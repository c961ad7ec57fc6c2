"""Tree all-reduce alone (BASELINE config 3): latency and bandwidth of the peer-to-peer tree kernels
against NCCL all_reduce and the all_gather + ordered-adds path, bf16, 8 KB ... 64 MB, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        tests/bench_allreduce.py [--iters 20] [--warmup 5] [--max-mb 64] [--min-kb 8]
                                 [--oneshot-max-kb K] [--max-blocks B] [--threads T] [--push-min-kb K] [--push-chunks C]
                                 [--vec-packs V] [--loads L] [--trace] [--only-p2p]

--oneshot-max-kb / --max-blocks / --threads / --vec-packs / --loads override the built-in choices (for tuning sweeps).
--trace adds, per size, the medians over CTAs of the kernel's phase stamps (GPU timer): first barrier, reduce
phase, middle barrier, gather phase -- the way a multi-rank kernel is profiled here, since ncu is never run on a
multi-rank command.

Counterpart of the reference's tests/bench_allreduce.py:19-135, with device timing (CUDA events, max
over ranks) instead of wall clock and without the clone inside the timed region.
Rank 0 prints one JSON line per size.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--max-mb", type=int, default=64)
    ap.add_argument("--min-kb", type=int, default=8)
    ap.add_argument("--oneshot-max-kb", type=int, default=0)
    ap.add_argument("--max-blocks", type=int, default=0)
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--push-min-kb", type=int, default=0)
    ap.add_argument("--push-chunks", type=int, default=0)
    ap.add_argument("--vec-packs", type=int, default=0)
    ap.add_argument("--loads", type=int, default=0)
    ap.add_argument("--trace", action="store_true")
    ap.add_argument("--only-p2p", action="store_true")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from llm_reproducibility_b200.mini_allreduce import CustomTreeAllreduce
    from llm_reproducibility_b200.tbik.tree_based_all_reduce import tree_all_reduce_sum_native

    max_bytes = args.max_mb << 20
    ar = CustomTreeAllreduce(group=dist.group.WORLD, device=dev, max_size=max_bytes + (1 << 20))
    assert not ar.disabled
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce_ops as ops
    if args.oneshot_max_kb:
        ops.configure(ar._ptr, ops.CFG_ONESHOT_MAX_BYTES, args.oneshot_max_kb << 10)
    if args.push_min_kb:
        ops.configure(ar._ptr, ops.CFG_PUSH_MIN_BYTES, args.push_min_kb << 10)
    if args.push_chunks:
        ops.configure(ar._ptr, ops.CFG_PUSH_CHUNKS, args.push_chunks)
    if args.threads:
        ops.configure(ar._ptr, ops.CFG_THREADS, args.threads)
    if args.max_blocks:
        ops.configure(ar._ptr, ops.CFG_MAX_BLOCKS, args.max_blocks)
    if args.vec_packs:
        ops.configure(ar._ptr, ops.CFG_VEC_PACKS, args.vec_packs)
    if args.loads:
        ops.configure(ar._ptr, ops.CFG_LOADS_IN_FLIGHT, args.loads)
    if args.trace:
        ops.configure(ar._ptr, ops.CFG_TRACE, 1)

    def phases():
        """Medians over the CTAs of the last launch, microseconds."""
        import statistics
        tr = ops.trace(ar._ptr)
        nb = len(tr) // 8
        if nb == 0:
            return None
        b = [tr[8 * i: 8 * i + 8] for i in range(nb)]
        med = lambda xs: statistics.median(xs) / 1e3
        out = {"ctas": nb, "kernel_us": (max(x[4] for x in b) - min(x[0] for x in b)) / 1e3,
               "first_barrier_us": med([x[1] - x[0] for x in b]), "reduce_us": med([x[2] - x[1] for x in b])}
        if all(x[3] for x in b):   # two-shot: a middle barrier, then the gather
            out["middle_barrier_us"] = med([x[3] - x[2] for x in b])
            out["gather_us"] = med([x[4] - x[3] for x in b])
        else:
            out["tail_us"] = med([x[4] - x[2] for x in b])
        return out

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) * 1e3  # us

    nbytes = args.min_kb << 10
    while nbytes <= max_bytes:
        numel = nbytes // 2
        g = torch.Generator(device=dev).manual_seed(1000 + rank)
        x = torch.randn(numel, generator=g, device=dev).to(torch.bfloat16)
        out = torch.empty_like(x)
        view = ar.registered_view((numel,), torch.bfloat16)
        view.copy_(x)
        nccl_buf = x.clone()
        res = {
            "bytes": nbytes, "world": world,
            "tree_p2p_staged_us": timed(lambda: ar.all_reduce(x, out=out)),
            "tree_p2p_registered_us": timed(lambda: ar.all_reduce(view, out=out, registered=True)),
        }
        if not args.only_p2p:
            res["nccl_allreduce_us"] = timed(lambda: dist.all_reduce(nccl_buf))
            res["allgather_adds_us"] = timed(lambda: tree_all_reduce_sum_native(x, None))
        if args.trace:
            res["phases_registered"] = phases()
        t = res["tree_p2p_registered_us"] * 1e-6
        res["algbw_GBs"] = nbytes / t / 1e9
        res["busbw_GBs"] = nbytes * 2 * (world - 1) / world / t / 1e9
        ar.check_status()
        if rank == 0:
            print(json.dumps(res), flush=True)
        nbytes *= 2
    dist.barrier()
    ar.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
