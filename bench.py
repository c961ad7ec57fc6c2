#!/usr/bin/env python
"""Benchmark of the TP-invariant row-split path: tree GEMM (+ tree all-reduce for N > 1).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--m 8192]

Workload (`config.workload`): the two row-split layers of a Qwen3-8B-shaped decoder at M tokens,
o_proj X[M,4096] x W[4096,4096] and down_proj X[M,12288] x W[12288,4096], bf16, activations
~N(0,1), weights ~N(0,0.02), synthetic and seeded.  One step = both layers once.  With N GPUs
the K dimension of both layers is split over the N ranks (TP = N, strong scaling) and each GEMM
is followed by the peer-to-peer tree all-reduce, so every rank ends with the full bf16 result,
bitwise equal to the N = 1 result.

Prints ONE JSON line (rank 0).  `value` is whole-job TFLOP/s = 2*M*4096*(4096+12288) / step time,
device-timed with CUDA events, max over ranks.  `e2e` is the same metric through the public
Python API with HOST activations: pinned host -> device copy of X, GEMM (+ all-reduce), device ->
pinned host copy of the result, all inside the timed region, every step (the copies run on two copy
streams beside the compute stream with double-buffered device inputs, so step i+1's input copy
overlaps step i's GEMMs and result copy; weights stay resident: they are parameters, not per-step
inputs).  `roofline` is for the dominant kernel (the down_proj GEMM):
algorithmic FLOPs per launch / mean launch duration measured live here, against the measured
dense-bf16 peak in MEASURED_PEAKS.json.  `cpu_baseline` times the CPU oracle on a bounded sample.

`--impl reference` times the CPU restatement of the reference's algorithm (oracle/tbik_ref.py) on
the host cores on a bounded sample of the same workload and prints the same line with
"impl": "reference" (the reference's own Triton kernel has no CPU execution path for bf16 and its
sources do not travel to the GPU box).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

HIDDEN = 4096
LAYERS = (("o_proj", 4096, HIDDEN), ("down_proj", 12288, HIDDEN))  # (name, K, N)
METRIC = "tp_invariant_row_split_gemm_plus_tree_allreduce_tflops"
L2_BYTES = 126 * 1024 * 1024


def step_flops(M: int) -> float:
    return sum(2.0 * M * N * K for _, K, N in LAYERS)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons through NVML while the timed region runs.
    Read-only: nothing about the GPU is changed."""

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None
        self.max_mhz = None

    def _run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[self.index]) if visible else self.index
            h = nv.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
        except Exception:
            return
        while not self._stop.is_set():
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                self.samples.append((mhz, reasons))
            except Exception:
                pass
            self._stop.wait(0.002)
        try:
            nv.nvmlShutdown()
        except Exception:
            pass

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        time.sleep(0.05)
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=10)

    def summary(self):
        # NVML clocks-event-reason bits
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        seen = set()
        for _, r in self.samples:
            for bit, n in names.items():
                if r & bit:
                    seen.add(n)
        return {"sm_mhz": statistics.median(m for m, _ in self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(seen), "samples": len(self.samples)}


# --------------------------------------------------------------------------- CPU arms
def cpu_port_tflops(sample_rows: int, repeats: int):
    """Oracle (CPU restatement of the reference algorithm) on `sample_rows` tokens of both layers."""
    from oracle.tbik_ref import normal_inputs, tbik_matmul_ref
    torch.set_num_threads(os.cpu_count() or 1)
    ops = []
    for i, (_, K, N) in enumerate(LAYERS):
        A, B = normal_inputs(sample_rows, K, N, torch.bfloat16, seed=100 + i)
        ops.append((A, B))
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        for A, B in ops:
            tbik_matmul_ref(A, B)
        best = min(best, time.perf_counter() - t0)
    return step_flops(sample_rows) / best / 1e12, best


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = 256
    torch.set_num_threads(os.cpu_count() or 1)
    from oracle.tbik_ref import normal_inputs, tbik_matmul_ref
    ops = [normal_inputs(rows, K, N, torch.bfloat16, seed=100 + i) for i, (_, K, N) in enumerate(LAYERS)]
    for _ in range(args.warmup):
        for A, B in ops:
            tbik_matmul_ref(A, B)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for A, B in ops:
            tbik_matmul_ref(A, B)
    dt = (time.perf_counter() - t0) / args.steps
    val = step_flops(rows) / dt / 1e12
    sample = f"{rows} of {args.m} token rows of both layers per step, bf16, all host threads"
    _emit({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, args.gpus),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })


def workload_config(args, n):
    return {
        "workload": f"Qwen3-8B row-split layers (o_proj 4096x4096, down_proj 12288x4096), M={args.m}, "
                    f"TP={n}: tree GEMM leaf 256 + tree all-reduce",
        "M": args.m, "tp": n, "leaf": 256, "node_dtype": "bf16",
        "l2": "rotating operand sets, working set > 2x L2",
    }


# --------------------------------------------------------------------------- GPU arm
_RESULT_FD = None


def _claim_stdout():
    """Keep the process's stdout for the one JSON line: everything else that writes to file descriptor 1 from here
    on (NCCL prints its version banner there) goes to stderr."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def _emit(line: dict) -> None:
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_RESULT_FD, data)


def main():
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch.distributed as dist
    from llm_reproducibility_b200.tbik.tree_based_all_reduce import reset_communicator, tree_matmul_all_reduce
    from llm_reproducibility_b200.tbik.tree_based_matmul import gemm_device_status, matmul_tp_persistent

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # keep stdout to the one JSON line: NCCL prints its version banner there at NCCL_DEBUG=VERSION
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    M, tp = args.m, world

    # operand sets: enough distinct copies that consecutive steps never find their inputs in L2
    per_set = sum(2 * (M * K // tp + N * K // tp + M * N) for _, K, N in LAYERS)
    nsets = max(2, -(-2 * L2_BYTES // per_set))
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    sets = []
    for _ in range(nsets):
        layers = []
        for _, K, N in LAYERS:
            X = torch.randn(M, K // tp, generator=g, device=dev).to(torch.bfloat16)
            W = (torch.randn(N, K // tp, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            C = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            layers.append((X, W, C))
        sets.append(layers)

    def step(i):
        for X, W, C in sets[i % nsets]:
            if tp > 1:
                out = tree_matmul_all_reduce(X, W.t(), None)
            else:
                out = matmul_tp_persistent(X, W.t(), out=C)
        return out

    def sync_all():
        torch.cuda.synchronize()
        if tp > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        if tp > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    for i in range(args.warmup):
        step(i)
    with ClockSampler(local_rank) as clocks:
        ms_step = timed(step, args.steps)
    value = step_flops(M) / (ms_step * 1e-3) / 1e12

    # ---- dominant kernel alone (down_proj GEMM), timed live with events on the launch stream
    Kd, Nd = LAYERS[1][1], LAYERS[1][2]

    def dom(i):
        X, W, C = sets[i % nsets][1]
        matmul_tp_persistent(X, W.t(), out=C)
    for i in range(3):
        dom(i)
    ms_dom = timed(dom, max(args.steps, 10))
    dom_flops = 2.0 * M * Nd * Kd / tp
    peak, peak_src = load_peaks()
    achieved = dom_flops / (ms_dom * 1e-3) / 1e12
    # dram__bytes_read.sum + dram__bytes_write.sum of this launch from one ncu capture of this command
    # (profiles/tree_gemm_pair256x128_m8192_dram_traffic.md); only known for the default shape
    traffic = 1313.0e6 if (M == 8192 and tp == 1) else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": traffic, "kernel": "tree_gemm_kernel (down_proj shard)", "peak_source": peak_src,
                "flops_per_launch": dom_flops, "ms_per_launch": ms_dom}

    # ---- end to end through the public API with host activations
    host_in = [torch.randn(M, K // tp).to(torch.bfloat16).pin_memory() for _, K, _ in LAYERS]
    host_out = [torch.empty(M, N, dtype=torch.bfloat16).pin_memory() for _, _, N in LAYERS]
    # The copies run on two copy streams beside the compute stream, inputs double-buffered on the device: the
    # host->device copy of step i+1 overlaps the GEMMs and the device->host copy of step i.  Every step still
    # moves its own inputs in and its own results out inside the timed region.
    NBUF = 2
    dev_in = [[torch.empty(M, K // tp, dtype=torch.bfloat16, device=dev) for _, K, _ in LAYERS] for _ in range(NBUF)]
    in_free = [[None] * len(LAYERS) for _ in range(NBUF)]   # event: the compute that last read dev_in[b][li]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def e2e_step(i):
        b = i % NBUF
        cur = torch.cuda.current_stream()
        leaving = []
        for li, (X, W, C) in enumerate(sets[i % nsets]):
            with torch.cuda.stream(s_in):
                if in_free[b][li] is not None:
                    s_in.wait_event(in_free[b][li])
                dev_in[b][li].copy_(host_in[li], non_blocking=True)
                arrived = s_in.record_event()
            cur.wait_event(arrived)
            if tp > 1:
                out = tree_matmul_all_reduce(dev_in[b][li], W.t(), None)
            else:
                out = matmul_tp_persistent(dev_in[b][li], W.t(), out=C)
            done = cur.record_event()
            in_free[b][li] = done
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                host_out[li].copy_(out, non_blocking=True)
                out.record_stream(s_out)
                leaving.append(s_out.record_event())
        # this step's results have left the device before the next step may overwrite C or the host buffers
        for ev in leaving:
            cur.wait_event(ev)
    for i in range(3):
        e2e_step(i)
    ms_e2e = timed(e2e_step, max(3, args.steps // 2))
    h2d = sum(t.numel() * 2 for t in host_in)
    d2h = sum(t.numel() * 2 for t in host_out)
    e2e = {"value": step_flops(M) / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e}

    status = gemm_device_status()
    if status[0] != 0:
        raise SystemExit(f"GEMM kernel reported a bounded-wait timeout: {status}")

    cpu = None
    if rank == 0 and tp == 1 and not args.no_cpu_baseline:
        rows = 2048
        v, secs = cpu_port_tflops(rows, repeats=3)
        cpu = {"value": v, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
               "sample": f"{rows} of {M} token rows of both layers, bf16, best of 3 ({secs:.2f} s per pass)"}

    if tp > 1:
        reset_communicator()
        dist.barrier()
    if rank == 0:
        launches_per_step = len(LAYERS) * (2 if tp > 1 else 1)
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": tp, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args, tp),
            "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks.summary(),
            "roofline": roofline, "frac_of_peak_whole_job": value / (peak * tp),
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        _emit(line)
    if tp > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
