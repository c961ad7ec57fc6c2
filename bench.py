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

With N > 1 the line also carries `parity_check`, computed outside the timed regions: the communicator's
peer-to-peer data plane must be active, rows of the TP = N result of both layers must equal, bit for bit, the
same rows computed with TP = 1 on every rank (operand shards gathered with NCCL for that purpose only), every
all-reduce schedule must reproduce the CPU oracle's rank-pair tree on a seeded 1 MiB message, and a
collective that a rank enters alone must time out cleanly.  Any mismatch ends the run with a non-zero exit code.

With N = 1 the line also carries `decode` (M = 1 and 16 of both layers, microseconds per call eager and under
a CUDA graph, fraction of the measured HBM bandwidth the weight stream reaches), `sustained` (the dominant
kernel back to back for two seconds with the SM clock sampled) and, when the reference's own Triton kernel
was staged under oracle/_ref by oracle/build_ref.py, `reference_triton_tflops`: that kernel on the same GPU
and the same operands (a comparator; nothing of it is on the product's path).

`--impl reference` times the CPU restatement of the reference's algorithm (oracle/tbik_ref.py) on
the host cores on a bounded sample of the same workload and prints the same line with
"impl": "reference" (the reference's own Triton kernel has no CPU execution path for bf16).
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
DOWN_PROJ_DRAM_BYTES = 1201.0e6  # ncu, M = 8192, 256x256 CTA-pair tiling (the automatic choice), 8 row-tiles per group


def step_flops(M: int) -> float:
    return sum(2.0 * M * N * K for _, K, N in LAYERS)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def load_other_peaks():
    """(sustained bf16 TFLOP/s, HBM GB/s, source)"""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return float(d.get("bf16_tflops_sustained", 1400.0)), float(d.get("hbm_gbs", 6650.0)), "measured"
    return 1400.0, 6650.0, "fallback"


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



def bits(t):
    return t.contiguous().view(torch.int16)


def parity_block(rank, tp, dev, sets, M):
    """Bitwise checks of the multi-GPU path, outside every timed region.  Raises SystemExit on a mismatch."""
    import torch.distributed as dist
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce_ops as ops
    from llm_reproducibility_b200.tbik import tree_based_all_reduce as tar
    from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent

    def fail(msg):
        raise SystemExit(f"parity check failed on rank {rank}: {msg}")

    ar = tar.custom_ar
    if ar is None or ar.disabled:
        fail("the peer-to-peer communicator is disabled: the timed steps ran the library fallback")
    ar.check_status()
    rows = 256
    slices = ((0, rows), (M - rows, M)) if M >= 2 * rows else ((0, M),)
    layer_ok = []
    for li, (X, W, _) in enumerate(sets[0]):
        got = tar.tree_matmul_all_reduce(X, W.t(), None)  # TP = N, the call the timed steps make
        # TP = 1 on every rank: gather the K-shards (setup through the library collective, not the product path)
        Wparts = [torch.empty_like(W) for _ in range(tp)]
        dist.all_gather(Wparts, W.contiguous())
        Wfull = torch.cat(Wparts, dim=1)
        for (r0, r1) in slices:
            Xs = X[r0:r1].contiguous()
            Xparts = [torch.empty_like(Xs) for _ in range(tp)]
            dist.all_gather(Xparts, Xs)
            want = matmul_tp_persistent(torch.cat(Xparts, dim=1), Wfull.t())
            torch.cuda.synchronize()
            if not torch.equal(bits(got[r0:r1]), bits(want)):
                fail(f"{LAYERS[li][0]}: rows {r0}:{r1} of the TP={tp} result differ from TP=1")
        layer_ok.append(LAYERS[li][0])
        del Wparts, Wfull
    # every schedule of the tree all-reduce against the CPU oracle's rank-pair tree (the checker)
    numel = 1 << 19  # 1 MiB of bf16
    g = torch.Generator(device=dev).manual_seed(4242 + rank)
    x = (torch.randn(numel, generator=g, device=dev) * 3.0).to(torch.bfloat16)
    gathered = [torch.empty_like(x) for _ in range(tp)]
    dist.all_gather(gathered, x)
    from oracle.tbik_ref import tree_allreduce_ref
    want = tree_allreduce_ref([t.cpu() for t in gathered])
    schedules = (("one-shot", 1 << 40, 0, 0, 0), ("two-shot", 1, 1 << 60, 0, 0), ("push-1", 1, 1, 1, 0),
                 ("push-4", 1, 1, 4, 0), ("two-shot-256bit", 1, 1 << 60, 0, 2))
    done = []
    for name, one_max, push_min, chunks, vec in schedules:
        ops.configure(ar._ptr, ops.CFG_ONESHOT_MAX_BYTES, one_max)
        ops.configure(ar._ptr, ops.CFG_PUSH_MIN_BYTES, push_min)
        ops.configure(ar._ptr, ops.CFG_PUSH_CHUNKS, chunks)
        ops.configure(ar._ptr, ops.CFG_VEC_PACKS, vec)
        y = ar.custom_tree_all_reduce(x)
        torch.cuda.synchronize()
        ar.check_status()
        if y is None or not torch.equal(bits(y.cpu()), bits(want)):
            fail(f"tree all-reduce, schedule {name}: result differs from the oracle")
        done.append(name)
    for key in (ops.CFG_ONESHOT_MAX_BYTES, ops.CFG_PUSH_MIN_BYTES, ops.CFG_PUSH_CHUNKS, ops.CFG_VEC_PACKS):
        ops.configure(ar._ptr, key, 0)
    return {"ok": True, "data_plane": "p2p", "tp_vs_tp1_rows": rows * len(slices), "layers": layer_ok,
            "schedules": done, "oracle": "oracle.tbik_ref.tree_allreduce_ref on gathered inputs"}


def timeout_probe(rank, tp, dev):
    """Last thing of a multi-GPU run: rank 0 enters one collective alone with a 20 ms limit.  Its kernel must
    return with a status record instead of hanging; the communicator is closed afterwards."""
    import torch.distributed as dist
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce_ops as ops
    from llm_reproducibility_b200.tbik import tree_based_all_reduce as tar
    ar = tar.custom_ar
    res = {"ok": True, "limit_ms": 20}
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        try:
            ops.configure(ar._ptr, ops.CFG_WAIT_LIMIT_NS, 20_000_000)
            x = torch.zeros(1 << 14, dtype=torch.bfloat16, device=dev)
            t0 = time.perf_counter()
            ar.custom_tree_all_reduce(x)
            torch.cuda.synchronize()
            res["returned_after_ms"] = (time.perf_counter() - t0) * 1e3
            st = ops.status(ar._ptr)
            res["status"] = {"code": st[0], "rank": st[1], "peer": st[3], "barrier": st[6]}
            refused = False
            try:
                ar.custom_tree_all_reduce(x)
            except RuntimeError:
                refused = True
            res["ok"] = bool(st[0] == 1 and st[1] == 0 and st[6] == 1 and refused and res["returned_after_ms"] < 1000)
        except Exception as exc:  # reported, not fatal: the timed numbers above stand on their own
            res = {"ok": False, "error": repr(exc)}
    dist.barrier()
    return res


def decode_record(dev, hbm_gbs):
    """M = 1 and 16 of both layers: microseconds per call eager and under a CUDA graph, weights rotating through
    more than L2 so that every call streams its weight from HBM."""
    from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent
    out = {"unit": "us", "hbm_peak_gbs": hbm_gbs, "cases": []}
    g = torch.Generator(device=dev).manual_seed(77)
    for name, K, N in LAYERS:
        copies = max(2, -(-2 * L2_BYTES // (N * K * 2)))
        Ws = [(torch.randn(N, K, generator=g, device=dev) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        for M in (1, 16):
            X = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
            C = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
            for W in Ws:
                matmul_tp_persistent(X, W.t(), out=C)
            torch.cuda.synchronize()
            reps = 10
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                for W in Ws:
                    matmul_tp_persistent(X, W.t(), out=C)
            e1.record()
            torch.cuda.synchronize()
            eager_us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
            t0 = time.perf_counter()
            for _ in range(reps):
                for W in Ws:
                    matmul_tp_persistent(X, W.t(), out=C)
            host_us = (time.perf_counter() - t0) * 1e6 / (reps * copies)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for W in Ws:
                        matmul_tp_persistent(X, W.t(), out=C)
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            graph_us = e0.elapsed_time(e1) * 1e3 / (reps * copies)
            weight_bytes = N * K * 2
            out["cases"].append({"layer": name, "M": M, "eager_us": eager_us, "host_us_per_call": host_us,
                                 "graph_us": graph_us,
                                 "hbm_frac_graph": weight_bytes / (graph_us * 1e-6) / (hbm_gbs * 1e9)})
            del graph
        del Ws
    return out


def sustained_record(dom, dom_flops, local_rank, sustained_peak, seconds=2.0):
    """The dominant kernel back to back for `seconds`, SM clock sampled meanwhile."""
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 0
    with ClockSampler(local_rank) as clk:
        t0 = time.perf_counter()
        e0.record()
        while time.perf_counter() - t0 < seconds:
            for _ in range(50):
                dom(n)
                n += 1
            torch.cuda.synchronize()  # keeps the launch queue short; costs microseconds per 50 launches
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    c = clk.summary()
    tf = dom_flops / (ms * 1e-3) / 1e12
    return {"seconds": seconds, "launches": n, "ms_per_launch": ms, "tflops": tf, "peak_sustained": sustained_peak,
            "frac_of_sustained_peak": tf / sustained_peak, "sm_mhz_median": c["sm_mhz"], "reasons": c["reasons"],
            "ms_times_mhz": (ms * c["sm_mhz"]) if c["sm_mhz"] else None}


def fp32_nodes_record(sets, M, steps):
    """The same step in the fp32-node mode (leaves and nodes fp32, one rounding at the root; leaf = K / 8): timed like
    the headline, plus its mean error against fp64 on a sample of rows beside the default mode's."""
    from llm_reproducibility_b200.tbik.tree_based_matmul import leaf_for_fp32_nodes, matmul_tp_persistent
    nsets = len(sets)

    def fstep(i):
        for X, W, C in sets[i % nsets]:
            matmul_tp_persistent(X, W.t(), out=C, leaf=leaf_for_fp32_nodes(X.shape[1], 8), node_dtype=torch.float32)
    for i in range(3):
        fstep(i)
    torch.cuda.synchronize()
    n = max(3, min(steps, 30))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(n):
        fstep(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    rec = {"ms_per_step": ms, "tflops": step_flops(M) / (ms * 1e-3) / 1e12, "steps": n,
           "leaf": [leaf_for_fp32_nodes(K, 8) for _, K, _ in LAYERS]}
    # accuracy on 256 rows of the down_proj operands
    X, W, _ = sets[0][-1]
    Xs = X[:256]
    exact = Xs.double() @ W.double().t()
    d16 = matmul_tp_persistent(Xs, W.t())
    d32 = matmul_tp_persistent(Xs, W.t(), leaf=leaf_for_fp32_nodes(X.shape[1], 8), node_dtype=torch.float32)
    rec["mean_abs_err_vs_fp64"] = {"rounded_nodes": float((d16.double() - exact).abs().mean()),
                                   "fp32_nodes": float((d32.double() - exact).abs().mean()),
                                   "one_rounding_of_fp64": float((exact.to(torch.bfloat16).double() - exact).abs().mean())}
    return rec


def reference_triton_record(sets, M, steps):
    """The reference's own Triton kernel (src/tbik/tree_based_matmul.py, staged unmodified under oracle/_ref by
    oracle/build_ref.py) on this GPU and these operands: a comparator, never on the product's path."""
    path = os.path.join(ROOT, "oracle", "_ref", "tree_based_matmul.py")
    if not os.path.isfile(path):
        return None
    try:
        import importlib.util
        spec = importlib.util.spec_from_file_location("tbik_reference_triton", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        ops = [(X, W.t()) for (X, W, _) in sets[0]]
        for A, B in ops:
            mod.matmul_tp_persistent(A, B)  # JIT compile
        torch.cuda.synchronize()
        n = max(3, min(steps, 10))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            for (X, W, _) in sets[i % len(sets)]:
                mod.matmul_tp_persistent(X, W.t())
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        return {"tflops": step_flops(M) / (ms * 1e-3) / 1e12, "ms_per_step": ms, "steps": n}
    except Exception as exc:
        return {"error": repr(exc)[:300]}


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
    ap.add_argument("--quick", action="store_true", help="skip the decode, sustained and reference-kernel records")
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
    parity = parity_block(rank, tp, dev, sets, M) if tp > 1 else None
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
    # dram__bytes_read.sum + dram__bytes_write.sum of one down_proj launch, from a one-pass ncu capture of this
    # command; it belongs to one tiling of one shape, so it is only reported while that tiling is what runs
    traffic = DOWN_PROJ_DRAM_BYTES if (M == 8192 and tp == 1 and os.environ.get("TBIK_LEAF") is None) else None
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": traffic, "kernel": "tree_gemm_kernel (down_proj shard)", "peak_source": peak_src,
                "flops_per_launch": dom_flops, "ms_per_launch": ms_dom}

    # ---- end to end through the public API with host activations
    host_in = [torch.randn(M, K // tp).to(torch.bfloat16).pin_memory() for _, K, _ in LAYERS]
    # the result is bit-identical on every rank, so rank r brings back only rows [r*M/tp, (r+1)*M/tp): together the
    # ranks return the whole result once
    row0, row1 = rank * M // tp, (rank + 1) * M // tp
    host_out = [torch.empty(row1 - row0, N, dtype=torch.bfloat16).pin_memory() for _, _, N in LAYERS]
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
                host_out[li].copy_(out[row0:row1], non_blocking=True)
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
    e2e = {"value": step_flops(M) / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d * tp,
           "d2h_bytes_per_step": d2h * tp, "h2d_bytes_per_step_per_rank": h2d, "d2h_bytes_per_step_per_rank": d2h,
           "ms_per_step": ms_e2e}

    status = gemm_device_status()
    if status[0] != 0:
        raise SystemExit(f"GEMM kernel reported a bounded-wait timeout: {status}")

    cpu = None
    if rank == 0 and tp == 1 and not args.no_cpu_baseline:
        rows = 2048
        v, secs = cpu_port_tflops(rows, repeats=3)
        cpu = {"value": v, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
               "sample": f"{rows} of {M} token rows of both layers, bf16, best of 3 ({secs:.2f} s per pass)"}

    decode = sustained = ref_triton = probe = fp32_nodes = None
    if tp == 1 and not args.quick:
        sustained_peak, hbm_gbs, _ = load_other_peaks()
        decode = decode_record(dev, hbm_gbs)
        sustained = sustained_record(dom, dom_flops, local_rank, sustained_peak)
        # the same achieved figure against the cuBLAS loop that ran for seconds under the power cap: with many steps the
        # timed region is itself tens of milliseconds of back-to-back GEMMs, between the two regimes
        roofline["peak_sustained"] = sustained_peak
        roofline["frac_of_sustained"] = achieved / sustained_peak
        ref_triton = reference_triton_record(sets, M, args.steps)
        fp32_nodes = fp32_nodes_record(sets, M, args.steps)
    if tp > 1:
        probe = timeout_probe(rank, tp, dev)
        reset_communicator()
        dist.barrier()
    if rank == 0:
        # kernels of this repository per step: one GEMM per layer, or per row block of a layer one GEMM and one
        # all-reduce when the layer is pipelined over row blocks
        if tp > 1:
            from llm_reproducibility_b200.tbik.tree_based_all_reduce import _pipeline_plan
            plans = [_pipeline_plan(M, N, K // tp, tp) for _, K, N in LAYERS]
            launches_per_step = sum(2 * (len(pl[0]) if pl else 1) for pl in plans)
        else:
            launches_per_step = len(LAYERS)
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": tp, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args, tp),
            "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks.summary(),
            "roofline": roofline, "frac_of_peak_whole_job": value / (peak * tp),
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        for key, val in (("parity_check", parity), ("timeout_probe", probe), ("decode", decode),
                         ("sustained", sustained), ("reference_triton", ref_triton), ("fp32_nodes", fp32_nodes)):
            if val is not None:
                line[key] = val
        if ref_triton is not None and "tflops" in ref_triton:
            line["reference_triton_tflops"] = ref_triton["tflops"]
        _emit(line)
    if tp > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
