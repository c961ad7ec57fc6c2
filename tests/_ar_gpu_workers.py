"""Per-rank bodies of the multi-GPU all-reduce tests (imported by spawned processes)."""
import os

import torch
import torch.distributed as dist


def _inputs(world, numel, dtype, seed, device):
    """Every rank regenerates all ranks' inputs (same Philox stream on every GPU)."""
    xs = []
    for r in range(world):
        g = torch.Generator(device=device).manual_seed(seed * 1000 + r)
        xs.append((torch.randn(numel, generator=g, device=device) * 3.0).to(dtype))
    return xs


def bits(t):
    return t.contiguous().view(torch.int16 if t.element_size() == 2 else torch.int32)


def tree_allreduce_parity(rank, world, cases, max_size):
    from llm_reproducibility_b200.mini_allreduce import CustomTreeAllreduce
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce_ops as ops
    from llm_reproducibility_b200.tbik.tree_based_all_reduce import tree_all_reduce_sum_native
    from oracle.tbik_ref import tree_allreduce_ref

    device = torch.device(f"cuda:{rank}")
    gloo = dist.new_group(backend="gloo")
    ar = CustomTreeAllreduce(group=gloo, device=device, max_size=max_size)
    assert not ar.disabled, "communicator disabled on a P2P-capable box"
    report = []
    for (numel, dtype, seed) in cases:
        xs = _inputs(world, numel, dtype, seed, device)
        want = tree_allreduce_ref(xs)
        # (name, one-shot limit, push from, push chunks, packs per access, packs in flight per thread, threads)
        for mode, one_max, push_min, chunks, vec, loads, threads in (
                ("auto", 0, 0, 0, 0, 0, 0), ("oneshot", 1 << 40, 0, 0, 0, 0, 0), ("twoshot", 1, 1 << 60, 0, 0, 0, 0),
                ("push", 1, 1, 0, 0, 0, 0), ("push1", 1, 1, 1, 0, 0, 0), ("push7", 1, 1, 7, 0, 0, 0),
                ("oneshot-256bit", 1 << 40, 0, 0, 2, 0, 0), ("twoshot-256bit", 1, 1 << 60, 0, 2, 0, 0),
                ("push1-256bit", 1, 1, 1, 2, 0, 0), ("twoshot-deep", 1, 1 << 60, 0, 1, 32, 0),
                ("oneshot-deep-256bit", 1 << 40, 0, 0, 2, 32, 0), ("twoshot-shallow", 1, 1 << 60, 0, 1, 4, 256)):
            if mode.startswith("oneshot") and numel * xs[0].element_size() > (8 << 20):
                continue
            ops.configure(ar._ptr, ops.CFG_ONESHOT_MAX_BYTES, one_max)
            ops.configure(ar._ptr, ops.CFG_PUSH_MIN_BYTES, push_min)
            ops.configure(ar._ptr, ops.CFG_PUSH_CHUNKS, chunks)
            ops.configure(ar._ptr, ops.CFG_VEC_PACKS, vec)
            ops.configure(ar._ptr, ops.CFG_LOADS_IN_FLIGHT, loads)
            ops.configure(ar._ptr, ops.CFG_THREADS, threads)
            got = ar.custom_tree_all_reduce(xs[rank])
            assert got is not None, (numel, dtype)
            torch.cuda.synchronize()
            ar.check_status()
            ok = torch.equal(bits(got), bits(want))
            report.append((numel, str(dtype), mode, ok))
            assert ok, f"rank {rank}: tree all-reduce differs from oracle: numel={numel} {dtype} {mode}"
        ops.configure(ar._ptr, ops.CFG_VEC_PACKS, 0)
        ops.configure(ar._ptr, ops.CFG_LOADS_IN_FLIGHT, 0)
        ops.configure(ar._ptr, ops.CFG_THREADS, 0)
        ops.configure(ar._ptr, ops.CFG_ONESHOT_MAX_BYTES, 0)
        ops.configure(ar._ptr, ops.CFG_PUSH_MIN_BYTES, 0)
        ops.configure(ar._ptr, ops.CFG_PUSH_CHUNKS, 0)
        # the reference's own cross-check: custom kernel vs all_gather + ordered adds
        native = tree_all_reduce_sum_native(xs[rank], None)
        assert torch.equal(bits(native), bits(want))
    # repeated calls reuse flags/epochs correctly
    xs = _inputs(world, 4096, torch.bfloat16, 77, device)
    want = tree_allreduce_ref(xs)
    for _ in range(50):
        got = ar.custom_tree_all_reduce(xs[rank])
    torch.cuda.synchronize()
    assert torch.equal(bits(got), bits(want))
    # the same with the push schedule, alternating inputs so that a stale chunk in the scratch would show
    ops.configure(ar._ptr, ops.CFG_ONESHOT_MAX_BYTES, 1)
    ops.configure(ar._ptr, ops.CFG_PUSH_MIN_BYTES, 1)
    ys = _inputs(world, 1 << 18, torch.bfloat16, 78, device)
    zs = _inputs(world, 1 << 18, torch.bfloat16, 79, device)
    want_y, want_z = tree_allreduce_ref(ys), tree_allreduce_ref(zs)
    for i in range(20):
        got_y = ar.custom_tree_all_reduce(ys[rank])
        got_z = ar.custom_tree_all_reduce(zs[rank])
    torch.cuda.synchronize()
    ar.check_status()
    assert torch.equal(bits(got_y), bits(want_y)) and torch.equal(bits(got_z), bits(want_z))
    ops.configure(ar._ptr, ops.CFG_ONESHOT_MAX_BYTES, 0)
    ops.configure(ar._ptr, ops.CFG_PUSH_MIN_BYTES, 0)
    # ineligible inputs return None (odd byte size; too large)
    assert ar.custom_tree_all_reduce(torch.zeros(3, dtype=torch.bfloat16, device=device)) is None
    assert ar.custom_tree_all_reduce(torch.zeros(max_size, dtype=torch.uint8, device=device).view(torch.bfloat16)) is None
    dist.barrier()
    ar.close()
    return report


def linear_allreduce_parity(rank, world):
    from llm_reproducibility_b200.mini_allreduce import CustomAllreduce

    device = torch.device(f"cuda:{rank}")
    gloo = dist.new_group(backend="gloo")
    ar = CustomAllreduce(group=gloo, device=device)
    assert not ar.disabled
    for numel, dtype in ((4096, torch.bfloat16), (1 << 20, torch.bfloat16), (8192, torch.float16), (2048, torch.float32)):
        xs = _inputs(world, numel, dtype, 5, device)
        acc = xs[0].float()
        for r in range(1, world):
            acc = acc + xs[r].float()
        want = acc.to(dtype)
        got = ar.custom_all_reduce(xs[rank])
        torch.cuda.synchronize()
        assert torch.equal(bits(got), bits(want)), (numel, dtype)
    dist.barrier()
    ar.close()
    return True


def graph_capture(rank, world):
    from llm_reproducibility_b200.mini_allreduce import CustomTreeAllreduce
    from oracle.tbik_ref import tree_allreduce_ref

    device = torch.device(f"cuda:{rank}")
    gloo = dist.new_group(backend="gloo")
    ar = CustomTreeAllreduce(group=gloo, device=device)
    xs = _inputs(world, 8192, torch.bfloat16, 9, device)
    want = tree_allreduce_ref(xs)
    static_in = xs[rank].clone()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with ar.capture():
        with torch.cuda.stream(stream):
            warm = ar.custom_tree_all_reduce(static_in)  # not capturing yet: zeros_like
            assert warm is not None and float(warm.abs().sum()) == 0.0
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                out = ar.custom_tree_all_reduce(static_in)
    dist.barrier()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    ar.check_status()
    assert torch.equal(bits(out), bits(want))
    # deferred registration: under capture an input that was never registered is taken as it is (no staging copy);
    # its peers' addresses are exchanged when the capture block ends and patched into the reserved slot
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce_ops as ops
    with ar.capture():
        with torch.cuda.stream(stream):
            graph2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph2, stream=stream):
                out2 = ar.all_reduce(static_in, registered=True)
            handles, offsets = ops.get_graph_buffer_ipc_meta(ar._ptr)
            assert len(offsets) == 1 and len(handles) == 64
    dist.barrier()
    for _ in range(3):
        graph2.replay()
    torch.cuda.synchronize()
    ar.check_status()
    assert torch.equal(bits(out2), bits(want))
    dist.barrier()
    ar.close()
    return True


def dispatcher(rank, world):
    """tree_all_reduce_sum end to end on the NCCL device group, plus the patched layer's forward."""
    from llm_reproducibility_b200.patch.patch_tp_invariant import row_parallel_forward
    from llm_reproducibility_b200.tbik import tree_based_all_reduce as tar
    from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent
    from oracle.tbik_ref import tree_allreduce_ref

    device = torch.device(f"cuda:{rank}")
    xs = _inputs(world, 1 << 18, torch.bfloat16, 3, device)
    y = tar.tree_all_reduce_sum(xs[rank], None)
    torch.cuda.synchronize()
    assert tar.custom_ar is not None and not tar.custom_ar.disabled
    assert torch.equal(bits(y), bits(tree_allreduce_ref(xs)))

    # row-parallel layer: TP result == single-device result, bit for bit
    M, K, N = 96, 4096, 512
    g = torch.Generator(device=device).manual_seed(1234)
    X = torch.randn(M, K, generator=g, device=device).to(torch.bfloat16)
    W = (torch.randn(N, K, generator=g, device=device) * 0.02).to(torch.bfloat16)
    ks = K // world

    class Layer:
        input_is_parallel = False
        tp_size = world
        tp_rank = rank
        weight = W[:, rank * ks:(rank + 1) * ks].contiguous()
        bias = None
        skip_bias_add = False
        reduce_results = True
        return_bias = False
        quant_method = object()

    out = row_parallel_forward(Layer(), X)
    full = matmul_tp_persistent(X, W.t())
    torch.cuda.synchronize()
    assert torch.equal(bits(out), bits(full)), "TP result differs from the single-device result"
    # GEMM then all-reduce as two calls gives the same bits, repeatedly (the registered buffer is reused)
    for _ in range(3):
        part = matmul_tp_persistent(X[:, rank * ks:(rank + 1) * ks], Layer.weight.t())
        assert torch.equal(bits(tar.tree_all_reduce_sum(part, None)), bits(full))
        assert torch.equal(bits(tar.tree_matmul_all_reduce(X[:, rank * ks:(rank + 1) * ks], Layer.weight.t(), None)), bits(full))
    # Qwen3-8B shapes at M = 2048 (two-shot schedule, 16 MiB message)
    g2 = torch.Generator(device=device).manual_seed(99)
    for (K2, N2) in ((4096, 4096), (12288, 4096)):
        X2 = torch.randn(2048, K2, generator=g2, device=device).to(torch.bfloat16)
        W2 = (torch.randn(N2, K2, generator=g2, device=device) * 0.02).to(torch.bfloat16)
        k2 = K2 // world
        got = tar.tree_matmul_all_reduce(X2[:, rank * k2:(rank + 1) * k2], W2[:, rank * k2:(rank + 1) * k2].t(), None)
        want = matmul_tp_persistent(X2, W2.t())
        torch.cuda.synchronize()
        assert torch.equal(bits(got), bits(want)), (K2, N2)
    # ragged sizes (edge tiles in M and N; the registered buffer is reused call after call)
    g3 = torch.Generator(device=device).manual_seed(5)
    X3 = torch.randn(300, 2048, generator=g3, device=device).to(torch.bfloat16)
    W3 = (torch.randn(520, 2048, generator=g3, device=device) * 0.05).to(torch.bfloat16)
    k3 = 2048 // world
    want3 = matmul_tp_persistent(X3, W3.t())
    for _ in range(4):
        y = tar.tree_matmul_all_reduce(X3[:, rank * k3:(rank + 1) * k3], W3[:, rank * k3:(rank + 1) * k3].t(), None)
        torch.cuda.synchronize()
        assert torch.equal(bits(y), bits(want3))
    # under a CUDA graph the GEMM writes into the registered buffer too (no staging copy, no late registration)
    Xs, Ws = X3[:, rank * k3:(rank + 1) * k3].contiguous(), W3[:, rank * k3:(rank + 1) * k3].contiguous()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            yg = tar.tree_matmul_all_reduce(Xs, Ws.t(), None)
    torch.cuda.current_stream().wait_stream(stream)
    dist.barrier()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(bits(yg), bits(want3))
    tar.custom_ar.check_status()
    dist.barrier()
    tar.reset_communicator()
    return True


def barrier_timeout(rank, world):
    """A cross-GPU wait that runs out: rank 0 enters a collective that no peer joins.  Its kernel must give up
    after the configured limit and return (nothing hangs, nothing faults), the status record must name the
    barrier, the communicator must refuse further use, close() must work, and a rebuilt one must be correct."""
    from llm_reproducibility_b200.mini_allreduce import CustomTreeAllreduce
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce_ops as ops
    from oracle.tbik_ref import tree_allreduce_ref
    import time

    device = torch.device(f"cuda:{rank}")
    gloo = dist.new_group(backend="gloo")
    ar = CustomTreeAllreduce(group=gloo, device=device, max_size=4 << 20)
    assert not ar.disabled
    xs = _inputs(world, 1 << 16, torch.bfloat16, 21, device)
    want = tree_allreduce_ref(xs)
    got = ar.custom_tree_all_reduce(xs[rank])
    torch.cuda.synchronize()
    assert torch.equal(bits(got), bits(want))
    ops.configure(ar._ptr, ops.CFG_WAIT_LIMIT_NS, 20_000_000)  # 20 ms
    dist.barrier(group=gloo)  # every rank is idle: no kernel in flight anywhere
    elapsed = None
    if rank == 0:
        t0 = time.perf_counter()
        lonely = ar.custom_tree_all_reduce(xs[rank])  # the peers skip this call
        torch.cuda.synchronize()                      # returns: the kernel gave up on its first barrier
        elapsed = time.perf_counter() - t0
        assert lonely is not None and elapsed < 1.0, elapsed
        st = ops.status(ar._ptr)
        assert st[0] == 1 and st[1] == 0 and 1 <= st[3] < world and st[6] == 1, st
        try:
            ar.check_status()
            raise AssertionError("check_status must raise after a timeout")
        except RuntimeError as e:
            assert "timed out" in str(e)
        try:
            ar.custom_tree_all_reduce(xs[rank])
            raise AssertionError("a communicator whose kernel timed out must refuse further calls")
        except RuntimeError as e:
            assert "(-7)" in str(e), str(e)
    dist.barrier(group=gloo)
    ar.close()
    dist.barrier(group=gloo)
    # a fresh communicator on the same GPUs works
    ar2 = CustomTreeAllreduce(group=gloo, device=device, max_size=4 << 20)
    assert not ar2.disabled
    for _ in range(3):
        got = ar2.custom_tree_all_reduce(xs[rank])
    torch.cuda.synchronize()
    ar2.check_status()
    assert torch.equal(bits(got), bits(want))
    dist.barrier(group=gloo)
    ar2.close()
    return elapsed if rank == 0 else True


def pipelined_layer(rank, world):
    """Row-block pipeline of tree_matmul_all_reduce (GEMM of block i+1 beside the all-reduce of block i on a second
    stream) against the single-device result, bit for bit; phase stamps of the all-reduce are sane."""
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce_ops as ops
    from llm_reproducibility_b200.tbik import tree_based_all_reduce as tar
    from llm_reproducibility_b200.tbik.tree_based_matmul import matmul_tp_persistent

    device = torch.device(f"cuda:{rank}")
    os.environ["TBIK_PIPELINE"] = "1"
    g = torch.Generator(device=device).manual_seed(4321)
    for (M, K, N) in ((4096, 4096, 4096), (4096 + 300, 2048, 1024), (8192, 2048, 2048)):
        X = torch.randn(M, K, generator=g, device=device).to(torch.bfloat16)
        W = (torch.randn(N, K, generator=g, device=device) * 0.02).to(torch.bfloat16)
        ks = K // world
        Xr, Wr = X[:, rank * ks:(rank + 1) * ks], W[:, rank * ks:(rank + 1) * ks]
        assert tar._pipeline_plan(M, N, ks, world) is not None
        want = matmul_tp_persistent(X, W.t())
        for _ in range(3):
            got = tar.tree_matmul_all_reduce(Xr, Wr.t(), None)
        torch.cuda.synchronize()
        tar.custom_ar.check_status()
        assert torch.equal(bits(got), bits(want)), (M, K, N)
        # other cuts: four blocks, a ragged last block, fewer CTAs for the all-reduce
        for forced in (([1024] * (M // 1024 - 1) + [M - 1024 * (M // 1024 - 1)], 20), ([M - 300, 300], 8)):
            tar._PIPE_FORCE = forced
            got = tar.tree_matmul_all_reduce(Xr, Wr.t(), None)
            torch.cuda.synchronize()
            assert torch.equal(bits(got), bits(want)), (M, K, N, forced)
        tar._PIPE_FORCE = None
        os.environ["TBIK_PIPELINE"] = "0"
        plain = tar.tree_matmul_all_reduce(Xr, Wr.t(), None)
        os.environ["TBIK_PIPELINE"] = "1"
        assert torch.equal(bits(plain), bits(want)), (M, K, N)
    # phase stamps: entry <= after the first barrier <= after the reduce phase <= exit, for every CTA
    ar = tar.custom_ar
    ops.configure(ar._ptr, ops.CFG_TRACE, 1)
    x = torch.randn(1 << 22, generator=g, device=device).to(torch.bfloat16)
    ar.custom_tree_all_reduce(x)
    torch.cuda.synchronize()
    tr = ops.trace(ar._ptr)
    assert len(tr) >= 8 and len(tr) % 8 == 0
    for b in range(len(tr) // 8):
        t = tr[8 * b: 8 * b + 8]
        assert 0 < t[0] <= t[1] <= t[2] <= t[4], t
    ops.configure(ar._ptr, ops.CFG_TRACE, 0)
    dist.barrier()
    tar.reset_communicator()
    return True


def fp32_nodes_layer(rank, world):
    """fp32-node mode across ranks: every rank's unrounded subtree root goes into the registered buffer, the
    rounding all-reduce adds the roots in fp32 in rank-pair tree order and rounds once.  Checked against the
    unsharded single-device call (bit for bit), against the CPU oracle on operands with exact leaves, and -- the
    all-reduce alone, both schedules -- against the same tree written with torch adds."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from oracle.tbik_ref import tbik_matmul_ref
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce_ops as ops
    from llm_reproducibility_b200.tbik import tree_based_all_reduce as tar
    from llm_reproducibility_b200.tbik.tree_based_matmul import leaf_for_fp32_nodes, matmul_tp_persistent

    device = torch.device(f"cuda:{rank}")
    g = torch.Generator(device=device).manual_seed(977)
    for dtype, (M, K, N) in ((torch.bfloat16, (1024, 4096, 4096)), (torch.bfloat16, (300, 12288, 1024)),
                             (torch.float16, (64, 4096, 512)), (torch.bfloat16, (4096, 4096, 4096))):
        leaf = leaf_for_fp32_nodes(K, 8)
        X = torch.randn(M, K, generator=g, device=device).to(dtype)
        W = (torch.randn(N, K, generator=g, device=device) * 0.02).to(dtype)
        ks = K // world
        want = matmul_tp_persistent(X, W.t(), leaf=leaf, node_dtype=torch.float32)
        for _ in range(2):
            got = tar.tree_matmul_all_reduce(X[:, rank * ks:(rank + 1) * ks], W[:, rank * ks:(rank + 1) * ks].t(), None,
                                             leaf=leaf, node_dtype=torch.float32)
        torch.cuda.synchronize()
        tar.custom_ar.check_status()
        assert got.dtype == dtype
        assert torch.equal(bits(got), bits(want)), (dtype, M, K, N)
    # operands with exact leaves and inexact node sums: the CPU oracle's fp32-node tree
    M, K, N, leaf = 128, 4096, 256, 512
    cg = torch.Generator().manual_seed(5)
    A = torch.randint(-15, 16, (M, K), generator=cg).float()
    B = torch.randint(-15, 16, (K, N), generator=cg).float()
    for i in range(K // leaf):
        A[:, i * leaf:(i + 1) * leaf] *= 2.0 ** (-5 * i)
    A, B = A.to(torch.bfloat16), B.to(torch.bfloat16)
    want = tbik_matmul_ref(A, B, leaf, torch.float32, torch.bfloat16)
    ks = K // world
    got = tar.tree_matmul_all_reduce(A[:, rank * ks:(rank + 1) * ks].to(device), B[rank * ks:(rank + 1) * ks].to(device),
                                     None, leaf=leaf, node_dtype=torch.float32)
    torch.cuda.synchronize()
    assert torch.equal(bits(got.cpu()), bits(want))

    # the rounding all-reduce alone, one-shot and two-shot, ragged part sizes
    ar = tar.custom_ar
    for numel, seed in ((8 * 1237, 61), (1 << 16, 62), (8 * 100003, 63), (1 << 22, 64)):
        xs = [t.float() * 1.37 for t in _inputs(world, numel, torch.bfloat16, seed, device)]
        parts = [x.clone() for x in xs]
        stride = 1
        while stride < world:
            for i in range(0, world, 2 * stride):
                parts[i] = parts[i] + parts[i + stride]
            stride *= 2
        for out_dtype in (torch.bfloat16, torch.float16):
            want = parts[0].to(out_dtype)
            for one_max in (1 << 30, 1024):   # everything one-shot / everything two-shot
                ops.configure(ar._ptr, ops.CFG_ONESHOT_MAX_BYTES, one_max)
                view = ar.registered_view((numel,), torch.float32)
                view.copy_(xs[rank])
                got = ar.all_reduce_rounding(view, out_dtype)
                torch.cuda.synchronize()
                ar.check_status()
                assert torch.equal(bits(got), bits(want)), (numel, out_dtype, one_max)
    ops.configure(ar._ptr, ops.CFG_ONESHOT_MAX_BYTES, 0)
    dist.barrier()
    tar.reset_communicator()
    return True
