"""Per-rank bodies of the CPU (gloo) tests of the all-reduce host logic."""
import torch
import torch.distributed as dist


def _bits(t):
    return t.contiguous().view(torch.int16 if t.element_size() == 2 else torch.int32)


def _inputs(world, numel, dtype, seed):
    out = []
    for r in range(world):
        g = torch.Generator().manual_seed(seed * 1000 + r)
        out.append((torch.randn(numel, generator=g) * 3).to(dtype))
    return out


def communicator_lifecycle(rank, world):
    import fake_backend
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce as car
    from oracle.tbik_ref import tree_allreduce_ref

    ops = fake_backend.install(car, dist.group.WORLD)
    try:
        ar = car.CustomTreeAllreduce(group=dist.group.WORLD, device=torch.device("cpu"), max_size=1 << 16)
        assert not ar.disabled and ar.rank == rank and ar.world_size == world
        assert len(ar.meta_ptrs) == world and len(ar.buffer_ptrs) == world
        assert ops.comms[ar._ptr]["cfg"][ops.CFG_SCRATCH_BYTES] == 1 << 16
        for dtype, numel in ((torch.bfloat16, 4096), (torch.float16, 512), (torch.float32, 256)):
            xs = _inputs(world, numel, dtype, 7)
            got = ar.custom_tree_all_reduce(xs[rank])
            assert torch.equal(_bits(got), _bits(tree_allreduce_ref(xs)))
        # eligibility: byte size not a multiple of 16; too large; non-contiguous
        assert ar.custom_tree_all_reduce(torch.zeros(3, dtype=torch.bfloat16)) is None
        assert ar.custom_tree_all_reduce(torch.zeros(1 << 15, dtype=torch.bfloat16)) is None      # == max_size
        assert ar.custom_tree_all_reduce(torch.zeros(64, 64, dtype=torch.bfloat16)[:, :32]) is None
        assert ar.should_custom_ar(torch.zeros(64, 64, dtype=torch.bfloat16)[8:].t())             # weakly contiguous
        # the explicit `out=` and registered paths of all_reduce
        xs = _inputs(world, 64, torch.bfloat16, 9)
        out = torch.empty(64, dtype=torch.bfloat16)
        assert ar.all_reduce(xs[rank], out=out) is out
        try:
            ar.all_reduce(xs[rank], registered=True)  # xs is not a registered buffer
            raise AssertionError("unregistered input must be rejected")
        except RuntimeError as e:
            assert "not registered" in str(e)
        ar.close()
        ar.close()  # idempotent
        assert ar.custom_tree_all_reduce(xs[rank]) is None
        # the non-tree class: world 1 is not supported there, fp32-accumulated linear order otherwise
        lin = car.CustomAllreduce(group=dist.group.WORLD, device="cpu")
        if world == 1:
            assert lin.disabled
        else:
            xs = _inputs(world, 128, torch.bfloat16, 11)
            acc = xs[0].float()
            for q in xs[1:]:
                acc = acc + q.float()
            assert torch.equal(_bits(lin.custom_all_reduce(xs[rank])), _bits(acc.to(torch.bfloat16)))
            lin.close()
    finally:
        fake_backend.FakeCudaRT.cleanup()
    return True


def disabled_paths(rank, world):
    import fake_backend
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce as car

    try:
        # different host names -> multi-node -> disabled, no exception
        fake_backend.install(car, dist.group.WORLD, hostname=f"node{rank}")
        ar = car.CustomTreeAllreduce(group=dist.group.WORLD, device="cpu")
        assert ar.disabled and ar.custom_tree_all_reduce(torch.zeros(8, dtype=torch.bfloat16)) is None
        ar.close()
        # P2P not possible -> disabled
        fake_backend.install(car, dist.group.WORLD, hostname="same", can_p2p=False)
        assert car.CustomTreeAllreduce(group=dist.group.WORLD, device="cpu").disabled
        # no full NVLink: fine for 2 ranks, disabled beyond
        fake_backend.install(car, dist.group.WORLD, hostname="same", full_nvlink=False)
        ar = car.CustomTreeAllreduce(group=dist.group.WORLD, device="cpu")
        assert ar.disabled == (world > 2)
        ar.close()
        # CUDA / native library absent -> disabled before any collective
        car.is_cuda = lambda: False
        assert car.CustomTreeAllreduce(group=dist.group.WORLD, device="cpu").disabled
    finally:
        fake_backend.FakeCudaRT.cleanup()
    return True


def dispatcher_paths(rank, world):
    """tree_all_reduce_sum: custom path when eligible, native path when disabled / not eligible / above the cut-off."""
    import os
    import fake_backend
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce as car
    from llm_reproducibility_b200.tbik import tree_based_all_reduce as tar
    from oracle.tbik_ref import tree_allreduce_ref

    ops = fake_backend.install(car, dist.group.WORLD, hostname="same")
    try:
        os.environ["TBIK_AR_MAX_SIZE"] = str(1 << 16)
        xs = _inputs(world, 2048, torch.bfloat16, 21)
        want = tree_allreduce_ref(xs)
        y = tar.tree_all_reduce_sum(xs[rank], dist.group.WORLD)
        assert torch.equal(_bits(y), _bits(want)) and ops.calls[-1] == ("tree", 2048)
        n_calls = len(ops.calls)
        # not eligible (odd size) -> native all_gather + ordered adds, same bits
        xs = _inputs(world, 2047, torch.bfloat16, 22)
        y = tar.tree_all_reduce_sum(xs[rank], dist.group.WORLD)
        assert torch.equal(_bits(y), _bits(tree_allreduce_ref(xs))) and len(ops.calls) == n_calls
        # above the optional cut-off -> native
        os.environ["TBIK_AR_NATIVE_CUTOFF"] = "1024"
        xs = _inputs(world, 2048, torch.bfloat16, 23)
        y = tar.tree_all_reduce_sum(xs[rank], dist.group.WORLD)
        assert torch.equal(_bits(y), _bits(tree_allreduce_ref(xs))) and len(ops.calls) == n_calls
        del os.environ["TBIK_AR_NATIVE_CUTOFF"]
        # a real error of the native op is raised, not swallowed
        def boom(*a):
            raise RuntimeError("kernel launch failed")
        ops.tree_all_reduce = boom
        try:
            tar.tree_all_reduce_sum(_inputs(world, 2048, torch.bfloat16, 24)[rank], dist.group.WORLD)
            raise AssertionError("error must propagate")
        except RuntimeError as e:
            assert "kernel launch failed" in str(e)
        tar.reset_communicator()
        assert tar.custom_ar is None
    finally:
        os.environ.pop("TBIK_AR_MAX_SIZE", None)
        fake_backend.FakeCudaRT.cleanup()
    return True


def native_rejects_non_power_of_two(rank, world):
    from llm_reproducibility_b200.tbik.tree_based_all_reduce import tree_all_reduce_sum_native
    try:
        tree_all_reduce_sum_native(torch.zeros(4), None)
    except ValueError:
        return True
    return False


def row_parallel_layer(rank, world):
    """Patched forward on CPU ranks with the GEMM replaced by the oracle: slicing, reduction, bias rules."""
    import fake_backend
    from llm_reproducibility_b200.mini_allreduce import custom_all_reduce as car
    import importlib
    pti = importlib.import_module("llm_reproducibility_b200.patch.patch_tp_invariant")
    from llm_reproducibility_b200.tbik import tree_based_all_reduce as tar
    from oracle.tbik_ref import exact_int_inputs, tbik_matmul_ref

    fake_backend.install(car, dist.group.WORLD, hostname="same")
    import llm_reproducibility_b200.tbik.tree_based_matmul as tbm

    def fake_matmul(a, b, bias=None, out=None, **kw):
        c = tbik_matmul_ref(a, b)
        if out is not None:
            out.copy_(c)
            return out
        return c
    pti.matmul_tp_persistent = fake_matmul
    tbm.matmul_tp_persistent = fake_matmul
    try:
        M, K, N = 6, 2048, 64
        A, B = exact_int_inputs(M, K, N, torch.bfloat16, seed=5, amax=7)
        W = B.t().contiguous()
        ks = K // world
        bias = torch.arange(N, dtype=torch.bfloat16)

        class Layer:
            input_is_parallel = False
            tp_size, tp_rank = world, rank
            weight = W[:, rank * ks:(rank + 1) * ks].contiguous()
            skip_bias_add = False
            reduce_results = True
            return_bias = True
            quant_method = object()
        Layer.bias = bias
        out, ob = pti.row_parallel_forward(Layer(), A.view(2, 3, K), device_group_fn=lambda: dist.group.WORLD)
        assert ob is None and out.shape == (2, 3, N)
        want = tbik_matmul_ref(A, B) + bias
        assert torch.equal(_bits(out.reshape(M, N)), _bits(want))
        Layer.skip_bias_add = True
        Layer.input_is_parallel = True
        out, ob = pti.row_parallel_forward(Layer(), A[:, rank * ks:(rank + 1) * ks].contiguous(),
                                           device_group_fn=lambda: dist.group.WORLD)
        assert ob is bias and torch.equal(_bits(out), _bits(tbik_matmul_ref(A, B)))
        tar.reset_communicator()
    finally:
        fake_backend.FakeCudaRT.cleanup()
    return True
