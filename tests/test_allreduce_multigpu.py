"""Multi-GPU parity of the peer-to-peer tree all-reduce (one process per GPU, no NCCL on the data path).

Skipped unless at least two GPUs are visible.  The world size is the largest of 2/4/8 that fits.
"""
import pytest
import torch

from _dist_utils import run_ranks
import _ar_gpu_workers as w

pytestmark = pytest.mark.gpu


def _world():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for cand in (8, 4, 2):
        if n >= cand:
            return cand
    return 0


needs_multi = pytest.mark.skipif(_world() < 2, reason="needs >= 2 GPUs")


@needs_multi
def test_tree_allreduce_matches_oracle_all_sizes():
    world = _world()
    # bf16 8 KB ... 64 MB doubling (config 3), plus fp16 / fp32 and a ragged pack count
    cases = [(4096 << i, torch.bfloat16, 10 + i) for i in range(0, 14)]
    cases += [(8192, torch.float16, 40), (1 << 20, torch.float16, 41), (2048, torch.float32, 42),
              (1 << 19, torch.float32, 43), (8 * 1237, torch.bfloat16, 44), (8 * 100003, torch.bfloat16, 45)]
    reports = run_ranks(w.tree_allreduce_parity, world, backend="nccl", args=(cases, 160 << 20), timeout=900)
    assert all(ok for rep in reports for (_, _, _, ok) in rep)


@needs_multi
def test_linear_allreduce_matches_fp32_rank_order():
    assert all(run_ranks(w.linear_allreduce_parity, _world(), backend="nccl"))


@needs_multi
def test_graph_capture_registers_buffers():
    assert all(run_ranks(w.graph_capture, _world(), backend="nccl"))


@needs_multi
def test_dispatcher_and_row_parallel_layer():
    assert all(run_ranks(w.dispatcher, _world(), backend="nccl"))


@needs_multi
def test_pipelined_row_blocks_match_single_device():
    assert all(run_ranks(w.pipelined_layer, _world(), backend="nccl"))


@needs_multi
def test_fp32_node_layer_matches_single_device_and_oracle():
    assert all(run_ranks(w.fp32_nodes_layer, _world(), backend="nccl"))


@needs_multi
def test_a_wait_that_runs_out_returns_and_reports():
    """No GPU hangs or faults here: the lonely kernel's bounded wait (20 ms) expires, it writes a status record
    and returns; the peers are idle on the host meanwhile."""
    reports = run_ranks(w.barrier_timeout, _world(), backend="nccl")
    assert reports[0] < 1.0
