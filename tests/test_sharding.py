"""Host logic of the N-sharded linear: shard arithmetic, the gathered layout, and a two-rank
run over gloo on the CPU in which the operators are replaced by the CPU checker (the device
kernels themselves are covered by the GPU tests)."""
import os
import sys
import types
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
for entry in (str(ROOT), str(ROOT / "consumer-int8-kernels_b200")):
    if entry not in sys.path:
        sys.path.insert(0, entry)

from consumer_int8.sharded import ShardPlan  # noqa: E402


def test_shard_plan_arithmetic():
    plan = ShardPlan(m=16384, n=34816, k=5120, world=8, rank=3, chunks=4)
    assert plan.shard_n == 4352 and plan.chunk_m == 4096
    assert plan.channels == slice(3 * 4352, 4 * 4352)
    assert plan.gathered_shape == (4, 8, 4096, 4352)
    assert plan.gather_bytes_received == 2 * 16384 * 4352 * 7 == 998_244_352
    for world in (1, 2, 4, 8):
        assert ShardPlan(16384, 34816, 5120, world, 0).shard_n % 256 == 0


def test_shard_plan_rejects_bad_splits():
    with pytest.raises(ValueError, match="evenly"):
        ShardPlan(8, 100, 32, 3, 0)
    with pytest.raises(ValueError, match="rank"):
        ShardPlan(8, 64, 32, 2, 2)
    with pytest.raises(ValueError, match="row chunks"):
        ShardPlan(10, 64, 32, 2, 0, chunks=4)
    with pytest.raises(ValueError, match="N % 4"):
        ShardPlan(8, 12, 32, 2, 0)
    plan = ShardPlan(8, 64, 32, 2, 0)
    with pytest.raises(ValueError, match="N rows"):
        plan.shard_weights(torch.zeros(60, 32, dtype=torch.int8), torch.zeros(64))


def test_row_major_inverts_the_gathered_layout():
    plan = ShardPlan(m=6, n=8, k=32, world=2, rank=0, chunks=3)
    full = torch.arange(48, dtype=torch.float32).view(6, 8)
    gathered = torch.empty(plan.gathered_shape)
    for c in range(3):
        for r in range(2):
            gathered[c, r] = full[c * 2:(c + 1) * 2, r * 4:(r + 1) * 4]
    assert torch.equal(plan.row_major(gathered), full)


def _checker_operators():
    from oracle import w8a8_ref as ref

    def quantize_rows(x, codes, scales):
        c, s = ref.quantize_rows_ref(x)
        codes.copy_(c)
        scales.copy_(s)

    def fused_channel_mm(a, w, sa, sw, out, schedule=0):
        out.copy_(ref.fused_channel_mm_ref(a, w, sa, sw, fast=True)[1])

    return types.SimpleNamespace(quantize_rows=quantize_rows, fused_channel_mm=fused_channel_mm)


def _rank_main(rank, world, port, chunks, fail_rank, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from consumer_int8 import workloads
        from consumer_int8.sharded import ColumnShardedLinear
        from oracle import w8a8_ref as ref

        m, n, k = 12, 64, 256
        inputs = workloads.linear_inputs(m, n, k, seed=0)
        plan = ShardPlan(m, n, k, world, rank, chunks)
        w_shard, sw_shard = plan.shard_weights(inputs.w, inputs.w_scale)
        if rank == fail_rank:
            w_shard = w_shard[:-4]     # a rank that shows up with the wrong shard size
        try:
            layer = ColumnShardedLinear(plan, w_shard, sw_shard, operators=_checker_operators())
        except ValueError as error:
            results[rank] = f"rejected: {error}"
            return
        if fail_rank is not None:
            results[rank] = "constructed"
            return
        gathered = layer.forward(inputs.x)
        codes, scales = ref.quantize_rows_ref(inputs.x)
        _, want = ref.fused_channel_mm_ref(codes, inputs.w, scales, inputs.w_scale)
        ok = bool(torch.equal(plan.row_major(gathered), want))
        # the column-sharded mode: no collective at all, every rank keeps its own [M, N/G] block
        if chunks == 1:
            alone = ColumnShardedLinear(plan, w_shard, sw_shard, operators=_checker_operators(), mode="none")
            block = alone.forward(inputs.x)[0, rank]
            ok = ok and bool(torch.equal(block, want[:, plan.channels]))
        with pytest.raises(ValueError, match="mode must be"):
            ColumnShardedLinear(plan, w_shard, sw_shard, operators=_checker_operators(), mode="ring")
        results[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("chunks", [1, 3])
def test_two_ranks_over_gloo_reassemble_the_unsharded_output(chunks):
    manager = mp.Manager()
    results = manager.dict()
    port = 29500 + os.getpid() % 1000 + chunks
    mp.spawn(_rank_main, args=(2, port, chunks, None, results), nprocs=2, join=True)
    assert dict(results) == {0: True, 1: True}


def test_wrong_shard_size_is_rejected_on_the_host_before_any_collective():
    manager = mp.Manager()
    results = manager.dict()
    port = 31500 + os.getpid() % 1000
    mp.spawn(_rank_main, args=(2, port, 1, 1, results), nprocs=2, join=True)
    assert results[0] == "constructed" and results[1].startswith("rejected")
