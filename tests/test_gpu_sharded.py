"""The N-sharded linear on real GPUs (2, 4 and 8 ranks, as many as the box has): every way of moving
the BF16 column blocks — the GEMM epilogue storing into every rank's symmetric-memory buffer (closed
by the in-kernel rendezvous or by an NCCL barrier) and a separate NCCL all-gather — must reproduce
the unsharded result of the CPU checker bit for bit on every rank, also when the call is replayed
from a CUDA graph, and at the benchmark's full shard size. NVLS is kept off: plain peer stores."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
for entry in (str(ROOT), str(ROOT / "consumer-int8-kernels_b200")):
    if entry not in sys.path:
        sys.path.insert(0, entry)

pytestmark = pytest.mark.gpu


def _same(got, want):
    return bool(torch.equal(got.view(torch.int16), want.view(torch.int16)))


def _small_shapes(rank, world, device, outcome):
    from consumer_int8 import workloads
    from consumer_int8.sharded import ColumnShardedLinear, ShardPlan
    from oracle import w8a8_ref as ref

    for m, n, k in [(300, 128 * world, 544), (1041, 512 * world, 1024)]:
        inputs = workloads.linear_inputs(m, n, k, seed=3)
        codes, scales = ref.quantize_rows_ref(inputs.x)
        _, want = ref.fused_channel_mm_ref(codes, inputs.w, scales, inputs.w_scale, fast=True)
        x = inputs.x.to(device)
        for mode, chunks in (("fused", 1), ("fused_flag", 1), ("fused_nccl_barrier", 1), ("nccl", 1), ("nccl", 3 if m % 3 == 0 else 1)):
            plan = ShardPlan(m, n, k, world, rank, chunks)
            w_shard, sw_shard = plan.shard_weights(inputs.w, inputs.w_scale)
            layer = ColumnShardedLinear(plan, w_shard.to(device), sw_shard.to(device), mode=mode)
            for s in layer._sets:
                s["gathered"].fill_(float("nan"))
            layer.gathered.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            for call in range(3):       # three calls: both buffer sets, then the first one again (overwritten)
                dist.barrier()          # the in-kernel rendezvous gives up after 2 s: enter together
                gathered = layer.forward(x)
                torch.cuda.synchronize()
                outcome[f"{mode}/{chunks}/{m}x{n}x{k}/call{call}"] = _same(plan.row_major(gathered).cpu(), want)
            dist.barrier()
        # the column-sharded form: nothing crosses NVLink, every rank holds its own block
        plan = ShardPlan(m, n, k, world, rank)
        w_shard, sw_shard = plan.shard_weights(inputs.w, inputs.w_scale)
        layer = ColumnShardedLinear(plan, w_shard.to(device), sw_shard.to(device), mode="none")
        block = layer.forward(x)[0, rank]
        torch.cuda.synchronize()
        outcome[f"none/{m}x{n}x{k}"] = _same(block.cpu(), want[:, plan.channels].contiguous())
        dist.barrier()


def _graph_replay(rank, world, device, outcome):
    """Two calls (one per buffer set) captured in one CUDA graph and replayed on fresh activations:
    the call counter of the rendezvous lives in device memory, so a replay is a new call."""
    from consumer_int8 import workloads
    from consumer_int8.sharded import ColumnShardedLinear, ShardPlan
    from oracle import w8a8_ref as ref

    m, n, k = 520, 256 * world, 512
    inputs = workloads.linear_inputs(m, n, k, seed=9)
    plan = ShardPlan(m, n, k, world, rank)
    w_shard, sw_shard = plan.shard_weights(inputs.w, inputs.w_scale)
    layer = ColumnShardedLinear(plan, w_shard.to(device), sw_shard.to(device), mode="fused")
    x = inputs.x.to(device)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        dist.barrier()
        layer.forward(x)
        layer.forward(x)
        torch.cuda.synchronize()
        dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            first = layer.forward(x)
            second = layer.forward(x)
        for replay in range(3):
            fresh = workloads.linear_inputs(m, n, k, seed=20 + replay)
            x.copy_(fresh.x.to(device))
            first.fill_(float("nan"))
            second.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            graph.replay()
            torch.cuda.synchronize()
            codes, scales = ref.quantize_rows_ref(fresh.x)
            _, want = ref.fused_channel_mm_ref(codes, inputs.w, scales, inputs.w_scale, fast=True)
            outcome[f"graph/replay{replay}/first"] = _same(plan.row_major(first).cpu(), want)
            outcome[f"graph/replay{replay}/second"] = _same(plan.row_major(second).cpu(), want)
            dist.barrier()


def _full_size_shard(rank, world, device, outcome):
    """The benchmark's shard at 8 GPUs (M=16384, N/G=4352, K=5120) on however many ranks are here: a
    seeded row sample of every rank's block, on every rank, against the CPU checker."""
    from consumer_int8 import workloads
    from consumer_int8.sharded import ColumnShardedLinear, ShardPlan
    from oracle import w8a8_ref as ref

    m, shard, k = 16384, 4352, 5120
    n = shard * world
    gen = torch.Generator().manual_seed(0)
    x_host = workloads.activations(m, k, gen)
    w, w_scale = workloads.weights(n, k, gen)
    plan = ShardPlan(m, n, k, world, rank)
    w_shard, sw_shard = plan.shard_weights(w, w_scale)
    layer = ColumnShardedLinear(plan, w_shard.to(device), sw_shard.to(device), mode="fused")
    x = x_host.to(device)
    rows = torch.randperm(m, generator=torch.Generator().manual_seed(1))[:48].sort().values
    codes, scales = ref.quantize_rows_ref(x_host[rows])
    _, want = ref.fused_channel_mm_ref(codes, w, scales, w_scale, fast=True)
    for call in range(2):
        dist.barrier()                  # the checker above takes a different time on every rank
        gathered = layer.forward(x)
        torch.cuda.synchronize()
        got = gathered[0][:, rows.to(device)].permute(1, 0, 2).reshape(len(rows), n).cpu()
        outcome[f"full/call{call}"] = _same(got, want)
    dist.barrier()


def _rank_main(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import ctypes

        from consumer_int8 import ops

        outcome = {}
        _small_shapes(rank, world, device, outcome)
        _graph_replay(rank, world, device, outcome)
        _full_size_shard(rank, world, device, outcome)
        word = ctypes.c_uint(0)
        outcome["status word clear"] = ops.libci8.ci8_device_status(ctypes.byref(word)) == 0 and word.value == 0
        results[rank] = outcome
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_linear_matches_unsharded_checker_on_every_rank(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    manager = mp.Manager()
    results = manager.dict()
    port = 29700 + (os.getpid() + 17 * world) % 500
    mp.spawn(_rank_main, args=(world, port, results), nprocs=world, join=True)
    for rank in range(world):
        assert rank in results, f"rank {rank} reported nothing"
        failed = [name for name, ok in results[rank].items() if not ok]
        assert not failed, (rank, failed)
