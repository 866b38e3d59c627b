"""The N-sharded linear on real GPUs (needs at least two): both ways of moving the BF16 column
blocks — the GEMM epilogue storing into every rank's symmetric-memory buffer, and a separate NCCL
all-gather — must reproduce the unsharded result of the CPU checker bit for bit."""
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


def _rank_main(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from consumer_int8 import workloads
        from consumer_int8.sharded import ColumnShardedLinear, ShardPlan
        from oracle import w8a8_ref as ref

        outcome = {}
        for m, n, k in [(300, 1024, 544), (1041, 2048, 1024)]:
            inputs = workloads.linear_inputs(m, n, k, seed=3)
            codes, scales = ref.quantize_rows_ref(inputs.x)
            _, want = ref.fused_channel_mm_ref(codes, inputs.w, scales, inputs.w_scale, fast=True)
            for mode, chunks in (("fused", 1), ("nccl", 1), ("nccl", 3 if m % 3 == 0 else 1)):
                plan = ShardPlan(m, n, k, world, rank, chunks)
                w_shard, sw_shard = plan.shard_weights(inputs.w, inputs.w_scale)
                layer = ColumnShardedLinear(plan, w_shard.to(device), sw_shard.to(device), mode=mode)
                layer.gathered.fill_(float("nan"))
                dist.barrier()
                for _ in range(2):       # twice: the second call overwrites a full buffer
                    gathered = layer.forward(inputs.x.to(device))
                torch.cuda.synchronize()
                got = plan.row_major(gathered).cpu()
                outcome[f"{mode}/{chunks}/{m}x{n}x{k}"] = bool(torch.equal(got.view(torch.int16), want.view(torch.int16)))
                dist.barrier()
        results[rank] = outcome
    finally:
        dist.destroy_process_group()


def test_sharded_linear_matches_unsharded_checker_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    manager = mp.Manager()
    results = manager.dict()
    port = 29700 + os.getpid() % 500
    mp.spawn(_rank_main, args=(2, port, results), nprocs=2, join=True)
    for rank in (0, 1):
        assert results[rank] and all(results[rank].values()), results[rank]
