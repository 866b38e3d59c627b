"""Output-channel (N) sharding of the W8A8 linear over the GPUs of one box.

The reference has no collective of its own; its serving stack runs these projections column-
parallel and gathers the result (benchmarks/microbench.py:187 "column parallel + gather").
Here rank r owns ``w[r*N/G:(r+1)*N/G]`` and its channel scales, the activations are replicated,
every rank quantizes them itself (cheap next to the GEMM) and computes a BF16 ``[M, N/G]`` column
block; only that BF16 block crosses NVLink, and afterwards the whole output is on every rank.
Ways to move it (``mode``):

* ``"fused"`` (the default on more than one GPU): the gathered buffers live in symmetric memory,
  every rank maps its peers' buffers, and the GEMM's epilogue stores each finished tile into block
  ``rank`` of every rank's buffer (``ops.fused_channel_mm_gather_sync``), so the transfers overlap the
  main loop and no communication kernel competes with the persistent GEMM for SMs. The kernel ends
  with a rendezvous over arrival counters in symmetric memory: when it returns on a rank, that rank's
  buffer is complete, and no collective follows. The layer owns TWO sets of buffers and alternates
  between them, so a rank that is already in its next call never writes into a result that a peer
  is still reading: the tensor ``forward`` returns stays valid until the second-next ``forward``.
* ``"fused_flag"``: the same stores; the GEMM kernel ends as soon as its own work is done and a
  one-thread kernel behind it (``ops.peer_rendezvous``) exchanges the arrival counts.
* ``"fused_nccl_barrier"``: the same stores, closed by a small stream-ordered NCCL all-reduce instead
  (the first form of this path; kept for comparison).
* ``"nccl"``: the GEMM writes its block locally and one NCCL all-gather moves it.
* ``"none"``: no gather at all: the result stays column-sharded, ``[M, N/G]`` per rank in block ``rank``
  of the returned buffer. A row-parallel layer that follows (the down projection after a column-
  parallel gate/up) consumes exactly that, and nothing crosses NVLink.

Layout of the gathered output: ``[chunks, G, M/chunks, N/G]``. Column blocks of a row-major
``[M, N]`` matrix are not contiguous, so each rank's block is kept contiguous instead and the
gather is done in place (a rank writes its block straight into its slot). ``chunks > 1`` (NCCL mode)
splits the rows so that the gather of a finished row chunk overlaps the GEMM of the next one on a
second stream. ``ShardPlan.row_major`` gives the ``[M, N]`` view as a copy when a caller needs it.

The bookkeeping (``ShardPlan``) is plain Python and is tested with CPU ranks over gloo; the
device work goes through ``consumer_int8.ops`` and fails loudly without the CUDA extension.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardPlan:
    m: int
    n: int
    k: int
    world: int
    rank: int
    chunks: int = 1

    def __post_init__(self):
        if self.world <= 0 or not 0 <= self.rank < self.world:
            raise ValueError(f"rank {self.rank} outside world of {self.world}")
        if self.n % self.world:
            raise ValueError(f"N={self.n} does not split evenly over {self.world} ranks")
        if (self.n // self.world) % 4:
            raise ValueError("each shard must keep N % 4 == 0 (fused_channel_mm geometry)")
        if self.chunks <= 0 or self.m % self.chunks:
            raise ValueError(f"M={self.m} does not split into {self.chunks} row chunks")

    @property
    def shard_n(self) -> int:
        return self.n // self.world

    @property
    def chunk_m(self) -> int:
        return self.m // self.chunks

    @property
    def channels(self) -> slice:
        """The output channels this rank owns."""
        return slice(self.rank * self.shard_n, (self.rank + 1) * self.shard_n)

    @property
    def gathered_shape(self) -> tuple[int, int, int, int]:
        return (self.chunks, self.world, self.chunk_m, self.shard_n)

    @property
    def gather_bytes_received(self) -> int:
        """BF16 bytes each rank receives per call."""
        return 2 * self.m * self.shard_n * (self.world - 1)

    def shard_weights(self, w: torch.Tensor, w_scale: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        if w.shape[0] != self.n or w_scale.shape[0] != self.n:
            raise ValueError("weight or scale does not have N rows")
        return w[self.channels].contiguous(), w_scale[self.channels].contiguous()

    def row_major(self, gathered: torch.Tensor) -> torch.Tensor:
        """[chunks, G, M/chunks, N/G] -> [M, N] (a copy)."""
        if tuple(gathered.shape) != self.gathered_shape:
            raise ValueError(f"expected {self.gathered_shape}, got {tuple(gathered.shape)}")
        return gathered.permute(0, 2, 1, 3).reshape(self.m, self.n)


MODES = ("fused", "fused_flag", "fused_nccl_barrier", "nccl", "none")
FUSED_MODES = ("fused", "fused_flag", "fused_nccl_barrier")


class ColumnShardedLinear:
    """quantize_rows -> fused_channel_mm on this rank's channels -> all-gather of the BF16 block.

    All buffers are allocated once here; ``forward`` allocates nothing. ``mode=None`` picks
    ``"fused"`` for CUDA weights on more than one rank and ``"nccl"`` otherwise.
    """

    def __init__(self, plan: ShardPlan, w_shard: torch.Tensor, w_scale_shard: torch.Tensor,
                 group: dist.ProcessGroup | None = None, schedule: int = 0, operators=None,
                 mode: str | None = None):
        if operators is None:
            from . import ops as operators  # the compiled operators; there is no fallback

        self.ops = operators   # tests of the host logic inject a stand-in here
        self.plan = plan
        self.group = group
        self.schedule = schedule
        if tuple(w_shard.shape) != (plan.shard_n, plan.k) or w_shard.dtype != torch.int8:
            raise ValueError("w_shard must be INT8 [N/G, K]")
        self.w = w_shard
        self.w_scale = w_scale_shard
        device = w_shard.device
        self.codes = torch.empty(plan.m, plan.k, dtype=torch.int8, device=device)
        self.scales = torch.empty(plan.m, dtype=torch.float32, device=device)
        if mode is None:
            mode = "fused" if plan.world > 1 and device.type == "cuda" else "nccl"
        if mode not in MODES:
            raise ValueError(f"mode must be one of {MODES}")
        self.mode = mode if plan.world > 1 else "nccl"
        self.calls = 0
        self._sets = []            # fused modes: two sets of (gathered, peer_ptrs, signal_ptrs, state, handles)
        if self.mode in FUSED_MODES:
            if plan.chunks != 1:
                raise ValueError("the fused gather overlaps tile by tile; use chunks=1")
            if plan.shard_n % 8:
                raise ValueError("the fused gather needs N/G % 8 == 0")
            import torch.distributed._symmetric_memory as symm_mem

            where = group if group is not None else dist.group.WORLD
            for _ in range(2):
                flat = symm_mem.empty(plan.world * plan.m * plan.shard_n, dtype=torch.bfloat16, device=device)
                handle = symm_mem.rendezvous(flat, group=where)
                counters = symm_mem.empty(8, dtype=torch.int64, device=device)   # one arrival counter per source rank
                counters.zero_()
                counter_handle = symm_mem.rendezvous(counters, group=where)
                self._sets.append(dict(
                    gathered=flat.view(plan.gathered_shape),
                    peer_ptrs=torch.tensor([int(p) for p in handle.buffer_ptrs], dtype=torch.int64),
                    signal_ptrs=torch.tensor([int(p) for p in counter_handle.buffer_ptrs], dtype=torch.int64),
                    state=torch.zeros(4, dtype=torch.int64, device=device),   # calls done, CTAs gone, tiles drawn, spare
                    keep=(handle, counter_handle, counters),     # keeps the peer mappings alive
                ))
            torch.cuda.synchronize(device)
            dist.barrier(group=group)       # every rank's counters are zero before anybody signals
            self.gathered = self._sets[0]["gathered"]
            self._barrier_word = torch.zeros(1, dtype=torch.float32, device=device)
        else:
            self.gathered = torch.empty(plan.gathered_shape, dtype=torch.bfloat16, device=device)
        overlap = self.mode == "nccl" and plan.chunks > 1 and plan.world > 1 and device.type == "cuda"
        self.comm_stream = torch.cuda.Stream(device=device) if overlap else None
        self._chunk_done = [torch.cuda.Event() for _ in range(plan.chunks)] if self.comm_stream else []

    def local_block(self, chunk: int = 0) -> torch.Tensor:
        return self.gathered[chunk, self.plan.rank]

    def compute(self, x: torch.Tensor) -> None:
        """Quantize and run this rank's GEMM (no communication)."""
        plan = self.plan
        self.ops.quantize_rows(x, self.codes, self.scales)
        for c in range(plan.chunks):
            rows = slice(c * plan.chunk_m, (c + 1) * plan.chunk_m)
            self.ops.fused_channel_mm(self.codes[rows], self.w, self.scales[rows], self.w_scale,
                                      self.local_block(c), self.schedule)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        plan = self.plan
        if plan.world == 1 or self.mode == "none":
            self.compute(x)
            return self.gathered
        self.ops.quantize_rows(x, self.codes, self.scales)
        if self.mode in FUSED_MODES:
            # every rank writes its block into every rank's buffer; the two sets alternate so that a
            # rank already in its next call cannot overwrite a result a peer still reads
            current = self._sets[self.calls % 2]
            self.calls += 1
            self.gathered = current["gathered"]
            if self.mode == "fused":
                self.ops.fused_channel_mm_gather_sync(self.codes, self.w, self.scales, self.w_scale, self.gathered[0],
                                                      current["peer_ptrs"], current["signal_ptrs"], current["state"],
                                                      plan.rank, self.schedule)
            else:
                self.ops.fused_channel_mm_gather(self.codes, self.w, self.scales, self.w_scale, self.gathered[0],
                                                 current["peer_ptrs"], plan.rank, self.schedule)
                if self.mode == "fused_flag":
                    self.ops.peer_rendezvous(current["signal_ptrs"], current["state"], plan.rank)
                else:
                    dist.all_reduce(self._barrier_word, group=self.group)   # stream-ordered, no host sync
            return self.gathered
        main = torch.cuda.current_stream() if self.comm_stream is not None else None
        for c in range(plan.chunks):
            rows = slice(c * plan.chunk_m, (c + 1) * plan.chunk_m)
            self.ops.fused_channel_mm(self.codes[rows], self.w, self.scales[rows], self.w_scale,
                                      self.local_block(c), self.schedule)
            flat = self.gathered[c].view(plan.world * plan.chunk_m, plan.shard_n)
            mine = self.local_block(c)
            if self.comm_stream is None:
                dist.all_gather_into_tensor(flat, mine, group=self.group)
            else:
                self._chunk_done[c].record(main)
                with torch.cuda.stream(self.comm_stream):
                    self.comm_stream.wait_event(self._chunk_done[c])
                    dist.all_gather_into_tensor(flat, mine, group=self.group)
        if self.comm_stream is not None:
            main.wait_stream(self.comm_stream)
        return self.gathered
