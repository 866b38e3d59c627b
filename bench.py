#!/usr/bin/env python
"""Benchmark of the W8A8 linear path: one JSON line per run.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one pass of the hot path over one batch of seeded synthetic input: quantize_rows on
BF16 activations, then the integer GEMM with the fused scale epilogue (and, on more than one
GPU, the all-gather of the BF16 output). Workloads (shapes of the five benchmark configs):

  sharded        M=16384 K=5120 N=34816, N split over the GPUs        (default, every --gpus)
  prefill_gate_up  M=4096 K=5120 N=34816       prefill_down   M=4096 K=17408 N=5120
  decode         M in {1,4,8,16} K=5120 N=34816 (HBM GB/s)            grouped  M=2048 K=8x4096 N=7168
  peer_store     the sharded output with K=32: times the epilogue's (peer) tile stores alone

``value`` is whole-job throughput with inputs resident in HBM; ``e2e`` is the same metric through
the public operators with host buffers (pinned host -> device copy of the activations and
device -> host copy of the result inside the timed region). ``--impl reference`` times the
reference's own host restatement of the path (torch on the CPU), on the whole workload when that
ends within a few minutes and on a bounded row sample otherwise.
Before anything is timed, a seeded sample of rows of the result on EVERY rank is compared bit for bit
with the CPU checker (the reference's discipline: benchmarks/microbench.py:206-214 asserts equality
before it times); a mismatch ends the run with a non-zero exit code, and the line carries
``"parity": true``. Inputs are synthetic (no dataset stands behind this path) and larger than L2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "consumer-int8-kernels_b200"))
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

WORKLOADS = {
    "sharded": dict(m=16384, k=5120, n=34816, config="configs[4]"),
    "prefill_gate_up": dict(m=4096, k=5120, n=34816, config="configs[2]"),
    "prefill_down": dict(m=4096, k=17408, n=5120, config="configs[2]"),
    "grouped": dict(m=2048, k=32768, n=7168, groups=8, config="configs[3]"),
    "decode": dict(m=16, k=5120, n=34816, config="configs[1]"),
    "decode_m8": dict(m=8, k=5120, n=34816, config="configs[1], M=8 (profile-only: the 8-row forms of the decode kernels)"),
    "q8_block": dict(m=4096, k=4096, n=1024, config="block-32 Q8_0 (the reference's benchmark shape)"),
    # the sharded output with next to no arithmetic (K = 32): what is left is the epilogue's tile stores,
    # i.e. on several GPUs the peer-store bandwidth of the fused gather
    "peer_store": dict(m=16384, k=32, n=34816, config="store-bandwidth probe of configs[4]'s output"),
}
METRIC = "W8A8 GEMM INT8 TOPS (quantize_rows + fused_channel_mm, whole job)"
RESULT_STREAM = sys.stdout     # main() replaces it by the original stdout and points fd 1 at stderr


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0), "fallback"


class ClockSampler:
    """Reads SM clock, power and throttle reasons through NVML while the timed region runs
    (read-only; nothing is set)."""

    def __init__(self, index: int):
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nvml = None

    def _run(self):
        n = self.nvml
        names = {
            "hw_slowdown": n.nvmlClocksEventReasonHwSlowdown if hasattr(n, "nvmlClocksEventReasonHwSlowdown") else 0x8,
            "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4, "hw_power_brake": 0x80,
        }
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def __enter__(self):
        if self.nvml:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self) -> dict:
        if not self.samples:
            return dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=[], samples=0)
        return dict(sm_mhz=statistics.median(self.samples), sm_max_mhz=self.max_mhz,
                    reasons=sorted(self.reasons), samples=len(self.samples))


# ----------------------------------------------------------------------------- CPU arm
def cpu_path(x, w_t, w_scale):
    """The reference's host restatement of the path: quantize, integer product, epilogue."""
    from oracle import w8a8_ref as ref

    codes, scales = ref.quantize_rows_ref(x)
    acc = torch._int_mm(codes, w_t) if codes.shape[0] > 16 else ref.int_mm_fast(codes, w_t.T)
    return ref.epilogue_ref(acc, scales, w_scale)


def cpu_sample(spec, target_seconds: float = 12.0):
    """Times the CPU path on a bounded row sample of the workload; returns a dict for JSON."""
    from consumer_int8 import workloads

    torch.set_num_threads(os.cpu_count() or 1)
    n, k = spec["n"], spec["k"]
    gen = torch.Generator().manual_seed(0)
    w, w_scale = workloads.weights(n, k, gen)
    w_t = w.T.contiguous()
    probe = 32
    x = workloads.activations(probe, k, gen)
    cpu_path(x, w_t, w_scale)
    t0 = time.perf_counter()
    cpu_path(x, w_t, w_scale)
    per_row = (time.perf_counter() - t0) / probe
    # the whole workload when three passes fit into about half a minute, else a bounded row sample
    rows = spec["m"] if per_row * spec["m"] * 3 <= 30.0 else int(max(32, min(spec["m"], target_seconds / 3 / max(per_row, 1e-9))))
    rows -= rows % 8
    x = workloads.activations(rows, k, gen)
    best = min(_timed(lambda: cpu_path(x, w_t, w_scale)) for _ in range(3))
    tops = 2.0 * rows * n * k / best / 1e12
    return dict(value=tops, unit="TOPS", cores=torch.get_num_threads(), kind="port",
                sample=f"{rows} of {spec['m']} rows x N={n} x K={k}, torch CPU (quantize_rows restatement + "
                       f"torch._int_mm + FP32 epilogue), best of 3, {best:.2f} s"), rows, best


def _timed(fn):
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0


def run_reference(args, spec, rank):
    """The reference arm: the host restatement of the path, K timed steps, each over a row sample
    sized so that warm-up plus K steps take about a minute and a half on this box's cores."""
    if rank != 0:
        return
    from consumer_int8 import workloads

    torch.set_num_threads(os.cpu_count() or 1)
    n, k = spec["n"], spec["k"]
    gen = torch.Generator().manual_seed(0)
    w, w_scale = workloads.weights(n, k, gen)
    w_t = w.T.contiguous()
    probe = workloads.activations(32, k, gen)
    cpu_path(probe, w_t, w_scale)
    per_row = _timed(lambda: cpu_path(probe, w_t, w_scale)) / 32
    warmup = max(args.warmup, 1)
    # every step is the whole workload when warm-up plus K steps then end within about four minutes
    # (so that both arms run the same configuration), else a row sample sized for a minute and a half
    if per_row * spec["m"] * (args.steps + warmup) <= 240.0:
        rows = spec["m"]
    else:
        rows = int(90.0 / (args.steps + warmup) / max(per_row, 1e-9))
        rows = max(24, min(spec["m"], rows - rows % 8))
    x = workloads.activations(rows, k, gen)
    for _ in range(warmup):
        cpu_path(x, w_t, w_scale)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_path(x, w_t, w_scale)
    seconds = (time.perf_counter() - t0) / args.steps
    tops = 2.0 * rows * n * k / seconds / 1e12
    sample = dict(value=tops, unit="TOPS", cores=torch.get_num_threads(), kind="port",
                  sample=f"{rows} of {spec['m']} rows x N={n} x K={k} per step, torch CPU (quantize_rows restatement + "
                         f"torch._int_mm + FP32 epilogue)")
    line = dict(metric=METRIC, value=tops, unit="TOPS", n_gpus=args.gpus, steps=args.steps, warmup=warmup,
                ms_per_step=seconds * 1e3, higher_is_better=True, scaling="strong", vs_baseline=None, dtype="int8",
                data="synthetic", impl="reference",
                config=dict(workload=f"{args.workload} {spec['config']} M={spec['m']} K={k} N={n}",
                            step=("the whole workload per step on the host CPU" if rows == spec["m"] else
                                  f"{rows}-row sample per step on the host CPU")),
                cpu_baseline=sample, e2e=dict(value=tops, unit="TOPS", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), file=RESULT_STREAM, flush=True)


# ----------------------------------------------------------------------------- GPU arm
NVLINK_PEER_GBS = 770.0      # measured peer copy on this pool, per direction per GPU (nominal 900)


def check_parity(plan, gathered, x_host, w, w_scale, device, rows_checked=32):
    """A seeded sample of rows of the whole [M, N] result on this rank against the CPU checker."""
    from oracle import w8a8_ref as ref

    rows = torch.randperm(plan.m, generator=torch.Generator().manual_seed(1234))[:rows_checked].sort().values
    codes, scales = ref.quantize_rows_ref(x_host[rows])
    _, want = ref.fused_channel_mm_ref(codes, w, scales, w_scale, fast=True)
    chunk, local = rows // plan.chunk_m, rows % plan.chunk_m
    got = gathered[chunk.to(device), :, local.to(device)]            # [rows, G, N/G]
    got = got.reshape(len(rows), plan.n).cpu()
    return bool(torch.equal(got.view(torch.int16), want.view(torch.int16)))


def source_tag() -> str:
    """Short hash of the GEMM kernel's code (comments and white space left out): DRAM-traffic figures
    from an ncu capture are only current while this matches the tag recorded with them."""
    import hashlib
    import re

    digest = hashlib.sha256()
    for name in ("gemm_tcgen05.cuh", "sm100_ptx.cuh"):
        text = (ROOT / "consumer-int8-kernels_b200" / "csrc" / name).read_text()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        digest.update("".join(text.split()).encode())
    return digest.hexdigest()[:12]


def run_ours(args, spec, rank, world, local_rank):
    import ctypes

    import torch.distributed as dist
    from consumer_int8 import ops, workloads
    from consumer_int8.sharded import ColumnShardedLinear, ShardPlan

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    m, n, k = spec["m"], spec["n"], spec["k"]
    gen = torch.Generator().manual_seed(0)
    x_host = workloads.activations(m, k, gen).pin_memory()
    w, w_scale = workloads.weights(n, k, gen)
    mode = args.gather if world > 1 else "nccl"
    fused = mode in ("fused", "fused_flag", "fused_nccl_barrier")     # symmetric memory, two buffer sets
    plan = ShardPlan(m, n, k, world, rank, chunks=args.chunks if mode == "nccl" and world > 1 else 1)
    w_shard, sw_shard = plan.shard_weights(w, w_scale)
    layer = ColumnShardedLinear(plan, w_shard.to(device), sw_shard.to(device), schedule=args.schedule, mode=mode)
    x = x_host.to(device)
    out_host = torch.empty(m, plan.shard_n, dtype=torch.bfloat16).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()       # the ranks enter the first call together (the in-kernel rendezvous gives up after 2 s)
    for _ in range(max(args.warmup, 3)):
        gathered = layer.forward(x)
    barrier()

    # ---- parity gate: nothing is timed before every rank's result has been checked
    ok = check_parity(plan, gathered, x_host, w, w_scale, device)
    if fused:     # the other buffer set as well (the ranks enter together: the rendezvous gives up after 2 s)
        barrier()
        second = layer.forward(x)
        barrier()
        ok = check_parity(plan, second, x_host, w, w_scale, device) and ok
    del w
    verdict = torch.tensor([1 if ok else 0], device=device)
    if world > 1:
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
    if verdict.item() != 1:
        print(f"bench: rank {rank}: the result differs from the CPU checker ({'this rank' if not ok else 'another rank'}); "
              "nothing was timed", file=sys.stderr, flush=True)
        raise SystemExit(3)
    barrier()

    # ---- device-resident timed region (K steps), GEMM timed per launch on the same stream
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    gemm0 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    gemm1 = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    end = torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        for i in range(args.steps):
            starts[i].record()
            if world == 1:
                ops.quantize_rows(x, layer.codes, layer.scales)
                gemm0[i].record()
                ops.fused_channel_mm(layer.codes, layer.w, layer.scales, layer.w_scale, layer.local_block(0), args.schedule)
                gemm1[i].record()
            else:
                layer.forward(x)
        end.record()
        barrier()
    step_ms = starts[0].elapsed_time(end) / args.steps
    gemm_ms = statistics.mean(a.elapsed_time(b) for a, b in zip(gemm0, gemm1)) if world == 1 else None
    sharded_ms = None
    if world > 1:
        # GEMM-only time of this rank's shard, and the step without any gather (the result stays
        # column-sharded, [M, N/G] per rank), each in a separate short loop
        barrier()
        a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        a.record()
        for _ in range(10):
            for ch in range(plan.chunks):
                rows = slice(ch * plan.chunk_m, (ch + 1) * plan.chunk_m)
                ops.fused_channel_mm(layer.codes[rows], layer.w, layer.scales[rows], layer.w_scale, layer.local_block(ch), args.schedule)
        b.record()
        for _ in range(10):
            ops.quantize_rows(x, layer.codes, layer.scales)
            ops.fused_channel_mm(layer.codes, layer.w, layer.scales, layer.w_scale, layer.gathered.view(world, m, plan.shard_n)[rank], args.schedule)
        c.record()
        barrier()
        gemm_ms, sharded_ms = a.elapsed_time(b) / 10, b.elapsed_time(c) / 10
        t = torch.tensor([step_ms, gemm_ms, sharded_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        step_ms, gemm_ms, sharded_ms = t.tolist()

    # ---- end-to-end region: host activations in, this rank's output block out, every step.
    # Two sets of device buffers and two copy streams: the device->host copy of step i runs while
    # step i+1's host->device copy and kernels run (both directions of the link in use at once).
    # The fused layer alternates its own two result buffers; the other modes get a second layer.
    e2e_steps = max(4, min(args.steps, 12))
    layers = [layer, layer if fused else ColumnShardedLinear(plan, layer.w, layer.w_scale, schedule=args.schedule, mode=mode)]
    xs = [x, torch.empty_like(x)]
    outs_host = [out_host, torch.empty_like(out_host).pin_memory()]
    main = torch.cuda.current_stream()
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    in_done = [torch.cuda.Event() for _ in range(2)]
    compute_done = [torch.cuda.Event() for _ in range(2)]
    out_done = [torch.cuda.Event() for _ in range(2)]
    for _ in range(2):
        layers[1].forward(xs[0])        # warm the second set
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(e2e_steps):
        s = i % 2
        with torch.cuda.stream(copy_in):
            copy_in.wait_event(compute_done[s])          # the kernels of step i-2 have read xs[s]
            xs[s].copy_(x_host, non_blocking=True)
            in_done[s].record()
        main.wait_event(in_done[s])
        main.wait_event(out_done[s])                     # step i-2's result has left its buffer
        gathered = layers[s].forward(xs[s])
        compute_done[s].record()
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(compute_done[s])
            for ch in range(plan.chunks):
                outs_host[s][ch * plan.chunk_m:(ch + 1) * plan.chunk_m].copy_(gathered[ch, rank], non_blocking=True)
            out_done[s].record()
    main.wait_stream(copy_out)
    b.record()
    barrier()
    e2e_ms = a.elapsed_time(b) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = t.item()

    word = ctypes.c_uint(0)
    ops.libci8.ci8_device_status(ctypes.byref(word))
    if rank != 0:
        return
    peaks, peak_kind = measured_peaks()
    ops_total = 2.0 * m * n * k
    # INT8 issues at twice the BF16 rate: the peak is 2 x the measured BF16 figure, the burst one for a
    # timed region shorter than a second, the sustained one for a longer loop
    region_s = step_ms * args.steps / 1e3
    burst_peak, sustained_peak = 2.0 * peaks["bf16_tflops"], 2.0 * peaks["bf16_tflops_sustained"]
    tensor_peak = burst_peak if region_s < 1.0 else sustained_peak
    gemm_tops = 2.0 * m * plan.shard_n * k / (gemm_ms * 1e-3) / 1e12
    traffic = KERNEL_TRAFFIC.get(args.workload if world == 1 else f"{args.workload}/{world}")
    # per GPU: the codes, this rank's weights and scales, and the BF16 result: its own block written once and,
    # on several GPUs, the other ranks' blocks arriving over NVLink (the whole [M, N] lands in every GPU's memory)
    algorithmic = float(m * k + plan.shard_n * k + 2 * m * n + 4 * m + 2 * plan.shard_n)
    # captures of the shard-shaped GEMM are taken on one GPU; the peers' blocks are added by construction
    traffic_bytes = (traffic["read"] + traffic["write"] + (plan.gather_bytes_received if world > 1 else 0)) if traffic else None
    roofline = dict(bound="tensor", achieved=gemm_tops, peak=tensor_peak, unit="TFLOP/s", frac=gemm_tops / tensor_peak,
                    frac_sustained=gemm_tops / sustained_peak, frac_nominal=gemm_tops / 4500.0,
                    traffic=traffic_bytes,
                    traffic_ratio=traffic_bytes / algorithmic if traffic else None,
                    traffic_source=traffic["source"] if traffic else None, kernel_source=source_tag(),
                    kernel="gemm_i8_kernel<2,fused>",
                    note=f"integer ops 2*M*N*K per launch / CUDA-event launch time ({gemm_ms:.3f} ms, per GPU); peak = 2 x "
                         f"{'bf16_tflops (burst' if region_s < 1.0 else 'bf16_tflops_sustained (long'} region, {region_s:.2f} s) of "
                         f"{peak_kind}; traffic is current when traffic_source equals kernel_source")
    line = dict(
        metric=METRIC, value=ops_total / (step_ms * 1e-3) / 1e12, unit="TOPS", n_gpus=world, steps=args.steps,
        warmup=max(args.warmup, 3), ms_per_step=step_ms, higher_is_better=True, scaling="strong", vs_baseline=None,
        dtype="int8", data="synthetic", parity=True,
        config=dict(workload=f"{args.workload} {spec['config']} M={m} K={k} N={n}", parallelism=f"N-sharded x{world}",
                    gather=("none" if world == 1 else
                            "fused: GEMM epilogue TMA-stores each tile into every rank's symmetric-memory buffer, closed by "
                            "an in-kernel rendezvous" if mode == "fused" else
                            "fused stores closed by a one-thread rendezvous kernel" if mode == "fused_flag" else
                            "fused stores closed by an NCCL barrier" if mode == "fused_nccl_barrier" else
                            "NCCL all-gather of BF16 [M,N/G] blocks"),
                    row_chunks=plan.chunks, schedule=args.schedule,
                    parity="32 seeded rows of the whole result on every rank, bit for bit against the CPU checker, before timing",
                    l2="inputs larger than L2 (weights+activations+output per step exceed 126 MB); no flush"),
        roofline=roofline,
        e2e=dict(value=ops_total / (e2e_ms * 1e-3) / 1e12, unit="TOPS", h2d_bytes_per_step=x_host.numel() * 2,
                 d2h_bytes_per_step=out_host.numel() * 2, ms_per_step=e2e_ms, steps=e2e_steps,
                 note="per rank: the activations in, this rank's [M, N/G] block out (the whole result reaches the host once)"),
        gpu_launches=args.steps * (1 + plan.chunks + (1 if mode == 'fused_flag' else 0)), clocks=clocks.summary(), device_status=word.value,
    )
    if world > 1:
        bytes_in = plan.gather_bytes_received
        floor_ms = bytes_in / NVLINK_PEER_GBS / 1e6
        line["gather"] = dict(bytes_in_per_gpu=bytes_in, achieved_gbs=bytes_in / step_ms / 1e6, floor_ms=floor_ms,
                              floor_ms_nominal_900=bytes_in / 900.0 / 1e6, frac=floor_ms / step_ms,
                              gemm_only_ms=gemm_ms,
                              note=f"every GPU must receive (G-1)/G of the BF16 result; floor = bytes / {NVLINK_PEER_GBS:.0f} GB/s "
                                   "(measured peer copy per direction); achieved over the whole step")
        line["column_sharded"] = dict(ms_per_step=sharded_ms, value=ops_total / (sharded_ms * 1e-3) / 1e12, unit="TOPS",
                                      note="the same step without the gather: the result stays [M, N/G] per rank "
                                           "(ColumnShardedLinear mode='none'), what a row-parallel consumer takes")
    if world == 1:
        sample, _, _ = cpu_sample(spec)
        line["cpu_baseline"] = sample
        if not args.no_extra:
            line["other_configs"] = other_configs(ops, workloads, device, peaks)
    print(json.dumps(line), file=RESULT_STREAM, flush=True)


# DRAM bytes per launch of the dominant kernel from ncu captures (dram__bytes_read.sum and
# dram__bytes_write.sum) summarised under profiles/, each tagged with source_tag() of the kernel
# source it was taken from: a figure whose tag differs from the running kernel's is stale.
KERNEL_TRAFFIC = {
    "sharded": dict(read=651.2e6, write=1104.0e6, source="a0da5dbd8d8b", profile="profiles/gemm_i8_kernel_sharded_traffic.md"),
    "prefill_gate_up": dict(read=199.5e6, write=246.7e6, source="a0da5dbd8d8b", profile="profiles/gemm_i8_kernel_prefill_gate_up.md"),
    "prefill_down": dict(read=381.1e6, write=32.9e6, source="a0da5dbd8d8b", profile="profiles/gemm_i8_kernel_prefill_down.md"),
    # one rank's channel shard of the sharded workload, captured on one GPU (--shard-of G): its own reads and the
    # writes of its own block; run_ours adds the peers' blocks that arrive over NVLink
    "sharded/2": dict(read=368.9e6, write=532.6e6, source="a0da5dbd8d8b", profile="profiles/gemm_i8_kernel_sharded_traffic.md"),
    "sharded/4": dict(read=227.2e6, write=248.3e6, source="a0da5dbd8d8b", profile="profiles/gemm_i8_kernel_sharded_traffic.md"),
    "sharded/8": dict(read=152.7e6, write=104.9e6, source="a0da5dbd8d8b", profile="profiles/gemm_i8_kernel_sharded_traffic.md"),
}


class Timing(float):
    """Median milliseconds per launch, with the fastest and slowest replay attached."""

    lo: float
    hi: float


def _time_graph(fn, launches, replays=7):
    """The reference's method (benchmarks/microbench.py:15-38): warm up, capture `launches` calls in
    one CUDA graph, replay it seven times, report the median (with min and max)."""
    for _ in range(3):
        fn(0)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(launches):
            fn(i)
    times = []
    for _ in range(replays):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b) / launches)
    result = Timing(statistics.median(times))
    result.lo, result.hi = min(times), max(times)
    return result


def _spread_us(t):
    return [t.lo * 1e3, t.hi * 1e3]


def other_configs(ops, workloads, device, peaks):
    """The remaining benchmark configs, each timed as a CUDA graph of back-to-back launches over
    rotating input copies larger than L2 (the reference's method, benchmarks/microbench.py:15-38)."""
    results = {}
    hbm = peaks["hbm_gbs"]
    tensor_peak = 2.0 * peaks["bf16_tflops"]      # each graph replay lasts milliseconds: the burst figure applies
    gen = torch.Generator().manual_seed(0)
    # decode: rotate four weight copies (4 x 178 MB) so every launch streams from HBM
    n, k = 34816, 5120
    w, w_scale = workloads.weights(n, k, gen)
    copies = [w.to(device) for _ in range(4)]
    copies_u8 = [(w.to(torch.int16) + 128).to(torch.uint8).to(device) for _ in range(2)]
    sw = w_scale.to(device)
    # one set of buffers for every M (views of their first rows), so that the four cases do not differ in
    # where the allocator happened to place them
    x16 = workloads.activations(16, k, gen).to(device)
    codes16 = torch.empty(16, k, dtype=torch.int8, device=device)
    scales16 = torch.empty(16, device=device)
    out16 = torch.empty(16, n, dtype=torch.bfloat16, device=device)
    for m in (1, 4, 8, 16):
        x, codes, scales, out = x16[:m], codes16[:m], scales16[:m], out16[:m]
        ops.quantize_rows(x, codes, scales)
        nbytes = n * k + 2 * n + m * k + 4 * m + 2 * m * n
        ms = _time_graph(lambda i: ops.fused_channel_mm(codes, copies[i % 4], scales, sw, out, 0), 40)
        ms_u8 = _time_graph(lambda i: ops.channel_mm(codes, copies_u8[i % 2], scales, sw, out), 40)
        ms_q = _time_graph(lambda i: (ops.quantize_rows(x, codes, scales), ops.fused_channel_mm(codes, copies[i % 4], scales, sw, out, 0)), 40)
        ms_gemv = _time_graph(lambda i: ops.channel_gemv(x, copies[i % 4], sw, out), 20)
        # BF16 activations in, one kernel: the quantizer runs inside the streaming kernel
        ms_dyn = _time_graph(lambda i: ops.dynamic_channel_mm(x, copies[i % 4], sw, codes, scales, out), 40)
        dyn_bytes = n * k + 2 * n + 2 * m * k + 2 * m * n
        results[f"decode_m{m}"] = dict(us=ms * 1e3, us_min_max=_spread_us(ms), gbs=nbytes / ms / 1e6, frac_hbm=nbytes / ms / 1e6 / hbm,
                                       frac_nominal_8000=nbytes / ms / 1e6 / 8000.0,
                                       channel_mm_u8_us=ms_u8 * 1e3, with_quantize_us=ms_q * 1e3,
                                       dynamic_us=ms_dyn * 1e3, dynamic_gbs=dyn_bytes / ms_dyn / 1e6,
                                       dynamic_frac_hbm=dyn_bytes / ms_dyn / 1e6 / hbm,
                                       channel_gemv_us=ms_gemv * 1e3,
                                       channel_gemv_gbs=(n * k + 2 * n + 2 * m * k + 2 * m * n) / ms_gemv / 1e6,
                                       channel_gemv_frac_hbm=(n * k + 2 * n + 2 * m * k + 2 * m * n) / ms_gemv / 1e6 / hbm)
    # rows between decode and a full tile: the streaming kernel up to 64 rows, the 128-row GEMM tile beyond
    for m in (32, 64, 128):
        x = workloads.activations(m, k, gen).to(device)
        codes = torch.empty(m, k, dtype=torch.int8, device=device)
        scales = torch.empty(m, device=device)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        ops.quantize_rows(x, codes, scales)
        nbytes = n * k + 2 * n + m * k + 4 * m + 2 * m * n
        ms = _time_graph(lambda i: ops.fused_channel_mm(codes, copies[i % 4], scales, sw, out, 0), 40)
        results[f"small_prefill_m{m}"] = dict(us=ms * 1e3, gbs=nbytes / ms / 1e6, frac_hbm=nbytes / ms / 1e6 / hbm)
    del copies, copies_u8
    # decode on the down-projection shape (few channels, long K: the split-K cluster path)
    n2, k2 = 5120, 17408
    w2, w2_scale = workloads.weights(n2, k2, gen)
    copies2 = [w2.to(device) for _ in range(4)]
    sw2 = w2_scale.to(device)
    for m in (1, 16):
        x = workloads.activations(m, k2, gen).to(device)
        codes = torch.empty(m, k2, dtype=torch.int8, device=device)
        scales = torch.empty(m, device=device)
        out = torch.empty(m, n2, dtype=torch.bfloat16, device=device)
        ops.quantize_rows(x, codes, scales)
        nbytes = n2 * k2 + 2 * n2 + m * k2 + 4 * m + 2 * m * n2
        ms = _time_graph(lambda i: ops.fused_channel_mm(codes, copies2[i % 4], scales, sw2, out, 0), 40)
        results[f"decode_down_m{m}"] = dict(us=ms * 1e3, gbs=nbytes / ms / 1e6, frac_hbm=nbytes / ms / 1e6 / hbm)
    del copies2
    for name in ("prefill_gate_up", "prefill_down"):
        spec = WORKLOADS[name]
        m, n, k = spec["m"], spec["n"], spec["k"]
        w, w_scale = workloads.weights(n, k, gen)
        wd, sw = w.to(device), w_scale.to(device)
        x = workloads.activations(m, k, gen).to(device)
        codes = torch.empty(m, k, dtype=torch.int8, device=device)
        scales = torch.empty(m, device=device)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        ops.quantize_rows(x, codes, scales)
        ms = _time_graph(lambda i: ops.fused_channel_mm(codes, wd, scales, sw, out, 0), 20)
        # the same product from UINT8 code+128 weights (channel_mm) and with the INT32 accumulators
        # written out as well (cutlass_channel_mm)
        wu8 = (w.to(torch.int16) + 128).to(torch.uint8).to(device)
        ms_u8 = _time_graph(lambda i: ops.channel_mm(codes, wu8, scales, sw, out), 20)
        del wu8
        workspace = torch.empty(m, n, dtype=torch.int32, device=device)
        ms_ws = _time_graph(lambda i: ops.cutlass_channel_mm(codes, wd, scales, sw, workspace, out), 10)
        del workspace
        xs = [x.clone() for _ in range(4)]
        ms_q = _time_graph(lambda i: ops.quantize_rows(xs[i % 4], codes, scales), 40)
        tops = 2.0 * m * n * k / ms / 1e9
        results[name] = dict(gemm_ms=ms, gemm_ms_min_max=[ms.lo, ms.hi], tops=tops, frac_tensor=tops / tensor_peak,
                             frac_tensor_sustained=tops / (2.0 * peaks["bf16_tflops_sustained"]),
                             frac_nominal_4500=tops / 4500,
                             channel_mm_u8_ms=ms_u8, channel_mm_u8_tops=2.0 * m * n * k / ms_u8 / 1e9,
                             channel_mm_u8_vs_fused=ms_u8 / ms,
                             cutlass_channel_mm_ms=ms_ws, cutlass_channel_mm_tops=2.0 * m * n * k / ms_ws / 1e9,
                             quantize_us=ms_q * 1e3, quantize_us_min_max=_spread_us(ms_q),
                             quantize_gbs=(3 * m * k + 4 * m) / ms_q / 1e6,
                             quantize_frac_hbm=(3 * m * k + 4 * m) / ms_q / 1e6 / hbm)
        del wd, x, xs, out, codes
    # the SwiGLU + quantizer between the two prefill GEMMs: [4096, 2*17408] BF16 -> INT8 [4096, 17408]
    m, k = 4096, 17408
    gate_up = [(torch.randn(m, 2 * k, generator=gen) * 3).bfloat16().to(device) for _ in range(2)]
    codes = torch.empty(m, k, dtype=torch.int8, device=device)
    scales = torch.empty(m, device=device)
    ms = _time_graph(lambda i: ops.silu_mul_quantize(gate_up[i % 2], codes, scales), 20)
    results["silu_mul_quantize_4096x17408"] = dict(us=ms * 1e3, gbs=(5 * m * k + 4 * m) / ms / 1e6,
                                                   frac_hbm=(5 * m * k + 4 * m) / ms / 1e6 / hbm)
    del gate_up, codes
    # the gate/up GEMM with the SwiGLU in its epilogue, then the row quantizer on its [4096, 17408] output:
    # the fused replacement of prefill_gate_up + silu_mul_quantize
    from consumer_int8.quantization import interleave_gate_up
    m, n, k = 4096, 34816, 5120
    w, w_scale = workloads.weights(n, k, gen)
    wi, swi = interleave_gate_up(w.to(device), w_scale.to(device))
    x = workloads.activations(m, k, gen).to(device)
    codes = torch.empty(m, k, dtype=torch.int8, device=device)
    scales = torch.empty(m, device=device)
    ops.quantize_rows(x, codes, scales)
    hidden = torch.empty(m, n // 2, dtype=torch.bfloat16, device=device)
    codes2 = torch.empty(m, n // 2, dtype=torch.int8, device=device)
    scales2 = torch.empty(m, device=device)
    ms = _time_graph(lambda i: ops.gate_up_silu_mm(codes, wi, scales, swi, hidden), 20)
    hiddens = [hidden, hidden.clone(), hidden.clone()]   # rotate, as for the other HBM-bound timings
    ms_q = _time_graph(lambda i: ops.quantize_rows(hiddens[i % 3], codes2, scales2), 20)
    del hiddens
    results["gate_up_silu_mm_4096"] = dict(gemm_ms=ms, tops=2.0 * m * n * k / ms / 1e9, quantize_us=ms_q * 1e3)
    del wi, swi, x, codes, hidden, codes2
    spec = WORKLOADS["grouped"]
    m, n, groups = spec["m"], spec["n"], spec["groups"]
    inputs = workloads.grouped_inputs(m, n, groups, seed=0)
    xs = [inputs.x.to(device) for _ in range(2)]
    wd, sw = inputs.w.to(device), inputs.w_scale.to(device)
    codes = torch.empty(groups, m, 4096, dtype=torch.int8, device=device)
    scales = torch.empty(groups, m, device=device)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=device)
    ms_q = _time_graph(lambda i: ops.quantize_grouped4096(xs[i % 2], codes, scales), 20)
    ms_plain = _time_graph(lambda i: ops.grouped_channel_mm(codes, wd, scales, sw, out), 10)
    # with a lent workspace the tiles of the thin last wave are split along the groups (same bits)
    need = ops.grouped_workspace_bytes(m, n, groups)
    ms = ms_plain
    if need:
        workspace = torch.zeros(need, dtype=torch.uint8, device=device)
        ms_ws = _time_graph(lambda i: ops.grouped_channel_mm_ws(codes, wd, scales, sw, workspace, out), 10)
        ms = ms_ws if ms_ws < ms_plain else ms_plain
    tops = 2.0 * m * n * groups * 4096 / ms / 1e9
    results["grouped"] = dict(gemm_ms=ms, gemm_ms_min_max=[ms.lo, ms.hi], plain_ms=ms_plain,
                              with_workspace_ms=ms_ws if need else None, workspace_bytes=need,
                              tops=tops, frac_tensor=tops / tensor_peak,
                              frac_tensor_sustained=tops / (2.0 * peaks["bf16_tflops_sustained"]), frac_nominal_4500=tops / 4500,
                              quantize_us=ms_q * 1e3, quantize_us_min_max=_spread_us(ms_q),
                              quantize_gbs=(3 * m * groups * 4096 + 4 * m * groups) / ms_q / 1e6,
                              quantize_frac_hbm=(3 * m * groups * 4096 + 4 * m * groups) / ms_q / 1e6 / hbm)
    del xs, wd, codes, out
    # block-32 (Q8_0) W8A8 through the C ABI, at the shapes of the reference's benchmark
    # (benchmarks/benchmark_q8_block_int8.py:44: n=1024, k=4096); quantizer + product per call
    import ctypes
    n, k = 1024, 4096
    w = torch.randint(-128, 128, (n, k), dtype=torch.int8, generator=gen).to(device)
    sw = (torch.randn(n, k // 32, generator=gen) * 0.01).half().to(device)
    for m in (16, 4096):
        x = (torch.randn(m, k, generator=gen) * 0.1).bfloat16().to(device)
        a = torch.empty(m, k, dtype=torch.int8, device=device)
        sa = torch.empty(m, k // 32, device=device)
        y = torch.empty(m, n, dtype=torch.bfloat16, device=device)

        def q8(_i, x=x, a=a, sa=sa, y=y, m=m):
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            rc = ops.libci8.ci8_q8_block_mm(*(ctypes.c_void_p(t.data_ptr()) for t in (x, a, sa, w, sw, y)), m, n, k, stream)
            assert rc == 0, rc

        ms = _time_graph(q8, 10)
        results[f"q8_block_m{m}"] = dict(us=ms * 1e3, tops=2.0 * m * n * k / ms / 1e9)
    return results


def profile_only(args, spec):
    """A few launches of one workload's kernels on cuda:0, nothing timed: the command line that
    ncu captures are taken from (weights rotate over copies larger than L2 for the decode case)."""
    from consumer_int8 import ops, workloads

    device = torch.device("cuda", 0)
    m, n, k = spec["m"], spec["n"], spec["k"]
    n //= args.shard_of       # one rank's channel shard of the workload, run on this one GPU
    if args.workload == "q8_block":
        import ctypes
        gen = torch.Generator().manual_seed(0)
        w = torch.randint(-128, 128, (n, k), dtype=torch.int8, generator=gen).to(device)
        sw = (torch.randn(n, k // 32, generator=gen) * 0.01).half().to(device)
        x = (torch.randn(m, k, generator=gen) * 0.1).bfloat16().to(device)
        a = torch.empty(m, k, dtype=torch.int8, device=device)
        sa = torch.empty(m, k // 32, device=device)
        y = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        for _ in range(args.steps):
            rc = ops.libci8.ci8_q8_block_mm(*(ctypes.c_void_p(t.data_ptr()) for t in (x, a, sa, w, sw, y)), m, n, k, stream)
            assert rc == 0, rc
    elif args.workload == "grouped":
        inputs = workloads.grouped_inputs(m, n, spec["groups"], seed=0)
        x, w, sw = inputs.x.to(device), inputs.w.to(device), inputs.w_scale.to(device)
        codes = torch.empty(spec["groups"], m, 4096, dtype=torch.int8, device=device)
        scales = torch.empty(spec["groups"], m, device=device)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        workspace = torch.zeros(max(ops.grouped_workspace_bytes(m, n, spec["groups"]), 16), dtype=torch.uint8, device=device)
        for _ in range(args.steps):
            ops.quantize_grouped4096(x, codes, scales)
            ops.grouped_channel_mm_ws(codes, w, scales, sw, workspace, out)
    else:
        inputs = workloads.linear_inputs(m, n, k, seed=0)
        x, sw = inputs.x.to(device), inputs.w_scale.to(device)
        decode = args.workload in ("decode", "decode_m8")
        copies = [inputs.w.to(device) for _ in range(3 if decode else 1)]
        codes = torch.empty(m, k, dtype=torch.int8, device=device)
        scales = torch.empty(m, device=device)
        out = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        for i in range(args.steps):
            ops.quantize_rows(x, codes, scales)
            ops.fused_channel_mm(codes, copies[i % len(copies)], scales, sw, out, args.schedule)
            if decode:
                ops.channel_gemv(x, copies[i % len(copies)], sw, out)
                ops.dynamic_channel_mm(x, copies[i % len(copies)], sw, codes, scales, out)
    torch.cuda.synchronize()
    print(json.dumps(dict(profile_only=args.workload, launches=args.steps)), file=RESULT_STREAM, flush=True)


def _claim_stdout():
    """Keeps stdout for the one JSON line: everything else that writes to file descriptor 1 (a library's
    version banner, for one) goes to stderr. Returns a file object on the original stdout."""
    sys.stdout.flush()
    kept = os.dup(1)
    os.dup2(2, 1)
    return os.fdopen(kept, "w")


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--workload", choices=list(WORKLOADS), default="sharded")
    parser.add_argument("--profile-only", action="store_true",
                        help="run --steps launches of the workload's kernels with no timing (for ncu captures)")
    parser.add_argument("--shard-of", type=int, default=1, choices=[1, 2, 4, 8],
                        help="--profile-only: run one rank's N/G channel shard of the workload (for DRAM-traffic captures "
                             "of the per-GPU GEMM of the sharded runs)")
    parser.add_argument("--schedule", type=int, default=0)
    parser.add_argument("--gather", choices=["fused", "fused_flag", "fused_nccl_barrier", "nccl"], default="fused",
                        help="N>1: peer stores from the GEMM epilogue (closed inside the kernel, or by an NCCL "
                             "barrier), or a separate NCCL all-gather")
    parser.add_argument("--chunks", type=int, default=4,
                        help="--gather nccl: row chunks whose gather overlaps the next GEMM")
    parser.add_argument("--no-extra", action="store_true", help="skip the other benchmark configs")
    args = parser.parse_args()
    spec = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    global RESULT_STREAM
    RESULT_STREAM = _claim_stdout()
    if args.impl == "reference":
        run_reference(args, spec, rank)
        return
    if args.profile_only:
        profile_only(args, spec)
        return
    if args.workload in ("decode", "decode_m8", "grouped", "q8_block"):
        raise SystemExit("the decode, grouped and q8_block workloads are timed inside the default run (other_configs) "
                         "or launched with --profile-only")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"     # keep NCCL's version banner off stdout (one JSON line)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, spec, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
