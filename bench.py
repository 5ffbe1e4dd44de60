#!/usr/bin/env python
"""Benchmark of the attention-and-linear hot path.

``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line for the headline metric: achieved HBM
GB/s of the paged-KV decode attention (config 2: 32 sequences with context lengths uniform in [128, 4096],
32 query / 8 KV heads, head_dim 128, 16-token pages, bf16).  A "step" is one decode call over the whole batch.

  * ``value``     device-resident: inputs already in HBM, K calls timed with CUDA events on the launching stream.
  * ``e2e``       the same call through the host-facing API with HOST buffers: the step's query, lengths and
                  block table are copied from pinned host memory and the output is copied back inside the
                  timed region (the KV cache itself is device state of the operator, as in the reference,
                  whose operators take device buffers).
  * ``roofline``  algorithmic bytes per launch / average launch duration against the measured HBM peak.
  * ``cpu_baseline`` the CPU restatement of the reference kernel timed on this host (rank 0, N=1 only).
  * ``also``      secondary figures of the same metric family (prefill TFLOP/s, GEMM TFLOP/s, cache-write GB/s).

With N > 1 (launched by torchrun, one rank per GPU) every rank decodes its own batch of the same shape
(different seed): sequences are independent, so there is no data-path collective and scaling is weak.
``--impl reference`` times the reference's own CPU algorithm (the restatement under oracle/) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "paged_decode_hbm_gbs"
UNIT = "GB/s"
WORKLOAD = ("config2 paged-decode bf16: 32 seqs, ctx U[128,4096] seed 1, 32Q/8KV heads, head_dim 128, "
            "block 16, pool +10%, permuted block table")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            data = json.load(handle)
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None

    def _run(self):
        nv = self._nvml
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": int(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def dist_setup(gpus: int):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = dist
    return rank, local, world, group


def barrier_sync(group):
    import torch

    if group is not None:
        group.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, group) -> float:
    import torch

    if group is None:
        return value
    tensor = torch.tensor([value], dtype=torch.float64, device="cuda")
    group.all_reduce(tensor, op=group.ReduceOp.MAX)
    return float(tensor.item())


def sum_over_ranks(value: float, group) -> float:
    import torch

    if group is None:
        return value
    tensor = torch.tensor([value], dtype=torch.float64, device="cuda")
    group.all_reduce(tensor, op=group.ReduceOp.SUM)
    return float(tensor.item())


# ----------------------------------------------------------------------------------------------------------
# headline: config 2 paged decode
# ----------------------------------------------------------------------------------------------------------

# DRAM bytes one launch of paged_decode_kernel moves on the config-2 workload (seed 1), from an ncu capture of this
# very command (dram__bytes_read.sum + dram__bytes_write.sum): 277.49 MB read + 7.69 MB written (split-K partials, output).
DECODE_DRAM_TRAFFIC = 285_181_184


def decode_device_inputs(case, seed: int):
    import torch

    generator = torch.Generator(device="cuda").manual_seed(seed)
    shape = (case.physical_blocks, case.block_size, case.kv_heads, case.head_dim)
    key_cache = torch.randn(shape, generator=generator, device="cuda").to(torch.bfloat16)
    value_cache = torch.randn(shape, generator=generator, device="cuda").to(torch.bfloat16)
    query = torch.randn((case.batch, case.heads, case.head_dim), generator=generator, device="cuda").to(torch.bfloat16)
    return query, key_cache, value_cache


def run_decode(args, rank, world, group):
    import torch

    from singe_b200 import ops, workloads

    # Weak scaling: every rank serves its own batch of config 2's shape - the same 32 context lengths and block
    # table (seed 1), its own K/V/Q values - so the work per GPU is fixed as N grows.
    case = workloads.paged_decode_case(seed=1)
    first_query, key_cache, value_cache = decode_device_inputs(case, seed=1 + rank)
    # The step's inputs (query, block table, lengths) live in ONE device allocation, so the end-to-end step uploads
    # them with a single copy from one pinned host buffer.
    host_table_array = case.block_table.view(np.int32)
    sizes = [first_query.numel() * 2, host_table_array.size * 4, case.lens.size * 4]
    starts = [0, sizes[0], sizes[0] + sizes[1]]
    assert all(start % 16 == 0 for start in starts)
    step_inputs = torch.empty(sum(sizes), dtype=torch.uint8, device="cuda")
    query = step_inputs[starts[0]:starts[1]].view(torch.bfloat16).view(first_query.shape)
    table = step_inputs[starts[1]:starts[2]].view(torch.int32).view(host_table_array.shape)
    lens = step_inputs[starts[2]:].view(torch.int32)
    query.copy_(first_query)
    table.copy_(torch.from_numpy(host_table_array))
    lens.copy_(torch.from_numpy(case.lens))
    out = torch.empty_like(query)
    config = ops.PagedKvDecodeAttentionConfig.contiguous(case.batch, case.heads, case.kv_heads, case.head_dim,
                                                         case.block_size, case.physical_blocks,
                                                         case.block_table_batch_stride, case.scale)
    stream = torch.cuda.current_stream()

    def step(on=None):
        ops.paged_kv_decode_attention(out, query, key_cache, value_cache, lens, table, config, stream=on or stream)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier_sync(group)

    # ---- device-resident region: exactly K steps, enqueued as one CUDA graph (a step is 61 us of kernels, less
    # than the host needs to issue two launches), CUDA events on the launching stream ----
    side = torch.cuda.Stream()
    side.wait_stream(stream)
    steps_graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(steps_graph, stream=side):
            for _ in range(args.steps):
                step(side)
    torch.cuda.synchronize()
    probe_start, probe_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps_graph.replay()  # untimed: the replay path itself warms up
    probe_start.record(stream)
    steps_graph.replay()
    probe_stop.record(stream)
    torch.cuda.synchronize()
    # The K-step graph is replayed back to back until the timed region is at least 50 ms long (K steps alone are
    # about a millisecond, too short for the clock sampler to see), and the time is divided by the replays.
    replays = max(1, int(math.ceil(50.0 / max(probe_start.elapsed_time(probe_stop), 1e-3))))
    replays = int(max_over_ranks(float(replays), group))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(torch.cuda.current_device())
    with sampler:
        barrier_sync(group)
        start.record(stream)
        for _ in range(replays):
            steps_graph.replay()
        stop.record(stream)
        barrier_sync(group)
    seconds = max_over_ranks(start.elapsed_time(stop) * 1e-3 / replays, group)
    my_bytes = float(case.algorithmic_bytes())
    total_bytes = sum_over_ranks(my_bytes, group)
    value = total_bytes * args.steps / seconds / 1e9

    # ---- spread: five more replays of the same graph, each timed on its own (median and p10-p90, as the
    # reference's Benches report, singe-testing/src/bench.rs:12-40) ----
    repeats = []
    for _ in range(5):
        again_start, again_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        again_start.record(stream)
        steps_graph.replay()
        again_stop.record(stream)
        torch.cuda.synchronize()
        repeats.append(again_start.elapsed_time(again_stop) / args.steps)
    spread = {"median": round(float(np.median(repeats)), 5), "p10": round(float(np.percentile(repeats, 10)), 5),
              "p90": round(float(np.percentile(repeats, 90)), 5), "replays": len(repeats)}

    # ---- the same K steps launched one by one from the host, for comparison ----
    eager_start, eager_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    eager_start.record(stream)
    for _ in range(args.steps):
        step()
    eager_stop.record(stream)
    torch.cuda.synchronize()
    eager_seconds = eager_start.elapsed_time(eager_stop) * 1e-3

    # ---- kernel duration for the roofline: this rank's own K launches inside the timed region (the step's two
    # kernels back to back; the small combine kernel is counted against the decode kernel) ----
    launch_seconds = start.elapsed_time(stop) * 1e-3 / replays / args.steps
    peaks = measured_peaks()
    achieved = my_bytes / launch_seconds / 1e9

    # ---- end to end through the host-facing call: pinned host inputs in, result out, every step ----
    host_inputs = step_inputs.cpu().pin_memory()
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = host_inputs.numel()
    d2h = host_out.numel() * 2

    # One step = copies in, the decode call, copy out: captured once, replayed and waited for every step.
    e2e_graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(e2e_graph, stream=side):
            step_inputs.copy_(host_inputs, non_blocking=True)
            step(side)
            host_out.copy_(out, non_blocking=True)
    torch.cuda.synchronize()

    def e2e_step():
        e2e_graph.replay()
        torch.cuda.current_stream().synchronize()  # the caller reads the result before the next step

    for _ in range(3):
        e2e_step()
    barrier_sync(group)
    begin = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier_sync(group)
    e2e_seconds = max_over_ranks(time.perf_counter() - begin, group)
    e2e_value = total_bytes * args.steps / e2e_seconds / 1e9

    # ---- the same end-to-end step with two steps in flight: while step i runs, step i + 1's inputs cross PCIe and the
    # host reads step i - 1's result.  Every step still uploads its inputs from pinned host memory and has its result
    # read back inside the timed region; only the waiting is one step behind.  All decode calls go through one stream
    # (the entry point's workspace is shared by the device's streams); the copies have streams of their own.
    in_stream, out_stream = torch.cuda.Stream(), torch.cuda.Stream()
    slots = []
    for _ in range(2):
        device_inputs = torch.empty_like(step_inputs)
        slots.append({
            "inputs": device_inputs,
            "query": device_inputs[starts[0]:starts[1]].view(torch.bfloat16).view(first_query.shape),
            "table": device_inputs[starts[1]:starts[2]].view(torch.int32).view(host_table_array.shape),
            "lens": device_inputs[starts[2]:].view(torch.int32),
            "out": torch.empty_like(out),
            "host_in": host_inputs.clone().pin_memory(),
            "host_out": torch.empty(out.shape, dtype=out.dtype).pin_memory(),
            "uploaded": torch.cuda.Event(), "computed": torch.cuda.Event(), "read": torch.cuda.Event(),
        })

    def pipelined_step(index):
        slot = slots[index % 2]
        if index >= 2:
            slot["read"].synchronize()  # the caller has the result of the step that used this slot before
        with torch.cuda.stream(in_stream):
            slot["inputs"].copy_(slot["host_in"], non_blocking=True)
            slot["uploaded"].record(in_stream)
        side.wait_event(slot["uploaded"])
        ops.paged_kv_decode_attention(slot["out"], slot["query"], key_cache, value_cache, slot["lens"], slot["table"],
                                      config, stream=side)
        slot["computed"].record(side)
        out_stream.wait_event(slot["computed"])
        with torch.cuda.stream(out_stream):
            slot["host_out"].copy_(slot["out"], non_blocking=True)
            slot["read"].record(out_stream)

    def pipelined_run(count):
        for index in range(count):
            pipelined_step(index)
        for slot in slots:
            slot["read"].synchronize()

    pipelined_run(4)
    torch.cuda.synchronize()
    if not torch.equal(slots[0]["host_out"], host_out) or not torch.equal(slots[1]["host_out"], host_out):
        raise RuntimeError("the pipelined end-to-end step differs from the step-by-step one")
    barrier_sync(group)
    begin = time.perf_counter()
    pipelined_run(args.steps)
    barrier_sync(group)
    pipelined_seconds = max_over_ranks(time.perf_counter() - begin, group)
    pipelined_value = total_bytes * args.steps / pipelined_seconds / 1e9

    if ops.take_device_error() != 0:
        raise RuntimeError("a device-side bounded wait ran out during the benchmark")

    line = {
        "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(seconds / args.steps * 1e3, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sequences_per_gpu": case.batch, "tokens_per_gpu": case.total_tokens,
                   "algorithmic_bytes_per_step_per_gpu": int(my_bytes), "l2": "inputs (277 MB) larger than L2",
                   "launch_mode": "the K timed steps are one CUDA graph; e2e issues each step from the host "
                                  "(one_step_at_a_time replays a one-step graph and waits for it)",
                   "timed_replays": replays,
                   "eager_ms_per_step": round(eager_seconds / args.steps * 1e3, 5),
                   "repeat_ms_per_step": spread,
                   "sharding": "by sequence, no collective"},
        "e2e": {"value": round(pipelined_value, 1), "unit": UNIT, "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h),
                "mode": "two steps in flight: every step uploads its inputs from pinned host memory, runs the decode "
                        "call and has its result read back; the host waits for a step's result one step later",
                "one_step_at_a_time": round(e2e_value, 1)},
        "gpu_launches": 2 * args.steps * replays,
        "clocks": sampler.summary(),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peaks["hbm_gbs"], 4), "traffic": DECODE_DRAM_TRAFFIC,
                     "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum of "
                                     "paged_decode_kernel on this workload)",
                     "algorithmic_bytes": int(my_bytes),
                     "peak_source": peaks["source"], "launch_us": round(launch_seconds * 1e6, 2),
                     "kernels": "paged_decode_kernel + decode_combine_kernel"},
    }
    return line, case


def cpu_baseline_decode(case, threads: int):
    """Times the CPU restatement of paged_kv_decode_attention_f32 on the full config-2 batch."""
    from oracle import oracle
    from singe_b200 import workloads

    rng = np.random.default_rng(1)
    q = workloads.normal_bf16(rng, (case.batch, case.heads, case.head_dim))
    shape = (case.physical_blocks, case.block_size, case.kv_heads, case.head_dim)
    k = workloads.normal_bf16(rng, shape)
    v = workloads.normal_bf16(rng, shape)
    oracle.set_threads(threads)
    best = float("inf")
    for _ in range(2):
        begin = time.perf_counter()
        oracle.paged_kv_decode_attention_f32(q, k, v, case.lens, case.block_table, batch=case.batch,
                                             heads=case.heads, kv_heads=case.kv_heads, head_dim=case.head_dim,
                                             block_size=case.block_size,
                                             block_table_batch_stride=case.block_table_batch_stride, scale=case.scale)
        best = min(best, time.perf_counter() - begin)
    return case.algorithmic_bytes() / best / 1e9, best


def run_reference(args):
    """The reference's CPU implementation of the path (restated under oracle/) on all host cores."""
    from oracle import oracle
    from singe_b200 import workloads

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    case = workloads.paged_decode_case(seed=1)
    # every core this process may run on (torchrun exports OMP_NUM_THREADS=1 to its ranks, which would otherwise
    # leave the reference on one thread)
    threads = max(oracle.max_threads(), len(os.sched_getaffinity(0)))
    rng = np.random.default_rng(1)
    q = workloads.normal_bf16(rng, (case.batch, case.heads, case.head_dim))
    shape = (case.physical_blocks, case.block_size, case.kv_heads, case.head_dim)
    k = workloads.normal_bf16(rng, shape)
    v = workloads.normal_bf16(rng, shape)
    oracle.set_threads(threads)

    def step():
        oracle.paged_kv_decode_attention_f32(q, k, v, case.lens, case.block_table, batch=case.batch,
                                             heads=case.heads, kv_heads=case.kv_heads, head_dim=case.head_dim,
                                             block_size=case.block_size,
                                             block_table_batch_stride=case.block_table_batch_stride, scale=case.scale)

    # one step = the whole config-2 batch (about 0.1 s on 16 threads): the run stays within minutes at any --steps
    # the driver uses; beyond 200 steps it is cut short and the line says so
    warmup = args.warmup
    steps = min(args.steps, 200)
    for _ in range(warmup):
        step()
    begin = time.perf_counter()
    for _ in range(steps):
        step()
    seconds = time.perf_counter() - begin
    value = case.algorithmic_bytes() * steps / seconds / 1e9
    world = int(os.environ.get("WORLD_SIZE", "1"))
    sample = f"full config-2 batch ({case.total_tokens} cached tokens), {steps} calls"
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": UNIT, "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": round(seconds / steps * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": round(value, 3), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def decode_step_parity(rank, world, group, collective: str):
    """Correctness of the tensor-parallel step on this very box, before anything is timed: two Llama-3-8B-wide layers,
    64 sequences at context 512, the same weights, cache contents and tokens everywhere.  The step with the fused
    peer-memory collective must agree with the step over NCCL's all-reduce, every rank must pick the same next tokens,
    and the gathered logits must agree with the same two layers run unsharded on rank 0."""
    import torch

    from singe_b200 import llama

    config = llama.LlamaConfig(layers=2)
    sequences, context = 64, 512
    weights = llama.random_weights(config, seed=11)          # same seed, same values on every rank
    shard = llama.Shard(rank, world, group)
    sharded = {kind: llama.LlamaDecoder(config, sequences, context + 16, shard=shard, weights=weights,
                                        collective=kind) for kind in (collective, "nccl")}
    whole = llama.LlamaDecoder(config, sequences, context + 16, weights=weights) if rank == 0 else None
    generator = torch.Generator(device="cuda").manual_seed(12)
    pages = sharded["nccl"].table.page_count()
    g = config.kv_heads // world
    for layer in range(config.layers):
        for which in ("key_caches", "value_caches"):
            full = torch.randn((pages, config.page_size, config.kv_heads, config.head_dim), generator=generator,
                               device="cuda").to(torch.bfloat16)
            for decoder in sharded.values():
                getattr(decoder, which)[layer].copy_(full[:, :, rank * g:(rank + 1) * g])
            if whole is not None:
                getattr(whole, which)[layer].copy_(full)
    tokens = np.random.default_rng(13).integers(0, config.vocab, size=sequences)
    outcome = {}
    logits = {}
    for kind, decoder in list(sharded.items()) + ([("whole", whole)] if whole is not None else []):
        decoder.table.place_prompts([context] * sequences)
        decoder._refresh_block_table()
        picked = decoder.step(tokens)
        torch.cuda.synchronize()
        logits[kind] = decoder.logits.float()
        outcome[kind] = picked.clone()
        if int(decoder.status.item()) != 0:
            raise RuntimeError(f"decode step ({kind}): status word {int(decoder.status.item())}")
    ours, nccl = logits[collective], logits["nccl"]
    # Two bf16 layer stacks that round partial sums in different places drift apart by a little noise on every one of
    # the 8 M logits (their standard deviation is about 1.3 here): the bound on a single logit leaves room for the
    # tail of that noise; the root-mean-square error (about 1 % of the logits' own rms, measured) must stay under 3 %.
    # A wrong sum -- a rank's partial rows missing or doubled -- is an error of order 1 on both counts.
    tolerance = lambda expect: 1e-1 + 2e-2 * expect.abs()
    relative_rms = lambda got, expect: float(((got - expect).pow(2).mean() / expect.pow(2).mean()).sqrt())
    problems = []
    versus_nccl = float((ours - nccl).abs().max())
    if not bool(((ours - nccl).abs() <= tolerance(nccl)).all()) or relative_rms(ours, nccl) > 3e-2:
        problems.append(f"logits differ from the NCCL step by {versus_nccl:.3e}")
    everyone = [torch.empty_like(outcome[collective]) for _ in range(world)]
    group.all_gather(everyone, outcome[collective])
    if any(not torch.equal(everyone[0], other) for other in everyone[1:]):
        problems.append("ranks picked different next tokens")
    gathered = [torch.empty_like(sharded[collective].logits) for _ in range(world)]
    group.all_gather(gathered, sharded[collective].logits)
    versus_whole = rms_whole = None
    if rank == 0:
        full_logits = torch.cat(gathered, dim=1).float() if sharded[collective].shard_lm_head else gathered[0].float()
        expect = logits["whole"]
        versus_whole = float((full_logits - expect).abs().max())
        rms_whole = relative_rms(full_logits, expect)
        if not bool(((full_logits - expect).abs() <= tolerance(expect)).all()) or rms_whole > 3e-2:
            problems.append(f"logits differ from the unsharded step by {versus_whole:.3e} (relative rms {rms_whole:.2e})")
        top = torch.sort(expect, dim=1).values[:, -2:]
        clear = (top[:, 1] - top[:, 0]) > 0.1
        if not torch.equal(outcome[collective][clear], expect.argmax(dim=1)[clear]):
            problems.append("next tokens differ from the unsharded step")
    for decoder in sharded.values():
        decoder.close()
    del sharded, whole, weights
    torch.cuda.empty_cache()
    flag = torch.tensor([len(problems)], dtype=torch.int32, device="cuda")
    group.all_reduce(flag)
    return {"tp_parity": "ok" if int(flag.item()) == 0 else "FAILED: " + "; ".join(problems or ["on another rank"]),
            "max_abs_vs_nccl_step": round(versus_nccl, 5),
            "max_abs_vs_unsharded_step": None if versus_whole is None else round(versus_whole, 5),
            "relative_rms_vs_unsharded_step": None if rms_whole is None else round(rms_whole, 6),
            "checked": "2 layers of the Llama-3-8B shape, 64 sequences x 512 context, same weights/cache/tokens on "
                       "every rank: fused collective vs NCCL all-reduce, every rank's next tokens, gathered logits "
                       "vs the unsharded step on rank 0"}


def run_decode_step(rank, world, group, steps: int = 20, warmup: int = 3, collective: str = "peer"):
    """Config 5: Llama-3-8B-shaped decode step, 64 sequences at context 2048, tensor-parallel over all ranks
    (KV heads and column/row-sharded linears, all-reduce after o_proj and down_proj).  Returns rank 0's figures."""
    import torch

    from singe_b200 import llama

    parity = None
    if world > 1:
        try:
            parity = decode_step_parity(rank, world, group, collective)
        except Exception as error:
            parity = {"tp_parity": "FAILED: " + repr(error)}
        if parity["tp_parity"] != "ok":
            return {"error": "the tensor-parallel step is wrong on this box, so it is not timed", **parity}
    config = llama.LlamaConfig()
    sequences, context = 64, 2048
    shard = llama.Shard(rank, world, group)
    decoder = llama.LlamaDecoder(config, sequences, context + 64, shard=shard, seed=4, collective=collective)
    decoder.fill_context(context, seed=4)
    rng = np.random.default_rng(4)
    tokens = rng.integers(0, config.vocab, size=sequences)
    decoder.plan(tokens)
    decoder.capture()
    for _ in range(warmup):
        decoder.graph.replay()
    barrier_sync(group)
    stream = torch.cuda.current_stream()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record(stream)
    for _ in range(steps):
        decoder.graph.replay()   # same positions every replay: the step's work does not depend on the token ids
    end.record(stream)
    barrier_sync(group)
    seconds = max_over_ranks(begin.elapsed_time(end) * 1e-3 / steps, group)
    # end to end: plan on the host, upload the step's index tensors, replay, read the next tokens back
    host_tokens = tokens
    barrier_sync(group)
    wall = time.perf_counter()
    e2e_steps = min(steps, 16)
    for _ in range(e2e_steps):
        next_tokens = decoder.step(host_tokens)
        host_tokens = next_tokens.cpu().numpy() % config.vocab
    barrier_sync(group)
    e2e_seconds = max_over_ranks((time.perf_counter() - wall) / e2e_steps, group)
    moved = llama.decode_step_bytes(config, sequences, context, world, decoder.shard_lm_head)
    peaks = measured_peaks()
    status = int(decoder.status.item())
    prompt = None
    if world == 1:
        # A prompt step through the same decoder: every sequence reads a prompt of 60 - 480 tokens (14 400 tokens in
        # all) in one step -- embedding, the linears at M = 14 400, rotary + cache write, the packed prefill kernel
        # over the paged cache, last-row logits.  Timed on its second run (the first allocates the step's buffers).
        lengths = [480, 240, 120, 60] * (sequences // 4)
        prompts = [rng.integers(0, config.vocab, size=n).tolist() for n in lengths]
        elapsed = None
        for _ in range(2):
            decoder.table.reset()
            torch.cuda.synchronize()
            begin = time.perf_counter()
            decoder.step_tokens(prompts)
            torch.cuda.synchronize()
            elapsed = time.perf_counter() - begin
        total = sum(lengths)
        linear_weights = config.layers * (config.hidden * (config.heads + 2 * config.kv_heads) * config.head_dim
                                          + config.heads * config.head_dim * config.hidden
                                          + 3 * config.hidden * config.ffn)
        flops = 2.0 * total * linear_weights
        prompt = {"tokens": total, "sequences": sequences, "ms": round(elapsed * 1e3, 2),
                  "tokens_per_s": round(total / elapsed, 1),
                  "linear_tflops": round(flops / elapsed / 1e12, 1),
                  "frac_of_bf16_peak": round(flops / elapsed / 1e12 / peaks["bf16_tflops_sustained"], 4),
                  "peak": "sustained cuBLAS figure (a step of 150 ms under the power cap)",
                  "status_word": int(decoder.status.item()),
                  "timing": "host wall clock around one eager step, including its buffer allocations"}
    decoder.close()
    how = "none (one GPU)"
    if world > 1:
        how = {"oneshot": "one kernel per collective: every rank reads all ranks' partial rows from peer memory, then "
                          "residual add + RMSNorm",
               "twophase": "one kernel per collective: partial rows pushed to the rank that owns them, summed there, "
                           "residual add + RMSNorm, normalised rows pushed to every rank",
               "pushall": "one kernel per collective: every partial row pushed to every rank, summed there, residual "
                          "add + RMSNorm",
               "nccl": "NCCL all-reduce, then the add + RMSNorm kernel"}[decoder.collective]
    figures = dict(parity or {})
    figures.update({
        "collective": how,
        "tokens_per_s": round(sequences / seconds, 1), "ms_per_step": round(seconds * 1e3, 3),
        "e2e_tokens_per_s": round(sequences / e2e_seconds, 1), "tp": world,
        "bytes_per_rank_per_step": moved["total"],
        "frac_of_hbm_bound_per_rank": round(moved["total"] / seconds / 1e9 / peaks["hbm_gbs"], 4),
        "lm_head": "vocab-sharded + (max, argmax) gather" if decoder.shard_lm_head else "replicated",
        "collectives_per_step": 2 * config.layers if world > 1 else 0, "status_word": status,
        "config": "Llama-3-8B shape, random bf16 weights, 64 seqs x ctx 2048, page 16, CUDA-graph replay",
    })
    if prompt is not None:
        figures["prompt_step"] = prompt
    return figures


def run_only(args):
    """Launches one kernel of the path `--steps` times after `--warmup` launches and exits: the small, bounded
    command the ncu captures of this repository are taken from."""
    import torch

    from singe_b200 import llama, ops, workloads

    kind, _, detail = args.only.partition(":")
    if kind == "decode":
        case = workloads.paged_decode_case(seed=1)
        query, key_cache, value_cache = decode_device_inputs(case, seed=1)
        lens = torch.from_numpy(case.lens).cuda()
        table = torch.from_numpy(case.block_table.view(np.int32)).cuda()
        out = torch.empty_like(query)
        config = ops.PagedKvDecodeAttentionConfig.contiguous(case.batch, case.heads, case.kv_heads, case.head_dim,
                                                             case.block_size, case.physical_blocks,
                                                             case.block_table_batch_stride, case.scale)
        call = lambda: ops.paged_kv_decode_attention(out, query, key_cache, value_cache, lens, table, config)
    elif kind == "paged_attention":
        import bench_extra

        call, _, _ = bench_extra.paged_attention_call()
    elif kind == "gemm":
        m, n, k = (int(v) for v in detail.split(","))
        x = torch.randn((m, k), device="cuda").to(torch.bfloat16)
        w = (torch.randn((n, k), device="cuda") * 0.02).to(torch.bfloat16)
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        call = lambda: ops.linear(x, w, y)
    elif kind in ("prefill", "kvwrite"):
        lens = tuple(int(v) for v in detail.split(",")) if detail else (8192, 4096, 2048, 1024)
        case = workloads.prefill_case(lens=lens)
        total = case.total_tokens
        q = torch.randn((total, case.heads, case.head_dim), device="cuda").to(torch.bfloat16)
        k = torch.randn((total, case.kv_heads, case.head_dim), device="cuda").to(torch.bfloat16)
        v = torch.randn((total, case.kv_heads, case.head_dim), device="cuda").to(torch.bfloat16)
        out = torch.empty_like(q)
        lse = torch.empty((total, case.heads), dtype=torch.float32, device="cuda")
        d_lens = torch.from_numpy(case.lens).cuda()
        d_offsets = torch.from_numpy(case.offsets).cuda()
        shape = (case.pages, case.page_size, case.kv_heads, case.head_dim)
        key_cache = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
        value_cache = torch.zeros(shape, dtype=torch.bfloat16, device="cuda")
        pages = torch.from_numpy(case.write_pages).cuda()
        slots = torch.from_numpy(case.write_slots).cuda()
        config = ops.RaggedKvPrefillAttentionConfig(len(lens), total, total, case.heads, case.kv_heads, case.head_dim,
                                                    True, case.scale)
        if kind == "prefill":
            call = lambda: ops.ragged_kv_prefill_attention(out, lse, q, k, v, d_lens, d_lens, d_offsets, config)
        else:
            call = lambda: ops.kv_cache_write(key_cache, value_cache, k, v, pages, slots)
    elif kind == "step":
        # step:LAYERS[:TP] - with TP > 1 one GPU runs the shapes of one rank of a TP-way split (no collective)
        layers, _, tp = (detail or "4").partition(":")
        tp = int(tp or 1)
        full = llama.LlamaConfig()
        config = llama.LlamaConfig(layers=int(layers), heads=full.heads // tp, kv_heads=full.kv_heads // tp,
                                   ffn=full.ffn // tp, vocab=full.vocab // tp)
        decoder = llama.LlamaDecoder(config, 64, 2048 + 64)
        decoder.fill_context(2048)
        decoder.plan(np.random.default_rng(4).integers(0, config.vocab, size=64))
        call = decoder.forward
    else:
        raise SystemExit(f"unknown --only target {args.only!r}")
    for _ in range(args.warmup + args.steps):
        call()
    torch.cuda.synchronize()
    print(json.dumps({"only": args.only, "launches": args.warmup + args.steps, "device_error": ops.take_device_error()}))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=500)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-also", action="store_true", help="skip the secondary figures")
    parser.add_argument("--no-decode-step", action="store_true", help="skip the Llama-shaped decode step figure")
    parser.add_argument("--collective", default="peer", choices=["peer", "oneshot", "twophase", "pushall", "nccl"],
                        help="how the decode step's two collectives per layer run at --gpus > 1")
    parser.add_argument("--only", default="", help="profiling aid: launch one kernel a few times and exit "
                        "(decode | paged_attention | gemm:M,N,K | prefill[:len,len,...] | kvwrite | step:LAYERS[:TP])")
    args = parser.parse_args()

    if args.impl == "reference":
        run_reference(args)
        return
    if args.only:
        run_only(args)
        return

    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path")
    rank, local, world, group = dist_setup(args.gpus)
    line, case = run_decode(args, rank, world, group)
    decode_step = None
    if not args.no_decode_step:
        try:
            decode_step = run_decode_step(rank, world, group, collective=args.collective)
        except Exception as error:
            decode_step = {"error": repr(error)}
    if rank == 0:
        if world == 1:
            threads = 1  # the reference's singe-kernel CPU decode is serial
            cpu_value, cpu_seconds = cpu_baseline_decode(case, threads)
            line["cpu_baseline"] = {"value": round(cpu_value, 3), "unit": UNIT, "cores": threads, "kind": "port",
                                    "sample": f"full config-2 batch, best of 2 calls ({cpu_seconds:.2f} s each)"}
        line["also"] = {}
        if not args.no_also:
            try:
                import bench_extra

                line["also"] = bench_extra.run_all(measured_peaks())
            except Exception as error:  # secondary figures never take the headline down
                line["also"] = {"error": repr(error)}
        if decode_step is not None:
            line["also"]["decode_step_config5"] = decode_step
        print(json.dumps(line), flush=True)
    if group is not None:
        group.barrier()
        group.destroy_process_group()


if __name__ == "__main__":
    main()
