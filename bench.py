#!/usr/bin/env python
"""Benchmark of the hot path on B200.

Headline (``--workload gpt2``, the default): the GPT-2-small-architecture forward pass — 12 pre-LN layers, d_model 768,
12 heads, MLP 3072 with tanh GELU, vocabulary 50257, batch 32 x 1024 tokens, fp32 parameters ~ N(0, 0.02), fp16 compute,
token ids uniform over the vocabulary — as tokens per second. One step = one forward pass over the whole batch. With N
GPUs the batch is split over the ranks BY THE COMPILER (every rank hands the full batch-32 module to
``mhlo_b200_compile_sharded``, which proves that the batch shards are independent and builds this rank's shard), so the
scaling is strong: total work is fixed, ``value`` = 32768 tokens / slowest rank's device time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload gpt2|norms]

For N > 1 launch under ``python -m torch.distributed.run --nproc-per-node N``; one rank per GPU, no collective on the
data path (the logits stay sharded; the column-split GEMM in ``extra`` is the one workload with an exchange step).

``value`` is timed on the device with inputs resident in HBM (CUDA events on the stream the program runs on, max over
ranks). ``e2e`` is the same metric through the PJRT plugin with HOST buffers: every step copies the token ids from pinned
host memory (PJRT_Client_BufferFromHostBuffer), executes, and copies the logits back (PJRT_Buffer_ToHostBuffer); the
parameters are device buffers created once, as a framework holds them.

``--impl reference`` times the CPU restatement of the reference's host kernels (oracle/gpt2_cpu.py: BLAS sgemm + the
OpenMP LayerNorm / GELU / attention kernels; the reference itself is Swift/Metal and cannot be built on Linux) on a
bounded sample of the same workload, on rank 0 only, with every host core.

Prints ONE JSON line on rank 0. The other metrics of the hot path (norm sweep GB/s, GEMM and attention TFLOP/s) ride
in ``extra``, each with its own roofline block.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, HIDDEN, EPS = 32768, 4096, 1e-5
BATCH, SEQ, VOCAB, LAYERS, D_MODEL, HEADS = 32, 1024, 50257, 12, 768, 12
# Algorithmic work of one token's forward pass: the dense products 2 * (12 * 7 077 888 + 768 * 50257) = 247 064 064 FLOP
# plus causal attention (each query meets on average half of the 1024 keys) 12 * 4 * 512 * 768 = 18 874 368 FLOP.
FLOP_PER_TOKEN = 2 * (LAYERS * 12 * D_MODEL * D_MODEL + D_MODEL * VOCAB) + LAYERS * 4 * (SEQ // 2) * D_MODEL
FLOP_PER_TOKEN_FULL_ATTENTION = FLOP_PER_TOKEN + LAYERS * 4 * (SEQ // 2) * D_MODEL  # counting the masked half too (2.85e8)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:  # pragma: no cover
        return os.cpu_count() or 1


def use_all_host_cores() -> int:
    """The CPU legs use every core this process may run on, whatever OMP_NUM_THREADS the launcher exported (torchrun sets
    it to 1): the OpenMP team of the oracle's kernels and the BLAS pool behind numpy are both set explicitly."""
    import oracle

    cores = host_cores()
    oracle.set_threads(cores)
    try:
        from threadpoolctl import threadpool_limits

        threadpool_limits(limits=cores)
    except Exception:  # pragma: no cover
        pass
    return cores


def gpt2_host_inputs(params, seed=7):
    import numpy as np

    rng = np.random.default_rng(seed)
    out = []
    for name, shape, dt in params:
        if dt == "i32":
            out.append(rng.integers(0, VOCAB, size=shape).astype(np.int32))
        elif name.endswith("_g"):
            out.append(np.ones(shape, np.float32))
        elif name.endswith(("ln1_b", "ln2_b", "lnf_b")):
            out.append(np.zeros(shape, np.float32))
        else:
            out.append((0.02 * rng.standard_normal(shape)).astype(np.float32))
    return out


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()  # the exact child this object started
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------
# CPU arm: the oracle's fp32 host kernels (operation order of the reference's CPU partition)
# ---------------------------------------------------------------------------------------------------------

def cpu_gpt2_forward(sample_sequences: int, steps: int, warmup: int):
    """Tokens per second of the fp32 CPU forward pass on `sample_sequences` sequences of 1024 tokens per step."""
    from metalhlo_b200 import modules
    from oracle import gpt2_cpu

    cores = use_all_host_cores()
    _, params = modules.gpt2_module(batch=sample_sequences, seq=SEQ)
    ins = gpt2_host_inputs(params)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        logits = gpt2_cpu.forward(ins, HEADS, EPS)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    assert logits.shape == (sample_sequences, SEQ, VOCAB)
    sec = sum(times) / len(times)
    return sample_sequences * SEQ / sec, sec, cores


def cpu_norm_sweep(sample_rows: int, steps: int, warmup: int):
    import numpy as np

    import oracle

    cores = use_all_host_cores()
    rng = np.random.default_rng(42)
    x = rng.standard_normal((sample_rows, HIDDEN), dtype=np.float32)
    gamma = (1 + 0.1 * rng.standard_normal(HIDDEN)).astype(np.float32)
    beta = (0.1 * rng.standard_normal(HIDDEN)).astype(np.float32)
    x4 = x * 4
    y = np.empty_like(x)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        oracle.cpu_layer_norm_f32(x, gamma, beta, y, EPS)
        oracle.cpu_rms_norm_f32(x, gamma, y, EPS)
        oracle.cpu_softmax_f32(x4, y)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    # same unit as the GPU arm: bf16-equivalent algorithmic bytes (2 B in + 2 B out per element and kernel)
    gbs = 3 * sample_rows * HIDDEN * 4 / sec / 1e9
    return gbs, sec, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload == "norms":
        sample_rows = 4096
        gbs, sec, cores = cpu_norm_sweep(sample_rows, args.steps, args.warmup)
        sample = (f"{sample_rows} of {ROWS} rows x {HIDDEN}, fp32 host arrays, LayerNorm+RMSNorm+softmax per step; "
                  "bytes counted as the bf16 workload's (4 B per element and kernel)")
        line = {
            "impl": "reference", "metric": "fused norm sweep throughput (LayerNorm+RMSNorm+softmax)", "value": gbs,
            "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": sec * 1e3 * ROWS / sample_rows, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "norms bf16-shaped [32768,4096] sweep, CPU restatement of the reference's host kernels",
                       "rows": ROWS, "hidden": HIDDEN, "eps": EPS},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
        print(json.dumps(line))
        return
    sample_sequences = 2
    tps, sec, cores = cpu_gpt2_forward(sample_sequences, args.steps, args.warmup)
    sample = (f"{sample_sequences} of {BATCH} sequences x {SEQ} tokens per step, full model extents, fp32 host arrays: BLAS sgemm + OpenMP "
              "LayerNorm / GELU / causal attention kernels")
    line = {
        "impl": "reference", "metric": "GPT-2-small forward throughput", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3 * BATCH / sample_sequences,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": gpt2_config(args.gpus, "CPU restatement of the reference's host kernels (the reference is Swift/Metal and cannot be built on Linux)"),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def gpt2_config(world, how):
    return {"workload": "GPT-2-small forward, batch 32 x seq 1024, vocab 50257, fp32 parameters, fp16 compute", "how": how,
            "global_batch": BATCH, "seq_len": SEQ, "layers": LAYERS, "d_model": D_MODEL, "heads": HEADS, "vocab": VOCAB,
            "parallelism": f"batch split x{world} by the compiler's batch-sharding analysis, parameters replicated, no collective",
            "l2": "inputs larger than L2 (497 MB of fp32 parameters, 3.3 GB of logits written per forward)"}


# ---------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------

class Ranks:
    """One process per GPU: rank / world from the launcher's environment, NCCL for the barriers and the max-over-ranks."""

    def __init__(self):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py: no CUDA device; the hot path has no CPU fallback")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            os.environ.setdefault("NCCL_DEBUG", "WARN")
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max(self, values):
        if self.world == 1:
            return list(values)
        t = self.torch.tensor(list(values), device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def tensor_block(flop, ms, world, peaks, sustained=False, **more):
    """Roofline block of a tensor-bound measurement: algorithmic FLOP / device time against the measured cuBLAS bf16 rate
    of `world` GPUs (burst figure for a kernel timed by itself, sustained figure inside a long step)."""
    peak = (peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]) * world
    achieved = flop / (ms * 1e-3) / 1e12
    out = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
           "peak_source": peaks["source"] + (" (sustained)" if sustained else " (burst)"), "traffic": None}
    out.update(more)
    return out


def hbm_block(nbytes, ms, world, peaks, **more):
    achieved = nbytes / (ms * 1e-3) / 1e9
    peak = peaks["hbm_gbs"] * world
    out = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peaks["source"], "traffic": None}
    out.update(more)
    return out


def measure_norms(r: Ranks, cuda, rows_total, steps, warmup, peaks):
    """The fused normalisation sweep with its rows split contiguously over the ranks: LayerNorm, RMSNorm and softmax(4x)
    over bf16 [rows_total / world, 4096]. Returns the aggregate GB/s of algorithmic bytes (one read + one write of the tensor
    per kernel), the per-kernel rates and the slowest kernel's roofline block."""
    torch = r.torch
    from metalhlo_b200 import sharding

    rows = sharding.contiguous_shard(rows_total, r.world, r.rank).count
    g = torch.Generator().manual_seed(42 + r.rank)
    x = torch.randn(rows, HIDDEN, generator=g).to(torch.bfloat16).to(r.dev)
    gamma = (1 + 0.1 * torch.randn(HIDDEN, generator=g)).to(torch.bfloat16).to(r.dev)
    beta = (0.1 * torch.randn(HIDDEN, generator=g)).to(torch.bfloat16).to(r.dev)
    x4 = (x.float() * 4).to(torch.bfloat16)
    y = [torch.empty_like(x) for _ in range(3)]
    stream = torch.cuda.current_stream()
    names = ["layer_norm", "rms_norm", "softmax"]
    calls = [lambda: cuda.layer_norm(x, gamma, beta, EPS, out=y[0]), lambda: cuda.rms_norm(x, gamma, EPS, out=y[1]),
             lambda: cuda.softmax(x4, out=y[2])]
    for _ in range(warmup):
        for c in calls:
            c()
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(steps)]
    r.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for k in range(steps):
        for i, c in enumerate(calls):
            marks[k][i].record(stream)
            c()
        marks[k][3].record(stream)
    t1.record(stream)
    r.barrier()
    elapsed = t0.elapsed_time(t1)
    per = [sum(marks[k][i].elapsed_time(marks[k][i + 1]) for k in range(steps)) / steps for i in range(3)]
    elapsed, *per = r.max([elapsed] + per)
    kernel_bytes_total = rows_total * HIDDEN * 4  # bf16 read + bf16 write, all ranks together
    per_kernel = {n: kernel_bytes_total / (per[i] * 1e-3) / 1e9 for i, n in enumerate(names)}
    dom = max(range(3), key=lambda i: per[i])
    traffic = TRAFFIC_BYTES.get(names[dom])
    block = hbm_block(kernel_bytes_total, per[dom], r.world, peaks, kernel=names[dom], per_kernel_gbs=per_kernel,
                      traffic=None if traffic is None else traffic * rows // ROWS)
    return {"gbs": 3 * kernel_bytes_total * steps / (elapsed * 1e-3) / 1e9, "ms_per_sweep": elapsed / steps, "rows_per_gpu": rows,
            "per_kernel_ms": dict(zip(names, per)), "roofline": block, "launches": 3 * steps}


def measure_gpt2(r: Ranks, args, peaks):
    """Device-resident and end-to-end (PJRT, host buffers) throughput of the GPT-2 forward pass, batch split over the ranks
    by the compiler."""
    import numpy as np

    torch = r.torch
    from metalhlo_b200 import capi, modules

    text, params = modules.gpt2_module(batch=BATCH, seq=SEQ)
    host_inputs = gpt2_host_inputs(params)
    client = capi.Client()
    exe = client.compile_sharded(text, r.world, r.rank, opt_level=3)
    count, index, in_axes, out_axes = exe.sharding
    assert (count, index) == (r.world, r.rank), exe.sharding
    if r.world > 1:  # the token ids and the logits are split along the batch, every parameter is replicated
        assert in_axes[0] == 0 and set(in_axes[1:]) == {-1} and out_axes == [0], exe.sharding
    shard_batch = BATCH // r.world
    assert exe.input_type(0)[0] == (shard_batch, SEQ) and exe.output_type(0)[0] == (shard_batch, SEQ, VOCAB)
    ids_shard = np.ascontiguousarray(np.split(host_inputs[0], r.world, axis=0)[r.rank])
    bufs = [client.buffer(ids_shard)] + [client.buffer(a) for a in host_inputs[1:]]
    in_ptrs = [b.device_pointer for b in bufs]
    logits = torch.empty(shard_batch, SEQ, VOCAB, device=r.dev, dtype=torch.float16)
    side = torch.cuda.Stream()  # its own stream, so that the executor may record the launch list once and replay it as a CUDA graph

    def step():
        exe.execute_on_device(in_ptrs, [logits.data_ptr()], side.cuda_stream)

    sampler = ClockSampler(r.local)
    if r.rank == 0:
        sampler.start()
        time.sleep(0.3)
    side.wait_stream(torch.cuda.current_stream())
    for _ in range(args.warmup):
        step()
    r.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(side)
    for _ in range(args.steps):
        step()
    e1.record(side)
    r.barrier()
    ms = r.max([e0.elapsed_time(e1) / args.steps])[0]
    clocks = sampler.stop() if r.rank == 0 else None
    from metalhlo_b200 import cuda

    assert cuda.device_error() == 0, "a tensor-core kernel gave up on a bounded wait"
    launches, replays, steps_list = exe.launch_count, exe.graph_replays, exe.steps
    finite = bool(torch.isfinite(logits[0, -1]).all())
    assert finite, "non-finite logits"
    del exe, bufs
    torch.cuda.empty_cache()

    # ---- end to end through the PJRT plugin (GetPjrtApi) with host buffers. The plugin's client reads the shard from the
    # environment, as a launcher would set it per process; the parameters become device buffers once.
    from metalhlo_b200 import pjrt

    os.environ["METALHLO_SHARD_COUNT"], os.environ["METALHLO_SHARD_INDEX"] = str(r.world), str(r.rank)
    os.environ["METALHLO_DEVICE"] = str(r.local)
    os.environ["METALHLO_OPT_LEVEL"] = "O3"  # the plugin compiles at O2 unless told otherwise, like the reference's (PJRTExecutable.swift:1755-1766)
    host = pjrt.Host()
    pexe = host.compile(text)
    param_bufs = [host.buffer(a) for a in host_inputs[1:]]
    ids_pinned = torch.from_numpy(ids_shard).pin_memory()
    logits_pinned = torch.empty(shard_batch, SEQ, VOCAB, dtype=torch.float16).pin_memory()
    nbytes_out = logits_pinned.numel() * 2

    def e2e_step(copy_back=True):
        ids_buf = host.buffer_from_pointer(ids_pinned.data_ptr(), np.int32, (shard_batch, SEQ))
        out = pexe.execute([ids_buf] + param_bufs)[0]
        if copy_back:
            out.to_host_pointer(logits_pinned.data_ptr(), nbytes_out)
        del out, ids_buf

    def time_e2e(n, copy_back):
        e2e_step(copy_back)
        r.barrier()
        t0 = time.perf_counter()
        for _ in range(n):
            e2e_step(copy_back)
        r.barrier()
        return r.max([(time.perf_counter() - t0) * 1e3 / n])[0]

    def time_e2e_overlapped(n):
        # Two steps in flight: PJRT_Buffer_ToHostBuffer returns while the logits of step i are still travelling (its event is
        # pending), the host sends the ids of step i + 1 and executes it, and awaits the event before it starts the next
        # transfer into the same pinned buffer. Every step still copies its ids up and its logits down inside the timed region.
        e2e_step(True)
        r.barrier()
        pending = None
        t0 = time.perf_counter()
        for _ in range(n):
            ids_buf = host.buffer_from_pointer(ids_pinned.data_ptr(), np.int32, (shard_batch, SEQ))
            out = pexe.execute([ids_buf] + param_bufs)[0]
            if pending is not None:
                pending[0]()  # the previous step's logits are in host memory
            pending = (out.to_host_pointer_start(logits_pinned.data_ptr(), nbytes_out), out, ids_buf)
        pending[0]()
        del pending
        r.barrier()
        return r.max([(time.perf_counter() - t0) * 1e3 / n])[0]

    e2e_steps = max(3, min(args.steps, 8))
    e2e_serial_ms = time_e2e(e2e_steps, True)
    e2e_ms = time_e2e_overlapped(e2e_steps)
    e2e_nocopy_ms = time_e2e(e2e_steps, False)
    # the first logits of the PJRT path equal the device-resident path's (same program, same kernels)
    same = bool(torch.equal(logits_pinned[0, -1].to(r.dev).view(torch.int16), logits[0, -1].view(torch.int16)))
    # the host-copy roof: the logits shard alone, device to pinned host memory, on every rank at once
    def copy_only():
        logits_pinned.copy_(logits, non_blocking=True)
    copy_only()
    r.barrier()
    t0 = time.perf_counter()
    for _ in range(3):
        copy_only()
    r.barrier()
    copy_ms = r.max([(time.perf_counter() - t0) * 1e3 / 3])[0]
    del pexe, param_bufs, host
    tokens = BATCH * SEQ
    return {
        "ms": ms, "tokens_per_s": tokens / (ms * 1e-3), "clocks": clocks, "launches_per_step": launches, "graph_replays": replays,
        "fused_steps": {k: steps_list.count(k) for k in sorted(set(s for s in steps_list if s.startswith("fused")))},
        "roofline": tensor_block(FLOP_PER_TOKEN * tokens, ms, r.world, peaks, sustained=True, kernel="whole forward pass (gemm_tcgen05 + attention_tcgen05 + row kernels)",
                                 flop_per_token=FLOP_PER_TOKEN, note="causal attention counted at the work it does (half of the score matrix); "
                                 f"with the masked half counted the figure would be {FLOP_PER_TOKEN_FULL_ATTENTION} FLOP per token"),
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": BATCH * SEQ * 4, "d2h_bytes_per_step": BATCH * SEQ * VOCAB * 2,
                "ms_per_step": e2e_ms, "steps": e2e_steps, "launches_per_step": launches,
                "path": "GetPjrtApi: BufferFromHostBuffer(token ids, pinned) -> LoadedExecutable_Execute -> Buffer_ToHostBuffer(fp16 logits, pinned); parameters resident; "
                        "the transfer's event is awaited after the next step's Execute, so the logits of step i travel while step i + 1 computes",
                "one_step_at_a_time": {"value": tokens / (e2e_serial_ms * 1e-3), "ms_per_step": e2e_serial_ms,
                                       "note": "the same calls with every transfer awaited before the next step starts"},
                "without_logits_copy": {"value": tokens / (e2e_nocopy_ms * 1e-3), "ms_per_step": e2e_nocopy_ms,
                                        "note": "ids up and execute only; the logits stay on the device"},
                "host_copy_roof": {"ms_per_step": copy_ms, "gbs_per_gpu": nbytes_out / (copy_ms * 1e-3) / 1e9,
                                   "value": tokens / (copy_ms * 1e-3),
                                   "note": "device-to-pinned-host copy of each rank's logits shard alone, all ranks at once: no e2e step can be faster"},
                "matches_device_resident_path": same},
    }


def run_ours(args):
    r = Ranks()
    torch, dist = r.torch, r.dist
    from metalhlo_b200 import cuda  # raises if libmhlo_cuda.so is missing: no fallback

    peaks = load_peaks()
    if args.workload == "norms":
        res = measure_norms(r, cuda, ROWS, args.steps, args.warmup, peaks)
        if args.kernels_only:
            if r.rank == 0:
                print(json.dumps({"kernels_only": True, "rows": ROWS, "per_kernel_gbs": res["roofline"]["per_kernel_gbs"]}))
            r.close()
            return
        cpu_gbs, _, cores = cpu_norm_sweep(2048, 3, 1) if r.rank == 0 else (None, None, None)
        if r.rank == 0:
            line = {"metric": "fused norm sweep throughput (LayerNorm+RMSNorm+softmax)", "value": res["gbs"], "unit": "GB/s", "n_gpus": r.world,
                    "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_sweep"], "higher_is_better": True, "scaling": "strong",
                    "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "config": {"workload": "norms bf16 [32768,4096]: LayerNorm, RMSNorm, softmax(x*4), fp32 statistics", "rows_per_gpu": res["rows_per_gpu"],
                               "hidden": HIDDEN, "eps": EPS, "l2": "inputs larger than L2 at up to 4 GPUs; 67 MB per GPU at 8",
                               "parallelism": f"rows split x{r.world}, no collective"},
                    "roofline": res["roofline"], "gpu_launches": res["launches"], "e2e": None,
                    "cpu_baseline": {"value": cpu_gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                                     "sample": f"2048 of {ROWS} rows x {HIDDEN}, fp32 host arrays, 3 timed sweeps"}}
            print(json.dumps(line))
        r.close()
        return

    g = measure_gpt2(r, args, peaks)
    extra = None
    if not args.no_extras:
        torch.cuda.empty_cache()
        extra = measure_extras(r, cuda, peaks)
    cpu = None
    if r.rank == 0:
        # the CPU baseline runs on rank 0 after the GPU legs, while the other ranks wait at the closing barrier
        tps, sec, cores = cpu_gpt2_forward(1, 2, 1)
        cpu = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"1 of {BATCH} sequences x {SEQ} tokens, full model extents, fp32 host arrays (BLAS sgemm + OpenMP LayerNorm / GELU / attention), "
                         "1 warm-up + 2 timed passes"}
    r.barrier()
    if r.rank == 0:
        line = {
            "metric": "GPT-2-small forward throughput", "value": g["tokens_per_s"], "unit": "tokens/s", "n_gpus": r.world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": g["ms"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": dict(gpt2_config(r.world, "mhlo_b200_compile_sharded of the full batch-32 module on every rank, O3, CUDA-graph replay on device-resident inputs"),
                           batch_per_gpu=BATCH // r.world, fused_steps=g["fused_steps"], graph_replays=g["graph_replays"]),
            "roofline": g["roofline"], "e2e": g["e2e"], "cpu_baseline": cpu,
            "gpu_launches": g["launches_per_step"] * args.steps, "clocks": g["clocks"],
        }
        if extra is not None:
            line["extra"] = extra
        print(json.dumps(line))
    r.close()


def measure_extras(r, cuda, peaks):
    """The other headline metrics of the hot path, each sharded the way its configuration prescribes and timed on the
    device (max over ranks): bf16 GEMM 8192^3 (column split + NCCL all-gather when world > 1), the HBM-limited batched
    GEMM, fused flash attention B8 H32 S4096 D128 (batch x head sharded), and the GPT-2-small forward pass (batch 32
    sharded). Returned as a dict for the "extra" key of the JSON line."""
    import math

    torch, dist, rank, world, dev = r.torch, r.dist, r.rank, r.world, r.dev
    out = {}
    # ---- the memory-bound normalisation sweep, rows split over the ranks
    n_res = measure_norms(r, cuda, ROWS, 20, 5, peaks)
    out["norm_sweep_bf16"] = {"gbs": n_res["gbs"], "ms_per_sweep": n_res["ms_per_sweep"], "rows_per_gpu": n_res["rows_per_gpu"],
                              "roofline": n_res["roofline"]}

    def timed(fn, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    g = torch.Generator(device=dev).manual_seed(42 + rank)
    # ---- GEMM 8192^3 bf16: B and C column-split across ranks, C slices all-gathered and interleaved to row-major
    n = 8192
    from metalhlo_b200 import sharding

    col_block = sharding.column_shard(n, world, rank)
    ncols = col_block.count
    a = (torch.randn(n, n, device=dev, generator=g) / math.sqrt(n)).to(torch.bfloat16)
    b = (torch.randn(n, n, device=dev, generator=g) / math.sqrt(n)).to(torch.bfloat16)
    c_slice = torch.empty(n, ncols, device=dev, dtype=torch.bfloat16)
    c_all = torch.empty(world, n, ncols, device=dev, dtype=torch.bfloat16) if world > 1 else None
    c_full = torch.empty(n, n, device=dev, dtype=torch.bfloat16) if world > 1 else None
    a_str, b_str = cuda._i64s([0, 0, n, 1]), cuda._i64s([0, 0, n, 1])
    b_ptr = b.data_ptr() + col_block.start * 2
    stream = torch.cuda.current_stream().cuda_stream

    def gemm_step():
        cuda.check(cuda.lib.mhlo_cuda_gemm(cuda.BF16, cuda.BF16, a.data_ptr(), a_str, b_ptr, b_str, c_slice.data_ptr(), 1, 1, n,
                                           ncols, n, None, 0, stream))
        if world > 1:
            dist.all_gather_into_tensor(c_all, c_slice)
            c_full.view(n, world, ncols).copy_(c_all.permute(1, 0, 2))

    ms = timed(gemm_step, 10)
    tf = 2 * n ** 3 / ms / 1e9
    out["gemm_bf16_8192"] = {"tflops": tf, "ms": ms, "roofline": tensor_block(2 * n ** 3, ms, world, peaks, kernel="gemm_tcgen05_kernel"),
                             "parallelism": f"column split x{world}" + (" + NCCL all-gather + interleave" if world > 1 else "")}
    if world > 1:
        # The same product with the exchange fused into the GEMM: every rank's epilogue stores its column block into all
        # ranks' copies of C through peer addresses; a one-CTA kernel behind it publishes this rank's epoch in the peers'
        # flag words and waits (bounded) for theirs, so the stream carries on once every copy is complete.
        import ctypes as C

        c_bytes = n * n * 2
        own = C.c_void_p()
        cuda.check(cuda.lib.mhlo_cuda_alloc(c_bytes + 256, C.byref(own)))  # C, then the eight flag words
        cuda.check(cuda.lib.mhlo_cuda_memset(own, 0, c_bytes + 256, stream))
        torch.cuda.synchronize()
        handle = C.create_string_buffer(64)
        cuda.check(cuda.lib.mhlo_cuda_ipc_export(own, handle))
        handles = sharding.exchange_handles(handle.raw, dist)
        peers = []
        for r in range(world):
            if r == rank:
                peers.append(own.value)
            else:
                ptr = C.c_void_p()
                cuda.check(cuda.lib.mhlo_cuda_ipc_open(handles[r], C.byref(ptr)))
                peers.append(ptr.value)
        c_ptrs = (C.c_void_p * world)(*peers)
        flag_ptrs = (C.c_void_p * world)(*[p + c_bytes for p in peers])
        ab_str = cuda._i64s([n, 1])
        flag = torch.zeros(1, device=dev)
        epoch = [0]
        dist.barrier()  # every rank's flag words are zero and mapped before the first epoch is published

        def fused_step(tuning=None, copy_stores=0, closing="flags"):
            cuda.check(cuda.lib.mhlo_cuda_gemm_all_gather_tuned(cuda.BF16, cuda.BF16, a.data_ptr(), ab_str, b_ptr, ab_str, c_ptrs, world, rank, n,
                                                                ncols, n, None, 0, None if tuning is None else C.addressof(tuning), copy_stores,
                                                                stream))
            if closing == "flags":
                epoch[0] += 1
                cuda.check(cuda.lib.mhlo_cuda_peer_barrier(flag_ptrs, world, rank, epoch[0], 2_000_000_000, stream))
            elif closing == "nccl":
                dist.all_reduce(flag)

        fused_step()
        torch.cuda.synchronize()
        # a device barrier that gave up (code 95 on any rank) takes the flag variants out of the comparison instead of
        # ending the benchmark: the exchange is then closed by the 1-element all-reduce
        code = torch.tensor([cuda.device_error()], device=dev, dtype=torch.int32)
        dist.all_reduce(code, op=dist.ReduceOp.MAX)
        flags_ok = int(code.item()) == 0
        dist.barrier()
        # correctness against the NCCL path of the same operands, on this rank's copy
        mine = torch.empty(n, n, device=dev, dtype=torch.bfloat16)
        cuda.check(cuda.lib.mhlo_cuda_copy(mine.data_ptr(), own, c_bytes, stream))
        torch.cuda.synchronize()
        same = bool(torch.equal(mine.view(torch.int16), c_full.view(torch.int16)))
        variants = {}
        for name, kw in (("lane_stores", {}), ("lane_stores_tile128", {"tuning": cuda.GemmTuning(128, 0, 0, 0)}),
                         ("bulk_stores", {"copy_stores": 2}), ("bulk_stores_tile128", {"tuning": cuda.GemmTuning(128, 0, 0, 0), "copy_stores": 2}),
                         ("pair_lane_stores", {"tuning": cuda.GemmTuning(256, 0, 2, 0)}),
                         ("pair_bulk_stores", {"tuning": cuda.GemmTuning(256, 0, 2, 0), "copy_stores": 2}),
                         ("lane_stores_nccl_closing", {"closing": "nccl"}), ("bulk_stores_nccl_closing", {"closing": "nccl", "copy_stores": 2}),
                         ("lane_stores_unclosed", {"closing": "none"})):
            if not flags_ok and kw.get("closing", "flags") == "flags":
                continue
            variants[name] = timed(lambda: fused_step(**kw), 10)
            dist.barrier()
        best = min((k for k in variants if not k.endswith("unclosed") and (not flags_ok or not k.endswith("nccl_closing"))), key=variants.get)
        ms_f = variants[best]
        tf_f = 2 * n ** 3 / ms_f / 1e9
        out["gemm_bf16_8192_fused_all_gather"] = {
            "tflops": tf_f, "ms": ms_f, "roofline": tensor_block(2 * n ** 3, ms_f, world, peaks, kernel="gemm_tcgen05_kernel + peer stores",
                                                                 link_floor_ms=(n * n * 2 / world) * (world - 1) / 770e9 * 1e3),
            "matches_nccl_path": same, "variant": best, "ms_by_variant": {k: round(v, 4) for k, v in variants.items()},
            "nvlink_bytes_per_rank": (n * n * 2 // world) * (world - 1), "device_barrier_code": int(code.item()),
            "parallelism": f"column split x{world}, epilogue stores into every rank's C over NVLink, " +
                           ("flag words in peer memory as completion barrier" if flags_ok else "1-element all-reduce as completion barrier")}
        out["gemm_bf16_8192_fused_all_gather"]["device_error_after"] = cuda.device_error()
        dist.barrier()
        for r in range(world):
            if r != rank:
                cuda.check(cuda.lib.mhlo_cuda_ipc_close(C.c_void_p(peers[r])))
        dist.barrier()
        cuda.check(cuda.lib.mhlo_cuda_free(own))
    del a, b, c_slice, c_all, c_full
    # ---- batched GEMM [64,2048,128].[64,128,2048]: batch sharded, HBM-limited
    nb = max(1, sharding.contiguous_shard(64, world, rank).count)
    a = (torch.randn(nb, 2048, 128, device=dev, generator=g) / math.sqrt(128)).to(torch.bfloat16)
    b = (torch.randn(nb, 128, 2048, device=dev, generator=g) / math.sqrt(128)).to(torch.bfloat16)
    c = torch.empty(nb, 2048, 2048, device=dev, dtype=torch.bfloat16)
    ms = timed(lambda: cuda.gemm(a, b, out=c), 10)
    bytes_total = 603_979_776
    out["gemm_bf16_batched"] = {"tflops": 68_719_476_736 / ms / 1e9, "gbs": bytes_total / ms / 1e6, "ms": ms,
                                "roofline": hbm_block(bytes_total, ms, world, peaks, kernel="gemm_tcgen05_kernel")}
    del a, b, c
    # ---- flash attention B8 H32 S4096 D128 bf16, batch sharded
    bsz = max(1, sharding.contiguous_shard(8, world, rank).count)
    q, k, v = (torch.randn(bsz, 32, 4096, 128, device=dev, generator=g).to(torch.bfloat16) for _ in range(3))
    o = torch.empty_like(q)
    for causal, flop in ((False, 2_199_023_255_552), (True, 1_099_780_063_232)):
        ms = timed(lambda: cuda.attention(q, k, v, 1 / math.sqrt(128), causal=causal, out=o), 5)
        tf = flop * (bsz * world / 8) / ms / 1e9
        out["attention_causal" if causal else "attention"] = {
            "tflops": tf, "ms": ms, "roofline": tensor_block(flop * (bsz * world / 8), ms, world, peaks, kernel="attention_tcgen05_kernel<128>")}
    assert cuda.device_error() == 0, "a tensor-core kernel gave up on a bounded wait"
    del q, k, v, o
    # ---- the model's own attention shape: f16, 12 heads of 64, 1024 tokens, causal, this rank's share of the 32 sequences
    bsz = max(1, sharding.contiguous_shard(BATCH, world, rank).count)
    q, k, v = (torch.randn(bsz, SEQ, HEADS, 64, device=dev, generator=g).to(torch.float16) for _ in range(3))
    o = torch.empty_like(q)
    ms = timed(lambda: cuda.attention(q, k, v, 0.125, causal=True, layout="BSHD", out=o), 10)
    flop = 4 * bsz * world * HEADS * SEQ * (SEQ // 2) * 64
    out["attention_gpt2_shape_f16_causal"] = {"ms": ms, "tflops": flop / ms / 1e9, "batch_per_gpu": bsz,
                                              "roofline": tensor_block(flop, ms, world, peaks, kernel="attention_tcgen05_kernel<64>")}
    del q, k, v, o
    # ---- the model's layer products at this rank's share of the tokens: [tokens, 768] . [768, 3072] and its transpose shape
    m_tok = bsz * SEQ
    for name, kk, nn, epi in (("gemm_f16_tokens_x768_x3072", D_MODEL, 4 * D_MODEL, "none"), ("gemm_f16_tokens_x3072_x768", 4 * D_MODEL, D_MODEL, "none"),
                              ("gemm_f16_tokens_x768_x2304", D_MODEL, 3 * D_MODEL, "none"),
                              # as the model runs them: bias in the epilogue, GELU behind the up-projection
                              ("gemm_f16_tokens_x768_x3072_bias_gelu", D_MODEL, 4 * D_MODEL, "gelu_tanh"),
                              ("gemm_f16_tokens_x768_x2304_bias", D_MODEL, 3 * D_MODEL, "bias")):
        a = (torch.randn(m_tok, kk, device=dev, generator=g) / math.sqrt(kk)).to(torch.float16)
        b = (torch.randn(kk, nn, device=dev, generator=g)).to(torch.float16)
        bias = None if epi == "none" else torch.randn(nn, device=dev, generator=g).to(torch.float16)
        c = torch.empty(m_tok, nn, device=dev, dtype=torch.float16)
        ms = timed(lambda: cuda.gemm(a, b, bias=bias, epilogue="gelu_tanh" if epi == "gelu_tanh" else "none", out=c), 20)
        flop = 2 * m_tok * world * kk * nn
        out[name] = {"ms": ms, "tflops": flop / ms / 1e9, "tokens_per_gpu": m_tok, "roofline": tensor_block(flop, ms, world, peaks, kernel="gemm_tcgen05_kernel")}
        del a, b, c, bias
    # the logits product: [tokens, 768] . [50257, 768]^T, rows of the result off the 16-byte grid (pitch 50257 f16)
    a = (torch.randn(m_tok, D_MODEL, device=dev, generator=g) / math.sqrt(D_MODEL)).to(torch.float16)
    b = torch.randn(VOCAB, D_MODEL, device=dev, generator=g).to(torch.float16)
    c = torch.empty(m_tok, VOCAB, device=dev, dtype=torch.float16)
    ms = timed(lambda: cuda.gemm(a, b, trans_b=True, out=c), 5)
    flop = 2 * m_tok * world * D_MODEL * VOCAB
    out["gemm_f16_tokens_x768_x50257_logits"] = {"ms": ms, "tflops": flop / ms / 1e9, "tokens_per_gpu": m_tok,
                                                 "roofline": tensor_block(flop, ms, world, peaks, kernel="gemm_tcgen05_kernel")}
    del a, b, c
    from metalhlo_b200 import capi

    client = capi.Client()
    if world == 1:
        # operators either side of the fused path, each as a one-operator module through the C API on device memory
        for kind in ("conv", "maxpool", "sort_rows", "scatter_add"):
            try:
                run, case_exe, work, unit, keep = module_case_runner(kind, client)
                stream = torch.cuda.current_stream().cuda_stream
                ms = timed(lambda: run(stream), 10)
                touched = sum(b.byte_count for b in keep[1]) + sum(o.numel() for o in keep[2]) + case_exe.arena_bytes
                out["module_" + kind] = {
                    "ms": ms, ("tflops" if unit == "TFLOP" else "gbs"): work / ms * 1e3, "launches": case_exe.launch_count,
                    "steps": case_exe.steps, "device_mb": round(touched / 1e6, 1),
                    "l2": "back-to-back executions on the same buffers: " +
                          ("the working set exceeds L2" if touched > 126e6 else "the working set fits L2 and stays warm")}
                del run, case_exe, keep
                torch.cuda.empty_cache()
            except Exception as e:  # a side measurement must not cost the benchmark line
                out["module_" + kind] = {"error": str(e)[:200]}
    return out


def _conv_text(dt="bf16"):
    from metalhlo_b200.modules import tt

    x, w, o = tt((32, 56, 56, 64), dt), tt((3, 3, 64, 64), dt), tt((32, 56, 56, 64), dt)
    return (f"func.func @main(%x: {x}, %w: {w}) -> {o} {{\n  %0 = stablehlo.convolution(%x, %w) dim_numbers = [b, 0, 1, f]x[0, 1, i, o]->[b, 0, 1, f], "
            f"window = {{stride = [1, 1], pad = [[1, 1], [1, 1]]}} {{batch_group_count = 1 : i64, feature_group_count = 1 : i64}} : ({x}, {w}) -> {o}\n"
            f"  return %0 : {o}\n}}\n")


def _pool_text(dt="bf16"):
    from metalhlo_b200.modules import tt

    x, o = tt((32, 112, 112, 64), dt), tt((32, 56, 56, 64), dt)
    return (f"func.func @main(%x: {x}) -> {o} {{\n  %i = stablehlo.constant dense<0xFF80> : tensor<{dt}>\n"
            f"  %0 = \"stablehlo.reduce_window\"(%x, %i) <{{window_dimensions = array<i64: 1, 3, 3, 1>, window_strides = array<i64: 1, 2, 2, 1>, "
            f"padding = dense<[[0, 0], [0, 1], [0, 1], [0, 0]]> : tensor<4x2xi64>}}> ({{\n  ^bb0(%a: tensor<{dt}>, %b: tensor<{dt}>):\n"
            f"    %m = stablehlo.maximum %a, %b : tensor<{dt}>\n    stablehlo.return %m : tensor<{dt}>\n  }}) : ({x}, tensor<{dt}>) -> {o}\n"
            f"  return %0 : {o}\n}}\n")


def _sort_text(rows, n):
    from metalhlo_b200.modules import tt

    t, ti = tt((rows, n), "f32"), tt((rows, n), "i32")
    return (f"func.func @main(%x: {t}) -> ({t}, {ti}) {{\n  %i = stablehlo.iota dim = 1 : {ti}\n"
            f"  %0:2 = \"stablehlo.sort\"(%x, %i) <{{dimension = 1 : i64, is_stable = true}}> ({{\n"
            f"  ^bb0(%a: tensor<f32>, %b: tensor<f32>, %c: tensor<i32>, %d: tensor<i32>):\n"
            f"    %p = stablehlo.compare  LT, %a, %b,  TOTALORDER : (tensor<f32>, tensor<f32>) -> tensor<i1>\n    stablehlo.return %p : tensor<i1>\n"
            f"  }}) : ({t}, {ti}) -> ({t}, {ti})\n  return %0#0, %0#1 : {t}, {ti}\n}}\n")


def _scatter_text():
    from metalhlo_b200.modules import tt

    table, idx, upd = tt((50257, 768), "f32"), tt((32768, 1), "i32"), tt((32768, 768), "f32")
    return (f"func.func @main(%t: {table}, %i: {idx}, %u: {upd}) -> {table} {{\n"
            f"  %0 = \"stablehlo.scatter\"(%t, %i, %u) <{{indices_are_sorted = false, scatter_dimension_numbers = #stablehlo.scatter<update_window_dims = [1], "
            f"inserted_window_dims = [0], scatter_dims_to_operand_dims = [0], index_vector_dim = 1>, unique_indices = false}}> ({{\n"
            f"  ^bb0(%a: tensor<f32>, %b: tensor<f32>):\n    %s = stablehlo.add %a, %b : tensor<f32>\n    stablehlo.return %s : tensor<f32>\n"
            f"  }}) : ({table}, {idx}, {upd}) -> {table}\n  return %0 : {table}\n}}\n")


# name -> (module text builder, work per execution, unit): operators either side of the fused path, as whole modules
MODULE_CASES = {
    "conv": (lambda: _conv_text(), 2 * 32 * 56 * 56 * 64 * 9 * 64 / 1e12, "TFLOP"),                    # ResNet 3x3, 64 -> 64 channels
    "maxpool": (lambda: _pool_text(), (32 * 112 * 112 * 64 + 32 * 56 * 56 * 64) * 2 / 1e9, "GB"),     # read once + write once
    "sort_rows": (lambda: _sort_text(4096, 4096), 4096 * 4096 * 4 * 4 / 1e9, "GB"),                    # keys + order out, keys in (+iota)
    "sort_long": (lambda: _sort_text(4, 4194304), 4 * 4194304 * 4 * 4 / 1e9, "GB"),
    "scatter_add": (lambda: _scatter_text(), (2 * 50257 * 768 + 3 * 32768 * 768) * 4 / 1e9, "GB"),     # copy of the table + read-modify-write of the rows
}


def module_case_runner(kind: str, client=None):
    """Compiles one module of MODULE_CASES and allocates seeded inputs and outputs on the device. Returns
    (run(stream), executable, work per execution, unit, keep-alive objects)."""
    import numpy as np
    import torch

    from metalhlo_b200 import capi

    build, work, unit = MODULE_CASES[kind]
    client = client or capi.Client()
    exe = client.compile(build(), 3)
    rng = np.random.default_rng(5)
    ins = []
    for i in range(exe.input_count):
        shape, code = exe.input_type(i)
        dt = capi.np_dtype(code)
        if np.issubdtype(dt, np.integer):
            arr = rng.integers(0, 50257, size=shape).astype(dt)
        else:
            arr = rng.standard_normal(shape).astype(np.float32).astype(dt)
        ins.append(client.buffer(arr))
    outs = []
    for i in range(exe.output_count):
        shape, code = exe.output_type(i)
        outs.append(torch.empty(int(np.prod(shape)) * capi.np_dtype(code).itemsize, dtype=torch.uint8, device="cuda"))
    in_ptrs, out_ptrs = [b.device_pointer for b in ins], [o.data_ptr() for o in outs]

    def run(stream):
        exe.execute_on_device(in_ptrs, out_ptrs, stream)

    return run, exe, work, unit, (client, ins, outs)


def profile_module_case(kind: str, launches: int):
    """One module of MODULE_CASES through the C API on device memory: compile, then `launches` timed executions."""
    import numpy as np
    import torch

    from metalhlo_b200 import capi

    torch.cuda.set_device(0)
    build, work, unit = MODULE_CASES[kind]
    client = capi.Client()
    exe = client.compile(build(), 3)
    rng = np.random.default_rng(5)
    ins = []
    for i in range(exe.input_count):
        shape, code = exe.input_type(i)
        dt = capi.np_dtype(code)
        if np.issubdtype(dt, np.integer):
            arr = rng.integers(0, 50257, size=shape).astype(dt)
        else:
            arr = rng.standard_normal(shape).astype(np.float32).astype(dt)
        ins.append(client.buffer(arr))
    outs = []
    for i in range(exe.output_count):
        shape, code = exe.output_type(i)
        outs.append(torch.empty(int(np.prod(shape)) * capi.np_dtype(code).itemsize, dtype=torch.uint8, device="cuda"))
    in_ptrs, out_ptrs = [b.device_pointer for b in ins], [o.data_ptr() for o in outs]
    print(f"{kind}: steps {exe.steps}, {exe.launch_count} launches per execution, arena {exe.arena_bytes / 1e6:.1f} MB", file=sys.stderr)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(launches):
        e0.record()
        exe.execute_on_device(in_ptrs, out_ptrs, torch.cuda.current_stream().cuda_stream)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        print(f"{kind} execution {i}: {ms:.3f} ms, {work / ms * 1e3:.1f} {unit}/s")


def profile_case(kind: str, launches: int):
    """A few launches of one tensor-core kernel on a profiler-sized case (a few hundred MB on the device, inputs
    larger than L2), for `ncu -k regex:<kernel>` captures. Prints the CUDA-event time per launch; no JSON line."""
    import math

    import torch

    from metalhlo_b200 import cuda

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(1)
    if kind in MODULE_CASES:
        return profile_module_case(kind, launches)
    if kind == "gemm":
        n = 8192
        a = (torch.randn(n, n, device=dev, generator=g) / math.sqrt(n)).to(torch.bfloat16)
        b = (torch.randn(n, n, device=dev, generator=g) / math.sqrt(n)).to(torch.bfloat16)
        c = torch.empty(n, n, device=dev, dtype=torch.bfloat16)
        fn = lambda: cuda.gemm(a, b, out=c)  # noqa: E731
        work, unit = 2 * n ** 3 / 1e12, "TFLOP"
    elif kind in ("gemm_layer", "gemm_layer_bias_gelu"):
        # the model's up-projection at the full batch: [32768, 768] . [768, 3072], f16
        m, k_, n = BATCH * SEQ, D_MODEL, 4 * D_MODEL
        a = (torch.randn(m, k_, device=dev, generator=g) / math.sqrt(k_)).to(torch.float16)
        b = torch.randn(k_, n, device=dev, generator=g).to(torch.float16)
        c = torch.empty(m, n, device=dev, dtype=torch.float16)
        bias = torch.randn(n, device=dev, generator=g).to(torch.float16)
        with_epilogue = kind == "gemm_layer_bias_gelu"  # bias + GELU, as the model's MLP runs it
        fn = (lambda: cuda.gemm(a, b, bias=bias, epilogue="gelu_tanh", out=c)) if with_epilogue else (lambda: cuda.gemm(a, b, out=c))  # noqa: E731
        work, unit = 2 * m * k_ * n / 1e12, "TFLOP"
    elif kind == "attention_gpt2":
        # the model's attention: f16, 32 sequences x 12 heads of 64, 1024 tokens, causal, [B,S,H,D] in place
        q, k, v = (torch.randn(BATCH, SEQ, HEADS, 64, device=dev, generator=g).to(torch.float16) for _ in range(3))
        o = torch.empty_like(q)
        fn = lambda: cuda.attention(q, k, v, 0.125, causal=True, layout="BSHD", out=o)  # noqa: E731
        work, unit = 4 * BATCH * HEADS * SEQ * (SEQ // 2) * 64 / 1e12, "TFLOP"
    elif kind == "gpt2":
        # the whole forward pass at 4 sequences (one GPU's share of the batch at 8 GPUs), launch by launch
        from metalhlo_b200 import capi, modules

        pb = int(os.environ.get("BENCH_PROFILE_BATCH", "4"))
        text, params = modules.gpt2_module(batch=pb, seq=SEQ)
        client = capi.Client()
        exe = client.compile(text, opt_level=3)
        bufs = [client.buffer(a) for a in gpt2_host_inputs(params)]
        ptrs = [b_.device_pointer for b_ in bufs]
        logits = torch.empty(pb, SEQ, VOCAB, device=dev, dtype=torch.float16)
        fn = lambda: exe.execute_on_device(ptrs, [logits.data_ptr()], torch.cuda.current_stream().cuda_stream)  # noqa: E731
        work, unit = FLOP_PER_TOKEN * pb * SEQ / 1e12, "TFLOP"
    else:
        causal = kind == "attention_causal"
        q, k, v = (torch.randn(2, 32, 4096, 128, device=dev, generator=g).to(torch.bfloat16) for _ in range(3))
        o = torch.empty_like(q)
        fn = lambda: cuda.attention(q, k, v, 1 / math.sqrt(128), causal=causal, out=o)  # noqa: E731
        work, unit = 4 * 2 * 32 * 4096 * 4096 * 128 / 1e12 * (0.5 if causal else 1.0), "TFLOP"
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(launches):
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        print(f"{kind} launch {i}: {ms:.3f} ms, {work / ms * 1e3:.1f} {unit}/s")
    assert cuda.device_error() == 0


# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu captures (profiles/), scaled to
# the full [32768, 4096] launch where the capture used fewer rows. None until a capture exists.
TRAFFIC_BYTES: dict = {
    # ncu, 8192-row capture: dram read 67.15 / 67.13 / 67.12 MB (x4 for 32768 rows) + the full 268 435 456 B result
    "layer_norm": 4 * 67_153_152 + 268_435_456,
    "rms_norm": 4 * 67_133_440 + 268_435_456,
    "softmax": 4 * 67_124_224 + 268_435_456,
}


def _reserve_stdout():
    """Stdout carries exactly one JSON line. Libraries (NCCL's version banner, for one) write to file descriptor 1
    directly, so descriptor 1 is pointed at stderr for the whole run and the JSON line goes to a private copy of the
    original descriptor."""
    sys.stdout.flush()
    keep = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(keep, "w", buffering=1)


def main():
    global ROWS
    _reserve_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["gpt2", "norms"], default="gpt2")
    ap.add_argument("--rows", type=int, default=ROWS,
                    help="rows of the norm sweep (default: the benchmark configuration; smaller for profiler captures)")
    ap.add_argument("--no-extras", action="store_true", help="skip the norm / GEMM / attention side measurements")
    ap.add_argument("--kernels-only", action="store_true",
                    help="norm workload: skip the CPU-baseline leg (profiler captures)")
    ap.add_argument("--profile-kernel", choices=["gemm", "attention", "attention_causal", "attention_gpt2", "gemm_layer", "gemm_layer_bias_gelu", "gpt2"] + sorted(MODULE_CASES),
                    help="run a few launches of one kernel (or one module) on a profiler-sized case and exit")
    args = ap.parse_args()
    # the CPU legs (rank 0) use every host core; torchrun exports OMP_NUM_THREADS=1, which the BLAS and OpenMP runtimes
    # read when they are loaded, so it is replaced before anything imports them
    if int(os.environ.get("RANK", "0")) == 0:
        os.environ["OMP_NUM_THREADS"] = str(host_cores())
        os.environ.pop("OPENBLAS_NUM_THREADS", None)
        os.environ.pop("MKL_NUM_THREADS", None)
    if args.profile_kernel:
        profile_case(args.profile_kernel, max(1, min(args.steps, 5)))
        return
    if args.warmup < 3 and args.impl == "ours" and not args.kernels_only:
        args.warmup = 3
    ROWS = args.rows
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
