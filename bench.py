#!/usr/bin/env python
"""Benchmark of the hot path on B200.

Default workload (``--workload norms``): the memory-bound fused normalisation sweep — LayerNorm, RMSNorm and
row softmax over bf16 rows [32768, 4096] with fp32 statistics (eps 1e-5, gamma ~ 1+N(0,0.1), beta ~ N(0,0.1),
softmax input scaled by 4). One step = the three kernels over one batch of rows. The metric is GB/s of
algorithmic traffic (one read + one write of the tensor per kernel = 536 870 912 B per kernel).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload norms|...]

For N > 1 launch under ``python -m torch.distributed.run --nproc-per-node N``; every rank runs the full
per-GPU workload (rows are independent, no collective on the data path) and the value is the sum over ranks
divided by the slowest rank's device time.

``--impl reference`` times the CPU restatement of the reference's host kernels (the oracle's fp32,
OpenMP-threaded kernels; the reference itself is Swift/Metal and cannot be built on Linux) on a bounded
sample of the same workload, on rank 0 only.

Prints ONE JSON line on rank 0.
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
KERNEL_BYTES = ROWS * HIDDEN * 2 * 2  # bf16 read + bf16 write = 536 870 912


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


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

def cpu_norm_sweep(sample_rows: int, steps: int, warmup: int):
    import numpy as np

    import oracle

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
    return gbs, sec, oracle.max_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_rows = 4096
    gbs, sec, cores = cpu_norm_sweep(sample_rows, args.steps, args.warmup)
    sample = (f"{sample_rows} of {ROWS} rows x {HIDDEN}, fp32 host arrays, LayerNorm+RMSNorm+softmax per step; "
              "bytes counted as the bf16 workload's (4 B per element and kernel)")
    line = {
        "impl": "reference", "metric": "fused norm sweep throughput (LayerNorm+RMSNorm+softmax)", "value": gbs,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3 * ROWS / sample_rows, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "norms bf16-shaped [32768,4096] sweep, CPU restatement of the reference's host kernels",
                   "rows": ROWS, "hidden": HIDDEN, "eps": EPS},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------------

def run_ours(args):
    import torch
    import torch.distributed as dist

    from metalhlo_b200 import cuda  # raises if libmhlo_cuda.so is missing: no fallback

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG", "WARN")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)

    g = torch.Generator().manual_seed(42 + rank)
    x_host = torch.randn(ROWS, HIDDEN, generator=g).to(torch.bfloat16).pin_memory()
    gamma = (1 + 0.1 * torch.randn(HIDDEN, generator=g)).to(torch.bfloat16).to(dev)
    beta = (0.1 * torch.randn(HIDDEN, generator=g)).to(torch.bfloat16).to(dev)
    x = x_host.to(dev)
    x4 = (x.float() * 4).to(torch.bfloat16)
    y = [torch.empty_like(x) for _ in range(3)]
    stream = torch.cuda.current_stream()

    def step():
        cuda.layer_norm(x, gamma, beta, EPS, out=y[0])
        cuda.rms_norm(x, gamma, EPS, out=y[1])
        cuda.softmax(x4, out=y[2])

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()

    # ---- device-resident throughput: K steps, one event pair around the region + one pair per kernel ----
    names = ["layer_norm", "rms_norm", "softmax"]
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t_start = torch.cuda.Event(enable_timing=True)
    t_stop = torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    for k in range(args.steps):
        marks[k][0].record(stream)
        cuda.layer_norm(x, gamma, beta, EPS, out=y[0])
        marks[k][1].record(stream)
        cuda.rms_norm(x, gamma, EPS, out=y[1])
        marks[k][2].record(stream)
        cuda.softmax(x4, out=y[2])
        marks[k][3].record(stream)
    t_stop.record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    elapsed_ms = t_start.elapsed_time(t_stop)
    per_kernel_ms = {n: sum(marks[k][i].elapsed_time(marks[k][i + 1]) for k in range(args.steps)) / args.steps
                     for i, n in enumerate(names)}
    clocks = sampler.stop() if rank == 0 else None

    if args.kernels_only:
        if rank == 0:
            print(json.dumps({"kernels_only": True, "rows": ROWS, "per_kernel_gbs":
                              {n: KERNEL_BYTES / (per_kernel_ms[n] * 1e-3) / 1e9 for n in names}}))
        return

    # ---- end to end through the mhlo_* C API with HOST buffers: per step, mhlo_buffer_create copies x / gamma / beta
    # from (pinned) host memory, mhlo_execute runs the O3-compiled norm-sweep module, mhlo_buffer_to_host brings the three
    # results back. The calls are synchronous, so the step is timed on the host clock.
    import numpy as np

    from metalhlo_b200 import capi, modules

    client = capi.Client()
    exe = client.compile(modules.norm_sweep_module(ROWS, HIDDEN, "bf16", EPS), opt_level=3)
    assert sorted(s for s in exe.steps if s.startswith("fused")) == ["fused_layer_norm", "fused_rms_norm", "fused_softmax"], exe.steps
    g_host, b_host = gamma.cpu().pin_memory(), beta.cpu().pin_memory()
    y_host = [torch.empty_like(x_host).pin_memory() for _ in range(3)]
    nbytes = x_host.numel() * 2

    def e2e_step():
        ins = [client.buffer(x_host), client.buffer(g_host), client.buffer(b_host)]
        outs = exe.execute(ins)
        for o, dst in zip(outs, y_host):
            capi._check(capi.lib.mhlo_buffer_to_host(o._h, dst.data_ptr(), nbytes))
        del ins, outs

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    e2e_launches = exe.launch_count

    extra = None
    if not args.no_extras:
        del x, x4, y, y_host
        torch.cuda.empty_cache()
        extra = measure_extras(torch, dist, cuda, rank, world, dev, load_peaks())

    if world > 1:
        t = torch.tensor([elapsed_ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, e2e_ms = t.tolist()
        pk = torch.tensor([per_kernel_ms[n] for n in names], device=dev, dtype=torch.float64)
        dist.all_reduce(pk, op=dist.ReduceOp.MAX)
        per_kernel_ms = dict(zip(names, pk.tolist()))

    if rank == 0:
        peaks = load_peaks()
        step_bytes = 3 * KERNEL_BYTES
        value = world * step_bytes * args.steps / (elapsed_ms * 1e-3) / 1e9
        e2e_value = world * step_bytes * e2e_steps / (e2e_ms * 1e-3) / 1e9
        dom = max(names, key=lambda n: per_kernel_ms[n])
        achieved = KERNEL_BYTES / (per_kernel_ms[dom] * 1e-3) / 1e9
        cpu_gbs, _, cores = cpu_norm_sweep(2048, 3, 1) if world == 1 else (None, None, None)
        line = {
            "metric": "fused norm sweep throughput (LayerNorm+RMSNorm+softmax)",
            "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "norms bf16 [32768,4096] per GPU: LayerNorm, RMSNorm, softmax(x*4), fp32 statistics",
                       "rows_per_gpu": ROWS, "hidden": HIDDEN, "eps": EPS,
                       "l2": "inputs larger than L2 (268 MB read + 268 MB written per kernel)",
                       "parallelism": f"rows sharded x{world}, no collective"},
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                         "traffic": TRAFFIC_BYTES.get(dom),
                         "per_kernel_gbs": {n: KERNEL_BYTES / (per_kernel_ms[n] * 1e-3) / 1e9 for n in names}},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": nbytes + 4 * HIDDEN, "d2h_bytes_per_step": 3 * nbytes,
                    "steps": e2e_steps, "launches_per_step": e2e_launches,
                    "path": "mhlo_buffer_create (host->device) -> mhlo_execute of the O3 module -> mhlo_buffer_to_host x3"},
            "gpu_launches": 3 * args.steps,
            "clocks": clocks,
        }
        if extra is not None:
            line["extra"] = extra
        if cpu_gbs is not None:
            line["cpu_baseline"] = {
                "value": cpu_gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                "sample": f"2048 of {ROWS} rows x {HIDDEN}, fp32 host arrays, 3 timed sweeps; bytes counted as the "
                          "bf16 workload's (4 B per element and kernel)"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def measure_extras(torch, dist, cuda, rank, world, dev, peaks):
    """The other headline metrics of the hot path, each sharded the way its configuration prescribes and timed on the
    device (max over ranks): bf16 GEMM 8192^3 (column split + NCCL all-gather when world > 1), the HBM-limited batched
    GEMM, fused flash attention B8 H32 S4096 D128 (batch x head sharded), and the GPT-2-small forward pass (batch 32
    sharded). Returned as a dict for the "extra" key of the JSON line."""
    import math

    import numpy as np

    out = {}

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
    out["gemm_bf16_8192"] = {"tflops": tf, "ms": ms, "frac_of_measured_peak": tf / (peaks["bf16_tflops"] * world),
                             "parallelism": f"column split x{world}" + (" + NCCL all-gather + interleave" if world > 1 else "")}
    if world > 1:
        # The same product with the exchange fused into the GEMM: every rank's epilogue stores its column block into all
        # ranks' copies of C through peer addresses, then one tiny all-reduce tells every rank that all copies are complete.
        import ctypes as C

        own = C.c_void_p()
        cuda.check(cuda.lib.mhlo_cuda_alloc(n * n * 2, C.byref(own)))
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
        ab_str = cuda._i64s([n, 1])
        flag = torch.zeros(1, device=dev)

        def fused_step():
            cuda.check(cuda.lib.mhlo_cuda_gemm_all_gather(cuda.BF16, cuda.BF16, a.data_ptr(), ab_str, b_ptr, ab_str, c_ptrs, world, rank, n,
                                                          ncols, n, None, 0, stream))
            dist.all_reduce(flag)

        fused_step()
        torch.cuda.synchronize()
        dist.barrier()
        # correctness against the NCCL path of the same operands, on this rank's copy
        mine = torch.empty(n, n, device=dev, dtype=torch.bfloat16)
        cuda.check(cuda.lib.mhlo_cuda_copy(mine.data_ptr(), own, n * n * 2, stream))
        torch.cuda.synchronize()
        same = bool(torch.equal(mine.view(torch.int16), c_full.view(torch.int16)))
        ms_f = timed(fused_step, 10)
        tf_f = 2 * n ** 3 / ms_f / 1e9
        out["gemm_bf16_8192_fused_all_gather"] = {
            "tflops": tf_f, "ms": ms_f, "frac_of_measured_peak": tf_f / (peaks["bf16_tflops"] * world), "matches_nccl_path": same,
            "parallelism": f"column split x{world}, epilogue stores into every rank's C over NVLink, 1-element all-reduce as completion barrier"}
        assert cuda.device_error() == 0
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
                                "frac_of_measured_hbm": bytes_total / ms / 1e6 / (peaks["hbm_gbs"] * world)}
    del a, b, c
    # ---- flash attention B8 H32 S4096 D128 bf16, batch sharded
    bsz = max(1, sharding.contiguous_shard(8, world, rank).count)
    q, k, v = (torch.randn(bsz, 32, 4096, 128, device=dev, generator=g).to(torch.bfloat16) for _ in range(3))
    o = torch.empty_like(q)
    for causal, flop in ((False, 2_199_023_255_552), (True, 1_099_780_063_232)):
        ms = timed(lambda: cuda.attention(q, k, v, 1 / math.sqrt(128), causal=causal, out=o), 5)
        tf = flop * (bsz * world / 8) / ms / 1e9
        out["attention_causal" if causal else "attention"] = {"tflops": tf, "ms": ms,
                                                              "frac_of_measured_peak": tf / (peaks["bf16_tflops"] * world)}
    assert cuda.device_error() == 0, "a tensor-core kernel gave up on a bounded wait"
    del q, k, v, o
    # ---- GPT-2-small forward through the C API (O3), batch 32 sharded across ranks, fp16 compute, fp32 parameters
    from metalhlo_b200 import capi, modules

    batch = max(1, sharding.contiguous_shard(32, world, rank).count)
    text, params = modules.gpt2_module(batch=batch, seq=1024)
    client = capi.Client()
    exe = client.compile(text, opt_level=3)
    rng = np.random.default_rng(7)
    ins = []
    for name, shape, dt in params:
        if dt == "i32":
            arr = rng.integers(0, 50257, size=shape).astype(np.int32)
        elif name.endswith("_g"):
            arr = np.ones(shape, np.float32)
        elif name.endswith(("ln1_b", "ln2_b", "lnf_b")):
            arr = np.zeros(shape, np.float32)
        else:
            arr = (0.02 * rng.standard_normal(shape)).astype(np.float32)
        ins.append(client.buffer(arr))
    logits = torch.empty(batch, 1024, 50257, device=dev, dtype=torch.float16)
    in_ptrs = [b_.device_pointer for b_ in ins]

    # on its own stream, so that the executor may record the launch list once and replay it as a CUDA graph
    side = torch.cuda.Stream()

    def gpt2_step():
        exe.execute_on_device(in_ptrs, [logits.data_ptr()], side.cuda_stream)

    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ms = timed(gpt2_step, 5)
    torch.cuda.current_stream().wait_stream(side)
    out["gpt2_small_fwd"] = {"tokens_per_s": batch * world * 1024 / (ms * 1e-3), "ms": ms, "batch_per_gpu": batch, "seq": 1024,
                             "launches": exe.launch_count, "graph_replays": exe.graph_replays, "compute": "fp16, fp32 parameters converted inside the module",
                             "logits": "fp16 [batch,1024,50257], left sharded"}
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
    global ROWS, KERNEL_BYTES
    _reserve_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", default="norms")
    ap.add_argument("--rows", type=int, default=ROWS,
                    help="rows of the norm sweep (default: the benchmark configuration; smaller for profiler captures)")
    ap.add_argument("--no-extras", action="store_true", help="skip the GEMM / attention / GPT-2 side measurements")
    ap.add_argument("--kernels-only", action="store_true",
                    help="skip the end-to-end and CPU-baseline legs (profiler captures)")
    ap.add_argument("--profile-kernel", choices=["gemm", "attention", "attention_causal"] + sorted(MODULE_CASES),
                    help="run a few launches of one kernel (or one single-operator module) on a profiler-sized case and exit")
    args = ap.parse_args()
    if args.profile_kernel:
        profile_case(args.profile_kernel, max(1, min(args.steps, 5)))
        return
    if args.warmup < 3 and args.impl == "ours" and not args.kernels_only:
        args.warmup = 3
    ROWS = args.rows
    KERNEL_BYTES = ROWS * HIDDEN * 2 * 2
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
