#!/usr/bin/env python
"""Attention-forward benchmark: TFLOPS = 4*B*H*Lq*Lk*D / time on synthetic inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload main|...] [--impl reference]

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE). A step is one pass of the
attention kernel over one resident batch; every rank owns `batch` independent (batch, head)
slices of the global problem (no data-path collective), so scaling is weak: the global batch
is `batch * N`. Rank 0 prints one JSON line.

    value          device-timed TFLOPS, whole job, inputs already in HBM
    e2e            the same metric through the public API with host buffers: pinned host ->
                   device copies of Q, K, V and the device -> host copy of O inside the timed
                   region, every step
    roofline       tensor-core roofline of the attention kernel: achieved TFLOP/s per launch
                   (CUDA events on the launch stream) over the measured cuBLAS bf16 peak
    cpu_baseline   torch SDPA (math backend, fp32) on the host cores over a bounded sample of the
                   same workload; it is what the reference project checks its kernels against
    k18_same_gpu   the reference project's final kernel, built unmodified into baseline/_ref/,
                   timed on the same GPU and inputs (null when that library is absent)

`--impl reference` times the CPU arm alone (rank 0 only) and prints the same line shape.
`--workload dit_1056` times the video-DiT call sequence (528 self- and 528 cross-attention
launches per step) as one CUDA-graph replay per step, with the eager time beside it;
`--workload sp_ring` the sequence-parallel K/V ring (needs --gpus >= 2); `--workload main_strong`
splits the headline problem itself over the ranks (strong scaling; the default `main` gives every
rank its own copy of it, weak scaling).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

HEAD_DIM = 128
METRIC = "attention fwd TFLOPS & % of B200 BF16 tensor peak at 1/2/4/8 GPUs"

# name -> per-GPU (batch, heads, len_q, len_kv, layout)
WORKLOADS = {
    "main": (4, 16, 8192, 8192, "bhld"),          # B=4 H=16 L=8192: the headline config
    "main_bshd": (4, 16, 8192, 8192, "bshd"),
    "l1k": (64, 16, 1024, 1024, "bhld"),
    "l2k": (32, 16, 2048, 2048, "bhld"),
    "l4k": (16, 16, 4096, 4096, "bhld"),
    "l16k": (4, 16, 16384, 16384, "bhld"),
    "l32k": (2, 16, 32768, 32768, "bhld"),
    "dit_self": (1, 12, 32768, 32768, "bshd"),
    "dit_cross": (1, 12, 32768, 512, "bshd"),
    "smoke": (1, 4, 1024, 1024, "bhld"),
    "causal": (4, 16, 8192, 8192, "bhld"),        # the headline shape with a causal mask
    "causal_gqa": (4, 16, 8192, 8192, "bshd"),    # causal, 4 query heads per K/V head, token-major
}
# Variants of the operator: causal mask (bottom-right aligned) and K/V heads (grouped-query).
WORKLOAD_OPTIONS = {
    "causal": {"causal": True},
    "causal_gqa": {"causal": True, "heads_kv": 4},
}
# Sequence-parallel long-context workload: the GLOBAL problem (batch, heads, len) is fixed and
# split by query rows / key rows over the ranks (strong scaling; needs --gpus >= 2 to be a ring).
RING_WORKLOADS = {
    "sp_ring": (1, 32, 131072),
    "sp_ring_small": (1, 8, 16384),
}
# Strong scaling of one fixed problem: the (batch, head) slices of the GLOBAL shape are dealt to the
# ranks by sharding.plan (contiguous, near-equal pieces), every rank launches only its own.
STRONG_WORKLOADS = {
    "main_strong": (4, 16, 8192, 8192),
}
# Video-DiT call sequence: per generation 528 self-attention calls (B, H, L, L) and 528
# cross-attention calls (B, H, L, Lc), issued back to back on one stream; a step is the whole
# sequence of 1056 launches (replayed from a CUDA graph, and once eagerly for comparison).
SEQUENCE_WORKLOADS = {
    "dit_1056": (1, 12, 32768, 512, 528),
    "dit_1056_small": (1, 12, 4096, 512, 16),
}


# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu summary of the
# workload (profiles/attn_fwd_ws_kernel_*.md); None where nothing was captured.
NCU_TRAFFIC_BYTES = {"main": 515.5e6, "dit_cross": 155.0e6, "causal": 659.0e6}


def flops(b, h, lq, lk, causal=False):
    """4 * B * H * D * (query, key) pairs; with a causal mask only the visible pairs count."""
    pairs = lq * lk if not causal else lq * (lq + 1) // 2 + (lk - lq) * lq
    return 4.0 * b * h * pairs * HEAD_DIM


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            return {"bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)),
                    "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
        except Exception:
            pass
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0,
            "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "25"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # keep the samples taken under load (upper half by power) for the median
        if sm:
            cut = statistics.median(power) if len(power) > 3 else 0.0
            loaded = [c for c, w in zip(sm, power) if w >= cut] or sm
        else:
            loaded = []
        return {"sm_mhz": statistics.median(loaded) if loaded else None,
                "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# --------------------------------------------------------------------------------------------
# CPU arm: the reference project's own check call, torch SDPA math backend in fp32
# --------------------------------------------------------------------------------------------
def cpu_sdpa_sample(b, h, lq, lk, budget_s: float, max_heads: int | None = None, causal: bool = False):
    """Times torch SDPA (math, fp32, CPU) head by head on inputs of the workload's distribution
    until `budget_s` is spent. Returns (tflops, heads_done, seconds, cores)."""
    import torch

    from oracle import sdpa_oracle as O

    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core it may run on
    try:
        usable = len(os.sched_getaffinity(0))
    except AttributeError:
        usable = os.cpu_count() or 1
    if torch.get_num_threads() < usable:
        torch.set_num_threads(usable)
    cores = torch.get_num_threads()
    g = torch.Generator().manual_seed(0)
    total = b * h if max_heads is None else min(b * h, max_heads)
    # cap the rows of one timed slice so the fp32 score matrix stays below ~1 GiB
    rows = min(lq, max(256, (1 << 28) // max(lk, 1)))
    done_flops, heads, t_total = 0.0, 0, 0.0
    q = torch.randn(1, 1, rows, HEAD_DIM, generator=g).to(torch.bfloat16)
    k = torch.randn(1, 1, lk, HEAD_DIM, generator=g).to(torch.bfloat16)
    v = torch.randn(1, 1, lk, HEAD_DIM, generator=g).to(torch.bfloat16)
    O.sdpa_torch_math(q[:, :, :64], k, v)  # warm the thread pool
    # the causal form of the call applies to whole square problems only; otherwise the dense call
    # is timed and credited with the dense FLOPs
    causal = causal and rows == lq == lk
    while heads < total and t_total < budget_s:
        t0 = time.perf_counter()
        for r0 in range(0, lq, rows):
            O.sdpa_torch_math(q[:, :, : min(rows, lq - r0)], k, v, causal=causal)
            if time.perf_counter() - t0 + t_total > 3 * budget_s:
                break
        dt = time.perf_counter() - t0
        t_total += dt
        done_flops += flops(1, 1, lq, lk, causal)
        heads += 1
    return done_flops / t_total / 1e12, heads, t_total, cores


def run_reference_arm(args, rank, world):
    b, h, lq, lk, layout = WORKLOADS[args.workload]
    causal = bool(WORKLOAD_OPTIONS.get(args.workload, {}).get("causal", False))
    if rank != 0:
        return
    per_step_budget = max(1.0, min(20.0, 90.0 / max(args.steps + args.warmup, 1)))
    for _ in range(args.warmup):
        cpu_sdpa_sample(b, h, lq, lk, budget_s=per_step_budget / 4, max_heads=1, causal=causal)
    vals, heads_done, secs, cores = [], 0, 0.0, 0
    for _ in range(args.steps):
        tf, heads, t, cores = cpu_sdpa_sample(b, h, lq, lk, budget_s=per_step_budget, causal=causal)
        vals.append(tf)
        heads_done += heads
        secs += t
    value = statistics.mean(vals)
    sample = (f"torch scaled_dot_product_attention, math backend, fp32, CPU, {heads_done} (batch, head) "
              f"slices of Lq={lq} x Lk={lk} over {args.steps} steps, {secs:.1f} s, scaled by FLOPs")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": flops(b * world, h, lq, lk, causal) / (value * 1e12) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic", "config": workload_config(args.workload, world),
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": cores, "kind": "reference",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(name, world):
    b, h, lq, lk, layout = WORKLOADS[name]
    opts = WORKLOAD_OPTIONS.get(name, {})
    kind = "causal (bottom-right aligned)" if opts.get("causal") else "non-causal"
    kv = f", {opts['heads_kv']} K/V heads" if "heads_kv" in opts else ""
    return {"workload": f"{name}: dense {kind} attention forward, B={b} per GPU, H={h}{kv}, Lq={lq}, "
                        f"Lk={lk}, D=128, bf16 N(0,1), scale 1/sqrt(128), layout {layout.upper()}",
            "global_batch": b * world, "heads": h, "heads_kv": opts.get("heads_kv", h),
            "causal": bool(opts.get("causal", False)), "len_q": lq, "len_kv": lk, "head_dim": HEAD_DIM,
            "layout": layout, "parallelism": f"(batch,head)-sharded x{world}, no collective",
            "l2_policy": "inputs+outputs per step (Q,K,V,O) exceed the 126 MB L2; no flush"}


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def run_ours(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist

    from b200_attention_b200 import _native, ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    b, h, lq, lk, layout = WORKLOADS[args.workload]
    opts = WORKLOAD_OPTIONS.get(args.workload, {})
    causal, hk = bool(opts.get("causal", False)), int(opts.get("heads_kv", h))
    shape_q = (b, h, lq, HEAD_DIM) if layout == "bhld" else (b, lq, h, HEAD_DIM)
    shape_k = (b, hk, lk, HEAD_DIM) if layout == "bhld" else (b, lk, hk, HEAD_DIM)

    # host-side inputs (pinned) are the source for the e2e leg and for the resident copies
    g = torch.Generator().manual_seed(1234 + rank)
    q_h = torch.randn(shape_q, generator=g).to(torch.bfloat16).pin_memory()
    k_h = torch.randn(shape_k, generator=g).to(torch.bfloat16).pin_memory()
    v_h = torch.randn(shape_k, generator=g).to(torch.bfloat16).pin_memory()
    o_h = torch.empty(shape_q, dtype=torch.bfloat16).pin_memory()
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    o = torch.empty_like(q)
    stream = torch.cuda.current_stream(dev)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing
    for _ in range(args.warmup):
        ops.attention(q, k, v, layout=layout, out=o, causal=causal)
    barrier()
    _native.device_check()
    launches0 = _native.launch_count()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    evs[0].record(stream)
    for i in range(args.steps):
        ops.attention(q, k, v, layout=layout, out=o, causal=causal)
        evs[i + 1].record(stream)
    barrier()
    total_ms = evs[0].elapsed_time(evs[-1])
    per_launch = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    launches = _native.launch_count() - launches0
    _native.device_check()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = max_over_ranks(total_ms)
    ms_per_step = total_ms / args.steps
    step_flops_global = flops(b * world, h, lq, lk, causal)
    value = step_flops_global / (ms_per_step * 1e-3) / 1e12
    kernel_ms = statistics.mean(per_launch)
    achieved = flops(b, h, lq, lk, causal) / (kernel_ms * 1e-3) / 1e12

    # ---- end to end: host buffers in, host buffer out, through the public API. Every step copies
    # its Q, K, V from pinned host memory and its O back; HostPipeline overlaps the copies of
    # neighbouring steps with the kernel (double-buffered device slots, three streams).
    from b200_attention_b200.pipeline import HostPipeline

    e2e_steps = max(4, min(args.steps, 12))
    pipe = HostPipeline(shape_q, shape_k, layout=layout, device=dev, causal=causal)
    for _ in range(2):
        pipe.submit(q_h, k_h, v_h, o_h)
    pipe.finish()
    barrier()
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record(stream)
    pipe.s_in.wait_event(t_begin)
    for _ in range(e2e_steps):
        pipe.submit(q_h, k_h, v_h, o_h)
    for st in (pipe.s_in, pipe.s_run, pipe.s_out):
        done = torch.cuda.Event()
        done.record(st)
        stream.wait_event(done)
    t_end.record(stream)
    pipe.finish()
    barrier()
    _native.device_check()
    e2e_ms = max_over_ranks(t_begin.elapsed_time(t_end)) / e2e_steps
    e2e_value = step_flops_global / (e2e_ms * 1e-3) / 1e12
    in_bytes = (q_h.numel() + k_h.numel() + v_h.numel()) * 2
    out_bytes = o_h.numel() * 2

    # ---- the reference project's final kernel on the same GPU and inputs (rank 0, BHLD only)
    k18 = None
    if rank == 0 and not args.no_k18 and not opts:  # the reference's final kernel is dense and ungrouped
        k18 = time_k18(torch, q, k, v, layout, args)
    # ---- CPU baseline on a bounded sample (rank 0, single-GPU runs only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        tf, heads, secs, cores = cpu_sdpa_sample(b, h, lq, lk, budget_s=args.cpu_budget, causal=causal)
        cpu = {"value": tf, "unit": "TFLOPS", "cores": cores, "kind": "reference",
               "sample": (f"torch scaled_dot_product_attention (math backend, fp32, CPU: the call the "
                          f"reference checks its kernels against), {heads} of {b * h} (batch, head) "
                          f"slices of this workload, {secs:.1f} s, scaled by FLOPs")}

    if rank == 0:
        peaks = measured_peaks()
        traffic = NCU_TRAFFIC_BYTES.get(args.workload)
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(args.workload, world),
            "pct_of_bf16_peak": 100.0 * value / world / peaks["bf16_tflops"],
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                         "frac_of_sustained_peak": (achieved / peaks["bf16_tflops_sustained"]
                                                    if peaks["bf16_tflops_sustained"] else None),
                         "peak_source": f"{peaks['source']} cuBLAS bf16 burst",
                         "kernel_ms": kernel_ms, "traffic": traffic,
                         "hbm_gbs_algorithmic": (in_bytes + out_bytes) / (kernel_ms * 1e-3) / 1e9},
            "e2e": {"value": e2e_value, "unit": "TFLOPS", "h2d_bytes_per_step": in_bytes * world,
                    "d2h_bytes_per_step": out_bytes * world, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "cpu_baseline": cpu,
            "k18_same_gpu": k18,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_ring(args, rank, local_rank, world):
    """K/V ring over `world` GPUs: Q rows and K/V rows sharded, shards pulled over NVLink P2P,
    partial (O, LSE) merged in the kernel epilogue. value = global FLOPs / max-over-ranks time."""
    import torch
    import torch.distributed as dist

    from b200_attention_b200 import _native
    from b200_attention_b200.ring import RingAttention

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", device_id=dev, rank=rank, world_size=world)
    B, H, L = RING_WORKLOADS[args.workload]
    n = L // world
    g = torch.Generator().manual_seed(4321 + rank)
    host = [torch.randn(B, H, n, HEAD_DIM, generator=g).to(torch.bfloat16).pin_memory() for _ in range(3)]
    q, k, v = (t.to(dev) for t in host)
    o_host = torch.empty(B, H, n, HEAD_DIM, dtype=torch.bfloat16).pin_memory()
    ra = RingAttention()
    stream = torch.cuda.current_stream(dev)

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(args.warmup, 3)):
        ra.forward(q, k, v)
    launches0 = _native.launch_count()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    if rank == 0:
        sampler.start()
    torch.cuda.synchronize(dev)
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        ra.forward(q, k, v)
    e1.record(stream)
    torch.cuda.synchronize(dev)
    dist.barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    launches = _native.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    # end to end: shards from pinned host memory in, O back out, every step
    e2e_steps = max(2, min(args.steps, 3))
    e0.record(stream)
    for _ in range(e2e_steps):
        for d, h in zip((q, k, v), host):
            d.copy_(h, non_blocking=True)
        o, _ = ra.forward(q, k, v)
        o_host.copy_(o, non_blocking=True)
    e1.record(stream)
    torch.cuda.synchronize(dev)
    dist.barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    ra.unbind()
    total = flops(B, H, L, L)
    if rank == 0:
        peaks = measured_peaks()
        value = total / (ms * 1e-3) / 1e12
        shard_bytes = 2 * B * H * n * HEAD_DIM * 2
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{args.workload}: sequence-parallel K/V ring, global B={B} H={H} "
                                   f"Lq=Lk={L} D=128 bf16 N(0,1), Q and K/V rows sharded x{world}",
                       "global_batch": B, "heads": H, "len_q": L, "len_kv": L, "head_dim": HEAD_DIM,
                       "parallelism": f"sequence-parallel ring x{world}: NVLink P2P pulls into a local "
                                      "double buffer, (O, LSE) merged in the kernel epilogue, no collective",
                       "l2_policy": "per-step operands exceed the 126 MB L2; no flush"},
            "pct_of_bf16_peak": 100.0 * value / world / peaks["bf16_tflops"],
            "roofline": {"bound": "tensor", "achieved": value / world, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": value / world / peaks["bf16_tflops"],
                         "peak_source": f"{peaks['source']} cuBLAS bf16 burst", "traffic": None,
                         "nvlink_bytes_per_gpu_per_step": shard_bytes * (world - 1),
                         "nvlink_gbs_needed": shard_bytes * (world - 1) / (ms * 1e-3) / 1e9},
            "e2e": {"value": total / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                    "h2d_bytes_per_step": 3 * host[0].numel() * 2 * world,
                    "d2h_bytes_per_step": o_host.numel() * 2 * world, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches), "clocks": clocks, "cpu_baseline": None, "k18_same_gpu": None,
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def video_dit_inputs(torch, b, length, h, seed):
    """Q/K RMS-normalised per head and scaled by a per-channel N(0,1) gain, V ~ N(0,1): the value
    distribution of a DiT block after its QK-norm, token-major [B, L, H, 128]."""
    g = torch.Generator().manual_seed(seed)
    gain = torch.randn(HEAD_DIM, generator=g)
    out = []
    for normed in (True, True, False):
        x = torch.randn(b, length, h, HEAD_DIM, generator=g)
        if normed:
            x = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + 1e-6) * gain
        out.append(x.to(torch.bfloat16))
    return out


def run_sequence(args, rank, local_rank, world):
    """The video-DiT workload: `pairs` x (self-attention, cross-attention) launches per step on one
    stream, token-major (BSHD) operands used in place. Every rank runs its own replica of the
    sequence (the calls of one generation are sequentially dependent in the model; replicas stand
    for independent generations). value = global FLOPs / max-over-ranks time of the graph replay."""
    import torch
    import torch.distributed as dist

    from b200_attention_b200 import _native, ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    b, h, length, lc, pairs = SEQUENCE_WORKLOADS[args.workload]
    q_h, k_h, v_h = (t.pin_memory() for t in video_dit_inputs(torch, b, length, h, 77 + rank))
    _, kc_h, vc_h = (t.pin_memory() for t in video_dit_inputs(torch, b, lc, h, 99 + rank))
    o_h = torch.empty_like(q_h).pin_memory()
    q, k, v, kc, vc = (t.to(dev) for t in (q_h, k_h, v_h, kc_h, vc_h))
    o_self, o_cross = torch.empty_like(q), torch.empty_like(q)
    stream = torch.cuda.current_stream(dev)

    def sequence():
        for _ in range(pairs):
            ops.attention(q, k, v, layout="bshd", out=o_self)
            ops.attention(q, kc, vc, layout="bshd", out=o_cross)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    steps = args.steps if args.steps_given else 3
    warmup = max(args.warmup if args.warmup_given else 3, 3)
    ops.attention(q, k, v, layout="bshd", out=o_self)      # tensor maps cached, device set up
    ops.attention(q, kc, vc, layout="bshd", out=o_cross)
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sequence()
    for _ in range(warmup):
        graph.replay()
    barrier()
    _native.device_check()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(steps):
        graph.replay()
    e1.record(stream)
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / steps
    clocks = sampler.stop() if rank == 0 else None
    _native.device_check()
    # the same sequence launched eagerly through the public API, once
    launches0 = _native.launch_count()
    barrier()
    e0.record(stream)
    sequence()
    e1.record(stream)
    barrier()
    eager_ms = max_over_ranks(e0.elapsed_time(e1))
    eager_launches = _native.launch_count() - launches0
    # end to end: operands from pinned host memory in, the last O back out, every step
    e2e_steps = 2
    barrier()
    e0.record(stream)
    for _ in range(e2e_steps):
        for d, src in ((q, q_h), (k, k_h), (v, v_h), (kc, kc_h), (vc, vc_h)):
            d.copy_(src, non_blocking=True)
        graph.replay()
        o_h.copy_(o_self, non_blocking=True)
    e1.record(stream)
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    _native.device_check()

    step_flops = pairs * (flops(b, h, length, length) + flops(b, h, length, lc))
    if rank == 0:
        peaks = measured_peaks()
        value = step_flops * world / (ms * 1e-3) / 1e12
        cpu = None
        if world == 1 and not args.no_cpu:
            tf, heads, secs, cores = cpu_sdpa_sample(b, h, length, length, budget_s=args.cpu_budget)
            cpu = {"value": tf, "unit": "TFLOPS", "cores": cores, "kind": "reference",
                   "sample": (f"torch scaled_dot_product_attention (math backend, fp32, CPU), {heads} of "
                              f"{b * h} (batch, head) slices of one self-attention call, {secs:.1f} s, "
                              "scaled by FLOPs")}
        in_bytes = (q_h.numel() + k_h.numel() + v_h.numel() + kc_h.numel() + vc_h.numel()) * 2
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": (f"{args.workload}: video-DiT call sequence per GPU, {pairs} x (self-attention "
                                    f"B={b} H={h} Lq=Lk={length}; cross-attention Lq={length} Lk={lc}), D=128 bf16, "
                                    "Q/K RMS-normalised per head with N(0,1) gains, V ~ N(0,1), token-major "
                                    "BSHD in place, one CUDA-graph replay per step"),
                       "calls_per_step": 2 * pairs, "heads": h, "len_q": length, "len_kv": [length, lc],
                       "head_dim": HEAD_DIM, "layout": "bshd",
                       "parallelism": f"independent replicas x{world}, no collective",
                       "l2_policy": "operands of a self-attention call (288 MiB at L=32768) exceed the 126 MB L2; no flush"},
            "pct_of_bf16_peak": 100.0 * value / world / peaks["bf16_tflops"],
            "roofline": {"bound": "tensor", "achieved": value / world, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": value / world / peaks["bf16_tflops"],
                         "peak_source": f"{peaks['source']} cuBLAS bf16 burst", "traffic": None},
            "eager": {"ms_per_step": eager_ms, "value": step_flops * world / (eager_ms * 1e-3) / 1e12,
                      "launches": int(eager_launches)},
            "e2e": {"value": step_flops * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                    "h2d_bytes_per_step": in_bytes * world, "d2h_bytes_per_step": o_h.numel() * 2 * world,
                    "ms_per_step": e2e_ms},
            "gpu_launches": int(2 * pairs * steps), "clocks": clocks, "cpu_baseline": cpu,
            "k18_same_gpu": None,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_strong(args, rank, local_rank, world):
    """The headline problem (global B=4, H=16) split by (batch, head) over the ranks: strong
    scaling, no data-path collective. value = global FLOPs / max-over-ranks time."""
    import torch
    import torch.distributed as dist

    from b200_attention_b200 import _native, sharding

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    b, h, lq, lk = STRONG_WORKLOADS[args.workload]
    ranges = sharding.plan(b, h, world, rank)
    g = torch.Generator().manual_seed(1234)
    q_h = torch.randn(b, h, lq, HEAD_DIM, generator=g).to(torch.bfloat16).pin_memory()
    k_h = torch.randn(b, h, lk, HEAD_DIM, generator=g).to(torch.bfloat16).pin_memory()
    v_h = torch.randn(b, h, lk, HEAD_DIM, generator=g).to(torch.bfloat16).pin_memory()
    o_h = torch.empty_like(q_h).pin_memory()
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)   # inputs resident on every GPU before timing
    o = torch.empty_like(q)
    stream = torch.cuda.current_stream(dev)

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(args.warmup):
        sharding.run_shard(q, k, v, ranges, out=o)
    barrier()
    _native.device_check()
    launches0 = _native.launch_count()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for _ in range(args.steps):
        sharding.run_shard(q, k, v, ranges, out=o)
    e1.record(stream)
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    launches = _native.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    _native.device_check()
    # end to end: this rank's slices from pinned host memory in, its slices of O back out
    e2e_steps = max(2, min(args.steps, 6))
    barrier()
    e0.record(stream)
    for _ in range(e2e_steps):
        for r in ranges:
            sl = (slice(r.batch, r.batch + 1), slice(r.head_begin, r.head_end))
            for d, src in ((q, q_h), (k, k_h), (v, v_h)):
                d[sl].copy_(src[sl], non_blocking=True)
        sharding.run_shard(q, k, v, ranges, out=o)
        for r in ranges:
            sl = (slice(r.batch, r.batch + 1), slice(r.head_begin, r.head_end))
            o_h[sl].copy_(o[sl], non_blocking=True)
    e1.record(stream)
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    total = flops(b, h, lq, lk)
    if rank == 0:
        peaks = measured_peaks()
        value = total / (ms * 1e-3) / 1e12
        units = sharding.units_of(ranges)
        tile_bytes = lq * HEAD_DIM * 2
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": (f"{args.workload}: dense non-causal attention forward, GLOBAL B={b} H={h} "
                                    f"Lq={lq} Lk={lk} D=128 bf16 N(0,1), {b * h} (batch, head) slices dealt to "
                                    f"{world} rank(s), {units} on rank 0"),
                       "global_batch": b, "heads": h, "len_q": lq, "len_kv": lk, "head_dim": HEAD_DIM,
                       "layout": "bhld", "parallelism": f"(batch,head)-sharded x{world}, no collective",
                       "work_items_per_gpu": units * ((lq + 255) // 256),
                       "l2_policy": "per-step operands exceed the 126 MB L2 up to 4 GPUs; no flush"},
            "pct_of_bf16_peak": 100.0 * value / world / peaks["bf16_tflops"],
            "roofline": {"bound": "tensor", "achieved": value / world, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": value / world / peaks["bf16_tflops"],
                         "peak_source": f"{peaks['source']} cuBLAS bf16 burst", "traffic": None},
            "e2e": {"value": total / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                    "h2d_bytes_per_step": 3 * b * h * tile_bytes, "d2h_bytes_per_step": b * h * tile_bytes,
                    "ms_per_step": e2e_ms},
            "gpu_launches": int(launches), "clocks": clocks, "cpu_baseline": None, "k18_same_gpu": None,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def time_k18(torch, q, k, v, layout, args):
    try:
        from baseline import k18 as R
    except Exception:
        return None
    fn = None
    if R.available(layout):
        fn = R.bhld if layout == "bhld" else R.bshd
    lq = q.shape[2] if layout == "bhld" else q.shape[1]
    lk = k.shape[2] if layout == "bhld" else k.shape[1]
    if fn is None or lq % 256 or lk % 128:
        return None
    b, h = (q.shape[0], q.shape[1]) if layout == "bhld" else (q.shape[0], q.shape[2])
    for _ in range(max(3, args.warmup)):
        fn(q, k, v)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn(q, k, v)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    return {"tflops": flops(b, h, lq, lk) / (ms * 1e-3) / 1e12, "ms": ms,
            "what": "reference final checkpoint kernel (18_tma_l2_promotion), unmodified, same GPU, "
                    "includes its per-call tensor-map encoding"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="main",
                    choices=sorted(WORKLOADS) + sorted(RING_WORKLOADS) + sorted(SEQUENCE_WORKLOADS)
                    + sorted(STRONG_WORKLOADS))
    ap.add_argument("--layout", default=None, choices=["bhld", "bshd"],
                    help="override the workload's operand layout (single-launch workloads)")
    ap.add_argument("--no-k18", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cpu-budget", type=float, default=12.0)
    args = ap.parse_args()
    args.steps_given, args.warmup_given = args.steps is not None, args.warmup is not None
    args.steps = 100 if args.steps is None else args.steps
    args.warmup = 5 if args.warmup is None else args.warmup
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.layout is not None and args.workload in WORKLOADS:
        WORKLOADS[args.workload] = WORKLOADS[args.workload][:4] + (args.layout,)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if args.workload in RING_WORKLOADS:
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  "the reference project has no sequence-parallel path; use --workload main"}))
            return
        run_ring(args, rank, local_rank, world)
        return
    if args.workload in STRONG_WORKLOADS:
        if args.impl == "reference":
            args.workload = "main"  # the CPU arm times the same global problem
            run_reference_arm(args, rank, 1)
            return
        run_strong(args, rank, local_rank, world)
        return
    if args.workload in SEQUENCE_WORKLOADS:
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  "the CPU arm times single calls; use --workload dit_self or dit_cross"}))
            return
        run_sequence(args, rank, local_rank, world)
        return
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
