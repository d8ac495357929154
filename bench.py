#!/usr/bin/env python
"""Attention-forward benchmark: TFLOPS = 4*B*H*Lq*Lk*D / time on synthetic inputs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload main|...] [--impl reference]

One process per GPU (torchrun sets RANK / LOCAL_RANK / WORLD_SIZE). A step is one pass of the
attention kernel over one resident problem. Rank 0 prints one JSON line.

Default workload `main` (B=4, H=16, Lq=Lk=8192, D=128, bf16, BHLD):
  * 1 GPU: the whole problem on the one GPU.
  * N GPUs: the ONE problem's 64 (batch, head) slices are dealt to the ranks (no data-path
    collective), `scaling` = "strong"; the figure for N independent copies of the problem (one per
    GPU) is reported beside it under `weak`.

Keys of the line:
    value          device-timed TFLOPS over exactly --steps launches, inputs already in HBM
    burst / sustained
                   the same kernel over the --steps launches (tens of milliseconds: the power
                   limiter has not engaged yet) and over >= 1 s of back-to-back launches after
                   >= 0.5 s of warm-up (the power-capped regime), each with the SM clock averaged
                   over exactly its own region (SM cycle counters against the global timer) and the
                   region's length in SM cycles, so the two regimes can be compared in cycles
    k18_same_gpu   the reference project's final kernel, built unmodified into baseline/_ref/,
                   against this library's kernel on the same GPU and inputs, arms alternated
                   A-B-B-A with a pause between arms, burst and sustained
    configs        the other benchmark configurations (sequence-length sweep in both layouts, the
                   video-DiT self- and cross-attention shapes), a few launches each: this kernel,
                   the reference kernel, % of the measured bf16 peak, algorithmic HBM GB/s
    e2e            the same metric through the public API with host buffers: pinned host -> device
                   copies of Q, K, V and the device -> host copy of O inside the timed region, every
                   step; `copy_floor_ms` is the time the same copies take with no kernel at all
    roofline       tensor-core roofline of the attention kernel: achieved TFLOP/s per launch
                   (CUDA events on the launch stream) over the measured cuBLAS bf16 peak
    cpu_baseline   torch SDPA (math backend, fp32) on the host cores over a bounded sample of the
                   same workload; it is what the reference project checks its kernels against

`--impl reference` times the CPU arm alone (rank 0 only) and prints the same line shape.
Other workloads: `--workload dit_1056` (the video-DiT call sequence, 528 self- and 528
cross-attention launches per step, one CUDA-graph replay per step), `--workload sp_ring` (the
sequence-parallel K/V ring, needs --gpus >= 2; `--check` verifies sampled rows of the result
against the CPU oracle), `--workload main_weak` (every rank its own copy of the main problem),
and the single shapes of the `configs` block by name.
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

# name -> (batch, heads, len_q, len_kv, layout)
WORKLOADS = {
    "main": (4, 16, 8192, 8192, "bhld"),          # B=4 H=16 L=8192: the headline config
    "main_weak": (4, 16, 8192, 8192, "bhld"),     # one copy of it per GPU
    "main_bshd": (4, 16, 8192, 8192, "bshd"),
    "main_rank8": (1, 8, 8192, 8192, "bhld"),     # what one of 8 GPUs owns of the headline problem
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
# The `configs` block of the default line: (name, layouts).
CONFIG_SWEEP = [("l1k", ("bhld", "bshd")), ("l2k", ("bhld", "bshd")), ("l4k", ("bhld", "bshd")),
                ("main", ("bhld", "bshd")), ("l16k", ("bhld", "bshd")), ("l32k", ("bhld", "bshd")),
                ("dit_self", ("bshd",)), ("dit_cross", ("bshd",))]
# Sequence-parallel long-context workload: the GLOBAL problem (batch, heads, len) is fixed and
# split by query rows / key rows over the ranks (strong scaling; needs --gpus >= 2 to be a ring).
RING_WORKLOADS = {
    "sp_ring": (1, 32, 131072),
    "sp_ring_small": (1, 8, 16384),
}
# Video-DiT call sequence: per generation 528 self-attention calls (B, H, L, L) and 528
# cross-attention calls (B, H, L, Lc), issued back to back on one stream; a step is the whole
# sequence of 1056 launches (replayed from a CUDA graph, and once eagerly for comparison).
SEQUENCE_WORKLOADS = {
    "dit_1056": (1, 12, 32768, 512, 528),
    "dit_1056_small": (1, 12, 4096, 512, 16),
}

# dram__bytes_read.sum + dram__bytes_write.sum per launch, copied from the committed ncu summary
# of the workload (an earlier capture of this kernel, not a measurement of this run).
NCU_TRAFFIC = {
    "main": (515.5e6, "profiles/attn_fwd_ws_kernel_main_B4_H16_L8192.md"),
    "dit_cross": (155.0e6, "profiles/attn_fwd_ws_kernel_dit_cross_B1_H12_Lq32768_Lk512.md"),
    "causal": (681.0e6, "profiles/attn_fwd_ws_kernel_causal_B4_H16_L8192.md"),
}


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
    """Samples nvidia-smi clocks and throttle reasons of one GPU while a timed region runs."""

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
                 "-i", str(self.index), "-lms", "20"],
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
        cut = statistics.median(power) if len(power) > 3 else 0.0
        loaded = [(c, w) for c, w in zip(sm, power) if w >= cut] or list(zip(sm, power))
        return {"sm_mhz": statistics.median(c for c, _ in loaded) if loaded else None,
                "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None,
                "power_w_median_loaded": statistics.median(w for _, w in loaded) if loaded else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_under_load": len(loaded)}


class SmClock:
    """Average SM clock over a stream-ordered region, from the SMs' own cycle counters: a tiny
    kernel of the library records (clock64, globaltimer) per SM before and after the region."""

    MAX_SMS = 256

    def __init__(self, torch, native, dev):
        self.lib = native.lib()
        self.check = native.check
        self.a = torch.zeros(2 * self.MAX_SMS, dtype=torch.int64, device=dev)
        self.b = torch.zeros(2 * self.MAX_SMS, dtype=torch.int64, device=dev)

    def before(self, stream):
        self.a.zero_()
        self.check(self.lib.b200attn_sample_sm_clocks(self.a.data_ptr(), self.MAX_SMS, stream.cuda_stream))

    def after(self, stream):
        self.b.zero_()
        self.check(self.lib.b200attn_sample_sm_clocks(self.b.data_ptr(), self.MAX_SMS, stream.cuda_stream))

    def mhz(self):
        """Median over the SMs seen by both samples; None if there is none. Synchronise first."""
        a = self.a.view(-1, 2).cpu()
        b = self.b.view(-1, 2).cpu()
        ok = (a[:, 1] > 0) & (b[:, 1] > a[:, 1])
        if not bool(ok.any()):
            return None
        cyc = (b[ok, 0] - a[ok, 0]).double()
        ns = (b[ok, 1] - a[ok, 1]).double()
        return float((cyc / ns * 1e3).median())


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
    """Times torch SDPA (math, fp32, CPU) head by head, in row blocks, on inputs of the workload's
    distribution until `budget_s` is spent; only the (row block x all keys) slices actually
    computed are credited. Returns (tflops, heads_started, seconds, cores, rows_done)."""
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
    q = torch.randn(1, 1, rows, HEAD_DIM, generator=g).to(torch.bfloat16)
    k = torch.randn(1, 1, lk, HEAD_DIM, generator=g).to(torch.bfloat16)
    v = torch.randn(1, 1, lk, HEAD_DIM, generator=g).to(torch.bfloat16)
    O.sdpa_torch_math(q[:, :, :64], k, v)  # warm the thread pool
    # the causal form of the call applies to whole square problems only; otherwise the dense call
    # is timed and credited with the dense FLOPs
    causal = causal and rows == lq == lk
    done_flops, heads, t_total, rows_done = 0.0, 0, 0.0, 0
    while heads < total and t_total < budget_s:
        heads += 1
        for r0 in range(0, lq, rows):
            n = min(rows, lq - r0)
            t0 = time.perf_counter()
            O.sdpa_torch_math(q[:, :, :n], k, v, causal=causal)
            t_total += time.perf_counter() - t0
            done_flops += flops(1, 1, lq, lk, True) if causal else flops(1, 1, n, lk)
            rows_done += n
            if t_total >= budget_s:
                break
    return done_flops / t_total / 1e12, heads, t_total, cores, rows_done


def run_reference_arm(args, rank, world):
    b, h, lq, lk, layout = WORKLOADS[args.workload]
    causal = bool(WORKLOAD_OPTIONS.get(args.workload, {}).get("causal", False))
    if rank != 0:
        return
    per_step_budget = max(1.0, min(20.0, 90.0 / max(args.steps + args.warmup, 1)))
    for _ in range(args.warmup):
        cpu_sdpa_sample(b, h, lq, lk, budget_s=per_step_budget / 4, max_heads=1, causal=causal)
    vals, rows_done, secs, cores = [], 0, 0.0, 0
    for _ in range(args.steps):
        tf, _, t, cores, rows = cpu_sdpa_sample(b, h, lq, lk, budget_s=per_step_budget, causal=causal)
        vals.append(tf)
        rows_done += rows
        secs += t
    value = statistics.mean(vals)
    sample = (f"torch scaled_dot_product_attention, math backend, fp32, CPU, {rows_done} query rows x "
              f"Lk={lk} of (batch, head) slices of this workload over {args.steps} steps, {secs:.1f} s, "
              "scaled by FLOPs")
    weak = args.workload != "main" and world > 1
    global_batch = b * world if weak else b
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": flops(global_batch, h, lq, lk, causal) / (value * 1e12) * 1e3,
        "higher_is_better": True, "scaling": scaling_of(args.workload, world), "vs_baseline": None,
        "dtype": "fp32", "data": "synthetic", "config": workload_config(args.workload, world),
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": cores, "kind": "reference",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def scaling_of(name, world):
    """`main` on several GPUs is one problem dealt to the ranks; every other single-launch
    workload gives each rank its own copy."""
    return "strong" if name == "main" else "weak"


def workload_config(name, world):
    b, h, lq, lk, layout = WORKLOADS[name]
    opts = WORKLOAD_OPTIONS.get(name, {})
    kind = "causal (bottom-right aligned)" if opts.get("causal") else "non-causal"
    kv = f", {opts['heads_kv']} K/V heads" if "heads_kv" in opts else ""
    split = name == "main" and world > 1
    weak = name != "main" and world > 1
    input_bytes = (b * h * lq + 2 * b * opts.get("heads_kv", h) * lk) * HEAD_DIM * 2 // (world if split else 1)
    where = (f"GLOBAL B={b}, its {b * h} (batch, head) slices dealt to {world} GPUs" if split
             else f"B={b} per GPU" if weak else f"B={b}")
    return {"workload": f"{name}: dense {kind} attention forward, {where}, H={h}{kv}, Lq={lq}, "
                        f"Lk={lk}, D=128, bf16 N(0,1), scale 1/sqrt(128), layout {layout.upper()}",
            "global_batch": b * world if weak else b, "heads": h, "heads_kv": opts.get("heads_kv", h),
            "causal": bool(opts.get("causal", False)), "len_q": lq, "len_kv": lk, "head_dim": HEAD_DIM,
            "layout": layout,
            "parallelism": (f"(batch,head)-sharded x{world}, no collective" if world > 1 else "single GPU"),
            "l2_policy": l2_policy_text(input_bytes)}


# --------------------------------------------------------------------------------------------
# timing helpers (device side)
# --------------------------------------------------------------------------------------------
L2_BYTES = 126e6
FLUSH_BYTES = 256 << 20


def flush_buffer_for(torch, dev, input_bytes):
    """Inputs that fit the L2 would be served from it by the second launch on: such workloads get
    a buffer twice the L2's size that is rewritten before every timed launch. None otherwise."""
    if input_bytes > L2_BYTES:
        return None
    return torch.empty(FLUSH_BYTES, dtype=torch.uint8, device=dev)


def l2_policy_text(input_bytes):
    if input_bytes > L2_BYTES:
        return f"inputs per step (Q,K,V: {input_bytes / 1e6:.0f} MB) exceed the 126 MB L2; no flush"
    return (f"inputs per step (Q,K,V: {input_bytes / 1e6:.0f} MB) fit the 126 MB L2: a {FLUSH_BYTES >> 20} MiB buffer "
            "is rewritten before every timed launch, outside the launch's own pair of events")


def time_launches(torch, call, n, stream, smclock=None, per_launch=False, flush=None):
    """n calls on `stream`; returns (total_ms, [per-launch ms] or None, sm_mhz). Back to back
    between two events; with a `flush` buffer every call has its own pair of events, the buffer
    is rewritten between the pairs and the total is the sum over the pairs."""
    if flush is not None:
        pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        if smclock is not None:
            smclock.before(stream)
        for a, b in pairs:
            flush.zero_()
            a.record(stream)
            call()
            b.record(stream)
        if smclock is not None:
            smclock.after(stream)
        stream.synchronize()
        each = [a.elapsed_time(b) for a, b in pairs]
        return sum(each), (each if per_launch else None), (smclock.mhz() if smclock is not None else None)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(n + 1 if per_launch else 2)]
    if smclock is not None:
        smclock.before(stream)
    evs[0].record(stream)
    for i in range(n):
        call()
        if per_launch:
            evs[i + 1].record(stream)
    if not per_launch:
        evs[1].record(stream)
    if smclock is not None:
        smclock.after(stream)
    stream.synchronize()
    total = evs[0].elapsed_time(evs[-1])
    each = [evs[i].elapsed_time(evs[i + 1]) for i in range(n)] if per_launch else None
    return total, each, (smclock.mhz() if smclock is not None else None)


def regime(total_ms, n, step_flops, mhz):
    ms = total_ms / n
    out = {"launches": n, "ms_per_launch": ms, "tflops": step_flops / (ms * 1e-3) / 1e12,
           "sm_mhz_avg": mhz}
    if mhz:
        out["sm_cycles_per_launch"] = ms * 1e-3 * mhz * 1e6
    return out


def sustained_region(torch, call, est_ms, stream, smclock, warm_s=0.5, timed_s=1.0, flush=None):
    warm = max(3, int(warm_s * 1e3 / max(est_ms, 1e-3)) + 1)
    n = max(10, int(timed_s * 1e3 / max(est_ms, 1e-3)) + 1)
    for _ in range(warm):
        call()
    total, _, mhz = time_launches(torch, call, n, stream, smclock, flush=flush)
    return total, n, mhz


def k18_call(torch, q, k, v, layout):
    """A zero-argument launcher of the reference's final kernel on these operands, or None."""
    try:
        from baseline import k18 as R
    except Exception:
        return None
    lq = q.shape[2] if layout == "bhld" else q.shape[1]
    lk = k.shape[2] if layout == "bhld" else k.shape[1]
    h_axis = 1 if layout == "bhld" else 2
    if not R.available(layout) or not R.supports(lq, lk) or q.shape[h_axis] != k.shape[h_axis]:
        return None  # (the reference kernel has no grouped K/V heads and needs Lq % 256 == Lk % 128 == 0)
    out = torch.empty_like(q)
    fn = R.bhld if layout == "bhld" else R.bshd
    return lambda: fn(q, k, v, out=out)


def compare_with_k18(torch, ours, theirs, step_flops, stream, smclock, burst_n, rounds=2, pause_s=1.0,
                     sustain_s=1.0):
    """Arms alternated ours, k18, k18, ours, ... with a pause before every arm (the reference's own
    harness alternates arm order and sleeps between arms, benchmarks/benchmark.py:255-260)."""
    res = {"ours": {"burst": [], "sustained": []}, "k18": {"burst": [], "sustained": []}}
    order = []
    for r in range(rounds):
        order += ["ours", "k18"] if r % 2 == 0 else ["k18", "ours"]
    for arm in order:
        call = ours if arm == "ours" else theirs
        time.sleep(pause_s)
        for _ in range(3):
            call()
        total, _, mhz = time_launches(torch, call, burst_n, stream, smclock)
        res[arm]["burst"].append(regime(total, burst_n, step_flops, mhz))
        total, n, mhz = sustained_region(torch, call, total / burst_n, stream, smclock, warm_s=0.3,
                                         timed_s=sustain_s)
        res[arm]["sustained"].append(regime(total, n, step_flops, mhz))
    out = {"what": "reference final checkpoint kernel (18_tma_l2_promotion), unmodified, same GPU and "
                   "inputs, includes its per-call tensor-map encoding; arms alternated "
                   + " ".join(order) + f", {pause_s:.1f} s pause before each arm",
           "order": order}

    def mean(arm, mode, key):
        vals = [x[key] for x in res[arm][mode] if x.get(key)]
        return statistics.mean(vals) if vals else None

    for mode in ("burst", "sustained"):
        o, t = mean("ours", mode, "tflops"), mean("k18", mode, "tflops")
        out[mode] = {"ours_tflops": o, "k18_tflops": t, "ratio": o / t,
                     "ours_runs": [round(x["tflops"], 1) for x in res["ours"][mode]],
                     "k18_runs": [round(x["tflops"], 1) for x in res["k18"][mode]],
                     "ours_sm_cycles_per_launch": mean("ours", mode, "sm_cycles_per_launch"),
                     "k18_sm_cycles_per_launch": mean("k18", mode, "sm_cycles_per_launch"),
                     "ours_sm_mhz": mean("ours", mode, "sm_mhz_avg"),
                     "k18_sm_mhz": mean("k18", mode, "sm_mhz_avg")}
    out["tflops"] = out["burst"]["k18_tflops"]
    return out


def configs_block(torch, ops, dev, stream, peaks, launches=10):
    """The other benchmark configurations, a few launches each (inputs drawn on the GPU), this
    kernel and the reference kernel alternated so that neither always runs on the warmer GPU."""
    out = {}
    g = torch.Generator(device=dev).manual_seed(7)
    for name, layouts in CONFIG_SWEEP:
        b, h, lq, lk, _ = WORKLOADS[name]
        for layout in layouts:
            def mk(length):
                shape = (b, h, length, HEAD_DIM) if layout == "bhld" else (b, length, h, HEAD_DIM)
                return torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)

            q, k, v = mk(lq), mk(lk), mk(lk)
            if name.startswith("dit_"):
                # the video model's QK-norm: per-head RMS normalisation times a per-channel gain
                gain = torch.randn(HEAD_DIM, generator=g, device=dev)
                q, k = ((x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
                         * gain).to(torch.bfloat16) for x in (q, k))
            o = torch.empty_like(q)

            def ours():
                ops.attention(q, k, v, layout=layout, out=o)

            fl = flops(b, h, lq, lk)
            flush = flush_buffer_for(torch, dev, (q.numel() + 2 * k.numel()) * 2)
            theirs = k18_call(torch, q, k, v, layout)
            arms = {"ours": ours} if theirs is None else {"ours": ours, "k18": theirs}
            times = {arm: [] for arm in arms}
            for order in (("ours", "k18"), ("k18", "ours")):   # each arm once first, once second
                for arm in order:
                    if arm not in arms:
                        continue
                    # every arm starts from the same short idle: without it the arm that runs last
                    # in a row of four inherits the others' heat and falls off the boost clock first
                    torch.cuda.synchronize(dev)
                    time.sleep(0.25)
                    for _ in range(3):
                        arms[arm]()
                    total, _, _ = time_launches(torch, arms[arm], launches, stream, flush=flush)
                    times[arm].append(total / launches)
            ms = statistics.mean(times["ours"])
            entry = {"tflops": fl / (ms * 1e-3) / 1e12, "ms": ms}
            entry["pct_of_bf16_peak"] = 100.0 * entry["tflops"] / peaks["bf16_tflops"]
            nbytes = (2 * q.numel() + 2 * k.numel()) * 2
            entry["hbm_gbs_algorithmic"] = nbytes / (ms * 1e-3) / 1e9
            entry["pct_of_hbm_peak"] = 100.0 * entry["hbm_gbs_algorithmic"] / peaks["hbm_gbs"]
            if theirs is not None:
                entry["k18_tflops"] = fl / (statistics.mean(times["k18"]) * 1e-3) / 1e12
                entry["ratio_to_k18"] = entry["tflops"] / entry["k18_tflops"]
            if flush is not None:
                entry["l2_flushed"] = True
            out[f"{name}_{layout}"] = {k_: (round(v_, 3) if isinstance(v_, float) else v_)
                                       for k_, v_ in entry.items()}
            del q, k, v, o, theirs, flush
            torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------------------------
# GPU arm: single-launch workloads
# --------------------------------------------------------------------------------------------
def run_ours(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist

    from b200_attention_b200 import _native, ops, sharding
    from b200_attention_b200.pipeline import HostPipeline

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    b, h, lq, lk, layout = WORKLOADS[args.workload]
    opts = WORKLOAD_OPTIONS.get(args.workload, {})
    causal, hk = bool(opts.get("causal", False)), int(opts.get("heads_kv", h))
    split = args.workload == "main" and world > 1   # the one problem dealt to the ranks
    shape_q = (b, h, lq, HEAD_DIM) if layout == "bhld" else (b, lq, h, HEAD_DIM)
    shape_k = (b, hk, lk, HEAD_DIM) if layout == "bhld" else (b, lk, hk, HEAD_DIM)

    # host-side inputs (pinned) are the source for the e2e leg and for the resident copies
    g = torch.Generator().manual_seed(1234 + (0 if split else rank))
    q_h = torch.randn(shape_q, generator=g).to(torch.bfloat16).pin_memory()
    k_h = torch.randn(shape_k, generator=g).to(torch.bfloat16).pin_memory()
    v_h = torch.randn(shape_k, generator=g).to(torch.bfloat16).pin_memory()
    o_h = torch.empty(shape_q, dtype=torch.bfloat16).pin_memory()
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    o = torch.empty_like(q)
    stream = torch.cuda.current_stream(dev)
    smclock = SmClock(torch, _native, dev)
    ranges = sharding.plan(b, h, world, rank) if split else None

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

    def whole():
        ops.attention(q, k, v, layout=layout, out=o, causal=causal)

    def shard():
        sharding.run_shard(q, k, v, ranges, out=o)

    step = shard if split else whole
    # a rank whose inputs fit the L2 rewrites a larger buffer before every timed launch
    rank_units = sharding.units_of(ranges) if split else b * h
    rank_input_bytes = (rank_units * lq + 2 * (rank_units * hk // h) * lk) * HEAD_DIM * 2
    flush = flush_buffer_for(torch, dev, rank_input_bytes)
    # FLOPs of one step on this rank and of one step of the whole job
    rank_flops = flops(sharding.units_of(ranges), 1, lq, lk) if split else flops(b, h, lq, lk, causal)
    job_flops = flops(b, h, lq, lk, causal) * (1 if split or world == 1 else world)

    # ---- the contract's region: W warm-up launches, exactly K timed launches
    for _ in range(args.warmup):
        step()
    barrier()
    _native.device_check()
    launches0 = _native.launch_count()
    barrier()
    # one event before the first launch and one after the last: an event between two launches
    # would keep the second from starting the moment the first ends
    total_ms, _, burst_mhz = time_launches(torch, step, args.steps, stream, smclock, flush=flush)
    launches = _native.launch_count() - launches0
    barrier()
    _native.device_check()
    kernel_ms = total_ms / args.steps   # this rank's own time per step
    total_ms = max_over_ranks(total_ms)
    ms_per_step = total_ms / args.steps
    value = job_flops / (ms_per_step * 1e-3) / 1e12
    achieved = rank_flops / (kernel_ms * 1e-3) / 1e12
    burst = regime(total_ms, args.steps, job_flops, burst_mhz)
    if args.only_timed:
        # profiling aid: the contract's region only (plus, if asked, a few launches of the reference
        # kernel for a counter-by-counter comparison under the same profiler)
        if rank == 0 and args.k18_launches > 0:
            theirs = k18_call(torch, q, k, v, layout)
            for _ in range(args.k18_launches if theirs is not None else 0):
                theirs()
            torch.cuda.synchronize(dev)
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world,
                              "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
                              "burst": burst, "gpu_launches": int(launches), "only_timed": True,
                              "config": workload_config(args.workload, world)}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- the power-capped regime: >= 0.5 s of warm-up, >= 1 s timed, clocks sampled over it
    sampler = ClockSampler(physical_gpu_index(local_rank))
    barrier()
    if rank == 0:
        sampler.start()
        time.sleep(0.15)
    for _ in range(max(3, int(500.0 / max(ms_per_step, 1e-3)) + 1)):
        step()
    barrier()
    n_sus = max(10, int(args.sustain_s * 1e3 / max(ms_per_step, 1e-3)) + 1)
    sus_ms, _, sus_mhz = time_launches(torch, step, n_sus, stream, smclock, flush=flush)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    _native.device_check()
    sustained = regime(max_over_ranks(sus_ms), n_sus, job_flops, sus_mhz)

    # ---- N > 1: N independent copies of the problem, one per GPU, beside the split
    weak = None
    if split:
        for _ in range(3):
            whole()
        barrier()
        w_ms, _, _ = time_launches(torch, whole, args.steps, stream)
        barrier()
        w_ms = max_over_ranks(w_ms) / args.steps
        weak = {"value": flops(b * world, h, lq, lk) / (w_ms * 1e-3) / 1e12, "unit": "TFLOPS",
                "ms_per_step": w_ms, "global_batch": b * world,
                "what": f"{world} independent copies of the problem, one per GPU, {args.steps} launches"}

    # ---- end to end: host buffers in, host buffer out, through the public API. Every step copies
    # its Q, K, V from pinned host memory and its O back; HostPipeline overlaps the copies of
    # neighbouring steps with the kernel (double-buffered device slots, three streams). With the
    # problem split over ranks, each rank moves only its own (batch, head) slices.
    if split:
        sl = [(slice(r.batch, r.batch + 1), slice(r.head_begin, r.head_end)) for r in ranges]
        views = [(q_h[s], k_h[s], v_h[s], o_h[s]) for s in sl]
        # a slice of the pinned tensors is contiguous here (whole heads of one batch entry)
        views = [tuple(t if t.is_contiguous() else t.contiguous().pin_memory() for t in view) for view in views]
    else:
        views = [(q_h, k_h, v_h, o_h)]
    in_bytes = sum((a.numel() + b_.numel() + c.numel()) * 2 for a, b_, c, _ in views)
    out_bytes = sum(d.numel() * 2 for _, _, _, d in views)
    e2e_steps = max(4, min(args.steps, 12))
    pipes = [HostPipeline(tuple(a.shape), tuple(b_.shape), layout=layout, device=dev, causal=causal)
             for a, b_, _, _ in views]

    def e2e_step():
        for pipe, (a, b_, c, d) in zip(pipes, views):
            pipe.submit(a, b_, c, d)

    def join(streams):
        for st in streams:
            done = torch.cuda.Event()
            done.record(st)
            stream.wait_event(done)

    for _ in range(2):
        e2e_step()
    for pipe in pipes:
        pipe.finish()
    barrier()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin.record(stream)
    for pipe in pipes:
        pipe.s_in.wait_event(t_begin)
    for _ in range(e2e_steps):
        e2e_step()
    join([st for pipe in pipes for st in (pipe.s_in, pipe.s_run, pipe.s_out)])
    t_end.record(stream)
    for pipe in pipes:
        pipe.finish()
    barrier()
    _native.device_check()
    e2e_ms = max_over_ranks(t_begin.elapsed_time(t_end)) / e2e_steps
    # the same copies with no kernel: what the host link alone allows
    s_in, s_out = pipes[0].s_in, pipes[0].s_out
    barrier()
    t_begin.record(stream)
    s_in.wait_event(t_begin)
    s_out.wait_event(t_begin)
    for _ in range(e2e_steps):
        for pipe, (a, b_, c, d) in zip(pipes, views):
            with torch.cuda.stream(s_in):
                for dst, src in ((pipe.slots[0]["q"], a), (pipe.slots[0]["k"], b_), (pipe.slots[0]["v"], c)):
                    dst.copy_(src, non_blocking=True)
            with torch.cuda.stream(s_out):
                d.copy_(pipe.slots[1 % pipe.depth]["o"], non_blocking=True)
    join([s_in, s_out])
    t_end.record(stream)
    barrier()
    copy_floor_ms = max_over_ranks(t_begin.elapsed_time(t_end)) / e2e_steps
    e2e_value = job_flops / (e2e_ms * 1e-3) / 1e12
    if world > 1:
        tot = torch.tensor([in_bytes, out_bytes], dtype=torch.int64, device=dev)
        dist.all_reduce(tot)
        job_in, job_out = int(tot[0]), int(tot[1])
    else:
        job_in, job_out = in_bytes, out_bytes
    e2e = {"value": e2e_value, "unit": "TFLOPS", "h2d_bytes_per_step": job_in,
           "d2h_bytes_per_step": job_out, "ms_per_step": e2e_ms, "copy_floor_ms": copy_floor_ms,
           "copy_floor_note": "the same pinned host->device and device->host copies with no kernel "
                              "in between: e2e sits on the host link, not on the kernel"}
    del pipes

    # ---- the reference project's final kernel on the same GPU and inputs (rank 0, one GPU)
    k18 = None
    configs = None
    if rank == 0 and world == 1 and not opts:
        theirs = None if args.no_k18 else k18_call(torch, q, k, v, layout)
        if theirs is not None:
            k18 = compare_with_k18(torch, whole, theirs, job_flops, stream, smclock,
                                   burst_n=min(max(args.steps, 10), 50), rounds=args.k18_rounds,
                                   sustain_s=args.sustain_s)
            del theirs
        if args.workload == "main" and not args.no_configs:
            del q, k, v, o
            torch.cuda.empty_cache()
            configs = configs_block(torch, ops, dev, stream, measured_peaks())
    _native.device_check()
    # ---- CPU baseline on a bounded sample (rank 0, single-GPU runs only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        tf, heads, secs, cores, rows = cpu_sdpa_sample(b, h, lq, lk, budget_s=args.cpu_budget, causal=causal)
        cpu = {"value": tf, "unit": "TFLOPS", "cores": cores, "kind": "reference",
               "sample": (f"torch scaled_dot_product_attention (math backend, fp32, CPU: the call the "
                          f"reference checks its kernels against), {rows} query rows x Lk={lk} "
                          f"({rows / lq:.2f} of the {b * h} (batch, head) slices of this workload), "
                          f"{secs:.1f} s, scaled by FLOPs")}

    if rank == 0:
        peaks = measured_peaks()
        traffic, traffic_source = NCU_TRAFFIC.get(args.workload, (None, None))
        if split:
            traffic = None
        per_gpu = value / world
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": scaling_of(args.workload, world), "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": workload_config(args.workload, world),
            "pct_of_bf16_peak": 100.0 * per_gpu / peaks["bf16_tflops"],
            "burst": burst, "sustained": sustained,
            "sustained_pct_of_sustained_bf16_peak": (
                100.0 * sustained["tflops"] / world / peaks["bf16_tflops_sustained"]
                if peaks["bf16_tflops_sustained"] else None),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                         "frac_of_sustained_peak": (achieved / peaks["bf16_tflops_sustained"]
                                                    if peaks["bf16_tflops_sustained"] else None),
                         "peak_source": f"{peaks['source']} cuBLAS bf16 burst",
                         "kernel_ms": kernel_ms, "traffic": traffic,
                         "traffic_source": (f"{traffic_source} (ncu capture of this kernel in an earlier "
                                            "run, not measured in this run)" if traffic else None),
                         "hbm_gbs_algorithmic": (in_bytes + out_bytes) / (kernel_ms * 1e-3) / 1e9},
            "e2e": e2e,
            "gpu_launches": int(launches),
            "clocks": clocks,
            "cpu_baseline": cpu,
            "k18_same_gpu": k18,
        }
        if weak is not None:
            line["weak"] = weak
            line["work_items_per_gpu"] = sharding.units_of(ranges) * ((lq + 255) // 256)
        if configs is not None:
            line["configs"] = configs
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def check_ring_rows(torch, o, lse, q_local, k_all, v_all, n_rows, heads, seed):
    """Sampled rows of this rank's result against the explicit CPU oracle over ALL keys."""
    from oracle import sdpa_oracle as O

    g = torch.Generator().manual_seed(seed)
    rows = torch.unique(torch.cat([torch.randperm(q_local.shape[2], generator=g)[:n_rows],
                                   torch.tensor([0, q_local.shape[2] - 1])]))
    worst = {"o_max_abs": 0.0, "o_mean_abs": 0.0, "lse_max_abs": 0.0}
    for hd in heads:
        qs = q_local[:, hd:hd + 1, rows].float().cpu()
        s = torch.matmul(qs, k_all[:, hd:hd + 1].float().transpose(-1, -2)) * O.default_scale()
        lse_ref = torch.logsumexp(s, dim=-1)
        o_ref = torch.matmul(torch.exp(s - lse_ref.unsqueeze(-1)), v_all[:, hd:hd + 1].float())
        st = O.compare(o[:, hd:hd + 1, rows].cpu(), o_ref, lse[:, hd:hd + 1, rows].cpu(), lse_ref)
        for key in worst:
            worst[key] = max(worst[key], st[key])
    ok = (worst["o_max_abs"] <= O.O_MAX_ABS and worst["o_mean_abs"] <= O.O_MEAN_ABS
          and worst["lse_max_abs"] <= O.LSE_MAX_ABS)
    return ok, worst, int(rows.numel()) * len(heads)


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
    ra.synchronize()
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
    ra.synchronize()
    dist.barrier()
    ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    launches = _native.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    # one more call with timing events on the copy stream: how long the peer pulls take and how
    # much of that the kernels hide
    o, lse = ra.forward(q, k, v, timing=True)
    ra.synchronize()
    timing = ra.last_timing()
    copy_ms = max_over_ranks(sum(timing["pull_ms"]))
    kernel_ms = max_over_ranks(sum(timing["kernel_ms"]))
    exposed_ms = max_over_ranks(timing["exposed_ms"])
    # correctness of this very run, on sampled rows of every rank (all keys: shards gathered on the host)
    checked = None
    if args.check:
        ks = [torch.empty(B, H, n, HEAD_DIM, dtype=torch.bfloat16, device=dev) for _ in range(world)]
        vs = [torch.empty_like(ks[0]) for _ in range(world)]
        dist.all_gather(ks, k)
        dist.all_gather(vs, v)
        heads = sorted({0, H // 2, H - 1})
        k_all = torch.cat([t[:, heads] for t in ks], dim=2).cpu()
        v_all = torch.cat([t[:, heads] for t in vs], dim=2).cpu()
        del ks, vs
        torch.set_num_threads(max(1, (os.cpu_count() or 8) // world))
        ok, worst, rows = check_ring_rows(torch, o[:, heads], lse[:, heads], q[:, heads], k_all, v_all,
                                          32, heads=range(len(heads)), seed=rank)
        flag = torch.tensor([int(ok)], device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        stats = torch.tensor([worst["o_max_abs"], worst["o_mean_abs"], worst["lse_max_abs"]],
                             dtype=torch.float64, device=dev)
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        checked = {"ok": bool(flag.item()), "rows_per_rank": rows, "ranks": world, "heads": heads,
                   "o_max_abs": float(stats[0]), "o_mean_abs": float(stats[1]),
                   "lse_max_abs": float(stats[2]),
                   "against": "explicit fp32 softmax(QK^T/sqrt(128))V on the host over all keys"}
    # end to end: shards from pinned host memory in, O back out, every step
    e2e_steps = max(2, min(args.steps, 3))
    e0.record(stream)
    for _ in range(e2e_steps):
        for d, hst in zip((q, k, v), host):
            d.copy_(hst, non_blocking=True)
        o, _ = ra.forward(q, k, v)
        o_host.copy_(o, non_blocking=True)
    e1.record(stream)
    ra.synchronize()
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
                         "peak_source": f"{peaks['source']} cuBLAS bf16 burst", "traffic": None},
            "nvlink": {"bytes_per_gpu_per_step": shard_bytes * (world - 1),
                       "gbs_needed": shard_bytes * (world - 1) / (ms * 1e-3) / 1e9,
                       "pull_ms_per_step": copy_ms, "kernel_ms_per_step": kernel_ms,
                       "pull_gbs_achieved": (shard_bytes * (world - 1) / (copy_ms * 1e-3) / 1e9
                                             if copy_ms > 0 else None),
                       "exposed_ms_per_step": exposed_ms,
                       "fraction_hidden": (1.0 - exposed_ms / copy_ms) if copy_ms > 0 else None,
                       "note": "max over ranks; pulls run on a side stream (copy engine), the kernel "
                               "of a step waits only for its own shard; exposed = time between a "
                               "kernel's predecessor ending and its shard's pull ending, where positive"},
            "fp32_partial_traffic_bytes_per_gpu_per_step": 2 * (world - 1) * B * H * n * (HEAD_DIM + 1) * 4,
            "check": checked,
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
            tf, heads, secs, cores, rows = cpu_sdpa_sample(b, h, length, length, budget_s=args.cpu_budget)
            cpu = {"value": tf, "unit": "TFLOPS", "cores": cores, "kind": "reference",
                   "sample": (f"torch scaled_dot_product_attention (math backend, fp32, CPU), {rows} query "
                              f"rows x Lk={length} of one self-attention call, {secs:.1f} s, scaled by FLOPs")}
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="main",
                    choices=sorted(WORKLOADS) + sorted(RING_WORKLOADS) + sorted(SEQUENCE_WORKLOADS)
                    + ["main_strong"])
    ap.add_argument("--layout", default=None, choices=["bhld", "bshd"],
                    help="override the workload's operand layout (single-launch workloads)")
    ap.add_argument("--no-k18", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the `configs` block of the main line")
    ap.add_argument("--check", action="store_true", help="sp_ring: verify sampled rows against the CPU oracle")
    ap.add_argument("--cpu-budget", type=float, default=12.0)
    ap.add_argument("--sustain-s", type=float, default=1.0, help="length of the sustained timed regions")
    ap.add_argument("--k18-rounds", type=int, default=2)
    ap.add_argument("--only-timed", action="store_true",
                    help="profiling aid: warm-up and the timed launches only, then stop")
    ap.add_argument("--k18-launches", type=int, default=0,
                    help="with --only-timed: also launch the reference kernel this many times")
    args = ap.parse_args()
    args.steps_given, args.warmup_given = args.steps is not None, args.warmup is not None
    args.steps = 100 if args.steps is None else args.steps
    args.warmup = 5 if args.warmup is None else args.warmup
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload == "main_strong":   # older name of what `main` does on more than one GPU
        args.workload = "main"
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
