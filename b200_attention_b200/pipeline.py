"""Host-resident batches through the GPU kernel with copies overlapped: a small double-buffered
pipeline (host -> device copy of step i+1, kernel of step i and device -> host copy of step i-1
run concurrently on three streams). For callers whose Q/K/V live in pinned host memory; the
reference project has no counterpart (its harness times device-resident tensors only,
benchmarks/benchmark.py:244-268)."""

from __future__ import annotations

from typing import Tuple

import torch

from . import ops


class HostPipeline:
    def __init__(self, shape_q: Tuple[int, ...], shape_kv: Tuple[int, ...], *, layout: str = "bhld",
                 device=None, depth: int = 2, softmax_scale: float = 0.0, causal: bool = False):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.layout = layout
        self.depth = depth
        self.scale = softmax_scale
        self.causal = causal
        mk = lambda shape: torch.empty(shape, dtype=torch.bfloat16, device=self.device)
        self.slots = [dict(q=mk(shape_q), k=mk(shape_kv), v=mk(shape_kv), o=mk(shape_q)) for _ in range(depth)]
        self.s_in = torch.cuda.Stream(self.device)
        self.s_run = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.ev_in = [torch.cuda.Event() for _ in range(depth)]
        self.ev_run = [torch.cuda.Event() for _ in range(depth)]
        self.ev_out = [torch.cuda.Event() for _ in range(depth)]
        self.n = 0

    def submit(self, q_host, k_host, v_host, o_host) -> None:
        """Queue one step: q/k/v are pinned host tensors, o_host (pinned) receives the result.
        Returns immediately; `finish()` waits for everything queued."""
        s = self.n % self.depth
        slot = self.slots[s]
        reused = self.n >= self.depth
        with torch.cuda.stream(self.s_in):
            if reused:
                self.s_in.wait_event(self.ev_run[s])  # the kernel that read this slot has finished
            slot["q"].copy_(q_host, non_blocking=True)
            slot["k"].copy_(k_host, non_blocking=True)
            slot["v"].copy_(v_host, non_blocking=True)
            self.ev_in[s].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_in[s])
            if reused:
                self.s_run.wait_event(self.ev_out[s])  # the previous result left this slot
            ops.attention(slot["q"], slot["k"], slot["v"], layout=self.layout, out=slot["o"],
                          softmax_scale=self.scale, causal=self.causal, stream=self.s_run)
            self.ev_run[s].record(self.s_run)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_run[s])
            o_host.copy_(slot["o"], non_blocking=True)
            self.ev_out[s].record(self.s_out)
        self.n += 1

    def finish(self) -> None:
        for st in (self.s_in, self.s_run, self.s_out):
            st.synchronize()
