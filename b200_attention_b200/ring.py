"""Sequence-parallel attention over a K/V ring, one process per GPU.

Q, O and LSE are sharded by query rows; rank r owns K/V shard r. At step s rank r attends to
shard (r + s) mod G, so every step each shard is read by exactly one rank and NVSwitch carries
G disjoint peer copies at once. A shard is pulled from its owner's memory (CUDA IPC mapping,
plain copy-engine `cudaMemcpyAsync`) into a local double buffer on a side stream while the
kernel works on the previous shard; the kernel's TMA only ever reads local HBM. Partial results
are chained in the kernel epilogue through an fp32 (O, LSE) scratch (`partial_merge` /
`partial_emit` of the C ABI): G launches, no merge kernel, no reduction collective.

Ordering is by stream events inside a rank and two host barriers between ranks per call: on
entry every rank first waits (on the host) until the stream that produced its own K/V shard has
caught up, then all ranks meet, so no peer can pull a shard that is still being written; on exit
every rank waits for its own pulls and all ranks meet again, so a shard may be rewritten (in
place, or by an allocator handing the address out again) as soon as `forward` has returned. The
barriers run on a host-side (gloo) group and do not wait for the attention kernels, which are
still in flight when `forward` returns. No device-side code waits on a peer, and no load with
cluster multicast is involved anywhere.

The reference project is single-GPU (no ring, no LSE); this is an addition on top of its
operator. `ring_schedule` / `chain_flags` are plain Python and tested on CPU.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Tuple


def ring_schedule(world: int, rank: int) -> List[int]:
    """Shard index rank attends to at steps 0..world-1 (its own shard first)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    return [(rank + s) % world for s in range(world)]


def chain_flags(world: int) -> List[Tuple[bool, bool]]:
    """(partial_merge, partial_emit) per step: the first step starts the chain, the last one
    writes the final bf16 O and LSE."""
    return [(s > 0, s < world - 1) for s in range(world)]


def pull_plan(world: int) -> List[List[Tuple[int, int]]]:
    """For each step s >= 1, the (reader, owner) pairs of the peer copies that run concurrently."""
    return [[(r, (r + s) % world) for r in range(world)] for s in range(1, world)]


@dataclass
class _Peer:
    k_ptr: int
    v_ptr: int
    mapped: List[int]  # bases to close


class RingAttention:
    """Ring attention for fixed shard shapes. Collective: construct and call on every rank.

    k_local, v_local: this rank's shard [B, H, Lk_shard, 128] bf16 contiguous ('bhld'); all
    ranks must use the same shard shape. q: [B, H, Lq_local, 128]. The contents of a shard may
    change between two `forward` calls (same tensors or new ones); they must not change while a
    call is in progress. The results are produced asynchronously on the current stream: call
    `synchronize()` (or synchronise the stream and `_native.device_check()`) before reading them
    on the host.
    """

    def __init__(self, group=None, native=None):
        """`native` replaces the ctypes binding module (tests of the host logic pass a stand-in
        whose IPC calls can be made to fail)."""
        import torch.distributed as dist

        if native is None:
            from . import _native as native
            self._require_cuda = True
        else:
            self._require_cuda = False
        self._native = native
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        # Host-only meeting point: a barrier on the NCCL group would queue behind the kernels.
        ranks = dist.get_process_group_ranks(group) if group is not None else None
        self._host_group = dist.new_group(ranks=ranks, backend="gloo") if self.world > 1 else None
        self._peers: List[Optional[_Peer]] = []
        self._bound = None
        self._keep = None
        self._staging = None
        self._partial = None
        self._out = None
        self._copy_stream = None
        self._events = None
        self._ready = None
        self._timing = None

    def _meet(self) -> None:
        import torch.distributed as dist

        if self._host_group is not None:
            dist.barrier(group=self._host_group)

    def _any_rank(self, flag: bool) -> bool:
        """True on every rank if `flag` is set on any rank (also a meeting point of all ranks)."""
        import torch
        import torch.distributed as dist

        if self._host_group is None:
            return flag
        t = torch.tensor([int(flag)], dtype=torch.int32)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self._host_group)
        return bool(t.item())

    # -- peer mapping ----------------------------------------------------------------------
    def bind(self, k_local, v_local) -> None:
        """Exchange IPC handles of this call's K/V shards and map every peer's shard. Raises on
        every rank if the shard shapes differ. (No ordering guarantee by itself: `forward` does
        the waiting.)"""
        import torch
        import torch.distributed as dist

        N = self._native
        lib = N.lib()
        if self._require_cuda and not (k_local.is_cuda and v_local.is_cuda):
            raise RuntimeError("ring shards must be CUDA tensors")
        if not (k_local.is_contiguous() and v_local.is_contiguous()):
            raise RuntimeError("ring shards must be contiguous")
        if tuple(k_local.shape) != tuple(v_local.shape):
            raise RuntimeError("k and v shards must have the same shape")
        self.unbind()
        mine = []
        for t in (k_local, v_local):
            handle = C.create_string_buffer(64)
            off = C.c_uint64(0)
            N.check(lib.b200attn_ipc_export(t.data_ptr(), handle, C.byref(off)))
            mine.append((handle.raw, int(off.value)))
        info = {"shape": tuple(k_local.shape), "handles": mine}
        gathered = [None] * self.world
        dist.all_gather_object(gathered, info, group=self._host_group if self._host_group is not None else self.group)
        for g in gathered:
            if g["shape"] != info["shape"]:
                raise RuntimeError(f"ring shards differ in shape: {g['shape']} vs {info['shape']}")
        self._peers = []
        try:
            for r, g in enumerate(gathered):
                if r == self.rank:
                    self._peers.append(_Peer(k_local.data_ptr(), v_local.data_ptr(), []))
                    continue
                peer = _Peer(0, 0, [])
                self._peers.append(peer)
                ptrs = []
                for raw, off in g["handles"]:
                    base = C.c_void_p()
                    N.check(lib.b200attn_ipc_open(raw, C.byref(base)))
                    peer.mapped.append(base.value)
                    ptrs.append(base.value + off)
                peer.k_ptr, peer.v_ptr = ptrs
        except Exception:
            self.unbind()  # close what was mapped before the failure
            raise
        self._bound = (tuple(k_local.shape), k_local.data_ptr(), v_local.data_ptr())
        self._keep = (k_local, v_local)
        if self._staging is None or tuple(self._staging[0][0].shape) != tuple(k_local.shape) \
                or self._staging[0][0].device != k_local.device:
            self._staging = [tuple(torch.empty_like(k_local) for _ in range(2)) for _ in range(2)]
        if self._copy_stream is None and k_local.is_cuda:
            self._copy_stream = torch.cuda.Stream(device=k_local.device)

    def unbind(self) -> None:
        N = self._native
        for peer in self._peers:
            if peer is None:
                continue
            for base in peer.mapped:
                N.lib().b200attn_ipc_close(C.c_void_p(base))
            peer.mapped = []
        self._peers = []
        self._bound = None
        self._keep = None

    def synchronize(self) -> None:
        """Wait for the kernels of the calls made so far and report a device-side wait that ran out."""
        import torch

        torch.cuda.current_stream().synchronize()
        self._native.device_check()

    # -- the ring ----------------------------------------------------------------------------
    def last_timing(self):
        """Of the last `forward(..., timing=True)` call, after `synchronize()`: per-step peer pull
        and kernel durations (ms) and the time the compute stream sat waiting for a pull."""
        if self._timing is None:
            return None
        pulls, kernels = self._timing
        pull_ms = [a.elapsed_time(b) for a, b in pulls[1:]]
        kernel_ms = [a.elapsed_time(b) for a, b in kernels]
        exposed = 0.0
        for s in range(1, len(kernels)):
            exposed += max(0.0, kernels[s - 1][1].elapsed_time(pulls[s][1]))
        return {"pull_ms": pull_ms, "kernel_ms": kernel_ms, "exposed_ms": exposed}

    def forward(self, q, k_local, v_local, *, softmax_scale: float = 0.0, return_lse: bool = True,
                out=None, timing: bool = False):
        import torch

        from . import ops

        N = self._native
        key = (tuple(k_local.shape), k_local.data_ptr(), v_local.data_ptr())
        lib = N.lib()
        dev = q.device
        B, H, Lq, D = q.shape
        nbytes = k_local.numel() * k_local.element_size()
        if self._partial is None or tuple(self._partial[0].shape) != (B, H, Lq, D):
            self._partial = (torch.empty(B, H, Lq, D, dtype=torch.float32, device=dev),
                             torch.empty(B, H, Lq, dtype=torch.float32, device=dev))
        if out is None:
            if self._out is None or self._out.shape != q.shape or self._out.device != dev:
                self._out = torch.empty_like(q)
            out = self._out
        main = torch.cuda.current_stream(dev)
        order = ring_schedule(self.world, self.rank)
        flags = chain_flags(self.world)
        if self._events is None or len(self._events[0]) != self.world:
            self._events = ([torch.cuda.Event() for _ in range(self.world)],
                            [torch.cuda.Event() for _ in range(self.world)])
            self._ready = torch.cuda.Event()
        copied, consumed = self._events
        result = None
        tev = lambda: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        self._timing = ([tev() for _ in range(self.world)], [tev() for _ in range(self.world)]) if timing else None

        # Entry: whatever wrote this rank's K/V (on the current stream) has finished, on every
        # rank, before anybody pulls. The ranks also agree here on whether the shards have to be
        # (re)mapped: binding is collective, so one rank whose shard moved makes all of them bind.
        if self.world > 1:
            self._ready.record(main)
            self._ready.synchronize()
            if self._any_rank(not self._peers or self._bound != key):
                self.bind(k_local, v_local)
        side = self._copy_stream

        def start_pull(step: int) -> None:
            buf = self._staging[step % 2]
            peer = self._peers[order[step]]
            with torch.cuda.stream(side):
                if step >= 2:
                    side.wait_event(consumed[step - 2])  # the buffer's previous occupant was read
                if timing:
                    self._timing[0][step][0].record(side)
                N.check(lib.b200attn_copy_async(buf[0].data_ptr(), peer.k_ptr, nbytes, side.cuda_stream))
                N.check(lib.b200attn_copy_async(buf[1].data_ptr(), peer.v_ptr, nbytes, side.cuda_stream))
                if timing:
                    self._timing[0][step][1].record(side)
                copied[step].record(side)

        if self.world > 1:
            start_pull(1)
        for step in range(self.world):
            if step == 0:
                k_cur, v_cur = k_local, v_local
            else:
                main.wait_event(copied[step])
                k_cur, v_cur = self._staging[step % 2]
            merge, emit = flags[step]
            if timing:
                self._timing[1][step][0].record(main)
            result = ops.attention(q, k_cur, v_cur, softmax_scale=softmax_scale, return_lse=True,
                                   out=out, partial=self._partial if self.world > 1 else None,
                                   partial_merge=merge, partial_emit=emit)
            if timing:
                self._timing[1][step][1].record(main)
            consumed[step].record(main)
            if step + 2 < self.world:
                start_pull(step + 2)
        # Exit: this rank's pulls have landed, on every rank, so every shard may change again.
        # (The last pull waits for the kernel two steps before the end; the last kernels are still
        # running when this returns.)
        if self.world > 1:
            side.synchronize()
            self._meet()
        return (result[0], result[1]) if return_lse else result[0]
