"""Sequence-parallel attention over a K/V ring, one process per GPU.

Q, O and LSE are sharded by query rows; rank r owns K/V shard r. At step s rank r attends to
shard (r + s) mod G, so every step each shard is read by exactly one rank and NVSwitch carries
G disjoint peer copies at once. A shard is pulled from its owner's memory (CUDA IPC mapping,
plain copy-engine `cudaMemcpyAsync`) into a local double buffer on a side stream while the
kernel works on the previous shard; the kernel's TMA only ever reads local HBM. Partial results
are chained in the kernel epilogue through an fp32 (O, LSE) scratch (`partial_merge` /
`partial_emit` of the C ABI): G launches, no merge kernel, no reduction collective.

Ordering is by stream events and two host barriers (inputs ready before anybody pulls, and
everybody done pulling before inputs may change); no device-side code waits on a peer, and no
load with cluster multicast is involved anywhere.

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
    ranks must use the same shard shape. q: [B, H, Lq_local, 128]. The K/V tensors must stay
    alive and unmodified from `bind` until the matching `forward` has returned.
    """

    def __init__(self, group=None):
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._peers: List[Optional[_Peer]] = []
        self._bound_shape = None
        self._staging = None
        self._partial = None
        self._copy_stream = None

    # -- peer mapping ----------------------------------------------------------------------
    def bind(self, k_local, v_local) -> None:
        """Exchange IPC handles of this call's K/V shards and map every peer's shard."""
        import torch
        import torch.distributed as dist

        from . import _native as N

        lib = N.lib()
        if not (k_local.is_cuda and v_local.is_cuda and k_local.is_contiguous() and v_local.is_contiguous()):
            raise RuntimeError("ring shards must be contiguous CUDA tensors")
        self.unbind()
        mine = []
        for t in (k_local, v_local):
            handle = C.create_string_buffer(64)
            off = C.c_uint64(0)
            N.check(lib.b200attn_ipc_export(t.data_ptr(), handle, C.byref(off)))
            mine.append((handle.raw, int(off.value)))
        info = {"shape": tuple(k_local.shape), "handles": mine}
        gathered = [None] * self.world
        dist.all_gather_object(gathered, info, group=self.group)
        for g in gathered:
            if g["shape"] != info["shape"]:
                raise RuntimeError(f"ring shards differ in shape: {g['shape']} vs {info['shape']}")
        self._peers = []
        for r, g in enumerate(gathered):
            if r == self.rank:
                self._peers.append(_Peer(k_local.data_ptr(), v_local.data_ptr(), []))
                continue
            ptrs, bases = [], []
            for raw, off in g["handles"]:
                base = C.c_void_p()
                N.check(lib.b200attn_ipc_open(raw, C.byref(base)))
                bases.append(base.value)
                ptrs.append(base.value + off)
            self._peers.append(_Peer(ptrs[0], ptrs[1], bases))
        self._bound_shape = tuple(k_local.shape)
        self._keep = (k_local, v_local)
        if self._staging is None or tuple(self._staging[0][0].shape) != self._bound_shape:
            self._staging = [tuple(torch.empty_like(k_local) for _ in range(2)) for _ in range(2)]
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=k_local.device)
        dist.barrier(group=self.group)  # every shard is final and mapped before anybody pulls

    def unbind(self) -> None:
        from . import _native as N

        for peer in self._peers:
            if peer is None:
                continue
            for base in peer.mapped:
                N.lib().b200attn_ipc_close(C.c_void_p(base))
        self._peers = []
        self._keep = None

    # -- the ring ----------------------------------------------------------------------------
    def forward(self, q, k_local, v_local, *, softmax_scale: float = 0.0, return_lse: bool = True):
        import torch
        import torch.distributed as dist

        from . import _native as N
        from . import ops

        if not self._peers or self._bound_shape != tuple(k_local.shape) or \
                self._peers[self.rank].k_ptr != k_local.data_ptr():
            self.bind(k_local, v_local)
        lib = N.lib()
        dev = q.device
        B, H, Lq, D = q.shape
        nbytes = k_local.numel() * k_local.element_size()
        if self._partial is None or tuple(self._partial[0].shape) != (B, H, Lq, D):
            self._partial = (torch.empty(B, H, Lq, D, dtype=torch.float32, device=dev),
                             torch.empty(B, H, Lq, dtype=torch.float32, device=dev))
        main = torch.cuda.current_stream(dev)
        side = self._copy_stream
        order = ring_schedule(self.world, self.rank)
        flags = chain_flags(self.world)
        copied = [torch.cuda.Event() for _ in range(self.world)]
        consumed = [torch.cuda.Event() for _ in range(self.world)]
        out = torch.empty_like(q)
        result = None

        def start_pull(step: int) -> None:
            buf = self._staging[step % 2]
            peer = self._peers[order[step]]
            with torch.cuda.stream(side):
                if step >= 2:
                    side.wait_event(consumed[step - 2])  # the buffer's previous occupant was read
                N.check(lib.b200attn_copy_async(buf[0].data_ptr(), peer.k_ptr, nbytes, side.cuda_stream))
                N.check(lib.b200attn_copy_async(buf[1].data_ptr(), peer.v_ptr, nbytes, side.cuda_stream))
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
            result = ops.attention(q, k_cur, v_cur, softmax_scale=softmax_scale, return_lse=True,
                                   out=out, partial=self._partial if self.world > 1 else None,
                                   partial_merge=merge, partial_emit=emit)
            consumed[step].record(main)
            if step + 2 < self.world:
                start_pull(step + 2)
        main.synchronize()
        N.device_check()
        dist.barrier(group=self.group)  # nobody may touch its shard while a peer still reads it
        return (result[0], result[1]) if return_lse else result[0]
