"""(batch, head) sharding across GPUs: every (batch, head) slice of attention is independent,
so each rank runs its slices with its own launches and nothing crosses the wire.

The reference kernel already treats batch*heads as one flat independent axis
(kernels/5_minor/18_tma_l2_promotion.cu:1016-1017, 1039); here that axis is cut into `world`
contiguous, near-equal pieces. The planning functions are plain Python (tested on CPU with
gloo ranks); `run_shard` is the only part that needs a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple


@dataclass(frozen=True)
class HeadRange:
    """Heads [head_begin, head_end) of one batch entry."""
    batch: int
    head_begin: int
    head_end: int

    @property
    def count(self) -> int:
        return self.head_end - self.head_begin


def flat_bounds(units: int, world: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of rank's piece when `units` items are cut into `world` near-equal pieces
    (the first units % world ranks get one more)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if units < 0:
        raise ValueError("units must be non-negative")
    base, extra = divmod(units, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def plan(batch: int, heads: int, world: int, rank: int) -> List[HeadRange]:
    """The (batch, head) slices rank owns, as per-batch head ranges in flat (b*heads + h) order."""
    begin, end = flat_bounds(batch * heads, world, rank)
    out: List[HeadRange] = []
    unit = begin
    while unit < end:
        b, h = divmod(unit, heads)
        h_end = min(heads, h + (end - unit))
        out.append(HeadRange(b, h, h_end))
        unit += h_end - h
    return out


def plan_all(batch: int, heads: int, world: int) -> List[List[HeadRange]]:
    return [plan(batch, heads, world, r) for r in range(world)]


def units_of(ranges: Sequence[HeadRange]) -> int:
    return sum(r.count for r in ranges)


def imbalance(batch: int, heads: int, world: int) -> float:
    """max over ranks of owned units divided by the ideal share (1.0 = perfectly even)."""
    total = batch * heads
    if total == 0:
        return 1.0
    most = max(units_of(p) for p in plan_all(batch, heads, world))
    return most / (total / world)


def launches_of(ranges: Sequence[HeadRange], heads: int) -> List[Tuple[int, int, int, int]]:
    """(batch_begin, batch_end, head_begin, head_end) per launch: consecutive batch entries owned
    with all their heads go into one launch (fewer, fuller waves of work items), a partial head
    range is a launch of its own."""
    out: List[Tuple[int, int, int, int]] = []
    for r in ranges:
        full = r.head_begin == 0 and r.head_end == heads
        if full and out and out[-1][2] == 0 and out[-1][3] == heads and out[-1][1] == r.batch:
            out[-1] = (out[-1][0], r.batch + 1, 0, heads)
        else:
            out.append((r.batch, r.batch + 1, r.head_begin, r.head_end))
    return out


def run_shard(q, k, v, ranges: Sequence[HeadRange], *, layout: str = "bhld", out=None,
              softmax_scale: float = 0.0, return_lse: bool = False):
    """Runs attention for `ranges` of q/k/v (full tensors resident on this rank's GPU) and
    writes the matching slices of `out` (allocated like q if None). One launch per run of whole
    batch entries and one per partial head range (`launches_of`), no copies: a slice is a strided view. Returns out (and LSE [B, H, Lq] with only the owned
    slices written, if asked)."""
    import torch

    from . import ops

    h_axis = 1 if layout == "bhld" else 2
    if out is None:
        out = torch.empty_like(q)
    lse = None
    if return_lse:
        lq = q.size(2) if layout == "bhld" else q.size(1)
        lse = torch.zeros(q.size(0), q.size(h_axis), lq, dtype=torch.float32, device=q.device)
    for b0, b1, h0, h1 in launches_of(ranges, q.size(h_axis)):
        sl = [slice(b0, b1), slice(None), slice(None), slice(None)]
        sl[h_axis] = slice(h0, h1)
        sl = tuple(sl)
        res = ops.attention(q[sl], k[sl], v[sl], layout=layout, out=out[sl],
                            softmax_scale=softmax_scale, return_lse=return_lse)
        if return_lse:
            lse[b0:b1, h0:h1] = res[1]
    return (out, lse) if return_lse else out
