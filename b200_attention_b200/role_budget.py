"""Where the cycles of the warp-specialised kernel go, role by role.

    python -m b200_attention_b200.role_budget [--shape B,H,Lq,Lk ...] [--no-split]

Builds an instrumented variant of the core library (B200ATTN_PROFILE: the MMA-issuing warp and the
first softmax warp of each Q tile accumulate clock deltas per category in registers, block 0
writes the totals once at the end; the shipped library carries none of this), runs one launch per
shape on the current GPU and prints, for block 0, the cycles per category, per K/V tile it worked
on and per work item. The instrumentation costs a clock read per boundary, which lengthens the
kernel by a few per cent: compare categories, not totals, with the shipped kernel.
"""

from __future__ import annotations

import argparse
import ctypes as C


MMA_LABELS = ["other", "wait pair (K/V)", "-", "wait P (+ accumulator free)", "issue PV", "issue QK",
              "commits", "-"]
SOFTMAX_LABELS = ["other", "wait S", "TMEM load", "exponentials + check", "store P + signal", "-", "-", "-"]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", nargs="*", default=["4,16,8192,8192"], help="B,H,Lq,Lk (BHLD)")
    ap.add_argument("--no-split", action="store_true", help="never use the tile-stream split")
    args = ap.parse_args()

    import torch

    from . import _native as N
    from . import build

    N.CORE_LIB = build.build_core(defines=("B200ATTN_PROFILE",), name="libb200attn_profile.so")
    from . import ops

    lib = N.lib()
    lib.b200attn_debug_set_trace.argtypes = [C.c_void_p]
    lib.b200attn_debug_set_trace.restype = None
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for shape in args.shape:
        b, h, lq, lk = (int(x) for x in shape.split(","))
        q = torch.randn(b, h, lq, 128, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(b, h, lk, 128, device="cuda", dtype=torch.bfloat16)
        v = torch.randn_like(k)
        ws = None if args.no_split else "auto"
        for _ in range(3):
            ops.attention(q, k, v, workspace=ws)
        torch.cuda.synchronize()
        buf = torch.zeros(64, dtype=torch.int64, device="cuda")
        lib.b200attn_debug_set_trace(buf.data_ptr())
        ops.attention(q, k, v, workspace=ws)
        torch.cuda.synchronize()
        lib.b200attn_debug_set_trace(None)
        N.device_check()
        t = buf.cpu().tolist()
        items = b * h * ((lq + 255) // 256)
        tiles_per_item = (lk + 127) // 128
        # what block 0 worked on when whole items are dealt round-robin (with the split its share
        # of tiles is total / SMs)
        items0 = (items + sms - 1) // sms
        tiles0 = items0 * tiles_per_item
        print(f"=== B={b} H={h} Lq={lq} Lk={lk}: {items} work items of {tiles_per_item} K/V tiles; "
              f"block 0: {items0} items = {tiles0} tiles when dealt whole items")
        for name, vals, labels in (("MMA-issuing warp", t[0:8], MMA_LABELS),
                                   ("softmax warp 0 of Q tile 0", t[8:16], SOFTMAX_LABELS)):
            total = sum(vals)
            print(f"{name}: {total} cycles = {total / tiles0:.0f} per tile")
            for label, val in zip(labels, vals):
                if val:
                    print(f"   {label:30s} {val / tiles0:8.1f} cycles/tile {val / items0:10.0f} cycles/item"
                          f" {100.0 * val / total:5.1f} %")


if __name__ == "__main__":
    main()
