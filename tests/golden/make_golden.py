"""Generates tests/golden/*.npz by running the reference project's own oracle call
(torch scaled_dot_product_attention, math backend, fp32, CPU: benchmarks/check_correctness.py:89-95
and capstone-project/tests/test_kernel.py:121-130) on seeded inputs drawn with the reference's
seeding protocols. LSE comes from torch.logsumexp over the fp32 scores. The causal_* files come from the same call
with `is_causal=True` (and `enable_gqa=True`) on square cases.

    python tests/golden/make_golden.py

Each file stores the generator name and arguments, a sha256 of the bf16 input bits (so a test can
tell a drifting random stream from a numerical regression), O in fp32 and LSE in fp32.
"""

from __future__ import annotations

import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))

from oracle import sdpa_oracle as O  # noqa: E402

# name -> (generator, kwargs)
CASES = {
    # BASELINE config 0: the CPU-runnable correctness case
    "bench_b1_h2_l256": ("benchmark", dict(batch=1, heads=2, len_q=256, len_kv=256, seed=0)),
    # cross-attention: more queries than keys, one K/V tile
    "bench_b2_h1_lq256_lk128": ("benchmark", dict(batch=2, heads=1, len_q=256, len_kv=128, seed=1)),
    # ragged: neither length is a multiple of the tile sizes
    "bench_b1_h2_lq200_lk333": ("benchmark", dict(batch=1, heads=2, len_q=200, len_kv=333, seed=2)),
    # capstone protocol (token-major, q/k scaled by 0.25)
    "capstone_h2_lq256_lk384": ("capstone", dict(heads=2, len_q=256, len_kv=384, seed=7)),
    # video-DiT stand-in (RMS-normalised q/k)
    "video_h2_lq256_lk256": ("video_dit", dict(heads=2, len_q=256, len_kv=256, seed=0)),
}


# Causal mask and grouped K/V heads (the reference's research operator, research/causal_gqa_2cta.cu):
# name -> (benchmark-generator kwargs, K/V heads). Square, so PyTorch's `is_causal` applies as is;
# K and V keep every (heads // heads_kv)-th head of the drawn tensors.
CAUSAL_CASES = {
    "causal_b1_h4_kv1_l384": (dict(batch=1, heads=4, len_q=384, len_kv=384, seed=11), 1),
    "causal_b2_h4_kv2_l256": (dict(batch=2, heads=4, len_q=256, len_kv=256, seed=12), 2),
}


def draw_causal(kwargs: dict, heads_kv: int):
    """q [B,H,L,128], k and v [B,Hkv,L,128], bf16 CPU."""
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(**kwargs))
    step = kwargs["heads"] // heads_kv
    return q, k[:, ::step].contiguous(), v[:, ::step].contiguous()


def draw(generator: str, kwargs: dict):
    """Returns q, k, v as BHLD bf16 CPU tensors."""
    if generator == "benchmark":
        q, k, v = O.make_inputs_benchmark(**kwargs)
        return tuple(O.to_bhld(t) for t in (q, k, v))
    if generator == "capstone":
        q, k, v = O.make_inputs_capstone(**kwargs)
        h = kwargs["heads"]
        return tuple(t.reshape(t.shape[0], t.shape[1], h, 128).transpose(1, 2).contiguous()
                     for t in (q, k, v))
    if generator == "video_dit":
        q, k, v = O.make_inputs_video_dit(**kwargs)
        return tuple(O.to_bhld(t) for t in (q, k, v))
    raise ValueError(generator)


def input_digest(q, k, v) -> str:
    h = hashlib.sha256()
    for t in (q, k, v):
        h.update(t.contiguous().view(torch.int16).numpy().tobytes())
    return h.hexdigest()


def main() -> None:
    for name, (generator, kwargs) in CASES.items():
        q, k, v = draw(generator, kwargs)
        o = O.sdpa_torch_math(q, k, v)
        s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * O.default_scale()
        lse = torch.logsumexp(s, dim=-1)
        np.savez_compressed(
            HERE / f"{name}.npz",
            generator=generator,
            kwargs=repr(kwargs),
            input_sha256=input_digest(q, k, v),
            o=o.numpy().astype(np.float32),
            lse=lse.numpy().astype(np.float32),
            torch_version=torch.__version__,
        )
        print(name, tuple(o.shape), input_digest(q, k, v)[:12])
    for name, (kwargs, heads_kv) in CAUSAL_CASES.items():
        q, k, v = draw_causal(kwargs, heads_kv)
        o = O.sdpa_torch_math(q, k, v, causal=True)
        _, lse = O.sdpa_explicit(q, k, v, causal=True)
        np.savez_compressed(
            HERE / f"{name}.npz",
            generator="benchmark",
            kwargs=repr(kwargs),
            heads_kv=heads_kv,
            input_sha256=input_digest(q, k, v),
            o=o.numpy().astype(np.float32),
            lse=lse.numpy().astype(np.float32),
            torch_version=torch.__version__,
        )
        print(name, tuple(o.shape), input_digest(q, k, v)[:12])


if __name__ == "__main__":
    main()
