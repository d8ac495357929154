"""CPU tests of the oracle: the restatements agree with the reference's own oracle call and with
the committed golden fixtures."""

import ast
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import native_refs as R
from oracle import sdpa_oracle as O
from tests.golden import make_golden as G

_ALL = sorted(Path(__file__).resolve().parent.joinpath("golden").glob("*.npz"))
GOLDEN = [p for p in _ALL if not p.stem.startswith("causal_")]
GOLDEN_CAUSAL = [p for p in _ALL if p.stem.startswith("causal_")]


def load_case(path):
    z = np.load(path, allow_pickle=False)
    generator = str(z["generator"])
    kwargs = ast.literal_eval(str(z["kwargs"]))
    q, k, v = G.draw(generator, kwargs)
    return z, q, k, v


def test_fixtures_exist():
    assert len(GOLDEN) >= 5


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_inputs_reproduce(path):
    z, q, k, v = load_case(path)
    assert G.input_digest(q, k, v) == str(z["input_sha256"]), (
        "the seeded CPU random stream no longer reproduces the fixture's inputs")


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_explicit_matches_golden(path):
    z, q, k, v = load_case(path)
    o, lse = O.sdpa_explicit(q, k, v)
    assert np.abs(o.numpy() - z["o"]).max() < 5e-6
    assert np.abs(lse.numpy() - z["lse"]).max() < 5e-6


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_torch_math_matches_golden(path):
    z, q, k, v = load_case(path)
    assert np.abs(O.sdpa_torch_math(q, k, v).numpy() - z["o"]).max() < 5e-6


@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
@pytest.mark.parametrize("block", [64, 100, 1024])
def test_streaming_matches_golden(path, block):
    z, q, k, v = load_case(path)
    o, lse = O.sdpa_streaming(q, k, v, block=block)
    assert np.abs(o.numpy() - z["o"]).max() < 5e-6
    assert np.abs(lse.numpy() - z["lse"]).max() < 5e-6


@pytest.mark.skipif(not R.c_ref_available(), reason="oracle/_ref/libsdpa_ref.so not built")
@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_c_restatement_matches_golden(path):
    z, q, k, v = load_case(path)
    b, h, lq, _ = q.shape
    o, lse = R.sdpa_c_ref(q.reshape(b * h, lq, 128), k.reshape(b * h, -1, 128),
                          v.reshape(b * h, -1, 128), O.default_scale())
    assert np.abs(o.reshape(z["o"].shape).numpy() - z["o"]).max() < 5e-6
    assert np.abs(lse.reshape(z["lse"].shape).numpy() - z["lse"]).max() < 5e-6


@pytest.mark.skipif(not R.c_ref_available(), reason="oracle/_ref/libsdpa_ref.so not built")
def test_c_restatement_row_window():
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(1, 1, 192, 320, seed=3))
    full, lse = O.sdpa_explicit(q, k, v)
    o, l = R.sdpa_c_ref(q[0], k[0], v[0], O.default_scale(), rows=(64, 160))
    assert (o - full[0, :, 64:160]).abs().max() < 5e-6
    assert (l - lse[0, :, 64:160]).abs().max() < 5e-6


def test_merge_of_partials_is_exact():
    # Splitting the keys in two and merging (O, LSE) pairs reproduces attention over all keys:
    # the identity the sequence-parallel ring relies on.
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(1, 2, 128, 384, seed=4))
    full, lse = O.sdpa_explicit(q, k, v)
    oa, la = O.sdpa_explicit(q, k[:, :, :256], v[:, :, :256])
    ob, lb = O.sdpa_explicit(q, k[:, :, 256:], v[:, :, 256:])
    om, lm = O.merge_partials(oa, la, ob, lb)
    assert (om - full).abs().max() < 5e-6
    assert (lm - lse).abs().max() < 5e-6


def test_scale_argument():
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(1, 1, 64, 64, seed=5))
    o1, _ = O.sdpa_explicit(q, k, v, scale=0.05)
    o2, _ = O.sdpa_streaming(q, k, v, scale=0.05, block=16)
    assert (o1 - o2).abs().max() < 5e-6
    ref = torch.softmax(q.float() @ k.float().transpose(-1, -2) * 0.05, dim=-1) @ v.float()
    assert (o1 - ref).abs().max() < 5e-6


# ------------------------------------------------------------- causal mask, grouped K/V heads
def load_causal_case(path):
    z = np.load(path, allow_pickle=False)
    q, k, v = G.draw_causal(ast.literal_eval(str(z["kwargs"])), int(z["heads_kv"]))
    return z, q, k, v


def test_causal_fixtures_exist():
    assert len(GOLDEN_CAUSAL) >= 2


@pytest.mark.parametrize("path", GOLDEN_CAUSAL, ids=lambda p: p.stem)
def test_causal_explicit_and_torch_match_golden(path):
    z, q, k, v = load_causal_case(path)
    assert G.input_digest(q, k, v) == str(z["input_sha256"])
    o, lse = O.sdpa_explicit(q, k, v, causal=True)
    assert np.abs(o.numpy() - z["o"]).max() < 5e-6
    assert np.abs(lse.numpy() - z["lse"]).max() < 5e-6
    assert np.abs(O.sdpa_torch_math(q, k, v, causal=True).numpy() - z["o"]).max() < 5e-6


def test_causal_alignment_is_bottom_right():
    # with more keys than queries the last query row sees every key and the first one
    # len_kv - len_q + 1 of them
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(1, 1, 4, 7, seed=5))
    o, _ = O.sdpa_explicit(q, k, v, causal=True)
    full, _ = O.sdpa_explicit(q[:, :, 3:], k, v)
    first, _ = O.sdpa_explicit(q[:, :, :1], k[:, :, :4], v[:, :, :4])
    assert torch.allclose(o[:, :, 3:], full, atol=1e-6) and torch.allclose(o[:, :, :1], first, atol=1e-6)
    with pytest.raises(ValueError):
        O.sdpa_explicit(k, q, q, causal=True)


def test_grouped_heads_equal_repeated_heads():
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(1, 6, 64, 96, seed=6))
    kg, vg = k[:, ::3].contiguous(), v[:, ::3].contiguous()
    a, la = O.sdpa_explicit(q, kg, vg)
    b, lb = O.sdpa_explicit(q, kg.repeat_interleave(3, dim=1), vg.repeat_interleave(3, dim=1))
    assert torch.equal(a, b) and torch.equal(la, lb)
    assert (O.sdpa_torch_math(q, kg, vg) - a).abs().max() < 5e-6
