"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle on the
same seeded inputs. Tolerances are the acceptance contract's: bf16 O within max-abs 2e-2 and
mean-abs 2e-3 of the fp32 oracle, LSE within 1e-3 (oracle.sdpa_oracle.O_MAX_ABS etc.)."""

import ast
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import sdpa_oracle as O
from tests.golden import make_golden as G

pytestmark = pytest.mark.gpu

GOLDEN = [p for p in sorted(Path(__file__).resolve().parent.joinpath("golden").glob("*.npz"))
          if not p.stem.startswith("causal_")]
WS, SERIAL = 0, 1


@pytest.fixture(scope="module")
def ops(native_built):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from b200_attention_b200 import _native, ops

    _native.lib()
    return ops


def run_and_check(ops, q, k, v, *, kernel, layout="bhld", scale=0.0, tag=""):
    """q, k, v: CPU bf16 in `layout`. Runs on cuda:0, compares with the explicit oracle."""
    from b200_attention_b200 import _native

    qd, kd, vd = (t.cuda() for t in (q, k, v))
    o, lse = ops.attention(qd, kd, vd, layout=layout, softmax_scale=scale, return_lse=True,
                           kernel=kernel)
    torch.cuda.synchronize()
    _native.device_check()
    to_bhld = (lambda t: t.transpose(1, 2)) if layout == "bshd" else (lambda t: t)
    o_ref, lse_ref = O.sdpa_explicit(to_bhld(q), to_bhld(k), to_bhld(v),
                                     scale=None if scale <= 0 else scale)
    stats = O.compare(to_bhld(o.cpu()), o_ref, lse.cpu(), lse_ref)
    O.assert_within_contract(stats)
    return o, lse, stats


@pytest.mark.parametrize("kernel", [SERIAL, WS], ids=["serial", "ws"])
@pytest.mark.parametrize("path", GOLDEN, ids=lambda p: p.stem)
def test_golden_fixtures(ops, path, kernel):
    from b200_attention_b200 import _native

    z = np.load(path, allow_pickle=False)
    q, k, v = G.draw(str(z["generator"]), ast.literal_eval(str(z["kwargs"])))
    assert G.input_digest(q, k, v) == str(z["input_sha256"])
    o, lse = ops.attention(q.cuda(), k.cuda(), v.cuda(), return_lse=True, kernel=kernel)
    torch.cuda.synchronize()
    _native.device_check()
    stats = O.compare(o.cpu(), torch.from_numpy(z["o"]), lse.cpu(), torch.from_numpy(z["lse"]))
    O.assert_within_contract(stats)


SHAPES = [
    # (batch, heads, len_q, len_kv)
    (1, 1, 128, 128),      # half a work item, one K/V tile
    (1, 1, 256, 128),      # one work item, one tile
    (1, 1, 256, 256),      # two tiles: ring prefill only
    (1, 2, 256, 640),      # five tiles: the two-slot (V, K) pair ring refills
    (2, 3, 512, 384),
    (1, 2, 200, 333),      # ragged in both lengths
    (1, 1, 1, 1),          # degenerate
    (1, 3, 257, 129),      # one row / one key past a tile boundary
    (1, 1, 256, 4096),     # many tiles, rescale statistics
    (1, 40, 1024, 384),    # 160 items: more than one item per persistent CTA
    (1, 64, 2048, 128),    # 512 items with a single K/V tile each (item seam, T == 1)
    (3, 50, 256, 256),     # 150 items: two CTAs get a second item
]


@pytest.mark.parametrize("kernel", [SERIAL, WS], ids=["serial", "ws"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "b%d_h%d_lq%d_lk%d" % s)
def test_shapes_bhld(ops, shape, kernel):
    b, h, lq, lk = shape
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(b, h, lq, lk, seed=11))
    run_and_check(ops, q, k, v, kernel=kernel)


@pytest.mark.parametrize("shape", [(2, 4, 512, 384), (1, 3, 200, 333), (1, 12, 1024, 512)],
                         ids=lambda s: "b%d_h%d_lq%d_lk%d" % s)
def test_shapes_bshd_in_place(ops, shape):
    b, h, lq, lk = shape
    q, k, v = O.make_inputs_benchmark(b, h, lq, lk, seed=12)  # [B, L, H, 128], no transposes
    run_and_check(ops, q, k, v, kernel=WS, layout="bshd")


def test_ws_and_serial_agree_closely(ops):
    q, k, v = (O.to_bhld(t).cuda() for t in O.make_inputs_benchmark(1, 4, 512, 1024, seed=13))
    a, la = ops.attention(q, k, v, return_lse=True, kernel=WS)
    b, lb = ops.attention(q, k, v, return_lse=True, kernel=SERIAL)
    torch.cuda.synchronize()
    assert (a.float() - b.float()).abs().max() <= 1e-2
    assert (la - lb).abs().max() <= 1e-3


def test_runtime_scale(ops):
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(1, 2, 256, 384, seed=14))
    run_and_check(ops, q, k, v, kernel=WS, scale=0.02)
    run_and_check(ops, q, k, v, kernel=WS, scale=0.3)   # peaky softmax: rescale path is busy


def test_large_magnitude_scores_trigger_rescale(ops):
    # Keys whose norm grows along the sequence keep raising the row maximum, so the conditional
    # rescale (threshold 8 in log2 units) has to fire many times and stay exact.
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(1, 2, 256, 1024, seed=15))
    ramp = torch.linspace(0.2, 3.0, 1024).view(1, 1, -1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    run_and_check(ops, q, k, v, kernel=WS, scale=0.25)
    run_and_check(ops, q, k, v, kernel=SERIAL, scale=0.25)


def test_deterministic_run_to_run(ops):
    q, k, v = (O.to_bhld(t).cuda() for t in O.make_inputs_benchmark(2, 8, 1024, 1024, seed=16))
    a, la = ops.attention(q, k, v, return_lse=True)
    b, lb = ops.attention(q, k, v, return_lse=True)
    torch.cuda.synchronize()
    assert torch.equal(a, b) and torch.equal(la, lb)


def test_canaries_around_outputs_survive(ops):
    # O and LSE sit inside larger buffers filled with a sentinel: nothing outside may change.
    b, h, lq, lk = 1, 2, 200, 333
    q, k, v = (O.to_bhld(t).cuda() for t in O.make_inputs_benchmark(b, h, lq, lk, seed=17))
    pad = 4096
    buf = torch.full((b * h * lq * 128 + 2 * pad,), 77.0, dtype=torch.bfloat16, device="cuda")
    out = buf[pad:-pad].view(b, h, lq, 128)
    ops.attention(q, k, v, out=out)
    torch.cuda.synchronize()
    assert torch.all(buf[:pad] == 77.0) and torch.all(buf[-pad:] == 77.0)
    assert torch.isfinite(out.float()).all()


def test_strided_views_without_copies(ops):
    # Q, K, V as slices of one fused [B, L, 3, H, 128] projection output.
    b, h, l = 2, 4, 384
    g = torch.Generator().manual_seed(18)
    qkv = torch.randn(b, l, 3, h, 128, generator=g).to(torch.bfloat16)
    q, k, v = (qkv[:, :, i] for i in range(3))            # [B, L, H, 128] views, not contiguous
    from b200_attention_b200 import _native

    qd = qkv.cuda()
    o = ops.attention(qd[:, :, 0], qd[:, :, 1], qd[:, :, 2], layout="bshd")
    torch.cuda.synchronize()
    _native.device_check()
    o_ref, _ = O.sdpa_explicit(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    O.assert_within_contract(O.compare(o.cpu().transpose(1, 2), o_ref))


def test_partial_chain_equals_single_call(ops):
    # Three K/V shards chained through the fp32 partial state == one call over all keys.
    b, h, lq, lk = 1, 4, 512, 1536
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(b, h, lq, lk, seed=19))
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    po = torch.empty(b, h, lq, 128, dtype=torch.float32, device="cuda")
    pl = torch.empty(b, h, lq, dtype=torch.float32, device="cuda")
    for kernel in (WS, SERIAL):
        shards = [(0, 512), (512, 1024), (1024, 1536)]
        out = None
        for i, (s0, s1) in enumerate(shards):
            last = i == len(shards) - 1
            res = ops.attention(qd, kd[:, :, s0:s1], vd[:, :, s0:s1], return_lse=True,
                                partial=(po, pl), partial_merge=i > 0, partial_emit=not last,
                                kernel=kernel)
            if last:
                out = res
        torch.cuda.synchronize()
        o_ref, lse_ref = O.sdpa_explicit(q, k, v)
        O.assert_within_contract(O.compare(out[0].cpu(), o_ref, out[1].cpu(), lse_ref))


def test_many_back_to_back_launches_stay_clean(ops):
    # Barrier-phase bookkeeping across persistent items is where a rare hang would come from:
    # hammer three shapes (many items per CTA, 1 / 2 / 64 tiles per item) and make sure no bounded
    # wait ever ran out and the result never changes.
    from b200_attention_b200 import _native

    for (b, h, lq, lk, reps) in [(2, 16, 4096, 128, 150), (2, 16, 4096, 256, 150), (1, 16, 8192, 8192, 40)]:
        q, k, v = (torch.randn(b, h, n, 128, device="cuda", dtype=torch.bfloat16) for n in (lq, lk, lk))
        first = ops.attention(q, k, v).clone()
        for n in range(reps):
            out = ops.attention(q, k, v)
            if n % 25 == 24:  # look often: a stalled launch costs a full wait limit each
                torch.cuda.synchronize()
                _native.device_check()
        torch.cuda.synchronize()
        _native.device_check()
        assert torch.equal(out, first)


@pytest.mark.parametrize("kernel", [WS, SERIAL], ids=["ws", "serial"])
def test_rebase_paths(ops, kernel):
    # The production kernel speculates that a row's reference maximum still holds and falls back
    # to an exact rebase (moving the maximum, rescaling l and O in TMEM) when a score exceeds it by
    # more than 32 log2 units. Drive that path hard: (1) key norms that grow 40x along the
    # sequence, (2) single outlier keys late in the sequence, placed in the first 96 columns of
    # a tile (speculated part) and in the last 32 (checked part), far beyond any earlier score.
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(1, 2, 256, 1024, seed=31))
    ramp = torch.linspace(0.2, 8.0, 1024).view(1, 1, -1, 1)
    run_and_check(ops, q, (k.float() * ramp).to(torch.bfloat16), v, kernel=kernel, scale=0.25)

    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(1, 2, 256, 1024, seed=32))
    k = k.float()
    k[:, :, 300] *= 30.0    # tile 2, column 44  -> part A
    k[:, :, 750] *= 60.0    # tile 5, column 110 -> part B
    k[:, :, 1023] *= 90.0   # last key of the last tile
    run_and_check(ops, q, k.to(torch.bfloat16), v, kernel=kernel, scale=0.5)
