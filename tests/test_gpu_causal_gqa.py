"""GPU parity tests of the causal mask and of grouped K/V heads (the operator of the reference's
research kernel, research/causal_gqa_2cta.cu: causal aligned to the bottom-right corner, query
head h reading K/V head h // group), through the C ABI, against the CPU oracle and the committed
fixtures. Same tolerances as the dense path."""

import ast
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import sdpa_oracle as O
from tests.golden import make_golden as G

pytestmark = pytest.mark.gpu

GOLDEN_CAUSAL = sorted(Path(__file__).resolve().parent.joinpath("golden").glob("causal_*.npz"))


@pytest.fixture(scope="module")
def ops(native_built):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from b200_attention_b200 import _native, ops

    _native.lib()
    return ops


def run_and_check(ops, q, k, v, *, causal, layout="bhld"):
    """q [B,H,Lq,128], k and v [B,Hkv,Lk,128] CPU bf16 (BHLD); `layout` is what the GPU is given."""
    from b200_attention_b200 import _native

    to_dev = (lambda t: t.transpose(1, 2).contiguous().cuda()) if layout == "bshd" else (lambda t: t.cuda())
    o, lse = ops.attention(to_dev(q), to_dev(k), to_dev(v), layout=layout, causal=causal, return_lse=True)
    torch.cuda.synchronize()
    _native.device_check()
    o = o.transpose(1, 2) if layout == "bshd" else o
    o_ref, lse_ref = O.sdpa_explicit(q, k, v, causal=causal)
    stats = O.compare(o.cpu(), o_ref, lse.cpu(), lse_ref)
    O.assert_within_contract(stats)
    return stats


@pytest.mark.parametrize("path", GOLDEN_CAUSAL, ids=lambda p: p.stem)
def test_causal_golden_fixtures(ops, path):
    from b200_attention_b200 import _native

    z = np.load(path, allow_pickle=False)
    q, k, v = G.draw_causal(ast.literal_eval(str(z["kwargs"])), int(z["heads_kv"]))
    assert G.input_digest(q, k, v) == str(z["input_sha256"])
    o, lse = ops.attention(q.cuda(), k.cuda(), v.cuda(), causal=True, return_lse=True)
    torch.cuda.synchronize()
    _native.device_check()
    O.assert_within_contract(O.compare(o.cpu(), torch.from_numpy(z["o"]), lse.cpu(), torch.from_numpy(z["lse"])))


CAUSAL_SHAPES = [
    # (batch, heads, heads_kv, len_q, len_kv)
    (1, 1, 1, 128, 128),     # half a work item, the diagonal tile only
    (1, 2, 2, 256, 256),     # one work item: the second Q tile sees one tile more than the first
    (2, 4, 4, 512, 512),     # two work items per head, longest first
    (1, 4, 1, 1024, 1024),   # multi-query: four query heads on one K/V head
    (1, 8, 2, 2048, 2048),   # grouped, many tiles, items of 2..16 tiles
    (1, 2, 2, 200, 333),     # ragged, 133 keys of history before the first row
    (1, 2, 1, 300, 300),     # ragged square
    (1, 2, 2, 256, 1000),    # long history: every row sees at least 745 keys
    (3, 6, 3, 640, 640),     # odd counts, items of a head spread over CTAs
    (1, 32, 8, 4096, 4096),  # more work items than CTAs: the persistent loop walks mixed lengths
    # 8192 keys make the head groups sixteen K/V heads wide, so these deal several groups, the
    # odd ones with the CTAs in reverse order and the last one smaller than the rest (rounds taken
    # back and forth inside a group: the full-size causal test, 512 items per group)
    (1, 40, 40, 640, 8192),  # groups of 16, 16 and 8 heads, three items each
    (1, 40, 20, 384, 8192),  # two query heads per K/V head: groups of 32 and 8 query heads
    (2, 20, 20, 768, 8192),  # the same groups over two batch entries (a group spans both)
]


@pytest.mark.parametrize("shape", CAUSAL_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_causal_shapes(ops, shape):
    b, h, hk, lq, lk = shape
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(b, h, lq, lk, seed=sum(shape)))
    step = h // hk
    run_and_check(ops, q, k[:, ::step].contiguous(), v[:, ::step].contiguous(), causal=True)


@pytest.mark.parametrize("layout", ["bhld", "bshd"])
@pytest.mark.parametrize("causal", [False, True], ids=["dense", "causal"])
def test_grouped_heads_both_layouts(ops, layout, causal):
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(2, 8, 512, 768, seed=21))
    run_and_check(ops, q, k[:, ::4].contiguous(), v[:, ::4].contiguous(), causal=causal, layout=layout)


def test_causal_first_rows_see_only_their_history(ops):
    """Row 0 of a square causal problem attends to key 0 alone: O[0] == V[0] and LSE[0] == score."""
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(1, 2, 384, 384, seed=31))
    o, lse = ops.attention(q.cuda(), k.cuda(), v.cuda(), causal=True, return_lse=True)
    torch.cuda.synchronize()
    assert torch.equal(o[:, :, 0].cpu(), v[:, :, 0])
    s00 = (q[:, :, 0].float() * k[:, :, 0].float()).sum(-1) * O.default_scale()
    assert (lse[:, :, 0].cpu() - s00).abs().max() < 1e-3


def test_causal_with_growing_scores_takes_the_rebase_path(ops):
    """Key norms grow along the sequence, so the running maximum keeps moving while the diagonal
    mask is active."""
    q, k, v = (O.to_bhld(t) for t in O.make_inputs_benchmark(1, 2, 1024, 1024, seed=41))
    ramp = torch.linspace(0.5, 12.0, 1024).view(1, 1, -1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    run_and_check(ops, q, k, v, causal=True)


def test_rejections(ops):
    q = torch.zeros(1, 4, 256, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(1, 4, 128, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="len_kv >= len_q"):
        ops.attention(q, k, k, causal=True)
    k3 = torch.zeros(1, 3, 256, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="whole number"):
        ops.attention(q, k3, k3)
    k2 = torch.zeros(1, 2, 256, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="warp-specialised"):
        ops.attention(q, k2, k2, kernel=1)
    with pytest.raises(RuntimeError, match="warp-specialised"):
        ops.attention(q, q, q, causal=True, kernel=1)


def test_torch_op_causal_gqa(native_built):
    """The shim's op with the call shape of the reference's research launcher: token-major Q with
    Hq heads, K/V with Hkv heads, returns O token-major and LSE [B, Hq, S]."""
    from b200_attention_b200 import _native

    torch.ops.load_library(str(native_built["torch_ops"]))
    q, k, v = O.make_inputs_benchmark(2, 8, 384, 384, seed=51)  # BSHD
    kg, vg = k[:, :, ::4].contiguous(), v[:, :, ::4].contiguous()
    o, lse = torch.ops.b200_attention_b200.sdpa_causal_gqa(q.cuda(), kg.cuda(), vg.cuda(), 0.0)
    torch.cuda.synchronize()
    _native.device_check()
    assert o.shape == q.shape and lse.shape == (2, 8, 384)
    o_ref, lse_ref = O.sdpa_explicit(O.to_bhld(q), O.to_bhld(kg), O.to_bhld(vg), causal=True)
    O.assert_within_contract(O.compare(O.to_bhld(o.cpu()), o_ref, lse.cpu(), lse_ref))
    with pytest.raises(RuntimeError, match="multiple of the number of K/V heads"):
        torch.ops.b200_attention_b200.sdpa_causal_gqa(q.cuda(), k[:, :, :3].contiguous().cuda(),
                                                      v[:, :, :3].contiguous().cuda(), 0.0)
