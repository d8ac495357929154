"""GPU tests of the tile-stream split: a dense call whose 256-row work items do not fill the SMs
evenly is cut into one equal run of K/V tiles per CTA; work items cut by a run boundary leave fp32
partials in the workspace and are merged by whichever piece finishes last. Checked against the CPU
oracle, against the unsplit kernel, for run-to-run equality, and for a workspace whose arrival
counters are back at zero afterwards."""

import pytest
import torch

from oracle import sdpa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(native_built):
    if not torch.cuda.is_available():
        pytest.fail("these tests need a CUDA device")
    from b200_attention_b200 import _native, ops

    _native.lib()
    return ops


def _inputs(b, h, lq, lk, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda n: torch.randn(b, h, n, 128, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    return mk(lq), mk(lk), mk(lk)


def _fresh_workspace(ops):
    import ctypes as C

    from b200_attention_b200 import _native as N

    size = C.c_uint64(0)
    N.check(N.lib().b200attn_workspace_bytes(C.byref(size)))
    return torch.zeros(int(size.value), dtype=torch.uint8, device="cuda")


def _counters(ws):
    """The arrival counters sit behind the partial slots (2 slots of 256 x 129 floats per SM)."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    return ws[sms * 2 * 256 * 129 * 4:].view(torch.int32)


SHAPES = [
    # (batch, heads, len_q, len_kv): work items = batch * heads * ceil(len_q / 256)
    (1, 149, 256, 2048),    # 149 items: one more than the SMs
    (1, 16, 4096, 8192),    # 256 items, 64 tiles each: 1.73 rounds of whole items
    (1, 27, 2816, 2048),    # 297 items, just over two rounds
    (1, 8, 512, 8192),      # 16 items on 148 SMs: every item is cut into four pieces
    (2, 3, 300, 16500),     # ragged in both lengths; the last K/V tile holds 116 keys
    (1, 2, 256, 16384),     # 2 items of 128 tiles
]


@pytest.mark.parametrize("b,h,lq,lk", SHAPES, ids=[f"B{b}_H{h}_Lq{lq}_Lk{lk}" for b, h, lq, lk in SHAPES])
def test_split_matches_oracle_and_unsplit_kernel(ops, b, h, lq, lk):
    from b200_attention_b200 import _native

    q, k, v = _inputs(b, h, lq, lk, seed=lq + lk)
    ws = _fresh_workspace(ops)
    whole, lse_whole = ops.attention(q, k, v, return_lse=True, workspace=None)
    split, lse_split = ops.attention(q, k, v, return_lse=True, workspace=ws)
    torch.cuda.synchronize()
    _native.device_check()
    assert bool(ws[: ws.numel() // 2].any()), "the split path was not taken for this shape"
    assert int(_counters(ws).abs().sum()) == 0
    assert float((lse_split - lse_whole).abs().max()) <= 1e-4
    d = (split.float() - whole.float()).abs()
    assert float(d.max()) <= O.O_MAX_ABS and float(d.mean()) <= 2e-4
    # against the oracle on a few heads
    for (bb, hh) in {(0, 0), (b - 1, h - 1), (0, h // 2)}:
        o_ref, lse_ref = O.sdpa_explicit(q[bb:bb + 1, hh:hh + 1].cpu(), k[bb:bb + 1, hh:hh + 1].cpu(),
                                         v[bb:bb + 1, hh:hh + 1].cpu())
        O.assert_within_contract(O.compare(split[bb:bb + 1, hh:hh + 1].cpu(), o_ref,
                                           lse_split[bb:bb + 1, hh:hh + 1].cpu(), lse_ref))
    # the same workspace again: counters were left at zero, and whoever merges, the result is the same
    again, lse_again = ops.attention(q, k, v, return_lse=True, workspace=ws)
    torch.cuda.synchronize()
    _native.device_check()
    assert torch.equal(again, split) and torch.equal(lse_again, lse_split)
    assert int(_counters(ws).abs().sum()) == 0


def test_split_token_major_in_place(ops):
    """The same through the token-major layout ([B, L, H, 128] used in place)."""
    b, h, lq, lk = 1, 16, 4096, 4096
    q, k, v = (t.transpose(1, 2).contiguous() for t in _inputs(b, h, lq, lk, seed=5))  # BSHD
    ws = _fresh_workspace(ops)
    whole = ops.attention(q, k, v, layout="bshd", workspace=None)
    split = ops.attention(q, k, v, layout="bshd", workspace=ws)
    torch.cuda.synchronize()
    assert bool(ws[: ws.numel() // 2].any())
    d = (split.float() - whole.float()).abs()
    assert float(d.max()) <= O.O_MAX_ABS and float(d.mean()) <= 2e-4


def test_balanced_shapes_and_chained_calls_do_not_split(ops):
    """When whole work items already fill the SMs evenly, or the call is part of a K/V chain or has
    a causal mask, the workspace stays untouched and the result is bit-identical."""
    q, k, v = _inputs(1, 37, 1024, 2048, seed=9)   # 148 items: exactly one round
    ws = _fresh_workspace(ops)
    a = ops.attention(q, k, v, workspace=ws)
    b_ = ops.attention(q, k, v, workspace=None)
    c = ops.attention(q, k, v, causal=True, workspace=ws)
    d = ops.attention(q, k, v, causal=True, workspace=None)
    torch.cuda.synchronize()
    assert torch.equal(a, b_) and torch.equal(c, d)
    assert not bool(ws.any())


def test_workspace_argument_checks(ops):
    q, k, v = _inputs(1, 2, 256, 256, seed=1)
    with pytest.raises(RuntimeError, match="workspace"):
        ops.attention(q, k, v, workspace=torch.zeros(1024, dtype=torch.uint8, device="cuda"))
    with pytest.raises(RuntimeError, match="uint8"):
        ops.attention(q, k, v, workspace=torch.zeros(1 << 20, dtype=torch.float32, device="cuda"))
