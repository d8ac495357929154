"""CPU tests of the C ABI: the library builds for sm_100a, loads, exports every symbol the
header declares, and rejects bad arguments before touching a device. No compute here."""

import ctypes as C
import re
from pathlib import Path

import pytest

from b200_attention_b200 import _native as N

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "b200_attention.h"


def declared_symbols():
    text = HEADER.read_text()
    return re.findall(r"B200ATTN_API\s+[\w\s\*]+?\b(b200attn_\w+)\s*\(", text)


def test_header_and_binding_agree():
    assert sorted(declared_symbols()) == sorted(N.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol(native_built):
    lib = C.CDLL(str(native_built["core"]))
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_version_and_status_strings(native_built):
    assert "sm_100a" in N.version()
    lib = N.lib()
    assert lib.b200attn_status_string(0) == b"ok"
    for code in range(1, 8):
        assert lib.b200attn_status_string(code) not in (b"ok", b"unknown status")
    assert lib.b200attn_status_string(99) == b"unknown status"


def test_struct_layout_matches_header(native_built):
    # 6 x 4 bytes, 4 operands of 32 bytes, lse ptr, scale + kernel, 2 ptrs, 2 ints, stream,
    # causal + heads_kv, workspace pointer + size
    assert C.sizeof(N.Operand) == 32
    assert C.sizeof(N.ForwardArgs) == 24 + 4 * 32 + 8 + 8 + 16 + 8 + 8 + 8 + 16


def _args(**over):
    a = N.ForwardArgs()
    a.struct_bytes = C.sizeof(N.ForwardArgs)
    a.batch, a.heads, a.len_q, a.len_kv, a.head_dim = 1, 1, 256, 256, 128
    for name in ("q", "k", "v", "o"):
        setattr(a, name, N.Operand(0x10000, 0, 256 * 128, 128))
    for key, val in over.items():
        setattr(a, key, val)
    return a


@pytest.mark.parametrize("over, status", [
    (dict(struct_bytes=4), N.STATUS_INVALID_ARGUMENT),
    (dict(head_dim=64), N.STATUS_UNSUPPORTED),
    (dict(len_q=0), N.STATUS_INVALID_ARGUMENT),
    (dict(len_kv=-5), N.STATUS_INVALID_ARGUMENT),
    (dict(kernel=7), N.STATUS_INVALID_ARGUMENT),
    (dict(q=N.Operand(0, 0, 256 * 128, 128)), N.STATUS_INVALID_ARGUMENT),       # null
    (dict(k=N.Operand(0x10008, 0, 256 * 128, 128)), N.STATUS_INVALID_ARGUMENT),  # misaligned
    (dict(v=N.Operand(0x10000, 0, 256 * 128, 132)), N.STATUS_INVALID_ARGUMENT),  # stride % 8
    (dict(o=N.Operand(0x10000, 0, 256 * 128, 64)), N.STATUS_INVALID_ARGUMENT),   # stride < 128
    (dict(partial_merge=1), N.STATUS_INVALID_ARGUMENT),                          # no scratch given
    (dict(softmax_scale=float("nan")), N.STATUS_INVALID_ARGUMENT),
    (dict(heads=4, heads_kv=3), N.STATUS_INVALID_ARGUMENT),                      # 4 % 3 != 0
    (dict(heads_kv=-1), N.STATUS_INVALID_ARGUMENT),
    (dict(causal=1, len_q=512), N.STATUS_UNSUPPORTED),                           # len_kv < len_q
    (dict(causal=1, kernel=1), N.STATUS_UNSUPPORTED),                            # serial kernel
    (dict(heads=4, heads_kv=2, kernel=1), N.STATUS_UNSUPPORTED),
    (dict(causal=1, partial_o=0x20000, partial_lse=0x30000, partial_emit=1), N.STATUS_UNSUPPORTED),
    (dict(causal=1, partial_o=0x20000, partial_lse=0x30000, partial_merge=1), N.STATUS_UNSUPPORTED),
])
def test_argument_errors_come_back_as_status_codes(native_built, over, status):
    a = _args(**over)
    rc = N.lib().b200attn_forward(C.byref(a))
    assert rc == status
    assert N.lib().b200attn_last_error() != b""
    with pytest.raises(N.B200AttnError) as info:
        N.check(rc)
    assert info.value.status == status


@pytest.mark.parametrize("over, splits, status", [
    (dict(partial_o=0x20000, partial_lse=0x30000), 2, N.STATUS_INVALID_ARGUMENT),  # scratch is built in
    (dict(partial_emit=1), 2, N.STATUS_INVALID_ARGUMENT),
    (dict(causal=1), 2, N.STATUS_UNSUPPORTED),
    (dict(heads=4, heads_kv=2), 2, N.STATUS_UNSUPPORTED),
    (dict(kernel=1), 2, N.STATUS_INVALID_ARGUMENT),                                # serial kernel
    (dict(len_q=N.NOALLOC_MAX_ROWS + 1), 2, N.STATUS_UNSUPPORTED),                 # beyond the array
    (dict(batch=2, heads=64, len_q=256), 2, N.STATUS_UNSUPPORTED),                 # 32768 rows
    (dict(), -1, N.STATUS_INVALID_ARGUMENT),
    (dict(), 65, N.STATUS_INVALID_ARGUMENT),
    (dict(head_dim=64), 1, N.STATUS_UNSUPPORTED),
    (dict(q=N.Operand(0, 0, 256 * 128, 128)), 1, N.STATUS_INVALID_ARGUMENT),
])
def test_no_alloc_entry_rejects_before_touching_a_device(native_built, over, splits, status):
    """Every argument rule of the allocation-free entry point is checked before its first CUDA
    call, so the refusals can be seen without a GPU."""
    a = _args(**over)
    rc = N.lib().b200attn_forward_kv_split_noalloc(C.byref(a), splits)
    assert rc == status
    assert N.lib().b200attn_last_error() != b""


def test_null_args(native_built):
    assert N.lib().b200attn_forward(None) == N.STATUS_INVALID_ARGUMENT


def test_wait_limit_bounds(native_built):
    assert N.lib().b200attn_set_wait_limit_ms(0) == N.STATUS_INVALID_ARGUMENT
    assert N.lib().b200attn_set_wait_limit_ms(2000) == N.STATUS_OK


def test_device_check_before_any_launch_is_clean(native_built):
    assert N.lib().b200attn_device_check(0, None) == N.STATUS_OK


def test_torch_shim_registers_reference_op_names(native_built):
    import torch

    torch.ops.load_library(str(native_built["torch_ops"]))
    ops = torch.ops.b200_attention_b200
    for name in ("sdpa", "sdpa_bshd", "sdpa_lse", "sdpa_causal_gqa", "device_check"):
        assert hasattr(ops, name)
    x = torch.zeros(1, 1, 256, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="must be CUDA tensors"):
        ops.sdpa(x, x, x)


def test_ops_refuse_cpu_tensors():
    import torch

    from b200_attention_b200 import ops

    x = torch.zeros(1, 1, 256, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.attention(x, x, x)


def test_reference_side_launcher_bindings_compile_and_link(native_built, tmp_path):
    """The forwarding translation unit a maintainer of the reference adds (the C++ launcher
    signatures of benchmarks/registry.py:272-282 and benchmarks/benchmark_bshd.py:151-160) builds
    against libb200attn.so and exports both launchers under the names the reference's generated
    glue would link."""
    from tests.integration import build_forwarders as B

    so = B.build(native_built["core"], tmp_path)
    lib = C.CDLL(str(so))
    assert hasattr(lib, B.BHLD_SYMBOL) and hasattr(lib, B.BSHD_SYMBOL)


def test_split_layout_invariants():
    """The host-side cuts of the tile-stream split: the runs cover the last round's units exactly,
    empty runs only trail, no piece of a cut item is shorter than four tiles, and no run exceeds
    the even share by more than a snap."""
    import random

    from b200_attention_b200 import _native as N

    rng = random.Random(5)
    cases = [(256, 64, 148), (512, 64, 148), (300, 9, 148), (149, 8, 148), (2, 130, 148), (100, 64, 148)]
    cases += [(rng.randint(1, 1200), rng.randint(1, 300), rng.choice([148, 132, 160, 16])) for _ in range(3000)]
    split = 0
    for items, tiles, sms in cases:
        grid, cuts = N.split_layout(items, tiles, sms)
        if grid == 0:
            assert cuts == []
            continue
        split += 1
        total = (items % sms) * tiles
        runs = len(cuts) - 1
        assert grid == (sms if items >= sms else runs) and 1 <= runs <= sms
        assert cuts[0] == 0 and cuts[-1] == total
        lengths = [b - a for a, b in zip(cuts, cuts[1:])]
        assert min(lengths) >= 0
        first_empty = lengths.index(0) if 0 in lengths else runs
        assert all(n == 0 for n in lengths[first_empty:]) and all(n >= 4 for n in lengths[:first_empty])
        for a, b in zip(cuts, cuts[1:]):
            u = a
            while u < b:
                end = min(b, (u // tiles + 1) * tiles)
                assert end - u >= 4 or end - u == tiles, (items, tiles, sms, a, b)
                u = end
        assert max(lengths) <= -(-total // runs) + 4
    assert split > 300
    assert N.split_layout(256, 64, 148)[0] == 148
    _, cuts = N.split_layout(256, 64, 148)
    assert max(b - a for a, b in zip(cuts, cuts[1:])) == 47  # 108 items x 64 tiles over 148 runs: 46.7 each
