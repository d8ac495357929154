"""A bounded device-side wait that actually runs out.

Every wait in the kernels gives up after the configured limit, records where it stopped and lets
the CTA leave (copies drained, TMEM freed); the host sees B200ATTN_ERR_DEVICE_TIMEOUT from
b200attn_device_check. The shipped library has no way to make that happen on purpose, so this test
compiles a variant of it with B200ATTN_TEST_DROP_P_READY (one softmax warp withholds one barrier
arrival on the second K/V tile of the first work item), runs a one-item launch with a 20 ms limit
and checks the status, the record, and that the device is fully usable afterwards. Nothing traps,
faults or spins without a limit: the kernel returns by itself after a few tens of milliseconds."""

import ctypes as C
import subprocess

import pytest
import torch

from oracle import sdpa_oracle as O

pytestmark = pytest.mark.gpu

TIMEOUT_SITES = {
    110, 111, 112, 100, 101,          # TMA warp: K/V pair slot or Q tile not released
    200, 201, 202, 210, 220, 221, 240, 241,   # MMA warp: pair, Q, P or accumulator not ready
    300, 301, 310, 311,               # softmax warps: scores or hand-off slot not ready
    410, 411, 420, 421,               # epilogue warps: final statistics or last PV not ready
}


def _build_variant(tmp_path):
    from b200_attention_b200 import build

    out = tmp_path / "libb200attn_drop.so"
    cmd = [build._nvcc(), "-std=c++17", "-O3", *build.ARCH_FLAGS, "-Xcompiler", "-fPIC,-fvisibility=hidden",
           "-DB200ATTN_TEST_DROP_P_READY", "-shared", "-o", str(out), *map(str, build.CORE_SOURCES)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    return out


def _forward(lib, N, q, k, v, o, lse):
    a = N.ForwardArgs()
    a.struct_bytes = C.sizeof(N.ForwardArgs)
    b, h, lq, _ = q.shape
    a.batch, a.heads, a.len_q, a.len_kv, a.head_dim = b, h, lq, k.shape[2], 128
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o)):
        setattr(a, name, N.Operand(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2)))
    a.lse = lse.data_ptr()
    a.stream = torch.cuda.current_stream().cuda_stream
    return lib.b200attn_forward(C.byref(a))


def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(native_built, tmp_path):
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    from b200_attention_b200 import _native as N
    from b200_attention_b200 import ops

    lib = C.CDLL(str(_build_variant(tmp_path)))
    lib.b200attn_forward.argtypes = [C.POINTER(N.ForwardArgs)]
    lib.b200attn_device_check.argtypes = [C.c_int, C.POINTER(C.c_int32)]
    lib.b200attn_set_wait_limit_ms.argtypes = [C.c_uint32]
    lib.b200attn_last_error.restype = C.c_char_p
    assert lib.b200attn_set_wait_limit_ms(20) == 0

    # one work item, four K/V tiles: the withheld arrival is on the second tile
    q, k, v = (O.to_bhld(t).cuda() for t in O.make_inputs_benchmark(1, 1, 256, 512, seed=80))
    o = torch.zeros_like(q)
    lse = torch.zeros(1, 1, 256, dtype=torch.float32, device="cuda")
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert _forward(lib, N, q, k, v, o, lse) == 0          # the launch itself succeeds
    t1.record()
    torch.cuda.synchronize()                                # and the kernel ends by itself
    assert t0.elapsed_time(t1) < 2000.0
    rec = (C.c_int32 * 8)()
    assert lib.b200attn_device_check(-1, rec) == N.STATUS_DEVICE_TIMEOUT
    code, site, block, warp, parity, item, tile = list(rec)[:7]
    assert code == 1 and site in TIMEOUT_SITES and block == 0 and 0 <= warp < 16 and item == 0
    assert 0 <= tile <= 4
    assert b"timed out" in lib.b200attn_last_error()
    # the record was cleared by the read
    assert lib.b200attn_device_check(-1, rec) == N.STATUS_OK

    # the same library, a launch that never reaches the withheld arrival (one K/V tile): clean and
    # correct, so the CTA that gave up released its TMEM and left no barrier or copy behind
    q1, k1, v1 = (O.to_bhld(t).cuda() for t in O.make_inputs_benchmark(1, 4, 512, 128, seed=81))
    o1 = torch.empty_like(q1)
    lse1 = torch.empty(1, 4, 512, dtype=torch.float32, device="cuda")
    assert _forward(lib, N, q1, k1, v1, o1, lse1) == 0
    torch.cuda.synchronize()
    assert lib.b200attn_device_check(-1, rec) == N.STATUS_OK
    o_ref, lse_ref = O.sdpa_explicit(q1.cpu(), k1.cpu(), v1.cpu())
    O.assert_within_contract(O.compare(o1.cpu(), o_ref, lse1.cpu(), lse_ref))

    # and the shipped library on the inputs that timed out above
    good, lse_good = ops.attention(q, k, v, return_lse=True)
    torch.cuda.synchronize()
    N.device_check()
    o_ref, lse_ref = O.sdpa_explicit(q.cpu(), k.cpu(), v.cpu())
    O.assert_within_contract(O.compare(good.cpu(), o_ref, lse_good.cpu(), lse_ref))
