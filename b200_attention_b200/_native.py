"""ctypes binding of the C ABI declared in include/b200_attention.h.

There is no fallback of any kind: if the shared library is missing or a call fails,
an exception is raised.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_DIR = PKG / "lib"
CORE_LIB = LIB_DIR / "libb200attn.so"
TORCH_LIB = LIB_DIR / "libb200attn_torch.so"
LTX_LIB = LIB_DIR / "libltx_sm100_attention.so"

KERNEL_WARP_SPECIALIZED = 0
KERNEL_SERIAL = 1

STATUS_OK = 0
STATUS_INVALID_ARGUMENT = 1
STATUS_UNSUPPORTED = 2
STATUS_ARCH = 3
STATUS_CUDA = 4
STATUS_DRIVER = 5
STATUS_DEVICE_TIMEOUT = 6
STATUS_DEVICE_FAULT = 7

NOALLOC_MAX_ROWS = 16384

# Every symbol include/b200_attention.h declares (the CPU tests check the library exports all).
EXPORTED_SYMBOLS = (
    "b200attn_forward",
    "b200attn_workspace_bytes",
    "b200attn_split_layout",
    "b200attn_bhld_launch",
    "b200attn_bshd_launch",
    "b200attn_forward_kv_split_noalloc",
    "b200attn_device_check",
    "b200attn_set_wait_limit_ms",
    "b200attn_launch_count",
    "b200attn_sample_sm_clocks",
    "b200attn_ipc_export",
    "b200attn_ipc_open",
    "b200attn_ipc_close",
    "b200attn_copy_async",
    "b200attn_status_string",
    "b200attn_last_error",
    "b200attn_version",
)


class B200AttnError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


class Operand(C.Structure):
    _fields_ = [
        ("ptr", C.c_void_p),
        ("stride_batch", C.c_int64),
        ("stride_head", C.c_int64),
        ("stride_row", C.c_int64),
    ]


class ForwardArgs(C.Structure):
    _fields_ = [
        ("struct_bytes", C.c_uint32),
        ("batch", C.c_int32),
        ("heads", C.c_int32),
        ("len_q", C.c_int32),
        ("len_kv", C.c_int32),
        ("head_dim", C.c_int32),
        ("q", Operand),
        ("k", Operand),
        ("v", Operand),
        ("o", Operand),
        ("lse", C.c_void_p),
        ("softmax_scale", C.c_float),
        ("kernel", C.c_int32),
        ("partial_o", C.c_void_p),
        ("partial_lse", C.c_void_p),
        ("partial_merge", C.c_int32),
        ("partial_emit", C.c_int32),
        ("stream", C.c_void_p),
        ("causal", C.c_int32),
        ("heads_kv", C.c_int32),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_uint64),
    ]


_lib = None


def lib() -> C.CDLL:
    """The loaded libb200attn.so; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not CORE_LIB.exists():
            raise ImportError(
                f"{CORE_LIB} is missing: build it with `python -m b200_attention_b200.build` "
                "(there is no fallback implementation)")
        handle = C.CDLL(str(CORE_LIB), mode=C.RTLD_GLOBAL)
        handle.b200attn_forward.argtypes = [C.POINTER(ForwardArgs)]
        handle.b200attn_forward.restype = C.c_int
        handle.b200attn_workspace_bytes.argtypes = [C.POINTER(C.c_uint64)]
        handle.b200attn_workspace_bytes.restype = C.c_int
        handle.b200attn_split_layout.argtypes = [C.c_int32] * 3 + [C.POINTER(C.c_int32)] * 3 + [C.c_int32]
        handle.b200attn_split_layout.restype = C.c_int
        launch8 = [C.c_void_p] * 4 + [C.c_int] * 3 + [C.c_void_p]
        handle.b200attn_bhld_launch.argtypes = launch8
        handle.b200attn_bhld_launch.restype = C.c_int
        handle.b200attn_bshd_launch.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_void_p]
        handle.b200attn_bshd_launch.restype = C.c_int
        handle.b200attn_forward_kv_split_noalloc.argtypes = [C.POINTER(ForwardArgs), C.c_int32]
        handle.b200attn_forward_kv_split_noalloc.restype = C.c_int
        handle.b200attn_device_check.argtypes = [C.c_int, C.POINTER(C.c_int32)]
        handle.b200attn_device_check.restype = C.c_int
        handle.b200attn_set_wait_limit_ms.argtypes = [C.c_uint32]
        handle.b200attn_set_wait_limit_ms.restype = C.c_int
        handle.b200attn_launch_count.argtypes = []
        handle.b200attn_launch_count.restype = C.c_uint64
        handle.b200attn_sample_sm_clocks.argtypes = [C.c_void_p, C.c_int32, C.c_void_p]
        handle.b200attn_sample_sm_clocks.restype = C.c_int
        handle.b200attn_ipc_export.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64)]
        handle.b200attn_ipc_export.restype = C.c_int
        handle.b200attn_ipc_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        handle.b200attn_ipc_open.restype = C.c_int
        handle.b200attn_ipc_close.argtypes = [C.c_void_p]
        handle.b200attn_ipc_close.restype = C.c_int
        handle.b200attn_copy_async.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]
        handle.b200attn_copy_async.restype = C.c_int
        handle.b200attn_status_string.argtypes = [C.c_int]
        handle.b200attn_status_string.restype = C.c_char_p
        handle.b200attn_last_error.argtypes = []
        handle.b200attn_last_error.restype = C.c_char_p
        handle.b200attn_version.argtypes = []
        handle.b200attn_version.restype = C.c_char_p
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != STATUS_OK:
        h = lib()
        raise B200AttnError(
            status,
            f"b200attn: {h.b200attn_status_string(status).decode()}: {h.b200attn_last_error().decode()}")


def device_check(device: int = -1) -> None:
    """Raise if a kernel launched on `device` left early. Synchronise the stream first."""
    rec = (C.c_int32 * 8)()
    status = lib().b200attn_device_check(device, rec)
    if status != STATUS_OK:
        # a kernel that left early may have left split counters behind: start from fresh workspaces
        from . import ops

        ops.drop_workspaces()
    check(status)


def split_layout(work_items: int, kv_tiles: int, sm_count: int = 148):
    """(grid, cuts) of the tile-stream split of a dense call, or (0, []) if it would not be split:
    CTA c of the first len(cuts) - 1 takes units [cuts[c], cuts[c + 1]) of the last round's
    (item, K/V tile) pairs. Host arithmetic only."""
    grid, runs = C.c_int32(0), C.c_int32(0)
    cuts = (C.c_int32 * 256)()
    check(lib().b200attn_split_layout(work_items, kv_tiles, sm_count, C.byref(grid), C.byref(runs), cuts, 256))
    return grid.value, list(cuts[: runs.value + 1]) if grid.value else []


def launch_count() -> int:
    return int(lib().b200attn_launch_count())


def version() -> str:
    return lib().b200attn_version().decode()
