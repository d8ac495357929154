"""ctypes access to what oracle/Makefile builds into oracle/_ref/. TEST INFRASTRUCTURE ONLY.

  libsdpa_ref.so       the plain-C restatement (oracle/sdpa_ref.c), a CPU checker

Nothing here is imported by the b200_attention_b200 package.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

REF_DIR = Path(__file__).resolve().parent / "_ref"

_cache: dict = {}


def _load(name: str):
    path = REF_DIR / name
    if not path.exists():
        return None
    if name not in _cache:
        _cache[name] = C.CDLL(str(path))
    return _cache[name]


def c_ref_available() -> bool:
    return (REF_DIR / "libsdpa_ref.so").exists()


def sdpa_c_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
               rows: tuple[int, int] | None = None):
    """q [BH, Lq, 128], k/v [BH, Lk, 128] bf16 CPU contiguous -> (O fp32 [BH, rows, 128], LSE)."""
    lib = _load("libsdpa_ref.so")
    if lib is None:
        raise RuntimeError("oracle/_ref/libsdpa_ref.so is missing: run `make -C oracle`")
    fn = lib.sdpa_ref_forward
    fn.argtypes = [C.c_void_p] * 5 + [C.c_int64] * 3 + [C.c_float, C.c_int64, C.c_int64]
    fn.restype = C.c_int
    q, k, v = (t.contiguous().cpu() for t in (q, k, v))
    assert q.dtype == torch.bfloat16 and q.dim() == 3
    bh, lq, _ = q.shape
    lk = k.shape[1]
    r0, r1 = rows if rows is not None else (0, lq)
    o = torch.empty(bh, r1 - r0, 128, dtype=torch.float32)
    lse = torch.empty(bh, r1 - r0, dtype=torch.float32)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), bh, lq, lk,
            float(scale), r0, r1)
    if rc != 0:
        raise RuntimeError(f"sdpa_ref_forward failed with {rc}")
    return o, lse
