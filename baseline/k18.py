"""ctypes access to the reference project's final checkpoint kernel as built by baseline/Makefile:

  _ref/libk18_ref.so        kernels/5_minor/18_tma_l2_promotion.cu, compiled unmodified
  _ref/libk18_bshd_ref.so   kernels/variants/18_tma_l2_promotion_bshd.cu, compiled unmodified

A comparison arm only (timed beside this library's kernel on the same GPU, and compared with it
on the same inputs by one GPU test). Nothing here is imported by the b200_attention_b200 package.
The launch symbols are the C++ functions the reference's generated glue binds
(benchmarks/registry.py:272-282, benchmarks/benchmark_bshd.py:151-160), looked up by mangled name.
"""

from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

REF_DIR = Path(__file__).resolve().parent / "_ref"
K18_SYMBOL = "_Z28attention_tcgen05_v18_launchPK13__nv_bfloat16S1_S1_PS_iiiP11CUstream_st"
K18_BSHD_SYMBOL = "_Z33attention_tcgen05_v18_bshd_launchPK13__nv_bfloat16S1_S1_PS_iiiiP11CUstream_st"

_cache: dict = {}


def _load(name: str):
    path = REF_DIR / name
    if not path.exists():
        return None
    if name not in _cache:
        _cache[name] = C.CDLL(str(path))
    return _cache[name]


def available(layout: str = "bhld") -> bool:
    return (REF_DIR / ("libk18_ref.so" if layout == "bhld" else "libk18_bshd_ref.so")).exists()


def supports(len_q: int, len_kv: int) -> bool:
    """The reference launcher's own shape rule (18_tma_l2_promotion.cu:1011-1015)."""
    return len_q % 256 == 0 and len_kv % 128 == 0 and len_q >= 256 and len_kv >= 128


def bhld(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Reference kernel on contiguous CUDA bf16 [B, H, L, 128]."""
    lib = _load("libk18_ref.so")
    if lib is None:
        raise RuntimeError("baseline/_ref/libk18_ref.so is missing")
    fn = getattr(lib, K18_SYMBOL)
    fn.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3 + [C.c_void_p]
    fn.restype = None
    assert q.is_cuda and q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    B, H, Lq, _ = q.shape
    Lk = k.shape[2]
    assert supports(Lq, Lk)
    o = torch.empty_like(q) if out is None else out
    fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), B * H, Lq, Lk,
       torch.cuda.current_stream().cuda_stream)
    return o


def bshd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Reference direct-BSHD kernel on contiguous CUDA bf16 [B, L, H, 128]."""
    lib = _load("libk18_bshd_ref.so")
    if lib is None:
        raise RuntimeError("baseline/_ref/libk18_bshd_ref.so is missing")
    fn = getattr(lib, K18_BSHD_SYMBOL)
    fn.argtypes = [C.c_void_p] * 4 + [C.c_int] * 4 + [C.c_void_p]
    fn.restype = None
    assert q.is_cuda and q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
    B, Lq, H, _ = q.shape
    Lk = k.shape[1]
    assert supports(Lq, Lk)
    o = torch.empty_like(q) if out is None else out
    fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), B, H, Lq, Lk,
       torch.cuda.current_stream().cuda_stream)
    return o
