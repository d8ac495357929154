"""Kernel registry with the surface of the reference benchmark registry.

The reference (IaroslavElistratov/b200-attention, benchmarks/registry.py) keeps a table of
`KernelSpec(number, label, source, launch_symbol, len_q_multiple)` (:63-73), resolves a kernel by
number / label (:202-212), a shape by name (:215-223), and `load_kernel(spec)` (:359-377) returns
`torch.ops.<namespace>` whose `.sdpa(Q, K, V)` is what benchmarks/benchmark.py:250-251 and
benchmarks/check_correctness.py:97 call. This module offers the same names for this library's
kernel, loading the prebuilt torch shim instead of JIT-compiling (there is nothing to compile
at run time and no fallback if the library is missing).
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass
from pathlib import Path

from . import _native

PKG = Path(__file__).resolve().parent
HEAD_DIM = 128


@dataclass(frozen=True)
class KernelSpec:
    number: int
    label: str
    source: str          # kernel source, relative to the package
    launch_symbol: str   # C-ABI entry point behind the op
    len_q_multiple: int  # 1: no length restriction (the reference's kernels need 128 or 256)
    op_name: str = "sdpa"
    layout: str = "bhld"

    @property
    def op_namespace(self) -> str:
        return "b200_attention_b200"


KERNELS = (
    KernelSpec(19, "b200", "csrc/attn_fwd_sm100.cu", "b200attn_bhld_launch", 1, "sdpa", "bhld"),
    KernelSpec(20, "b200_bshd", "csrc/attn_fwd_sm100.cu", "b200attn_bshd_launch", 1, "sdpa_bshd", "bshd"),
)

# Shapes of the reference benchmark (benchmarks/registry.py:188-192): (batch, heads, len_q, len_kv)
SHAPES = {
    "paper4k": (8, 16, 4096, 4096),
    "paper8k": (4, 16, 8192, 8192),
    "paper16k": (2, 16, 16384, 16384),
}


def resolve_kernel(value: str | int) -> KernelSpec:
    key = str(value).strip()
    if not key:
        raise ValueError("Pass a kernel: " + ", ".join(s.label for s in KERNELS))
    for spec in KERNELS:
        if key in {str(spec.number), spec.label, spec.launch_symbol}:
            return spec
    raise ValueError(f"Unknown kernel {value!r}; choose one of: " + ", ".join(s.label for s in KERNELS))


def resolve_shape(value: str) -> tuple[str, int, int, int, int]:
    name = value.strip().lower()
    try:
        batch, heads, len_q, len_kv = SHAPES[name]
    except KeyError as exc:
        raise ValueError(f"Unknown shape {value!r}; choose one of: {', '.join(SHAPES)}") from exc
    return name, batch, heads, len_q, len_kv


def sha256_file(path: Path) -> str:
    return hashlib.sha256(Path(path).read_bytes()).hexdigest()


def source_closure_sha256(spec: KernelSpec) -> str:
    """Fingerprint of the kernel source and every header it includes (cf. registry.py:230-255)."""
    h = hashlib.sha256()
    names = ["csrc/attn_fwd_sm100.cu", "csrc/capi.cu", "csrc/noalloc.cu", "csrc/attn_kernels.cuh",
             "csrc/ptx_sm100.cuh", "csrc/host_common.cuh", "../include/b200_attention.h"]
    for name in names:
        p = (PKG / name).resolve()
        h.update(name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


class _KernelModule:
    """What `load_kernel` returns: `.sdpa(Q, K, V)` like the reference's op namespace."""

    def __init__(self, spec: KernelSpec, ops_namespace):
        self.spec = spec
        self._ns = ops_namespace
        self._op = getattr(ops_namespace, spec.op_name)

    def sdpa(self, q, k, v):
        return self._op(q, k, v)

    def sdpa_lse(self, q, k, v, scale: float = 0.0):
        return self._ns.sdpa_lse(q, k, v, float(scale), self.spec.layout == "bshd", 0)

    def device_check(self) -> None:
        self._ns.device_check()


_loaded = False


def load_kernel(spec: KernelSpec) -> _KernelModule:
    """Loads libb200attn.so and the torch shim (once) and returns the module-like wrapper."""
    global _loaded
    import torch

    _native.lib()  # raises if the core library has not been built
    if not _loaded:
        if not _native.TORCH_LIB.exists():
            raise ImportError(f"{_native.TORCH_LIB} is missing: run `python -m b200_attention_b200.build`")
        torch.ops.load_library(str(_native.TORCH_LIB))
        _loaded = True
    return _KernelModule(spec, torch.ops.b200_attention_b200)
