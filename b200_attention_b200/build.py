"""Builds the native libraries in-tree with nvcc / g++ (no JIT cache, no build system).

    python -m b200_attention_b200.build            # everything that is out of date
    python -m b200_attention_b200.build --force

Outputs (git-ignored, next to the sources they come from):
    b200_attention_b200/lib/libb200attn.so              kernels + C ABI (no torch dependency)
    b200_attention_b200/lib/libb200attn_torch.so        torch ops `b200_attention_b200::*`
    b200_attention_b200/lib/libltx_sm100_attention.so   torch op  `ltx_sm100::attention`
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
INCLUDE = PKG.parent / "include"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
CORE_SOURCES = [CSRC / "attn_fwd_sm100.cu", CSRC / "capi.cu", CSRC / "noalloc.cu"]
CORE_HEADERS = [CSRC / "attn_kernels.cuh", CSRC / "ptx_sm100.cuh", CSRC / "host_common.cuh",
                INCLUDE / "b200_attention.h"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _digest(paths, extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(Path(p).name.encode())
        h.update(Path(p).read_bytes())
    return h.hexdigest()


def _stale(target: Path, digest: str) -> bool:
    stamp = target.with_suffix(target.suffix + ".sha256")
    return not (target.exists() and stamp.exists() and stamp.read_text().strip() == digest)


def _run(cmd, verbose: bool) -> None:
    if verbose:
        print("+", " ".join(map(str, cmd)), flush=True)
    proc = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed ({proc.returncode}):\n{' '.join(map(str, cmd))}\n"
                           f"{proc.stdout}\n{proc.stderr}")
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout, proc.stderr, flush=True)


def build_core(force: bool = False, verbose: bool = False, defines: tuple[str, ...] = (),
               name: str = "libb200attn.so") -> Path:
    """Kernels + C ABI -> libb200attn.so (links the CUDA runtime statically). `defines` and `name`
    build an instrumented variant beside it (see role_budget.py)."""
    LIB.mkdir(exist_ok=True)
    out = LIB / name
    flags = ["-std=c++17", "-O3", "-lineinfo", *ARCH_FLAGS, "-Xcompiler", "-fPIC,-fvisibility=hidden",
             "-Xptxas", "-v", *[f"-D{d}" for d in defines]]
    digest = _digest(CORE_SOURCES + CORE_HEADERS, " ".join(flags))
    if force or _stale(out, digest):
        _run([_nvcc(), *flags, "-shared", "-o", out, *CORE_SOURCES], verbose)
        out.with_suffix(".so.sha256").write_text(digest)
    return out


def _torch_flags():
    import torch
    from torch.utils import cpp_extension as ce

    inc = [f"-I{p}" for p in ce.include_paths("cuda")]
    libdir = Path(torch.__file__).resolve().parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cflags = ["-std=c++17", "-O2", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
              "-DTORCH_API_INCLUDE_EXTENSION_H", *inc]
    ldflags = [f"-L{libdir}", f"-Wl,-rpath,{libdir}", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch",
               f"-L{LIB}", "-Wl,-rpath,$ORIGIN", "-lb200attn"]
    return cflags, ldflags, torch.__version__


def _build_torch_lib(src: Path, out: Path, force: bool, verbose: bool) -> Path:
    cflags, ldflags, tver = _torch_flags()
    digest = _digest([src, INCLUDE / "b200_attention.h"], tver + " ".join(cflags))
    if force or _stale(out, digest):
        _run([os.environ.get("CXX", "g++"), *cflags, "-o", out, src, *ldflags], verbose)
        out.with_suffix(".so.sha256").write_text(digest)
    return out


def build_torch_ops(force: bool = False, verbose: bool = False) -> Path:
    build_core(False, verbose)
    return _build_torch_lib(CSRC / "torch_ops.cpp", LIB / "libb200attn_torch.so", force, verbose)


def build_ltx_op(force: bool = False, verbose: bool = False) -> Path:
    build_core(False, verbose)
    return _build_torch_lib(CSRC / "ltx_sm100_op.cpp", LIB / "libltx_sm100_attention.so", force, verbose)


def build_all(force: bool = False, verbose: bool = False) -> dict[str, Path]:
    return {
        "core": build_core(force, verbose),
        "torch_ops": build_torch_ops(force, verbose),
        "ltx_op": build_ltx_op(force, verbose),
    }


if __name__ == "__main__":
    built = build_all(force="--force" in sys.argv, verbose=True)
    for name, path in built.items():
        print(f"{name}: {path}")
