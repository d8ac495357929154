"""Compiles tests/integration/b200attn_forwarders.cu (the reference-side launcher bindings)
against libb200attn.so. Host-only C++: g++ with the CUDA headers, no GPU needed."""

from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
SOURCE = HERE / "b200attn_forwarders.cu"

# The mangled names of the two launchers: the reference's generated glue declares these C++
# functions and the linker resolves them by exactly these symbols.
BHLD_SYMBOL = "_Z29attention_b200attn_v19_launchPK13__nv_bfloat16S1_S1_PS_iiiP11CUstream_st"
BSHD_SYMBOL = "_Z34attention_b200attn_v19_bshd_launchPK13__nv_bfloat16S1_S1_PS_iiiiP11CUstream_st"


def cuda_include() -> Path:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and (Path(cand) / "include" / "cuda_bf16.h").exists():
            return Path(cand) / "include"
    nvcc = shutil.which("nvcc")
    if nvcc:
        return Path(nvcc).resolve().parents[1] / "include"
    raise RuntimeError("CUDA headers not found")


def build(core_lib: Path, out_dir: Path) -> Path:
    out = out_dir / "libb200attn_forwarders.so"
    cmd = [os.environ.get("CXX", "g++"), "-std=c++17", "-O2", "-shared", "-fPIC", "-x", "c++",
           f"-I{ROOT / 'include'}", f"-I{cuda_include()}", str(SOURCE), "-o", str(out),
           f"-L{core_lib.parent}", "-lb200attn", f"-Wl,-rpath,{core_lib.parent}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"forwarder build failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    return out
