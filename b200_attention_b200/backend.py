"""Attention callable for the video-generation model, with the contract of the reference's
`SM100Attention` (capstone-project/src/ltx_sm100/backend.py:180-263): call signature
`(query, key, value, heads, mask=None)` on token-major `[B, T, H*128]` bf16 CUDA tensors, a
`label`, lazy loading, strict validation (a mask is rejected before anything touches CUDA),
and process-wide call statistics with the same keys and signature-string format that the
reference CLI checks (capstone-project/src/ltx_sm100/cli.py:167-208).

Difference: `[B, T, H*128]` is read and written in place as the `[B, T, H, 128]` view it already
is (strided BSHD through the C ABI), so the reference's four `.contiguous()` layout passes per
call (backend.py:226-228, 247-252) do not exist here, and sequence lengths need not be
multiples of 256 / 128.
"""

from __future__ import annotations

import threading
from collections import Counter
from typing import TYPE_CHECKING, Any

if TYPE_CHECKING:
    import torch

HEAD_DIM = 128


class _CallLog:
    """Process-wide record of successful attention calls. What the reference's CLI reads from it
    (capstone-project/src/ltx_sm100/cli.py:167-208) is the contract: the three keys of
    `snapshot()` and the text of a signature."""

    def __init__(self) -> None:
        self._guard = threading.Lock()
        self._calls = 0
        self._by_signature: Counter = Counter()
        self._layouts: set = set()

    def clear(self) -> None:
        with self._guard:
            self._calls = 0
            self._by_signature.clear()
            self._layouts.clear()

    def add(self, tensors, dims) -> None:
        query = tensors[0]
        signature = ("B={0},Lq={1},Lkv={2},H={3},D={4},".format(*dims)
                     + f"dtype={query.dtype},device={query.device}")
        layout = "; ".join(f"{name}_shape={tuple(t.shape)} {name}_stride={tuple(t.stride())}"
                           for name, t in zip("qkv", tensors))
        with self._guard:
            self._calls += 1
            self._by_signature[signature] += 1
            self._layouts.add(layout)

    def snapshot(self) -> dict[str, Any]:
        with self._guard:
            return {"total_calls": self._calls, "signatures": dict(self._by_signature),
                    "unique_inputs": sorted(self._layouts)}


_LOG = _CallLog()


def reset_stats() -> None:
    """Reset the process-wide statistics of successful attention calls."""
    _LOG.clear()


def get_stats() -> dict[str, Any]:
    """JSON-serialisable snapshot: total_calls, signatures, unique_inputs."""
    return _LOG.snapshot()


def ensure_loaded() -> None:
    """Load the native library now (otherwise the first valid call does). Raises if it is missing."""
    from . import _native

    _native.lib()


def _refuse(kind, text):
    raise kind("B200Attention " + text)


def _check_call(query, key, value, heads, mask):
    """The rules of the reference callable (capstone-project/src/ltx_sm100/backend.py:64-141), in an
    order that keeps its promise that a mask is refused before torch or CUDA are touched, minus its
    length rules (no multiple-of-256 / multiple-of-128 requirement here). Returns
    (batch, len_q, len_kv, head_dim). The wording callers match on is kept: "unmasked attention
    only", "BF16", "head dimension 128"."""
    if mask is not None:
        _refuse(RuntimeError, "supports dense, unmasked attention only.")
    import torch

    qkv = (query, key, value)
    if not all(isinstance(t, torch.Tensor) for t in qkv):
        _refuse(TypeError, "requires query, key, and value to be torch.Tensor instances.")
    if isinstance(heads, bool) or not isinstance(heads, int) or heads <= 0:
        _refuse(ValueError, f"requires a positive integer head count, got {heads!r}.")
    if not all(t.is_cuda for t in qkv):
        _refuse(RuntimeError, "requires CUDA query/key/value tensors.")
    if len({t.device for t in qkv}) != 1:
        _refuse(RuntimeError, "requires query/key/value on the same CUDA device.")
    major, minor = torch.cuda.get_device_capability(query.device)
    if (major, minor) != (10, 0):
        _refuse(RuntimeError, "requires an NVIDIA B200-class SM100 GPU (compute capability 10.0), "
                              f"got {major}.{minor}.")
    shapes = ", ".join(f"{n}={tuple(t.shape)}" for n, t in zip(("query", "key", "value"), qkv))
    if any(t.dtype != torch.bfloat16 for t in qkv):
        _refuse(RuntimeError, "requires BF16 query/key/value tensors; got "
                + ", ".join(f"{n}={t.dtype}" for n, t in zip(("query", "key", "value"), qkv)) + ".")
    if any(t.ndim != 3 for t in qkv):
        _refuse(RuntimeError, f"expects query/key/value shaped [B, T, H*D]; got {shapes}.")
    batch, len_q, hidden = query.shape
    len_kv = key.shape[1]
    if min(batch, len_q, len_kv) <= 0:
        _refuse(RuntimeError, "requires non-empty batch and sequence dimensions.")
    if key.shape[0] != batch or value.shape[0] != batch:
        _refuse(RuntimeError, f"requires matching query/key/value batch dimensions; got {shapes}.")
    if value.shape[1] != len_kv:
        _refuse(RuntimeError, f"requires matching key/value sequence lengths; got {shapes}.")
    if key.shape[2] != hidden or value.shape[2] != hidden:
        _refuse(RuntimeError, f"requires matching query/key/value hidden dimensions; got {shapes}.")
    head_dim, rest = divmod(hidden, heads)
    if rest:
        _refuse(RuntimeError, f"cannot split hidden dimension {hidden} across {heads} heads.")
    if head_dim != HEAD_DIM:
        _refuse(RuntimeError, f"supports head dimension 128 only, got {head_dim}.")
    if max(batch * heads, len_q, len_kv) >= 2**31:
        _refuse(RuntimeError, "dimensions exceed 32-bit integer limits.")
    return batch, len_q, len_kv, head_dim


class B200Attention:
    """Callable accepted by the video model's `DiffusionStage.with_attention(...)`."""

    label = "B200Attention"

    def __init__(self, *, softmax_scale: float = 0.0) -> None:
        self._softmax_scale = float(softmax_scale)
        self._loaded = False

    def __call__(self, query, key, value, heads: int, mask=None):
        batch, lq, lk, head_dim = _check_call(query, key, value, heads, mask)
        if not self._loaded:
            ensure_loaded()
            self._loaded = True
        from . import ops

        def as_bshd(t):
            # token-major [B, T, H*128] -> [B, T, H, 128] view; copy only if the view is unusable
            if t.stride(2) != 1:
                t = t.contiguous()
            v = t.unflatten(2, (heads, head_dim))
            ok = v.data_ptr() % 16 == 0 and all(
                v.size(d) == 1 or (v.stride(d) % 8 == 0 and v.stride(d) >= head_dim) for d in range(3))
            return v if ok else v.contiguous()

        q4, k4, v4 = as_bshd(query), as_bshd(key), as_bshd(value)
        out = ops.attention(q4, k4, v4, layout="bshd", softmax_scale=self._softmax_scale)
        output = out.view(batch, lq, heads * head_dim)
        _LOG.add((query, key, value), (batch, lq, lk, heads, head_dim))
        return output


__all__ = ["B200Attention", "ensure_loaded", "get_stats", "reset_stats"]
