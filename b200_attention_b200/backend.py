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

_STATS_LOCK = threading.Lock()
_TOTAL_CALLS = 0
_SIGNATURES: Counter = Counter()
_UNIQUE_INPUTS: set = set()


def reset_stats() -> None:
    """Reset the process-wide statistics of successful attention calls."""
    global _TOTAL_CALLS
    with _STATS_LOCK:
        _TOTAL_CALLS = 0
        _SIGNATURES.clear()
        _UNIQUE_INPUTS.clear()


def get_stats() -> dict[str, Any]:
    """JSON-serialisable snapshot: total_calls, signatures, unique_inputs."""
    with _STATS_LOCK:
        return {
            "total_calls": _TOTAL_CALLS,
            "signatures": dict(_SIGNATURES),
            "unique_inputs": sorted(_UNIQUE_INPUTS),
        }


def ensure_loaded() -> None:
    """Load the native library now (otherwise the first valid call does). Raises if it is missing."""
    from . import _native

    _native.lib()


def _validate_inputs(query, key, value, heads, mask):
    # Order matters: the mask check comes first so that it needs neither torch nor CUDA.
    if mask is not None:
        raise RuntimeError("B200Attention supports dense, unmasked attention only.")
    import torch

    if not all(isinstance(t, torch.Tensor) for t in (query, key, value)):
        raise TypeError("B200Attention requires query, key, and value to be torch.Tensor instances.")
    if not isinstance(heads, int) or isinstance(heads, bool) or heads <= 0:
        raise ValueError(f"B200Attention requires a positive integer head count, got {heads!r}.")
    if not (query.is_cuda and key.is_cuda and value.is_cuda):
        raise RuntimeError("B200Attention requires CUDA query/key/value tensors.")
    if query.device != key.device or query.device != value.device:
        raise RuntimeError("B200Attention requires query/key/value on the same CUDA device.")
    capability = torch.cuda.get_device_capability(query.device)
    if capability != (10, 0):
        raise RuntimeError(
            "B200Attention requires an NVIDIA B200-class SM100 GPU (compute capability 10.0), "
            f"got {capability[0]}.{capability[1]}.")
    if any(t.dtype != torch.bfloat16 for t in (query, key, value)):
        raise RuntimeError(
            "B200Attention requires BF16 query/key/value tensors; "
            f"got query={query.dtype}, key={key.dtype}, value={value.dtype}.")
    if query.ndim != 3 or key.ndim != 3 or value.ndim != 3:
        raise RuntimeError(
            "B200Attention expects query/key/value shaped [B, T, H*D]; "
            f"got query={tuple(query.shape)}, key={tuple(key.shape)}, value={tuple(value.shape)}.")
    batch, query_length, hidden = query.shape
    if batch <= 0 or query_length <= 0 or key.shape[1] <= 0:
        raise RuntimeError("B200Attention requires non-empty batch and sequence dimensions.")
    if key.shape[0] != batch or value.shape[0] != batch:
        raise RuntimeError(
            "B200Attention requires matching query/key/value batch dimensions; "
            f"got query={batch}, key={key.shape[0]}, value={value.shape[0]}.")
    if value.shape[1] != key.shape[1]:
        raise RuntimeError(
            "B200Attention requires matching key/value sequence lengths; "
            f"got key={key.shape[1]}, value={value.shape[1]}.")
    if key.shape[2] != hidden or value.shape[2] != hidden:
        raise RuntimeError(
            "B200Attention requires matching query/key/value hidden dimensions; "
            f"got query={hidden}, key={key.shape[2]}, value={value.shape[2]}.")
    if hidden % heads != 0:
        raise RuntimeError(f"B200Attention cannot split hidden dimension {hidden} across {heads} heads.")
    head_dim = hidden // heads
    if head_dim != HEAD_DIM:
        raise RuntimeError(f"B200Attention supports head dimension 128 only, got {head_dim}.")
    if max(batch * heads, query_length, key.shape[1]) > 2**31 - 1:
        raise RuntimeError("B200Attention dimensions exceed 32-bit integer limits.")
    return batch, query_length, key.shape[1], head_dim


def _record_success(query, key, value, *, batch, query_length, key_value_length, heads, head_dim):
    global _TOTAL_CALLS
    signature = (f"B={batch},Lq={query_length},Lkv={key_value_length},H={heads},D={head_dim},"
                 f"dtype={query.dtype},device={query.device}")
    input_record = (f"q_shape={tuple(query.shape)} q_stride={tuple(query.stride())}; "
                    f"k_shape={tuple(key.shape)} k_stride={tuple(key.stride())}; "
                    f"v_shape={tuple(value.shape)} v_stride={tuple(value.stride())}")
    with _STATS_LOCK:
        _TOTAL_CALLS += 1
        _SIGNATURES[signature] += 1
        _UNIQUE_INPUTS.add(input_record)


class B200Attention:
    """Callable accepted by the video model's `DiffusionStage.with_attention(...)`."""

    label = "B200Attention"

    def __init__(self, *, softmax_scale: float = 0.0) -> None:
        self._softmax_scale = float(softmax_scale)
        self._loaded = False

    def __call__(self, query, key, value, heads: int, mask=None):
        batch, lq, lk, head_dim = _validate_inputs(query, key, value, heads, mask)
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
        _record_success(query, key, value, batch=batch, query_length=lq, key_value_length=lk,
                        heads=heads, head_dim=head_dim)
        return output


__all__ = ["B200Attention", "ensure_loaded", "get_stats", "reset_stats"]
