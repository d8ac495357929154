"""Tensor-level entry points: torch tensors in, C ABI underneath.

`attention()` goes straight to `b200attn_forward` through ctypes with the tensors' device
pointers and strides (no copies, any layout whose head_dim axis is dense). The
`torch.ops.b200_attention_b200.*` ops registered by the C++ shim are reached through
`registry.load_kernel()`.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _native as N

HEAD_DIM = 128

# Workspaces of the tile-stream split, one per (device, stream): kernels on one stream run one
# after the other and may share it, kernels on different streams may overlap and may not.
_workspaces: dict = {}


def workspace_for(device: torch.device, stream: torch.cuda.Stream) -> Optional[torch.Tensor]:
    """The cached split workspace of (device, stream), allocated (zeroed) on first use; None while
    the stream is being captured and nothing has been allocated for it yet."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream.cuda_stream)
    ws = _workspaces.get(key)
    if ws is None:
        if torch.cuda.is_current_stream_capturing():
            return None
        size = C.c_uint64(0)
        N.check(N.lib().b200attn_workspace_bytes(C.byref(size)))
        with torch.cuda.stream(stream):
            ws = torch.zeros(int(size.value), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def drop_workspaces() -> None:
    """Forget every cached workspace (after a device-side timeout their counters may be stale)."""
    _workspaces.clear()


def _operand(t: torch.Tensor, layout: str) -> N.Operand:
    if layout == "bhld":
        sb, sh, sl = t.stride(0), t.stride(1), t.stride(2)
    elif layout == "bshd":
        sb, sl, sh = t.stride(0), t.stride(1), t.stride(2)
    else:
        raise ValueError(f"layout must be 'bhld' or 'bshd', got {layout!r}")
    return N.Operand(t.data_ptr(), sb, sh, sl)


def _dims(t: torch.Tensor, layout: str) -> Tuple[int, int, int]:
    if layout == "bhld":
        return t.size(0), t.size(1), t.size(2)
    return t.size(0), t.size(2), t.size(1)


def attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    layout: str = "bhld",
    softmax_scale: float = 0.0,
    causal: bool = False,
    return_lse: bool = False,
    out: Optional[torch.Tensor] = None,
    kernel: int = N.KERNEL_WARP_SPECIALIZED,
    partial: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    partial_merge: bool = False,
    partial_emit: bool = False,
    stream: Optional[torch.cuda.Stream] = None,
    workspace="auto",
):
    """O = softmax(Q K^T * scale) V on the current CUDA stream.

    q: [B, H, Lq, 128] ('bhld') or [B, Lq, H, 128] ('bshd'), bf16, CUDA; k, v likewise with Lk.
    Returns O (same layout as q) and, if asked, LSE [B, H, Lq] fp32 (natural log).
    k and v may have fewer heads than q (grouped-query attention: query head h reads K/V head
    h // (H // Hkv)). `causal=True` masks key j for query row i unless j <= i + (Lk - Lq)
    (bottom-right aligned, needs Lk >= Lq).
    `partial=(o_fp32 [B,H,Lq,128], lse_fp32 [B,H,Lq])` with the two flags chains calls over K/V
    shards; see include/b200_attention.h.
    `workspace`: "auto" (a zeroed device buffer cached per stream, which lets a dense call whose
    work items do not fill the SMs evenly be cut into equal runs of K/V tiles), None (never
    split), or a uint8 CUDA tensor of at least b200attn_workspace_bytes() zeroed bytes.
    """
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"{name} must be a torch.Tensor")
        if not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor (this library has no CPU path)")
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name} must be bfloat16, got {t.dtype}")
        if t.dim() != 4 or t.size(3) != HEAD_DIM:
            raise RuntimeError(f"{name} must be 4-D with head_dim {HEAD_DIM}, got {tuple(t.shape)}")
        if t.stride(3) != 1:
            raise RuntimeError(f"{name}: the head_dim axis must be contiguous")
    if q.device != k.device or q.device != v.device:
        raise RuntimeError("q, k, v must be on the same device")
    B, H, Lq = _dims(q, layout)
    Bk, Hk, Lk = _dims(k, layout)
    if Bk != B or tuple(k.shape) != tuple(v.shape):
        raise RuntimeError("q, k, v disagree on batch, or k and v differ in shape")
    if Hk < 1 or H % Hk != 0:
        raise RuntimeError(f"q has {H} heads, k and v have {Hk}: not a whole number of query heads per K/V head")

    with torch.cuda.device(q.device):
        if out is None:
            out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        elif out.shape != q.shape or out.dtype != q.dtype or out.device != q.device or out.stride(3) != 1:
            raise RuntimeError("out must match q in shape, dtype and device with a dense head_dim axis")
        lse = torch.empty((B, H, Lq), dtype=torch.float32, device=q.device) if return_lse else None

        a = N.ForwardArgs()
        a.struct_bytes = C.sizeof(N.ForwardArgs)
        a.batch, a.heads, a.len_q, a.len_kv, a.head_dim = B, H, Lq, Lk, HEAD_DIM
        a.q, a.k, a.v, a.o = (_operand(t, layout) for t in (q, k, v, out))
        a.lse = lse.data_ptr() if lse is not None else None
        a.softmax_scale = float(softmax_scale)
        a.kernel = int(kernel)
        a.causal = int(bool(causal))
        a.heads_kv = Hk
        if partial is not None:
            po, pl = partial
            if po.dtype != torch.float32 or pl.dtype != torch.float32 or not po.is_contiguous() \
                    or not pl.is_contiguous() or tuple(po.shape) != (B, H, Lq, HEAD_DIM) \
                    or tuple(pl.shape) != (B, H, Lq) or po.device != q.device or pl.device != q.device:
                raise RuntimeError("partial must be (fp32 [B,H,Lq,128], fp32 [B,H,Lq]), contiguous, on q's device")
            a.partial_o, a.partial_lse = po.data_ptr(), pl.data_ptr()
        a.partial_merge = int(bool(partial_merge))
        a.partial_emit = int(bool(partial_emit))
        s = stream if stream is not None else torch.cuda.current_stream(q.device)
        a.stream = s.cuda_stream
        if isinstance(workspace, str):
            if workspace != "auto":
                raise ValueError("workspace must be 'auto', None or a uint8 CUDA tensor")
            workspace = workspace_for(q.device, s) if (partial is None and not causal) else None
        if workspace is not None:
            if workspace.dtype != torch.uint8 or workspace.device != q.device or not workspace.is_contiguous():
                raise RuntimeError("workspace must be a contiguous uint8 tensor on q's device")
            a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
        N.check(N.lib().b200attn_forward(C.byref(a)))
    return (out, lse) if return_lse else out
