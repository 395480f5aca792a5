"""Fused family: one call for the forward launches of model.mojo:668-699 (RoPE on q, k
then flash attention) and one for the backward launches of model.mojo:915-964
(D, dQ, dK/dV, inverse RoPE), on bf16 or fp32 CUDA tensors of shape [B, T, H, 128].
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from . import _lib

_DT = {torch.float32: _lib.AR_F32, torch.bfloat16: _lib.AR_BF16}


@dataclass
class AttnParams:
    """Arguments shared by attn_fwd / attn_bwd.

    window: the reference's window_size (<= 0 or >= T: full causal; else keys q-window..q).
    rope:   (cos, sin) fp32 CUDA tables [rows >= T, 64] to rotate q and k with position t on
            the way in (gradients come back for the un-rotated q, k); None if q, k are
            already rotated.
    rope_prepass: rotate in a separate kernel instead of inside the attention kernel.
    grad_dtype: dtype of dq, dk, dv (float32 like the reference's grad buffers, or bfloat16).
    sync: wait for completion and check the device status word before returning.
    """
    window: int = 0
    rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
    rope_prepass: bool = False
    grad_dtype: torch.dtype = torch.float32
    sync: bool = False
    stream: Optional[int] = None
    skip_d: bool = False     # attn_bwd: d_buf already holds D
    skip_dq: bool = False    # attn_bwd: do not compute dq
    skip_dkv: bool = False   # attn_bwd: do not compute dk, dv
    # optional bf16 [B,T,H,D] buffers for the rotated q, k (the reference's saved_q / saved_k):
    # attn_fwd fills them, attn_bwd given the same params reads them instead of rotating again
    q_rot: Optional[torch.Tensor] = None
    k_rot: Optional[torch.Tensor] = None


def _layout(q: torch.Tensor):
    """Element strides (b, t, h) of a [B, T, H, D] tensor for ar_attn_params, or None when it is
    contiguous.  Accepted besides contiguous tensors: a head range cut out of a wider contiguous
    [B, T, H_all, D] tensor, i.e. strides (T * H_all * D, H_all * D, D, 1)."""
    if q.is_contiguous():
        return None
    sb, st, sh, sd = q.stride()
    D = q.shape[3]
    if sd != 1 or sh != D or st % D != 0 or sb % D != 0 or st < q.shape[2] * D or sb < q.shape[1] * st:
        raise ValueError(f"unsupported strides {q.stride()}: only a head range of a contiguous [B,T,H,D] tensor")
    return (sb, st, sh)


def _check(t: torch.Tensor, name: str, shape=None, dtype=None, device=None, layout=None) -> int:
    """layout: None = must be contiguous; else the (b, t, h) element strides every [B,T,H,D] tensor of
    the call shares (a [B,T,H] tensor has them divided by D)."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if layout is None:
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    else:
        D = layout[2]
        want = (layout[0], layout[1], D, 1) if t.dim() == 4 else (layout[0] // D, layout[1] // D, 1)
        if tuple(t.stride()) != want:
            raise ValueError(f"{name} has strides {tuple(t.stride())}, expected {want} (all tensors of a call share "
                             "one layout)")
    if device is not None and t.device != device:
        raise ValueError(f"{name} is on {t.device}, expected {device} (all tensors of a call share one device)")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
    if dtype is not None and t.dtype != dtype:
        raise ValueError(f"{name} has dtype {t.dtype}, expected {dtype}")
    return t.data_ptr()


def _new(shape, dtype, device, layout):
    """An output tensor in the call's layout (contiguous, or the same cut of a wider tensor)."""
    if layout is None:
        return torch.empty(shape, dtype=dtype, device=device)
    D = layout[2]
    strides = (layout[0], layout[1], D, 1) if len(shape) == 4 else (layout[0] // D, layout[1] // D, 1)
    return torch.empty_strided(shape, strides, dtype=dtype, device=device)


def _workspace(c: "_lib.ArAttnParams", which_pass: int, device) -> Optional[torch.Tensor]:
    """Scratch for one call, taken from torch's stream-aware caching allocator (so that calls on
    different streams never share it and nothing synchronises the device) and handed to the
    library as caller workspace.  Returns the tensor, which the caller keeps alive until the call
    has been enqueued (the allocator then defers its reuse to the stream it was allocated on)."""
    need = int(_lib.lib().ar_attn_workspace_bytes(ctypes.byref(c), which_pass))
    if need == 0 or c.stream != torch.cuda.current_stream(device).cuda_stream:
        return None     # nothing needed, or a foreign stream: the library's own per-device scratch serves
    buf = torch.empty(need + 1024, dtype=torch.uint8, device=device)
    base = (buf.data_ptr() + 1023) // 1024 * 1024      # the library wants 1024-byte alignment
    c.workspace = base
    c.workspace_bytes = need
    return buf


def check_device_status(device=None) -> None:
    """Per-step hook: waits for `device` (default: the current one) and raises ArattnError if any
    attention kernel since the last check abandoned a bounded wait.  After such an event the
    kernels of later calls return without writing their outputs until this check has been made,
    so a training loop calls it once per step before it trusts the step's results."""
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        _lib.check(_lib.lib().ar_device_status())


def _c_params(p: AttnParams, q: torch.Tensor) -> _lib.ArAttnParams:
    if not isinstance(q, torch.Tensor) or not q.is_cuda:
        raise ValueError("q must be a CUDA tensor")
    if q.dim() != 4:
        raise ValueError("q must be [B, T, H, D]")
    if q.dtype not in _DT:
        raise ValueError(f"unsupported dtype {q.dtype}")
    if p.grad_dtype not in _DT:
        raise ValueError(f"unsupported grad dtype {p.grad_dtype}")
    B, T, H, D = q.shape
    c = _lib.ArAttnParams()
    c.struct_size = ctypes.sizeof(_lib.ArAttnParams)
    c.flags = ((_lib.AR_FLAG_SYNC if p.sync else 0) | (_lib.AR_FLAG_ROPE_PREPASS if p.rope_prepass else 0)
               | (_lib.AR_FLAG_BWD_SKIP_D if p.skip_d else 0) | (_lib.AR_FLAG_BWD_SKIP_DQ if p.skip_dq else 0)
               | (_lib.AR_FLAG_BWD_SKIP_DKV if p.skip_dkv else 0))
    c.io_dtype = _DT[q.dtype]
    c.grad_dtype = _DT[p.grad_dtype]
    c.B, c.T, c.H, c.D = B, T, H, D
    c.window = int(p.window)
    if p.rope is not None:
        cos, sin = p.rope
        c.rope_mode = 1
        c.cos_buf = _check(cos, "cos", dtype=torch.float32, device=q.device)
        c.sin_buf = _check(sin, "sin", dtype=torch.float32, device=q.device)
        if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != D // 2:
            raise ValueError("rope tables must both be [rows, D/2]")
        c.rope_rows = cos.shape[0]
    else:
        c.rope_mode = 0
    if (p.q_rot is None) != (p.k_rot is None):
        raise ValueError("q_rot and k_rot must be given together")
    lay = _layout(q)
    if lay is not None:
        c.stride_b, c.stride_t, c.stride_h = lay
    if p.q_rot is not None:
        if p.rope is None:
            raise ValueError("q_rot / k_rot need rope tables")
        c.q_rot = _check(p.q_rot, "q_rot", tuple(q.shape), torch.bfloat16, q.device, lay)
        c.k_rot = _check(p.k_rot, "k_rot", tuple(q.shape), torch.bfloat16, q.device, lay)
    c.workspace = None
    c.workspace_bytes = 0
    c.stream = p.stream if p.stream is not None else torch.cuda.current_stream(q.device).cuda_stream
    return c


def attn_fwd(q, k, v, params: AttnParams, out=None, lse=None):
    """Returns (o [B,T,H,D] in q's dtype, lse [B,T,H] fp32)."""
    c = _c_params(params, q)
    shape, dev, lay = tuple(q.shape), q.device, _layout(q)
    if out is None:
        out = _new(shape, q.dtype, dev, lay)
    if lse is None:
        lse = _new(shape[:3], torch.float32, dev, lay)
    args = (_check(q, "q", layout=lay), _check(k, "k", shape, q.dtype, dev, lay), _check(v, "v", shape, q.dtype, dev, lay),
            _check(out, "out", shape, q.dtype, dev, lay), _check(lse, "lse", shape[:3], torch.float32, dev, lay))
    # the library works on the CURRENT device (status word, launches): make it the tensors' device
    with torch.cuda.device(dev):
        ws = _workspace(c, 0, dev)
        _lib.check(_lib.lib().ar_attn_fwd(ctypes.byref(c), *args))
        del ws
    return out, lse


def attn_bwd(q, k, v, o, d_o, lse, params: AttnParams, d_buf=None, dq=None, dk=None, dv=None):
    """Returns (dq, dk, dv, d_buf)."""
    c = _c_params(params, q)
    shape, dev, lay = tuple(q.shape), q.device, _layout(q)
    gd = params.grad_dtype
    if d_buf is None:
        d_buf = _new(shape[:3], torch.float32, dev, lay)
    dq = _new(shape, gd, dev, lay) if dq is None else dq
    dk = _new(shape, gd, dev, lay) if dk is None else dk
    dv = _new(shape, gd, dev, lay) if dv is None else dv
    args = (_check(q, "q", layout=lay), _check(k, "k", shape, q.dtype, dev, lay), _check(v, "v", shape, q.dtype, dev, lay),
            _check(o, "o", shape, q.dtype, dev, lay), _check(d_o, "d_o", shape, q.dtype, dev, lay),
            _check(lse, "lse", shape[:3], torch.float32, dev, lay), _check(d_buf, "d_buf", shape[:3], torch.float32, dev, lay),
            _check(dq, "dq", shape, gd, dev, lay), _check(dk, "dk", shape, gd, dev, lay), _check(dv, "dv", shape, gd, dev, lay))
    with torch.cuda.device(dev):
        ws = _workspace(c, 1, dev)
        _lib.check(_lib.lib().ar_attn_bwd(ctypes.byref(c), *args))
        del ws
    return dq, dk, dv, d_buf


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, params: AttnParams):
        o, lse = attn_fwd(q, k, v, params)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.params = params
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv, _ = attn_bwd(q, k, v, o, d_o.contiguous(), lse, ctx.params)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), None


def attention(q, k, v, params: AttnParams):
    """Differentiable attention (for harnesses that drive the path from PyTorch autograd)."""
    return _Attention.apply(q, k, v, params)
