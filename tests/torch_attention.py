"""A plain-torch stand-in for the attention back end of autoresearch_b200.train_step (test
infrastructure, CPU): RoPE, per-head RMSNorm and masked softmax attention with the contract of
LibraryAttention - backward returns dq, dk with rope_bwd applied and the normalisation passed
straight through, plus rms_q / rms_k in the context."""
import math

import torch

from autoresearch_b200 import precompute_rope
from autoresearch_b200.train_step import NORM_EPS


def rope(x, cos, sin, inverse=False):
    """ops.mojo:237-238 (forward) / 1119-1120 (its transpose); x [B,T,H,D], tables [T, D/2]."""
    D = x.shape[-1]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    if inverse:
        s = -s
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return torch.cat([x1 * c + x2 * s, -x1 * s + x2 * c], dim=-1)


def masked_attention(q, k, v, window):
    """softmax(mask(q k^T / sqrt(D))) v on [B,T,H,D]; window as in ops.mojo:290-293."""
    B, T, H, D = q.shape
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(D)
    qi, ki = torch.arange(T, device=q.device)[:, None], torch.arange(T, device=q.device)[None, :]
    mask = ki <= qi
    if 0 < window < T:
        mask &= ki >= qi - window
    s = s.masked_fill(~mask, float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), v)


class TorchAttention:
    def __init__(self, cfg, seq_len, dtype=torch.float64):
        cos, sin = precompute_rope(seq_len, cfg.head_dim)
        self.cos, self.sin = torch.from_numpy(cos).to(dtype), torch.from_numpy(sin).to(dtype)
        self.dtype = dtype

    def forward(self, q, k, v, window):
        q, k, v = (t.to(self.dtype) for t in (q, k, v))
        rq, rk = rope(q, self.cos, self.sin), rope(k, self.cos, self.sin)
        rms_q = torch.sqrt(rq.pow(2).mean(-1) + NORM_EPS)
        rms_k = torch.sqrt(rk.pow(2).mean(-1) + NORM_EPS)
        yq = (rq / rms_q.unsqueeze(-1)).detach().requires_grad_(True)
        yk = (rk / rms_k.unsqueeze(-1)).detach().requires_grad_(True)
        vv = v.detach().requires_grad_(True)
        with torch.enable_grad():
            o = masked_attention(yq, yk, vv, window)
        return o.detach(), dict(yq=yq, yk=yk, v=vv, o=o, rms_q=rms_q, rms_k=rms_k)

    def backward(self, ctx, d_o):
        gq, gk, gv = torch.autograd.grad(ctx["o"], [ctx["yq"], ctx["yk"], ctx["v"]], d_o.to(self.dtype))
        return (rope(gq, self.cos, self.sin, inverse=True), rope(gk, self.cos, self.sin, inverse=True), gv)
