"""Plain PyTorch (fp32) statements of every hand-written op: the references the GPU tests compare against."""

from __future__ import annotations

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: (..., S, hd) float; cos/sin: (S, hd)."""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos + rot * sin


def qknorm_rope(qkv, qw, kw, cos, sin, B, S, Hq, Hkv, hd, eps, use_norm=True):
    """qkv (B*S, (Hq+2Hkv)*hd) -> (B*S, (Hq+Hkv)*hd) fp32: per-head norm then RoPE on q and k."""
    x = qkv.float().view(B, S, Hq + 2 * Hkv, hd)
    q, k = x[:, :, :Hq], x[:, :, Hq:Hq + Hkv]
    if use_norm:
        q, k = rmsnorm(q, qw, eps), rmsnorm(k, kw, eps)
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    q = q * c + torch.cat((-q[..., hd // 2:], q[..., :hd // 2]), -1) * s
    k = k * c + torch.cat((-k[..., hd // 2:], k[..., :hd // 2]), -1) * s
    return torch.cat([q, k], dim=2).reshape(B * S, (Hq + Hkv) * hd)


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    g, u = gu.float().chunk(2, dim=-1)
    return F.silu(g) * u


def attention(q, k, v, causal=True):
    """q (B,S,Hq,hd), k/v (B,S,Hkv,hd) float -> (B,S,Hq,hd), lse (B,Hq,S) natural log."""
    B, S, Hq, hd = q.shape
    Hkv = k.shape[2]
    rep = Hq // Hkv
    qf, kf, vf = q.float().transpose(1, 2), k.float().transpose(1, 2), v.float().transpose(1, 2)
    kf, vf = kf.repeat_interleave(rep, 1), vf.repeat_interleave(rep, 1)
    s = qf @ kf.transpose(-1, -2) / hd ** 0.5
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.softmax(s, dim=-1) @ vf
    return o.transpose(1, 2), lse


def adamw(p, g, m, v, lr, b1, b2, eps, wd, step):
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    p = p * (1 - lr * wd) - (lr / (1 - b1 ** step)) * m / (v.sqrt() / (1 - b2 ** step) ** 0.5 + eps)
    return p, m, v
