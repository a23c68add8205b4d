"""Plain-PyTorch fp32 reference implementations of every op in :mod:`monarch_b200.ops`.

They serve three purposes: the numerics oracle for the CUDA kernels, the CPU path that
keeps the engines testable without a GPU, and the definition of each op's semantics.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def gemm(a, b, a_mn=False, b_mn=False, residual=None, accumulate_into=None):
    A = a.float().t() if a_mn else a.float()
    B = b.float() if b_mn else b.float().t()
    c = A @ B
    if residual is not None:
        c = c + residual.float()
    if accumulate_into is not None:
        c = c + accumulate_into.float()
    return c


def rmsnorm_fwd(x, w, eps):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
    return xf * rstd[:, None] * w.float(), rstd


def rmsnorm_bwd(dy, x, w, rstd):
    xh = x.float() * rstd[:, None]
    g = dy.float() * w.float()
    dx = rstd[:, None] * (g - xh * (g * xh).mean(-1, keepdim=True))
    dw = (dy.float() * xh).sum(0)
    return dx, dw


def rope_tables(seq_len: int, hd: int, theta: float, device=None):
    inv = 1.0 / (theta ** (torch.arange(0, hd, 2, dtype=torch.float32, device=device) / hd))
    ang = torch.arange(seq_len, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


def rope(x, cos, sin, seq_len, inverse=False):
    """x: [rows, heads, hd] float; rotate-half convention; position = row % seq_len."""
    rows, _, hd = x.shape
    pos = torch.arange(rows, device=x.device) % seq_len
    c = cos[pos][:, None, :]
    s = sin[pos][:, None, :]
    if inverse:
        s = -s
    x1, x2 = x[..., : hd // 2], x[..., hd // 2:]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


def swiglu_fwd(gu):
    Fdim = gu.shape[-1] // 2
    g, u = gu[..., :Fdim].float(), gu[..., Fdim:].float()
    return F.silu(g) * u


def swiglu_bwd(gu, dh):
    Fdim = gu.shape[-1] // 2
    g, u, d = gu[..., :Fdim].float(), gu[..., Fdim:].float(), dh.float()
    sg = torch.sigmoid(g)
    return torch.cat([d * u * sg * (1 + g * (1 - sg)), d * g * sg], dim=-1)


def cross_entropy(logits, targets, grad_scale):
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    loss = lse - lf.gather(1, targets[:, None]).squeeze(1)
    p = torch.softmax(lf, dim=-1)
    p[torch.arange(lf.shape[0], device=lf.device), targets] -= 1
    return loss, p * grad_scale


def adamw(p, m, v, g, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    g = g.float() * grad_scale
    p = p * (1 - lr * wd)
    m = beta1 * m + (1 - beta1) * g
    v = beta2 * v + (1 - beta2) * g * g
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = v.sqrt() / (bc2 ** 0.5) + eps
    p = p - (lr / bc1) * m / denom
    return p, m, v


def attention(q, k, v, scale, causal=True):
    """q: [B,S,Hq,hd]; k,v: [B,S,Hkv,hd] -> o [B,S,Hq,hd], lse [B,Hq,S] (natural log)."""
    B, S, Hq, hd = q.shape
    Hkv = k.shape[2]
    rep = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.softmax(s, dim=-1) @ vf
    return o.permute(0, 2, 1, 3), lse
