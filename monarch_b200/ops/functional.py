"""Tensor-level entry points of the hand-written sm_100a kernels.

Every function dispatches on the device of its inputs: CUDA tensors go to the kernel
library (and fail loudly if it is missing), CPU tensors go to the fp32 PyTorch
reference so that engines and tests run without a GPU.
"""
from __future__ import annotations

import os

import torch

from . import kernels as K
from . import reference as R

bf16 = torch.bfloat16


def _p(t):
    return 0 if t is None else t.data_ptr()


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    assert t.dim() == 2
    if t.stride(1) != 1 or t.stride(0) < t.shape[1]:
        t = t.contiguous()
    return t


def gemm(a, b, *, a_mn=False, b_mn=False, out=None, residual=None, accumulate=False):
    """out[M,N] = opA(a) @ opB(b) (+ residual) (+ out when ``accumulate``).

    ``a`` is [M,K] (``a_mn=False``) or [K,M] (``a_mn=True``); ``b`` is [N,K]
    (``b_mn=False``, i.e. out = a @ b.T) or [K,N] (``b_mn=True``).  bf16 in, fp32
    accumulation on the tensor cores (tcgen05, accumulator in TMEM), bf16 out.
    """
    a = _rowmajor(a)
    b = _rowmajor(b)
    M, Ka = (a.shape[1], a.shape[0]) if a_mn else a.shape
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else b.shape
    assert Ka == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        assert not accumulate
        out = torch.empty(M, N, dtype=a.dtype, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1
    if not a.is_cuda:
        out.copy_(R.gemm(a, b, a_mn, b_mn, residual, out if accumulate else None).to(out.dtype))
        return out
    assert a.dtype == bf16 and b.dtype == bf16 and out.dtype == bf16
    if residual is not None:
        assert residual.shape == (M, N) and residual.stride(1) == 1 and residual.dtype == bf16
    rc = K.lib().mb200_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), _p(residual), M, N, Ka, a.stride(0),
        b.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
        int(a_mn), int(b_mn), int(accumulate), K.status_word(a.device).data_ptr(), K.stream_ptr())
    K.check(rc, "gemm_bf16")
    return out


def rmsnorm_fwd(x, w, eps=1e-5):
    rows, d = x.shape
    if not x.is_cuda:
        y, rstd = R.rmsnorm_fwd(x, w, eps)
        return y.to(x.dtype), rstd
    x = x.contiguous()
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    K.check(K.lib().mb200_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(),
                                      rows, d, eps, K.stream_ptr()), "rmsnorm_fwd")
    return y, rstd


_scratch: dict = {}


def _rms_scratch(device, nblocks, d):
    key = (device, "rms")
    t = _scratch.get(key)
    if t is None or t.numel() < nblocks * d:
        t = torch.empty(nblocks * d, dtype=torch.float32, device=device)
        _scratch[key] = t
    return t


def rmsnorm_bwd(dy, x, w, rstd, dw_out, accumulate=False, dres=None):
    """Returns dx (+ ``dres``); writes (or adds) the weight gradient into ``dw_out``."""
    rows, d = x.shape
    if not x.is_cuda:
        dx, dw = R.rmsnorm_bwd(dy, x, w, rstd)
        if dres is not None:
            dx = dx + dres.float()
        if accumulate:
            dw = dw + dw_out.float()
        dw_out.copy_(dw.to(dw_out.dtype))
        return dx.to(x.dtype)
    dy = dy.contiguous()
    dx = torch.empty_like(x)
    nb = K.lib().mb200_rmsnorm_bwd_blocks(rows)
    part = _rms_scratch(x.device, nb, d)
    K.check(K.lib().mb200_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                      _p(dres), dx.data_ptr(), part.data_ptr(), dw_out.data_ptr(),
                                      int(accumulate), rows, d, K.stream_ptr()),
            "rmsnorm_bwd", 2)
    return dx


def rope_(qkv, cos, sin, seq_len, n_rot_heads, hd, inverse=False):
    """In-place rotary embedding on the first ``n_rot_heads`` heads of each row."""
    rows = qkv.shape[0]
    if not qkv.is_cuda:
        x = qkv[:, : n_rot_heads * hd].float().reshape(rows, n_rot_heads, hd)
        y = R.rope(x, cos, sin, seq_len, inverse)
        qkv[:, : n_rot_heads * hd] = y.reshape(rows, -1).to(qkv.dtype)
        return qkv
    assert qkv.stride(1) == 1
    K.check(K.lib().mb200_rope_inplace(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), rows,
                                       seq_len, n_rot_heads, hd, qkv.stride(0), int(inverse),
                                       K.stream_ptr()), "rope")
    return qkv


def swiglu_fwd(gu):
    rows, F2 = gu.shape
    if not gu.is_cuda:
        return R.swiglu_fwd(gu).to(gu.dtype)
    h = torch.empty(rows, F2 // 2, dtype=gu.dtype, device=gu.device)
    K.check(K.lib().mb200_swiglu_fwd(gu.data_ptr(), h.data_ptr(), rows, F2 // 2, K.stream_ptr()),
            "swiglu_fwd")
    return h


def swiglu_bwd(gu, dh, out=None):
    rows, F2 = gu.shape
    if not gu.is_cuda:
        r = R.swiglu_bwd(gu, dh).to(gu.dtype)
        if out is not None:
            out.copy_(r)
            return out
        return r
    dgu = torch.empty_like(gu) if out is None else out
    K.check(K.lib().mb200_swiglu_bwd(gu.data_ptr(), dh.data_ptr(), dgu.data_ptr(), rows, F2 // 2,
                                     K.stream_ptr()), "swiglu_bwd")
    return dgu


def cross_entropy_(logits, targets, grad_scale):
    """Per-row loss; ``logits`` is overwritten with d(loss_sum * grad_scale)/d(logits)."""
    rows, V = logits.shape
    if not logits.is_cuda:
        loss, g = R.cross_entropy(logits, targets, grad_scale)
        logits.copy_(g.to(logits.dtype))
        return loss
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    assert targets.dtype == torch.int64 and logits.stride(1) == 1
    K.check(K.lib().mb200_cross_entropy_fwd_bwd(logits.data_ptr(), targets.data_ptr(),
                                                loss.data_ptr(), rows, V, logits.stride(0),
                                                grad_scale, K.stream_ptr()), "cross_entropy")
    return loss


def adamw_(p, m, v, g, p_bf16, *, lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, step=1,
           grad_scale=1.0):
    """Fused AdamW step on flat fp32 master/moment buffers; refreshes the bf16 copy."""
    if not p.is_cuda:
        np_, nm, nv = R.adamw(p, m, v, g, lr, beta1, beta2, eps, wd, step, grad_scale)
        p.copy_(np_)
        m.copy_(nm)
        v.copy_(nv)
        if p_bf16 is not None:
            p_bf16.copy_(p.to(p_bf16.dtype))
        return
    assert p.dtype == torch.float32 and p.is_contiguous() and g.is_contiguous()
    K.check(K.lib().mb200_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(),
                                _p(p_bf16), p.numel(), int(g.dtype == bf16), lr, beta1, beta2, eps,
                                wd, step, grad_scale, K.stream_ptr()), "adamw")


def embedding_fwd(table, ids):
    rows, d = ids.numel(), table.shape[1]
    if not table.is_cuda:
        return table[ids.reshape(-1)]
    out = torch.empty(rows, d, dtype=table.dtype, device=table.device)
    K.check(K.lib().mb200_embedding_fwd(table.data_ptr(), ids.data_ptr(), out.data_ptr(), rows, d,
                                        K.stream_ptr()), "embedding_fwd")
    return out


def embedding_bwd_(dout, ids, dtable):
    """dtable[ids[r]] += dout[r] (atomic)."""
    rows, d = dout.shape
    if not dout.is_cuda:
        dtable.index_add_(0, ids.reshape(-1), dout.to(dtable.dtype))
        return
    K.check(K.lib().mb200_embedding_bwd(dout.data_ptr(), ids.data_ptr(), dtable.data_ptr(), rows,
                                        d, K.stream_ptr()), "embedding_bwd")


def sumsq(x, out=None):
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    if not x.is_cuda:
        out += x.float().pow(2).sum()
        return out
    K.check(K.lib().mb200_sumsq(x.data_ptr(), x.numel(), int(x.dtype == bf16), out.data_ptr(),
                                K.stream_ptr()), "sumsq")
    return out


def have_attention_kernel() -> bool:
    """True when the tcgen05 flash-attention kernels (forward and backward) are in the
    loaded library and not disabled with ``MB200_ATTN=sdpa``."""
    if not torch.cuda.is_available() or os.environ.get("MB200_ATTN", "") == "sdpa":
        return False
    l = K.lib()
    return hasattr(l, "mb200_attn_fwd") and hasattr(l, "mb200_attn_bwd")


class AttnCtx:
    """What attention_bwd needs from attention_fwd."""
    __slots__ = ("qkv", "o", "lse", "B", "S", "Hq", "Hkv", "hd", "scale", "graph")


def attention_fwd(qkv, B, S, Hq, Hkv, hd, scale=None, need_bwd=True):
    """Causal GQA attention on a fused post-RoPE qkv buffer [B*S, (Hq+2Hkv)*hd].

    Returns (o [B*S, Hq*hd], ctx).  On sm_100a the hand-written tcgen05 flash kernel is
    used when the library exports it; otherwise (CPU, or library built without it) the
    math is done by torch SDPA.
    """
    scale = scale if scale is not None else hd ** -0.5
    ctx = AttnCtx()
    ctx.qkv, ctx.B, ctx.S, ctx.Hq, ctx.Hkv, ctx.hd, ctx.scale = qkv, B, S, Hq, Hkv, hd, scale
    ctx.graph = None
    T = B * S
    if qkv.is_cuda and have_attention_kernel():
        o = torch.empty(T, Hq * hd, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(B, Hq, S, dtype=torch.float32, device=qkv.device)
        q = qkv
        k = qkv[:, Hq * hd:]
        v = qkv[:, (Hq + Hkv) * hd:]
        K.check(K.lib().mb200_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                       lse.data_ptr(), B, S, Hq, Hkv, hd, qkv.stride(0),
                                       o.stride(0), scale, K.status_word(qkv.device).data_ptr(),
                                       K.stream_ptr()), "attn_fwd")
        ctx.o, ctx.lse = o, lse
        return o, ctx
    q = qkv[:, : Hq * hd].reshape(B, S, Hq, hd).transpose(1, 2)
    k = qkv[:, Hq * hd: (Hq + Hkv) * hd].reshape(B, S, Hkv, hd).transpose(1, 2)
    v = qkv[:, (Hq + Hkv) * hd:].reshape(B, S, Hkv, hd).transpose(1, 2)
    if need_bwd:
        q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
    with torch.enable_grad() if need_bwd else torch.no_grad():
        o = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True, scale=scale,
                                                             enable_gqa=True)
        o2 = o.transpose(1, 2).reshape(T, Hq * hd)
    if need_bwd:
        ctx.graph = (q, k, v, o2)
    ctx.o, ctx.lse = o2.detach(), None
    return ctx.o, ctx


def attention_ctx_from_saved(qkv, saved, B, S, Hq, Hkv, hd, scale=None):
    """Rebuild the backward context from a recomputed qkv and the (o, lse) that the first
    forward kept, without running the attention kernel again."""
    ctx = AttnCtx()
    ctx.qkv, ctx.B, ctx.S, ctx.Hq, ctx.Hkv, ctx.hd = qkv, B, S, Hq, Hkv, hd
    ctx.scale = scale if scale is not None else hd ** -0.5
    ctx.graph = None
    ctx.o, ctx.lse = saved
    return ctx.o, ctx


def attention_bwd(ctx: AttnCtx, do):
    """Gradient w.r.t. the fused (post-RoPE) qkv buffer: [B*S, (Hq+2Hkv)*hd]."""
    B, S, Hq, Hkv, hd = ctx.B, ctx.S, ctx.Hq, ctx.Hkv, ctx.hd
    T = B * S
    dqkv = torch.empty_like(ctx.qkv)
    if ctx.graph is None and ctx.lse is not None:
        qkv = ctx.qkv
        delta = torch.empty(B, Hq, S, dtype=torch.float32, device=qkv.device)
        k = qkv[:, Hq * hd:]
        v = qkv[:, (Hq + Hkv) * hd:]
        dk = dqkv[:, Hq * hd:]
        dv = dqkv[:, (Hq + Hkv) * hd:]
        K.check(K.lib().mb200_attn_bwd(qkv.data_ptr(), k.data_ptr(), v.data_ptr(),
                                       ctx.o.data_ptr(), do.data_ptr(), ctx.lse.data_ptr(),
                                       delta.data_ptr(), dqkv.data_ptr(), dk.data_ptr(),
                                       dv.data_ptr(), B, S, Hq, Hkv, hd, qkv.stride(0),
                                       ctx.o.stride(0), dqkv.stride(0), ctx.scale,
                                       K.status_word(qkv.device).data_ptr(), K.stream_ptr()),
                "attn_bwd", 3)
        return dqkv
    q, k, v, o2 = ctx.graph
    dq, dk, dv = torch.autograd.grad(o2, (q, k, v), do)
    dqkv[:, : Hq * hd] = dq.transpose(1, 2).reshape(T, Hq * hd)
    dqkv[:, Hq * hd: (Hq + Hkv) * hd] = dk.transpose(1, 2).reshape(T, Hkv * hd)
    dqkv[:, (Hq + Hkv) * hd:] = dv.transpose(1, 2).reshape(T, Hkv * hd)
    ctx.graph = None
    return dqkv
