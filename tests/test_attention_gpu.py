"""The tcgen05 flash-attention kernels against an fp32 PyTorch computation of the same
causal grouped-query attention (forward output, log-sum-exp and all three gradients)."""
import math

import pytest
import torch

from monarch_b200.ops import kernels as K

pytestmark = pytest.mark.gpu
bf16 = torch.bfloat16


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _reference(qkv, B, S, Hq, Hkv, hd, scale):
    """fp32 causal GQA attention with autograd; returns (o [T, Hq*hd], lse [B,Hq,S], q,k,v)."""
    T = B * S
    x = qkv.float()
    q = x[:, : Hq * hd].reshape(B, S, Hq, hd).transpose(1, 2).detach().requires_grad_(True)
    k = x[:, Hq * hd: (Hq + Hkv) * hd].reshape(B, S, Hkv, hd).transpose(1, 2).detach()
    v = x[:, (Hq + Hkv) * hd:].reshape(B, S, Hkv, hd).transpose(1, 2).detach()
    k.requires_grad_(True)
    v.requires_grad_(True)
    g = Hq // Hkv
    kk = k.repeat_interleave(g, dim=1)
    vv = v.repeat_interleave(g, dim=1)
    s = (q @ kk.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.softmax(s, dim=-1) @ vv
    return o.transpose(1, 2).reshape(T, Hq * hd), lse, q, k, v


CASES = [(1, 256, 4, 2, 64), (2, 512, 8, 2, 128), (1, 384, 4, 4, 128), (1, 1024, 2, 2, 64),
         (1, 2048, 8, 2, 128)]


def _run_fwd(qkv, B, S, Hq, Hkv, hd, scale):
    T = B * S
    lib = K.lib()
    o = torch.empty(T, Hq * hd, dtype=bf16, device="cuda")
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    k = qkv[:, Hq * hd:]
    v = qkv[:, (Hq + Hkv) * hd:]
    K.check(lib.mb200_attn_fwd(qkv.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                               lse.data_ptr(), B, S, Hq, Hkv, hd, qkv.stride(0), o.stride(0),
                               scale, K.status_word().data_ptr(), K.stream_ptr()), "attn_fwd")
    torch.cuda.synchronize()
    K.check_status()
    return o, lse


@pytest.mark.parametrize("B,S,Hq,Hkv,hd", CASES)
def test_attention_forward(B, S, Hq, Hkv, hd):
    torch.manual_seed(0)
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * hd, device="cuda").to(bf16)
    scale = 1.0 / math.sqrt(hd)
    o, lse = _run_fwd(qkv, B, S, Hq, Hkv, hd, scale)
    o_ref, lse_ref, *_ = _reference(qkv, B, S, Hq, Hkv, hd, scale)
    assert _rel(o, o_ref) < 1e-2, _rel(o, o_ref)
    assert (lse - lse_ref).abs().max().item() < 2e-2


def test_attention_forward_large_logits():
    """Row maxima that grow along the KV axis force the lazy rescale of O to trigger."""
    torch.manual_seed(1)
    B, S, Hq, Hkv, hd = 1, 512, 2, 1, 128
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * hd, device="cuda")
    ramp = torch.linspace(0.5, 6.0, S, device="cuda")[:, None]
    qkv[:, Hq * hd: (Hq + Hkv) * hd] *= ramp      # later keys score higher
    qkv = qkv.to(bf16)
    scale = 1.0 / math.sqrt(hd)
    o, lse = _run_fwd(qkv, B, S, Hq, Hkv, hd, scale)
    o_ref, lse_ref, *_ = _reference(qkv, B, S, Hq, Hkv, hd, scale)
    assert _rel(o, o_ref) < 1e-2, _rel(o, o_ref)
    assert ((lse - lse_ref).abs() / (1 + lse_ref.abs())).max().item() < 1e-2


@pytest.mark.parametrize("B,S,Hq,Hkv,hd", CASES)
def test_attention_backward(B, S, Hq, Hkv, hd):
    lib = K.lib()
    if not hasattr(lib, "mb200_attn_bwd"):
        pytest.skip("library built without the backward kernels")
    torch.manual_seed(2)
    T = B * S
    qkv = torch.randn(T, (Hq + 2 * Hkv) * hd, device="cuda").to(bf16)
    do = torch.randn(T, Hq * hd, device="cuda").to(bf16)
    scale = 1.0 / math.sqrt(hd)
    o, lse = _run_fwd(qkv, B, S, Hq, Hkv, hd, scale)
    dqkv = torch.empty_like(qkv)
    delta = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
    k = qkv[:, Hq * hd:]
    v = qkv[:, (Hq + Hkv) * hd:]
    dk = dqkv[:, Hq * hd:]
    dv = dqkv[:, (Hq + Hkv) * hd:]
    K.check(lib.mb200_attn_bwd(qkv.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                               do.data_ptr(), lse.data_ptr(), delta.data_ptr(), dqkv.data_ptr(),
                               dk.data_ptr(), dv.data_ptr(), B, S, Hq, Hkv, hd, qkv.stride(0),
                               o.stride(0), dqkv.stride(0), scale, K.status_word().data_ptr(),
                               K.stream_ptr()), "attn_bwd", 3)
    torch.cuda.synchronize()
    K.check_status()
    o_ref, _, q, kk, vv = _reference(qkv, B, S, Hq, Hkv, hd, scale)
    gq, gk, gv = torch.autograd.grad(o_ref, (q, kk, vv), do.float())
    ref = torch.cat([gq.transpose(1, 2).reshape(T, -1), gk.transpose(1, 2).reshape(T, -1),
                     gv.transpose(1, 2).reshape(T, -1)], dim=1)
    n_q, n_k = Hq * hd, Hkv * hd
    assert _rel(dqkv[:, :n_q], ref[:, :n_q]) < 2e-2, ("dq", _rel(dqkv[:, :n_q], ref[:, :n_q]))
    assert _rel(dqkv[:, n_q:n_q + n_k], ref[:, n_q:n_q + n_k]) < 2e-2, "dk"
    assert _rel(dqkv[:, n_q + n_k:], ref[:, n_q + n_k:]) < 2e-2, "dv"
