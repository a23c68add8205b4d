"""Stock-PyTorch Llama (``nn.Module`` + autograd, ATen ops only) with Hugging Face
parameter names.  It is the numerics oracle for :class:`LlamaEngine`, the module that
``state_dict`` checkpoints interchange with, and the "library path" (cuBLAS + SDPA via
ATen) that the hand-written kernels are measured against."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .llama import LlamaConfig


class RMSNorm(nn.Module):
    def __init__(self, d, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
                * self.weight.float()).to(x.dtype)


def _rope(x, cos, sin):
    # x: [B, H, S, hd]
    hd = x.shape[-1]
    x1, x2 = x[..., : hd // 2].float(), x[..., hd // 2:].float()
    c, s = cos[None, None], sin[None, None]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class Attention(nn.Module):
    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        hd = cfg.hd
        self.q_proj = nn.Linear(cfg.d, cfg.n_heads * hd, bias=False)
        self.k_proj = nn.Linear(cfg.d, cfg.n_kv_heads * hd, bias=False)
        self.v_proj = nn.Linear(cfg.d, cfg.n_kv_heads * hd, bias=False)
        self.o_proj = nn.Linear(cfg.n_heads * hd, cfg.d, bias=False)

    def forward(self, x, cos, sin):
        B, S, _ = x.shape
        cfg = self.cfg
        q = self.q_proj(x).view(B, S, cfg.n_heads, cfg.hd).transpose(1, 2)
        k = self.k_proj(x).view(B, S, cfg.n_kv_heads, cfg.hd).transpose(1, 2)
        v = self.v_proj(x).view(B, S, cfg.n_kv_heads, cfg.hd).transpose(1, 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        return self.o_proj(o.transpose(1, 2).reshape(B, S, -1))


class MLP(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.gate_proj = nn.Linear(cfg.d, cfg.ffn, bias=False)
        self.up_proj = nn.Linear(cfg.d, cfg.ffn, bias=False)
        self.down_proj = nn.Linear(cfg.ffn, cfg.d, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class Block(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.d, cfg.eps)
        self.self_attn = Attention(cfg)
        self.post_attention_layernorm = RMSNorm(cfg.d, cfg.eps)
        self.mlp = MLP(cfg)

    def forward(self, x, cos, sin):
        x = x + self.self_attn(self.input_layernorm(x), cos, sin)
        return x + self.mlp(self.post_attention_layernorm(x))


class _Inner(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.embed_tokens = nn.Embedding(cfg.vocab, cfg.d)
        self.layers = nn.ModuleList(Block(cfg) for _ in range(cfg.n_layers))
        self.norm = RMSNorm(cfg.d, cfg.eps)


class TorchLlama(nn.Module):
    def __init__(self, cfg: LlamaConfig, checkpoint: bool = False):
        super().__init__()
        self.cfg = cfg
        self.checkpoint = checkpoint
        self.model = _Inner(cfg)
        self.lm_head = nn.Linear(cfg.d, cfg.vocab, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    def forward(self, tokens, targets=None):
        from ..ops.reference import rope_tables
        B, S = tokens.shape
        cos, sin = rope_tables(S, self.cfg.hd, self.cfg.theta, device=tokens.device)
        x = self.model.embed_tokens(tokens)
        for blk in self.model.layers:
            if self.checkpoint and self.training:
                x = torch.utils.checkpoint.checkpoint(blk, x, cos, sin, use_reentrant=False)
            else:
                x = blk(x, cos, sin)
        logits = self.lm_head(self.model.norm(x))
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(B * S, -1), targets.reshape(-1))
