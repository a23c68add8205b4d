#!/usr/bin/env python
"""Data-parallel Llama training written as ONE single-controller program over distributed
tensors: the model is plain torch code (``F.rms_norm``, matmuls, SDPA, cross-entropy) run
under ``mesh.activate()``, autograd runs on the controller over the tensors' metadata, the
gradients are flattened into 25 MB buckets and averaged with ``bucket.reduce_("dp", "avg")``
(on GPUs: this package's NVLink all-reduce kernels), AdamW runs as ``torch._foreach_*`` ops
on fp32 master weights.  The whole step is traced once with ``compile`` and replayed on the
workers with one message per step.

    python examples/llama_ddp_distributed_tensors.py --cuda --procs 8 --model llama3.2-1b \
        --seq 4096 --micro-batch 2 --steps 8 --warmup 3

The operators themselves are the stock ATen ones (cuBLAS, SDPA): this is the path a user of
the tensor engine gets without touching the kernel engine; ``bench.py --parallelism ddp``
runs the same configuration on the hand-written kernels.

Parity: docs/source/examples/distributed_tensors.py:192-342 of the reference (DDP over
distributed tensors with ``reduce_`` on the data-parallel dim)."""
import argparse
import json
import math
import os
import sys
import time

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200 import tensor_engine as te  # noqa: E402
from monarch_b200.actor import this_host  # noqa: E402
from monarch_b200.models import PRESETS  # noqa: E402

BUCKET_BYTES = 25 << 20


def init_params(cfg, dev):
    """fp32 master weights, the same on every worker (the seed is)."""
    d, hd = cfg.d, cfg.d // cfg.n_heads
    qkv = (cfg.n_heads + 2 * cfg.n_kv_heads) * hd
    p = {"emb": torch.randn(cfg.vocab, d, device=dev) * 0.02,
         "norm": torch.ones(d, device=dev)}
    if not cfg.tie_embeddings:
        p["head"] = torch.randn(cfg.vocab, d, device=dev) * 0.02
    for i in range(cfg.n_layers):
        p[f"l{i}.n1"] = torch.ones(d, device=dev)
        p[f"l{i}.wqkv"] = torch.randn(qkv, d, device=dev) * 0.02
        p[f"l{i}.wo"] = torch.randn(d, cfg.n_heads * hd, device=dev) * (0.02 / math.sqrt(2 * cfg.n_layers))
        p[f"l{i}.n2"] = torch.ones(d, device=dev)
        p[f"l{i}.wgu"] = torch.randn(2 * cfg.ffn, d, device=dev) * 0.02
        p[f"l{i}.wd"] = torch.randn(d, cfg.ffn, device=dev) * (0.02 / math.sqrt(2 * cfg.n_layers))
    return p


def rope_tables(cfg, seq, dev, dtype):
    hd = cfg.d // cfg.n_heads
    inv = 1.0 / (cfg.theta ** (torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd))
    ang = torch.arange(seq, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos().to(dtype), ang.sin().to(dtype)


def rotate_half(x):
    a, b = x.chunk(2, dim=-1)
    return torch.cat([-b, a], dim=-1)


def forward_loss(cfg, w, tokens, targets, cos, sin):
    B, S = tokens.shape
    H, Hkv, hd = cfg.n_heads, cfg.n_kv_heads, cfg.d // cfg.n_heads
    x = F.embedding(tokens, w["emb"])
    for i in range(cfg.n_layers):
        h = F.rms_norm(x, (cfg.d,), w[f"l{i}.n1"], cfg.eps)
        qkv = h @ w[f"l{i}.wqkv"].t()
        q, k, v = qkv.split([H * hd, Hkv * hd, Hkv * hd], dim=-1)
        q = q.view(B, S, H, hd).transpose(1, 2)
        k = k.view(B, S, Hkv, hd).transpose(1, 2)
        v = v.view(B, S, Hkv, hd).transpose(1, 2)
        q = q * cos + rotate_half(q) * sin
        k = k * cos + rotate_half(k) * sin
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=Hkv != H)
        x = x + a.transpose(1, 2).reshape(B, S, H * hd) @ w[f"l{i}.wo"].t()
        h = F.rms_norm(x, (cfg.d,), w[f"l{i}.n2"], cfg.eps)
        g, u = (h @ w[f"l{i}.wgu"].t()).chunk(2, dim=-1)
        x = x + (F.silu(g) * u) @ w[f"l{i}.wd"].t()
    x = F.rms_norm(x, (cfg.d,), w["norm"], cfg.eps)
    logits = x @ w["head" if "head" in w else "emb"].t()
    return F.cross_entropy(logits.float().view(B * S, -1), targets.reshape(B * S))


def buckets_of(names, params, elem_bytes):
    """Consecutive parameters (backward order: last layer first) up to BUCKET_BYTES each."""
    out, cur, size = [], [], 0
    for n in reversed(names):
        nb = params[n].numel() * elem_bytes
        if cur and size + nb > BUCKET_BYTES:
            out.append(cur)
            cur, size = [], 0
        cur.append(n)
        size += nb
    if cur:
        out.append(cur)
    return out


def run(model="llama3.2-1b", procs=2, cuda=False, seq=4096, micro_batch=2, steps=8, warmup=3,
        lr=3e-4, compiled=True):
    cfg = PRESETS[model]
    pm = this_host().spawn_procs(per_host={"gpus": procs})
    mesh = te.spawn_tensor_engine(pm, use_cuda=cuda).rename(gpus="dp")
    dev = "cuda" if cuda else "cpu"
    cdt = torch.bfloat16 if cuda else torch.float32      # compute dtype
    b1, b2, eps, wd = 0.9, 0.95, 1e-8, 0.1
    try:
        with mesh.activate():
            from monarch_b200 import random as mrandom
            mrandom.manual_seed(0)
            master = init_params(cfg, dev)
            names = list(master)
            m = {n: torch.zeros_like(master[n]) for n in names}
            v = {n: torch.zeros_like(master[n]) for n in names}
            step_t = torch.zeros((), device=dev)
            cos, sin = rope_tables(cfg, seq, dev, cdt)
            mrandom.manual_seed(1, per_rank=True)           # every rank trains on its own data
            tokens = torch.randint(0, cfg.vocab, (micro_batch, seq), device=dev)
            targets = torch.randint(0, cfg.vocab, (micro_batch, seq), device=dev)
            buckets = buckets_of(names, master, 2 if cuda else 4)

            def train_step(tokens, targets):
                w = {n: master[n].to(cdt, copy=True).requires_grad_(True) for n in names}
                loss = forward_loss(cfg, w, tokens, targets, cos, sin)
                grads = dict(zip(names, torch.autograd.grad(loss, [w[n] for n in names])))
                g32 = {}
                for b in buckets:
                    flat = torch.cat([grads[n].reshape(-1) for n in b])
                    flat.reduce_("dp", "avg")
                    flat = flat.float()
                    off = 0
                    for n in b:
                        k = master[n].numel()
                        g32[n] = flat[off: off + k].view_as(master[n])
                        off += k
                # AdamW on the fp32 masters; the step count lives on the workers, so the bias
                # corrections stay right when this function is replayed as a recording
                P, G = [master[n] for n in names], [g32[n] for n in names]
                M, V = [m[n] for n in names], [v[n] for n in names]
                with torch.no_grad():
                    step_t.add_(1.0)
                    bc1 = 1.0 - torch.pow(b1, step_t)
                    bc2_sqrt = (1.0 - torch.pow(b2, step_t)).sqrt()
                    torch._foreach_mul_(P, 1.0 - lr * wd)
                    torch._foreach_lerp_(M, G, 1.0 - b1)
                    torch._foreach_mul_(V, b2)
                    torch._foreach_addcmul_(V, G, G, 1.0 - b2)
                    D = torch._foreach_sqrt(V)
                    torch._foreach_div_(D, bc2_sqrt)
                    torch._foreach_add_(D, eps)
                    torch._foreach_mul_(D, bc1 / lr)
                    torch._foreach_addcdiv_(P, M, D, -1.0)
                return loss.detach()

            step = te.compile(train_step) if compiled else train_step
            losses = []
            for _ in range(warmup):
                losses.append(step(tokens, targets))
            te.inspect(losses[-1])                      # everything so far has run
            t0 = time.perf_counter()
            for _ in range(steps):
                losses.append(step(tokens, targets))
            last = te.inspect(losses[-1].reduce("dp", "avg")).item()
            wall = time.perf_counter() - t0
            first = te.inspect(losses[0].reduce("dp", "avg")).item()
            name0 = names[-1]
            spread = (master[name0].reduce("dp", "max") - master[name0].reduce("dp", "min")).abs().max()
            in_sync = te.inspect(spread).item() == 0.0
        tok = procs * micro_batch * seq * steps
        return {"model": model, "procs": procs, "device": dev, "seq_len": seq,
                "micro_batch": micro_batch, "steps": steps, "warmup": warmup,
                "tokens_per_s": tok / wall, "ms_per_step": wall * 1e3 / steps,
                "loss_first": first, "loss_last": last, "replicas_in_sync": in_sync,
                "grad_buckets": len(buckets), "compiled": compiled,
                "timing": "controller wall clock around the steps, closed by fetching the last loss"}
    finally:
        mesh.exit()
        pm.stop().get()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--cuda", action="store_true")
    ap.add_argument("--procs", type=int, default=2)
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--micro-batch", type=int, default=2)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--eager", action="store_true", help="dispatch op by op instead of compiling")
    a = ap.parse_args()
    print(json.dumps(run(a.model, a.procs, a.cuda, a.seq, a.micro_batch, a.steps, a.warmup,
                         compiled=not a.eager)))
