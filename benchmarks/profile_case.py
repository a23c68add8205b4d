#!/usr/bin/env python
"""Small, self-terminating cases of each hand-written kernel for `ncu` captures.

    python benchmarks/profile_case.py gemm            # 3 launches of one 8192x4096x4096 GEMM
    python benchmarks/profile_case.py elementwise     # one launch of each memory-bound kernel
    python benchmarks/profile_case.py attn            # attention forward + backward, S=4096, 16q/4kv
    python benchmarks/profile_case.py step            # 2-layer Llama-3-8B-shaped training steps
    python benchmarks/profile_case.py collectives     # the NVLink kernels as a group of one rank
    python benchmarks/profile_case.py fused           # the fused compute+collective kernels, one rank

A profiler replays each captured launch many times, so kernels that wait for a peer cannot be
captured in a multi-rank run; ``collectives`` runs them as a group of one rank on one GPU (the
flag waits see the rank's own signal).  What such a capture shows is the kernels' own cost --
instruction mix, registers, the HBM side of the traffic; NVLink traffic needs peers and is
measured with CUDA events in the multi-GPU harnesses instead.

Inputs are larger than the 126 MB L2 but only a few hundred MB, so a multi-pass capture
finishes in about a minute.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200 import ops  # noqa: E402
from monarch_b200.ops import kernels as K  # noqa: E402
from monarch_b200.ops import reference as R  # noqa: E402

bf16 = torch.bfloat16


def gemm_case(variant="nt"):
    T, N, Kd = 8192, 4096, 4096
    a_mn, b_mn = {"nt": (False, False), "nn": (False, True), "tn": (True, True)}[variant]
    a = torch.randn((Kd, T) if a_mn else (T, Kd), device="cuda", dtype=bf16)
    b = torch.randn((Kd, N) if b_mn else (N, Kd), device="cuda", dtype=bf16)
    out = torch.empty(T, N, device="cuda", dtype=bf16)
    for _ in range(3):
        ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out)
    torch.cuda.synchronize()


def elementwise_case():
    T, d, F, V = 8192, 4096, 14336, 32064
    x = torch.randn(T, d, device="cuda", dtype=bf16)
    w = torch.ones(d, device="cuda", dtype=bf16)
    y, rstd = ops.rmsnorm_fwd(x, w)
    dw = torch.zeros(d, device="cuda", dtype=bf16)
    ops.rmsnorm_bwd(y, x, w, rstd, dw, dres=x)
    gu = torch.randn(T, 2 * F, device="cuda", dtype=bf16)
    h = ops.swiglu_fwd(gu)
    ops.swiglu_bwd(gu, h)
    cos, sin = R.rope_tables(T, 128, 500000.0, device="cuda")
    qkv = torch.randn(T, 6144, device="cuda", dtype=bf16)
    ops.rope_(qkv, cos, sin, T, 40, 128)
    logits = torch.randn(T, V, device="cuda", dtype=bf16)
    tg = torch.randint(0, V, (T,), device="cuda")
    ops.cross_entropy_(logits, tg, 1.0 / T)
    n = 64 << 20
    p = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    g = torch.randn(n, device="cuda", dtype=bf16)
    pb = torch.empty(n, device="cuda", dtype=bf16)
    ops.adamw_(p, m, v, g, pb, lr=1e-3, step=1)
    torch.cuda.synchronize()


def attn_case(S=4096, Hq=16, Hkv=4):
    B, hd = 1, 128   # qkv + o + do + dqkv = 56 MB at the default size: a short capture
    qkv = torch.randn(B * S, (Hq + 2 * Hkv) * hd, device="cuda", dtype=bf16)
    o, ctx = ops.attention_fwd(qkv, B, S, Hq, Hkv, hd)
    do = torch.randn_like(o)
    ops.attention_bwd(ctx, do)
    torch.cuda.synchronize()


def step_case(layers=2, steps=2):
    from dataclasses import replace
    from monarch_b200.models import PRESETS, LlamaEngine, LocalParamStore, ParamLayout
    cfg = replace(PRESETS["llama3-8b"], n_layers=layers, vocab=32064)
    layout = ParamLayout(cfg)
    st = LocalParamStore(layout, "cuda", seed=0)
    eng = LlamaEngine(cfg, st, 8192)
    tok = torch.randint(0, cfg.vocab, (1, 8192), device="cuda")
    for _ in range(steps):
        eng.forward_backward(tok, tok)
        eng.optimizer_step(1e-4)
    torch.cuda.synchronize()


def collectives_case():
    """allreduce / reduce-scatter+AdamW / all-gather on symmetric buffers and the staged mesh
    collectives, 64 MiB each, world size 1."""
    import torch.distributed as dist
    from monarch_b200.parallel.meshcomm import MeshComm
    from monarch_b200.parallel.symm import FlagArray, SymmBuffer
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    lib, st = K.lib(), K.status_word(dev)
    n = 32 << 20                                   # bf16 elements: 64 MiB
    flags = FlagArray(8, dev)
    buf = SymmBuffer(n, bf16, dev, zero=False)
    buf.tensor.normal_()
    for epoch in (1, 2):
        K.check(lib.mb200_allreduce_scale_cast(buf.ptrs_at(0), buf.ptrs_at(0), None, None,
                                               flags.ptrs, n, 0, 0, 1, 1.0, 0, epoch,
                                               flags.counter.data_ptr(), 0, st.data_ptr(),
                                               K.stream_ptr()), "allreduce")
    master = torch.randn(n, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    shard = torch.empty(n, dtype=bf16, device=dev)
    for epoch in (1, 2):
        K.check(lib.mb200_rs_adamw(buf.ptrs_at(0), None, flags.ptrs, master.data_ptr(),
                                   m.data_ptr(), v.data_ptr(), shard.data_ptr(), n, 0, 1, 2, 3,
                                   epoch, 1e-3, 0.9, 0.95, 1e-8, 0.1, epoch, 1.0,
                                   flags.counter.data_ptr(), 0, st.data_ptr(), K.stream_ptr()),
                "rs_adamw")
    full = torch.empty(n, dtype=bf16, device=dev)
    for _ in range(2):
        K.check(lib.mb200_allgather_pull(full.data_ptr(), buf.ptrs_at(0), n, 0, 1, flags.my_ptr,
                                         0, 0, None, 0, 0, 0, st.data_ptr(), K.stream_ptr()),
                "allgather_pull")
    comm = MeshComm.from_process_group(None, dev, 64 << 20)
    x = torch.randn(n // 2, device=dev)             # 64 MiB of fp32
    comm.all_reduce(x, "sum")                       # stage + two-shot reduce + copy-out
    comm.all_gather(x)
    torch.cuda.synchronize()
    dist.destroy_process_group()


def fused_case():
    """The fused compute+collective kernels as a group of one rank: tensor-parallel
    all-gather->GEMM and GEMM->reduce-scatter (TPComm), the FSDP step with the parameter
    gather inside the GEMM launches, the MoE dispatch->GEMM / GEMM->combine pair (EPComm)."""
    from dataclasses import replace
    import torch.distributed as dist
    from monarch_b200.models import PRESETS, LlamaEngine, ParamLayout
    from monarch_b200.parallel.ep import EPComm
    from monarch_b200.parallel.fsdp import FSDPParamStore
    from monarch_b200.parallel.tp import TPComm
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29578")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    # tensor parallel: Llama-2-13B shapes at tp=1 (4096 rows, d 5120, ffn 13824)
    T, d, F = 4096, 5120, 13824
    tp = TPComm(dist.group.WORLD, dev, T, d)
    tp.gather = "kernel"      # the form with copy CTAs inside the GEMM launch (the default,
    #                           "dma", moves the rows with the copy engines: nothing to capture)
    x = torch.randn(T, d, device=dev, dtype=bf16)
    w_gu = torch.randn(2 * F, d, device=dev, dtype=bf16) * 0.02
    w_dn = torch.randn(d, F, device=dev, dtype=bf16) * 0.02
    for _ in range(2):
        gu, _ = tp.ag_gemm(x, w_gu)
        h = ops.swiglu_fwd(gu)
        tp.gemm_rs(h, w_dn, residual_local=x)
    # FSDP, two layers of Llama-3-8B shape, gather inside the consuming GEMMs
    cfg = replace(PRESETS["llama3-8b"], n_layers=2, vocab=32064)
    st = FSDPParamStore(ParamLayout(cfg), dev, seed=0, gather="gemm")
    eng = LlamaEngine(cfg, st, 8192)
    tok = torch.randint(0, cfg.vocab, (1, 8192), device=dev)
    st.set_hyper(lr=1e-4)
    eng.forward_backward(tok, tok)
    eng.optimizer_step(1e-4)
    # expert parallel: Mixtral shapes, one expert on this rank
    Tm, dm, Fm = 4096, 4096, 14336
    ep = EPComm(dist.group.WORLD, dev, Tm, dm, Fm, top_k=1)
    xm = torch.randn(Tm, dm, device=dev, dtype=bf16)
    idx = torch.zeros(Tm, 1, dtype=torch.int32, device=dev)
    wts = torch.ones(Tm, 1, device=dev)
    e_gu = torch.randn(2 * Fm, dm, device=dev, dtype=bf16) * 0.02
    e_dn = torch.randn(dm, Fm, device=dev, dtype=bf16) * 0.02
    for _ in range(2):
        ep.forward(xm, idx, wts, e_gu, e_dn, residual=xm)
    torch.cuda.synchronize()
    dist.destroy_process_group()


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    if what == "gemm":
        gemm_case(sys.argv[2] if len(sys.argv) > 2 else "nt")
    elif what == "elementwise":
        elementwise_case()
    elif what == "attn":
        attn_case()
    elif what == "step":
        step_case()
    elif what == "collectives":
        collectives_case()
    elif what == "fused":
        fused_case()
    K.check_status()
    print("ok", what)
