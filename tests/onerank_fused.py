#!/usr/bin/env python
"""The fused compute+collective kernels as a group of ONE rank on one GPU, checked against
plain PyTorch / the resident store: tensor-parallel all-gather->GEMM and GEMM->reduce-scatter,
the FSDP store in its three gather modes, the DDP store, the MoE dispatch/combine pair.  The
flag handshakes see the rank's own signals and the "peer" loads hit the rank's own memory, so
every kernel runs exactly as it does in a larger group.  (Groups of 2-8 ranks:
tests/multigpu_selftest.py.)  Run by tests/test_fused_one_rank_gpu.py in a process of its own,
because it initialises torch.distributed."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

bf16 = torch.bfloat16


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def main() -> int:
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29591")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    from monarch_b200.models import PRESETS, LlamaEngine, LocalParamStore, ParamLayout
    from monarch_b200.ops import kernels as K
    from monarch_b200.parallel.ddp import DDPParamStore
    from monarch_b200.parallel.ep import EPComm
    from monarch_b200.parallel.fsdp import FSDPParamStore
    from monarch_b200.parallel.tp import TPComm
    out = {}
    torch.manual_seed(0)

    # ---- tensor parallel primitives
    T, d, N = 512, 512, 1024
    tp = TPComm(dist.group.WORLD, dev, T, d)
    x = torch.randn(T, d, device=dev, dtype=bf16)
    w = torch.randn(N, d, device=dev, dtype=bf16) * 0.05
    for _ in range(3):                       # both buffers of the double-buffered pair
        y, x_full = tp.ag_gemm(x, w)
    assert torch.equal(x_full, x)
    out["ag_gemm_rel"] = _rel(y, x.float() @ w.float().t())
    tp.gather = "dma"                        # rows by the copy engines, no copy CTAs
    for _ in range(3):
        y2, x_full2 = tp.ag_gemm(x, w)
    torch.cuda.synchronize()
    assert torch.equal(x_full2, x) and torch.equal(y2, y)
    tp.gather = "kernel"
    a = torch.randn(T, N, device=dev, dtype=bf16)
    w2 = torch.randn(d, N, device=dev, dtype=bf16) * 0.05
    for _ in range(3):
        z = tp.gemm_rs(a, w2, residual_local=x)
    out["gemm_rs_rel"] = _rel(z, a.float() @ w2.float().t() + x.float())
    assert out["ag_gemm_rel"] < 1e-2 and out["gemm_rs_rel"] < 1e-2, out

    # ---- sharded / replicated stores against the resident one
    cfg = PRESETS["tiny"]
    layout = ParamLayout(cfg)
    S = 128
    g = torch.Generator().manual_seed(7)
    toks = torch.randint(0, cfg.vocab, (3, 2, S), generator=g).to(dev)

    def run(store):
        eng = LlamaEngine(cfg, store, S)
        p0 = store.full_params().float().clone()
        losses = []
        for step in range(2):
            if hasattr(store, "set_hyper"):
                store.set_hyper(lr=1.0, eps=1.0)
            losses.append(float(eng.forward_backward(toks[step], toks[step + 1])))
            eng.optimizer_step(1.0, eps=1.0)
        torch.cuda.synchronize()
        K.check_status()
        return store.full_params().float() - p0, losses

    ref_upd, ref_loss = run(LocalParamStore(layout, dev, seed=3, init_std=0.05))
    for mode in ("dma", "prefetch", "gemm"):
        upd, loss = run(FSDPParamStore(layout, dev, seed=3, init_std=0.05, gather=mode,
                                       gather_chunk=1 << 15))
        out[f"fsdp_{mode}_rel"] = _rel(upd, ref_upd)
        assert out[f"fsdp_{mode}_rel"] < 2e-2, out
        assert all(abs(p - q) < 2e-2 * abs(q) for p, q in zip(loss, ref_loss)), (loss, ref_loss)
    upd, loss = run(DDPParamStore(layout, dev, seed=3, init_std=0.05))
    out["ddp_rel"] = _rel(upd, ref_upd)
    assert out["ddp_rel"] < 2e-2, out

    # ---- expert parallel: one expert on this rank, every token routed to it
    Tm, dm, Fm = 256, 256, 512
    ep = EPComm(dist.group.WORLD, dev, Tm, dm, Fm, top_k=1)
    xm = torch.randn(Tm, dm, device=dev, dtype=bf16)
    idx = torch.zeros(Tm, 1, dtype=torch.int32, device=dev)
    wts = torch.rand(Tm, 1, device=dev) + 0.5
    e_gu = torch.randn(2 * Fm, dm, device=dev, dtype=bf16) * 0.05
    e_dn = torch.randn(dm, Fm, device=dev, dtype=bf16) * 0.05
    ym, _ = ep.forward(xm, idx, wts, e_gu, e_dn, residual=xm)
    gu = xm.float() @ e_gu.float().t()
    gate, up = gu[:, :Fm], gu[:, Fm:]
    h = (torch.nn.functional.silu(gate) * up * wts).to(bf16).float()
    want = h @ e_dn.float().t() + xm.float()
    out["moe_rel"] = _rel(ym, want)
    torch.cuda.synchronize()
    K.check_status()
    assert out["moe_rel"] < 2e-2, out
    out["launches"] = K.launch_count
    print("ONERANK FUSED OK " + json.dumps(out))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
