"""Expert-parallel mixture of experts on CPU ranks (gloo, all-to-all path): the layer's
forward and both gradients must equal a dense single-process computation in which every
token evaluates its top-k experts locally."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _dense(x, top_i, wts, wgu, wdown):
    """x [W, T, d] tokens of all ranks; expert e = (wgu[e], wdown[e])."""
    F = wgu[0].shape[0] // 2
    y = torch.zeros_like(x)
    for e in range(len(wgu)):
        gu = x @ wgu[e].t()
        h = torch.nn.functional.silu(gu[..., :F]) * gu[..., F:]
        ye = h @ wdown[e].t()
        w_e = (wts * (top_i == e)).sum(-1, keepdim=True)
        y = y + w_e * ye
    return y


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from monarch_b200.parallel.ep import EPComm
    T, d, F, k = 24, 16, 32, 2
    g = torch.Generator().manual_seed(3)
    x_all = torch.randn(world, T, d, generator=g)
    wgu = [torch.randn(2 * F, d, generator=g) * 0.3 for _ in range(world)]
    wdown = [torch.randn(d, F, generator=g) * 0.3 for _ in range(world)]
    logits = torch.randn(world, T, world, generator=g)
    top_p, top_i = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    wts_all = top_p / top_p.sum(-1, keepdim=True)
    dy_all = torch.randn(world, T, d, generator=g)
    # dense oracle with autograd
    xa = x_all.clone().requires_grad_(True)
    wa = wts_all.clone().requires_grad_(True)
    wg = [w.clone().requires_grad_(True) for w in wgu]
    wd = [w.clone().requires_grad_(True) for w in wdown]
    y_ref = _dense(xa, top_i, wa, wg, wd)
    y_ref.backward(dy_all)

    ep = EPComm(dist.group.WORLD, "cpu", T, d, F, k, comm="nccl")
    g_gu, g_down = torch.zeros_like(wgu[rank]), torch.zeros_like(wdown[rank])
    y, sv = ep.forward(x_all[rank], top_i[rank].int(), wts_all[rank], wgu[rank], wdown[rank])
    d_x, d_w = ep.backward(dy_all[rank], sv, wgu[rank], wdown[rank], g_gu, g_down, acc=False)
    errs = [
        (y - y_ref[rank]).abs().max().item(),
        (d_x - xa.grad[rank]).abs().max().item(),
        (d_w - wa.grad[rank]).abs().max().item(),
        (g_gu - wg[rank].grad).abs().max().item(),
        (g_down - wd[rank].grad).abs().max().item(),
    ]
    out.put((rank, errs))
    dist.barrier()
    dist.destroy_process_group()


def test_ep_layer_matches_dense():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    world, port = 4, _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for _ in range(world):
        rank, errs = out.get(timeout=10)
        assert max(errs) < 1e-3, (rank, errs)


def _train_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from monarch_b200.parallel.ep import MoETrainer
    tr = MoETrainer("tiny-moe", 32, 2, device="cpu", comm="nccl", lr=3e-3, init_std=0.05)
    g = torch.Generator().manual_seed(10 + rank)
    tok = torch.randint(0, tr.cfg.vocab, (2, 32), generator=g)
    losses = [tr.step(tok, tok.roll(-1, 1)) for _ in range(6)]
    out.put((rank, losses))
    dist.barrier()
    dist.destroy_process_group()


def test_moe_training_reduces_loss():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    world, port = 2, _free_port()
    procs = [ctx.Process(target=_train_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    for _ in range(world):
        rank, losses = out.get(timeout=10)
        assert losses[-1] < losses[0], losses
