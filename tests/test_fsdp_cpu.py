"""FSDP store on CPU ranks (gloo, world_size 2): the sharded schedule (gather ahead,
reduce-scatter + AdamW per unit during backward) must reproduce single-process training."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from monarch_b200.models import PRESETS, LlamaEngine, LocalParamStore, ParamLayout


def _worker(rank, world, port, preset, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from monarch_b200.parallel.fsdp import FSDPParamStore
    cfg = PRESETS[preset]
    layout = ParamLayout(cfg)
    st = FSDPParamStore(layout, "cpu", seed=7, init_std=0.05, comm="nccl")
    eng = LlamaEngine(cfg, st, seq_len=16)
    g = torch.Generator().manual_seed(100)
    toks = torch.randint(0, cfg.vocab, (world, 3, 2, 16), generator=g)
    losses = []
    for step in range(3):
        st.set_hyper(lr=1e-2)
        losses.append(eng.forward_backward(toks[rank, step], toks[rank, (step + 1) % 3]).item())
        eng.optimizer_step(1e-2)
        if step == 0:
            # an evaluation pass between two training steps must move neither the flag
            # epoch nor AdamW's step
            before = st.step_count
            ev = eng.forward_loss(toks[rank, 2], toks[rank, 0])
            assert st.step_count == before
            dist.all_reduce(ev)
            eval_loss = ev.item() / world
    full = st.full_params()
    if rank == 0:
        torch.save({"params": full, "losses": losses, "eval": eval_loss},
                   os.path.join(out_dir, "r0.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("preset", ["tiny", "tiny-tied"])
def test_fsdp_two_ranks_matches_single_process(preset):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    world = 2
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, port, preset, d), nprocs=world, join=True)
        got = torch.load(os.path.join(d, "r0.pt"))
    cfg = PRESETS[preset]
    layout = ParamLayout(cfg)
    st = LocalParamStore(layout, "cpu", seed=7, init_std=0.05)
    eng = LlamaEngine(cfg, st, seq_len=16)
    g = torch.Generator().manual_seed(100)
    toks = torch.randint(0, cfg.vocab, (world, 3, 2, 16), generator=g)
    for step in range(3):
        tok = torch.cat([toks[r, step] for r in range(world)])
        tgt = torch.cat([toks[r, (step + 1) % 3] for r in range(world)])
        eng.forward_backward(tok, tgt)
        eng.optimizer_step(1e-2)
        if step == 0:
            ev = eng.forward_loss(torch.cat([toks[r, 2] for r in range(world)]),
                                  torch.cat([toks[r, 0] for r in range(world)])).item()
            assert abs(ev - got["eval"]) < 2e-2 * abs(ev), (ev, got["eval"])
    ref = st.params.float()
    out = got["params"].float()
    rel = ((out - ref).norm() / ref.norm()).item()
    assert rel < 2e-2, rel
    assert got["losses"][-1] < got["losses"][0] + 1.0
