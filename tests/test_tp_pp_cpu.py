"""Tensor parallel x pipeline parallel training on CPU ranks (gloo): a {pp: 2, tp: 2} mesh
running 1F1B over 4 micro-batches must reproduce the loss and the updated parameters of
the single-process engine on the same weights and data."""
import os
import socket
import sys

import pytest
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


def _worker(rank, world, port, pp, tp, out, schedule="1f1b"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    from monarch_b200.models import PRESETS, LlamaEngine, LocalParamStore, ParamLayout
    from monarch_b200.models.llama import to_hf_state_dict
    from monarch_b200.parallel.pipelining import PipelineTrainer
    cfg = PRESETS["tiny"]
    S, B, M = 32, 1, 4
    torch.manual_seed(7)
    tok = torch.randint(0, cfg.vocab, (M, B, S))
    tgt = torch.randint(0, cfg.vocab, (M, B, S))
    # single-process oracle
    layout = ParamLayout(cfg)
    ref_store = LocalParamStore(layout, "cpu", seed=5, init_std=0.05)
    sd0 = to_hf_state_dict(cfg, layout, ref_store.params)
    ref = LlamaEngine(cfg, ref_store, S)
    ref_loss = float(ref.forward_backward(tok.reshape(M * B, S), tgt.reshape(M * B, S)))
    ref.optimizer_step(1e-2, eps=1e-3)
    sd_ref = to_hf_state_dict(cfg, layout, ref_store.params)

    tr = PipelineTrainer(cfg, pp, tp, S, B, M, device="cpu", lr=1e-2, comm="nccl",
                         schedule=schedule)
    tr.load_state_dict(sd0)
    orig = tr.engine.store.optimizer_step
    tr.engine.store.optimizer_step = lambda lr, **kw: orig(lr, eps=1e-3, **kw)
    loss = float(tr.step_device(tok, tgt))
    sd = tr.state_dict()
    if rank == world - 1:
        worst = max(((sd[k].float() - sd_ref[k].float()).norm() /
                     (sd_ref[k].float().norm() + 1e-9)).item() for k in sd_ref)
        out.put((loss, ref_loss, worst))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("pp,tp,schedule", [(2, 2, "1f1b"), (1, 2, "1f1b"), (2, 1, "1f1b"),
                                            (2, 1, "zb-h1"), (2, 2, "zb-h1"), (2, 1, "gpipe")])
def test_tp_pp_matches_single_process(pp, tp, schedule):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    world = pp * tp
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, pp, tp, out, schedule)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    loss, ref_loss, worst = out.get(timeout=10)
    assert abs(loss - ref_loss) < 2e-2 * abs(ref_loss), (loss, ref_loss)
    assert worst < 3e-2, worst


def test_schedules_are_complete_and_deadlock_free():
    from monarch_b200.parallel.pipelining import schedule_ir as ir
    for P, M in [(2, 8), (4, 8), (4, 4), (3, 7)]:
        for name, gen in ir.GENERATORS.items():
            s = gen(P, M)
            ir.validate(s, P, M)
            span, ev = ir.simulate(ir.add_communication(s, P), P)
            assert span > 0 and len(ev) == sum(1 for a in sum(s.values(), []))
    s = ir.interleaved_1f1b(4, 8, 2)
    ir.validate(s, 8, 8)
    assert ir.bubble_fraction(s, 8) < ir.bubble_fraction(ir.one_f_one_b(4, 8), 4)
    assert ir.bubble_fraction(ir.zero_bubble_h1(4, 8), 4) < ir.bubble_fraction(ir.gpipe(4, 8), 4)
    assert str(ir.Action.parse("3SEND_F12")) == "3SEND_F12"
