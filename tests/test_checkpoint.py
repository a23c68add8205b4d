"""Checkpoint / resume: a trainer restored from per-rank shards continues exactly as the one
that kept running (single process, and FSDP over two gloo ranks), and the Hugging
Face-named ``state_dict`` round-trips through the stock torch module."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _data(cfg, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg.vocab, (2, 32), generator=g) for _ in range(n + 1)]


def _run_resume(tmp, rank=0):
    from monarch_b200.parallel.trainer import Trainer
    a = Trainer("tiny", seq_len=32, micro_batch=2, device="cpu", lr=1e-2)
    d = _data(a.cfg, 6, seed=rank)
    for i in range(3):
        a.step(d[i], d[i + 1])
    a.save_checkpoint(tmp)
    cont = [a.step(d[i], d[i + 1]) for i in range(3, 6)]
    b = Trainer("tiny", seq_len=32, micro_batch=2, device="cpu", lr=1e-2, seed=99)
    assert b.load_checkpoint(tmp) == 3
    res = [b.step(d[i], d[i + 1]) for i in range(3, 6)]
    return cont, res


def test_single_process_resume_is_exact(tmp_path):
    cont, res = _run_resume(str(tmp_path))
    assert cont == res
    assert sorted(os.listdir(tmp_path)) == ["manifest.json", "shard_0.pt"]


def test_state_dict_roundtrip_with_stock_torch_module():
    from monarch_b200.models import TorchLlama
    from monarch_b200.parallel.trainer import Trainer
    t = Trainer("tiny", seq_len=32, micro_batch=2, device="cpu")
    sd = t.state_dict()
    m = TorchLlama(t.cfg)
    missing = m.load_state_dict({k: v.float() for k, v in sd.items()}, strict=True)
    assert not missing.missing_keys
    t2 = Trainer("tiny", seq_len=32, micro_batch=2, device="cpu", seed=5)
    t2.load_state_dict(m.state_dict())
    for k, v in t2.state_dict().items():
        assert torch.equal(v.float(), sd[k].float()), k


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tmp, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    cont, res = _run_resume(tmp, rank)
    out.put((rank, cont, res))
    dist.barrier()
    dist.destroy_process_group()


def test_fsdp_resume_is_exact(tmp_path):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path), out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
        assert p.exitcode == 0
    for _ in range(2):
        rank, cont, res = out.get(timeout=10)
        assert cont == res, (rank, cont, res)
    assert sorted(os.listdir(tmp_path)) == ["manifest.json", "shard_0.pt", "shard_1.pt"]
