#!/usr/bin/env python
"""FSDP training driven from one controller over an actor mesh.

The controller spawns one proc per GPU (or per CPU rank), a ``TrainerActor`` on each, and then
only sends ``step`` messages: every actor owns its shard of the parameters, gradients and
AdamW state (``monarch_b200.parallel.trainer.Trainer`` with ``parallelism="fsdp"``), generates
its own synthetic batch and runs the sharded step with this package's NVLink kernels (or gloo
collectives on CPU).  The controller gets the per-rank losses back as a ``ValueMesh``.

    python examples/fsdp_on_mesh.py --gpus 2 --model llama3.2-1b --seq 2048 --steps 5
    python examples/fsdp_on_mesh.py --cpu --gpus 2 --model tiny --seq 64 --steps 3

This is the shape of the headline configuration ("Llama-3-8B FSDP on a mesh"): the control
plane is the actor runtime, the data plane never leaves the GPUs.
"""
import argparse
import os
import socket
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200.actor import Actor, current_rank, endpoint, proc_mesh  # noqa: E402


class TrainerActor(Actor):
    def __init__(self, model: str, seq: int, micro_batch: int, world: int, use_cuda: bool):
        import torch.distributed as dist
        self.rank = current_rank().rank
        os.environ.update(RANK=str(self.rank), WORLD_SIZE=str(world), LOCAL_RANK=str(self.rank))
        if use_cuda:
            torch.cuda.set_device(self.rank)      # before any allocation of this proc
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=self.rank, world_size=world)
        from monarch_b200.parallel.trainer import Trainer
        self.trainer = Trainer(model, seq_len=seq, micro_batch=micro_batch, parallelism="fsdp",
                               device=torch.device("cuda", self.rank) if use_cuda else "cpu",
                               comm="fused" if use_cuda else "nccl", lr=1e-3)
        # a fixed synthetic batch per rank (random token ids): repeating it lets the loss show
        # that the sharded optimizer step learns
        gen = torch.Generator().manual_seed(100 + self.rank)
        vocab = self.trainer.cfg.vocab
        self.tok = torch.randint(0, vocab, (micro_batch, seq), generator=gen)
        self.tgt = torch.randint(0, vocab, (micro_batch, seq), generator=gen)
        if use_cuda:
            self.tok, self.tgt = self.tok.pin_memory(), self.tgt.pin_memory()

    @endpoint
    def step(self, i: int) -> float:
        return self.trainer.step(self.tok, self.tgt)

    @endpoint
    def shutdown(self) -> None:
        import torch.distributed as dist
        if self.trainer.device.type == "cuda":
            torch.cuda.synchronize()
        dist.destroy_process_group()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run(model: str = "tiny", gpus: int = 2, seq: int = 64, micro_batch: int = 1, steps: int = 3,
        use_cuda: bool = False):
    procs = proc_mesh(gpus=gpus, env={"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(_free_port())})
    try:
        trainers = procs.spawn("trainers", TrainerActor, model, seq, micro_batch, gpus, use_cuda)
        losses, times = [], []
        for i in range(steps):
            t = time.perf_counter()
            vm = trainers.step.call(i).get(timeout=600)
            times.append(time.perf_counter() - t)
            losses.append([v for _, v in vm.items()])
        trainers.shutdown.call().get(timeout=120)
        steady = times[1:] or times
        return {"losses_first": losses[0], "losses_last": losses[-1],
                "tokens_per_s": gpus * micro_batch * seq / (sum(steady) / len(steady)),
                "ms_per_step": 1e3 * sum(steady) / len(steady)}
    finally:
        procs.stop().get()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--gpus", type=int, default=2)
    ap.add_argument("--seq", type=int, default=64)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args()
    print(run(a.model, a.gpus, a.seq, a.micro_batch, a.steps, use_cuda=not a.cpu))
