#!/usr/bin/env python
"""SPMD inside actors: every actor of a mesh joins a torch.distributed process group and
trains a DistributedDataParallel replica.  The controller only sets the job up, starts the
steps and collects results; the gradient all-reduce runs between the procs (NCCL over NVLink
when every proc has a GPU, gloo otherwise).

    python examples/spmd_ddp.py

Parity: docs/source/examples/spmd_ddp.py of the reference (re-created on this package's
actor API)."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200.actor import Actor, current_rank, endpoint, proc_mesh  # noqa: E402


class ToyModel(nn.Module):
    def __init__(self):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(10, 32), nn.ReLU(), nn.Linear(32, 5))

    def forward(self, x):
        return self.net(x)


class DDPActor(Actor):
    def __init__(self, world_size: int):
        self.rank = current_rank().rank
        self.world = world_size
        self.model = self.opt = None

    @endpoint
    def setup(self) -> str:
        use_cuda = torch.cuda.is_available() and torch.cuda.device_count() >= self.world
        backend = "nccl" if use_cuda else "gloo"
        if use_cuda:
            torch.cuda.set_device(self.rank)
        dist.init_process_group(backend, rank=self.rank, world_size=self.world)
        self.device = torch.device("cuda", self.rank) if use_cuda else torch.device("cpu")
        torch.manual_seed(0)                       # same initial weights on every replica
        model = ToyModel().to(self.device)
        self.model = nn.parallel.DistributedDataParallel(
            model, device_ids=[self.rank] if use_cuda else None)
        self.opt = torch.optim.SGD(self.model.parameters(), lr=0.05)
        return backend

    @endpoint
    def train(self, steps: int):
        g = torch.Generator().manual_seed(1000 + self.rank)   # a different shard per rank
        w = torch.randn(10, 5, generator=torch.Generator().manual_seed(5))
        losses = []
        for _ in range(steps):
            x = torch.randn(64, 10, generator=g)
            y = (x @ w).to(self.device)
            loss = nn.functional.mse_loss(self.model(x.to(self.device)), y)
            self.opt.zero_grad()
            loss.backward()                        # DDP all-reduces the gradients here
            self.opt.step()
            losses.append(float(loss))
        flat = torch.cat([p.detach().flatten() for p in self.model.parameters()])
        return losses[0], losses[-1], float(flat.double().sum())

    @endpoint
    def cleanup(self) -> None:
        dist.destroy_process_group()


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run(world_size: int = 2, steps: int = 40):
    procs = proc_mesh(gpus=world_size,
                      env={"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(_free_port())})
    try:
        actors = procs.spawn("ddp_actor", DDPActor, world_size)
        backends = [b for _, b in actors.setup.call().get(timeout=120).items()]
        res = [r for _, r in actors.train.call(steps).get(timeout=300).items()]
        actors.cleanup.call().get(timeout=60)
        sums = [r[2] for r in res]
        return {"backend": backends[0], "loss_first": sum(r[0] for r in res) / len(res),
                "loss_last": sum(r[1] for r in res) / len(res),
                "replicas_in_sync": max(sums) - min(sums) < 1e-6 * max(1.0, abs(sums[0]))}
    finally:
        procs.stop().get()


if __name__ == "__main__":
    print(run())
