#!/usr/bin/env python
"""CPU-only data-parallel training over an actor mesh.

A ProcMesh of 4 processes each hosts a ``Trainer`` actor holding a 2-layer MLP
(784 -> 1024 -> 10, ReLU, fp32, Kaiming-uniform init, seed 0).  Every step is one
``train`` call broadcast to the mesh: each actor runs forward/backward on a batch of 32
N(0,1) inputs with uniform labels and returns its flattened gradient; the gradients are
summed by the native accumulating port of the caller's mailbox (C++ reducer), the mean is
broadcast back and every actor applies plain SGD (lr 0.01).  Also copies a 1 MiB fp32
buffer between two actors' host memory through an RDMABuffer.

    python examples/mlp_actor_mesh.py [--steps 100] [--procs 4] [--in-process]
"""
import argparse
import json
import os
import statistics
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200.actor import Actor, current_rank, endpoint, local_proc_mesh, this_host  # noqa: E402
from monarch_b200.tensor_engine import RDMABuffer  # noqa: E402


class Trainer(Actor):
    def __init__(self, lr: float = 0.01):
        torch.manual_seed(0)
        torch.set_num_threads(1)
        self.model = torch.nn.Sequential(torch.nn.Linear(784, 1024), torch.nn.ReLU(),
                                         torch.nn.Linear(1024, 10))
        self.lr = lr
        self.rank = current_rank().rank
        self.gen = torch.Generator().manual_seed(1000 + self.rank)
        self.blob = None

    @endpoint
    def train(self, step: int) -> torch.Tensor:
        x = torch.randn(32, 784, generator=self.gen)
        y = torch.randint(0, 10, (32,), generator=self.gen)
        self.model.zero_grad(set_to_none=True)
        loss = torch.nn.functional.cross_entropy(self.model(x), y)
        loss.backward()
        self.last_loss = float(loss)
        return torch.cat([p.grad.reshape(-1) for p in self.model.parameters()])

    @endpoint
    def apply(self, mean_grad: torch.Tensor) -> None:
        off = 0
        with torch.no_grad():
            for p in self.model.parameters():
                n = p.numel()
                p.sub_(self.lr * mean_grad[off: off + n].view_as(p))
                off += n

    @endpoint
    def loss(self) -> float:
        return self.last_loss

    @endpoint
    def fingerprint(self) -> float:
        return float(sum(p.double().sum() for p in self.model.parameters()))

    @endpoint
    def export_blob(self) -> RDMABuffer:
        self.blob = torch.arange(262144, dtype=torch.float32)
        return RDMABuffer(self.blob.view(torch.uint8))

    @endpoint
    def fetch_blob(self, buf: RDMABuffer) -> dict:
        dst = torch.empty(262144, dtype=torch.float32)
        t0 = time.perf_counter()
        buf.read_into(dst.view(torch.uint8)).get()
        dt = time.perf_counter() - t0
        return {"ok": bool(torch.equal(dst, torch.arange(262144, dtype=torch.float32))),
                "seconds": dt}


def run(steps: int = 100, procs: int = 4, in_process: bool = False) -> dict:
    pm = local_proc_mesh(gpus=procs) if in_process else \
        this_host().spawn_procs(per_host={"gpus": procs})
    try:
        trainers = pm.spawn("trainer", Trainer)
        lat = []
        t_start = time.perf_counter()
        first = last = None
        for step in range(steps):
            t0 = time.perf_counter()
            g = trainers.train.reduce(step, reducer="sum_f32").get(timeout=60)
            trainers.apply.broadcast(g / procs)
            lat.append(time.perf_counter() - t0)
            if step in (0, steps - 1):
                ls = trainers.loss.call().get(timeout=60).values()
                if step == 0:
                    first = sum(ls) / procs
                last = sum(ls) / procs
        total = time.perf_counter() - t_start
        prints = trainers.fingerprint.call().get(timeout=60).values()
        # cast round-trip latency of a trivial endpoint
        cast = []
        for _ in range(200):
            t0 = time.perf_counter()
            trainers.loss.call().get(timeout=60)
            cast.append((time.perf_counter() - t0) * 1e6)
        cast.sort()
        buf = trainers.slice(gpus=0).export_blob.call_one().get(timeout=60)
        copy = trainers.slice(gpus=1).fetch_blob.call_one(buf).get(timeout=60)
        return {"steps": steps, "procs": procs, "steps_per_s": steps / total,
                "loss_first": first, "loss_last": last,
                "replicas_in_sync": max(prints) - min(prints) < 1e-6,
                "step_ms_p50": statistics.median(lat) * 1e3,
                "cast_us_p50": cast[len(cast) // 2], "cast_us_p99": cast[int(len(cast) * 0.99)],
                "rdma_1mib_ok": copy["ok"],
                "rdma_1mib_gbs": 1048576 / copy["seconds"] / 1e9}
    finally:
        pm.stop().get()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--procs", type=int, default=4)
    ap.add_argument("--in-process", action="store_true")
    a = ap.parse_args()
    print(json.dumps(run(a.steps, a.procs, a.in_process)))
