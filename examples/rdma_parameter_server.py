#!/usr/bin/env python
"""Parameter server over one-sided buffers.

The server owns the weights and one gradient slot per worker and hands out RDMABuffer handles
to them.  Each step a worker pulls the weights with ``read_into``, computes a gradient of a
least-squares problem on its own data shard and pushes it into its slot with ``write_from``;
the server then averages the slots and applies SGD.  No tensor ever travels in an actor
message: only the small handles do.

    python examples/rdma_parameter_server.py

Parity: monarch_rdma/examples/parameter_server of the reference (re-created on this
package's RDMABuffer; GPU tensors are first-class here, host tensors are used so that the
example also runs without a GPU)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200.actor import Actor, current_rank, endpoint, this_host  # noqa: E402
from monarch_b200.tensor_engine import RDMABuffer  # noqa: E402

DIM = 64


class ParameterServer(Actor):
    def __init__(self, n_workers: int, lr: float):
        self.w = torch.zeros(DIM)
        self.grads = torch.zeros(n_workers, DIM)
        self.lr = lr
        self._handles = None

    @endpoint
    def handles(self):
        if self._handles is None:
            self._handles = (RDMABuffer(self.w.view(torch.uint8)),
                             [RDMABuffer(self.grads[i].view(torch.uint8))
                              for i in range(self.grads.shape[0])])
        return self._handles

    @endpoint
    def apply(self) -> float:
        g = self.grads.mean(0)
        self.w -= self.lr * g
        return float(g.norm())

    @endpoint
    def weights(self) -> torch.Tensor:
        return self.w.clone()


class Worker(Actor):
    def __init__(self, w_true: torch.Tensor):
        self.rank = current_rank().rank
        g = torch.Generator().manual_seed(100 + self.rank)
        self.x = torch.randn(256, DIM, generator=g)
        self.y = self.x @ w_true
        self.w = torch.zeros(DIM)
        self.w_buf = self.slot = None

    @endpoint
    def connect(self, w_buf: RDMABuffer, slots) -> None:
        self.w_buf, self.slot = w_buf, slots[self.rank]

    @endpoint
    def step(self) -> float:
        self.w_buf.read_into(self.w.view(torch.uint8)).get()
        err = self.x @ self.w - self.y
        grad = (2.0 / len(self.y)) * (self.x.t() @ err)
        self.slot.write_from(grad.contiguous().view(torch.uint8)).get()
        return float((err ** 2).mean())


def run(n_workers: int = 2, steps: int = 60):
    w_true = torch.randn(DIM, generator=torch.Generator().manual_seed(7))
    server_procs = this_host().spawn_procs(per_host={"gpus": 1})
    worker_procs = this_host().spawn_procs(per_host={"gpus": n_workers})
    try:
        server = server_procs.spawn("server", ParameterServer, n_workers, 0.2)
        workers = worker_procs.spawn("workers", Worker, w_true)
        w_buf, slots = server.handles.call_one().get(timeout=30)
        workers.connect.call(w_buf, slots).get(timeout=30)
        losses = []
        for _ in range(steps):
            vals = workers.step.call().get(timeout=30)
            losses.append(sum(v for _, v in vals.items()) / n_workers)
            server.apply.call_one().get(timeout=30)
        w = server.weights.call_one().get(timeout=30)
        return {"loss_first": losses[0], "loss_last": losses[-1],
                "weight_error": float((w - w_true).norm() / w_true.norm())}
    finally:
        worker_procs.stop().get()
        server_procs.stop().get()


if __name__ == "__main__":
    print(run())
