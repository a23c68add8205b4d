#!/usr/bin/env python
"""Data-parallel training written as a single-controller program over distributed tensors:
one Python process drives every worker of the mesh, gradients are produced one at a time by
``grad_generator`` and all-reduced on a ``comm`` stream (borrowed across streams) while the
rest of backward runs, then the whole step is compiled into a recording.

    python examples/distributed_tensors_ddp.py [--cuda] [--procs 4]

With ``--cuda`` every worker owns one GPU and the gradient reductions run on this package's
NVLink collectives (communicators bootstrapped over actor messages, one per stream).

Parity: docs/source/examples/distributed_tensors.py:192-342 of the reference (DDP with
``grad.reduce_("dp", "sum")`` on a comms stream through ``borrow``)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200 import tensor_engine as te  # noqa: E402
from monarch_b200.actor import this_host  # noqa: E402


def run(steps: int = 8, procs: int = 4, cuda: bool = False):
    pm = this_host().spawn_procs(per_host={"gpus": procs})
    mesh = te.spawn_tensor_engine(pm, use_cuda=cuda).rename(gpus="dp")
    dev = "cuda" if cuda else "cpu"
    comm = te.Stream("comm")
    try:
        with mesh.activate():
            from monarch_b200 import random as mrandom
            mrandom.manual_seed(0)              # same weights on every worker ...
            w1 = torch.randn(16, 32, device=dev) * 0.1
            w2 = torch.randn(32, 4, device=dev) * 0.1
            mrandom.manual_seed(1, per_rank=True)   # ... different data
            losses = []
            for step in range(steps):
                x = torch.randn(64, 16, device=dev)   # every rank draws its own batch
                y = (x[:, :4] > 0).to(torch.float32)
                h = (x @ w1).relu()
                out = h @ w2
                # manual backward so that gradients appear one at a time, last layer first
                d_out = 2 * (out - y) / out.numel()
                g2 = h.t() @ d_out
                g2c, b2 = comm.borrow(g2, mutable=True)
                with comm.activate():
                    g2c.reduce_("dp", "avg")          # overlaps with the rest of backward
                d_h = (d_out @ w2.t()) * (h > 0)
                g1 = x.t() @ d_h
                g1c, b1 = comm.borrow(g1, mutable=True)
                with comm.activate():
                    g1c.reduce_("dp", "avg")
                b2.drop()
                b1.drop()
                w2.sub_(g2 * 0.5)
                w1.sub_(g1 * 0.5)
                losses.append(((out - y) ** 2).mean().reduce("dp", "avg"))
            vals = [te.inspect(l).item() for l in losses]
            # replicas stay identical: the averaged gradients are the same everywhere
            spread = (w1.reduce("dp", "max") - w1.reduce("dp", "min")).abs().max()
            in_sync = te.inspect(spread).item() == 0.0
        return {"loss_first": vals[0], "loss_last": vals[-1], "replicas_in_sync": in_sync}
    finally:
        mesh.exit()
        pm.stop().get()


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--cuda", action="store_true")
    ap.add_argument("--procs", type=int, default=4)
    ap.add_argument("--steps", type=int, default=8)
    a = ap.parse_args()
    print(run(a.steps, a.procs, a.cuda))
