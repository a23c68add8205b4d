#!/usr/bin/env python
"""A tour of distributed tensors: one Python program drives every device of a mesh.

    python examples/distributed_tensors.py

Covers: meshes and `inspect`; commands that fail without taking the workers down;
collectives as `reduce` over named mesh dims; reshaping a mesh for several kinds of
parallelism; moving tensors between sub-meshes (pipelining); remote functions; compiled
blocks.  Every step checks what it shows.

Parity: docs/source/examples/distributed_tensors.py of the reference (the same tour on this
package's API; the DDP part of that tour is examples/distributed_tensors_ddp.py)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200 import tensor_engine as te  # noqa: E402
from monarch_b200.actor import this_host  # noqa: E402


def _rank_banner(t):
    """Runs on every worker: any Python may run there, not only torch operators."""
    return t + t.numel()


def _fails_on_rank_two(t, rank):
    if int(rank.item()) == 2:
        raise ValueError("rank two is out today")
    return t


def run():
    out = {}
    procs = this_host().spawn_procs(per_host={"gpus": 4})
    mesh = te.spawn_tensor_engine(procs, use_cuda=False)
    try:
        # ---- meshes: without an active mesh torch runs here, with one it runs everywhere
        local = torch.ones(2) * 3
        assert not isinstance(local, te.Tensor)
        with mesh.activate():
            t = torch.ones(2, 3) * (mesh.rank("gpus") + 1).to(torch.float32)
            assert isinstance(t, te.Tensor) and t.shape == (2, 3)
            out["rank0"] = te.inspect(t)[0, 0].item()              # rank 0's copy
            out["rank3"] = te.inspect(t, gpus=3)[0, 0].item()      # another rank's copy
            assert (out["rank0"], out["rank3"]) == (1.0, 4.0)

            # ---- shape errors are caught here, before anything is sent ...
            try:
                t @ t                                              # 2x3 @ 2x3
                raise AssertionError("expected a shape error")
            except RuntimeError as e:
                assert "reduction dim" in str(e) or "shapes" in str(e)

            # ---- ... and a command that fails on a worker poisons its results, not the worker
            picky = te.remote(_fails_on_rank_two, propagate=lambda t, r: t)
            bad = picky(t, mesh.rank("gpus"))
            worse = bad * 2                                        # depends on the failure
            out["error_caught"] = False
            try:
                te.inspect(worse, gpus=2)
            except te.RemoteException as e:
                out["error_caught"] = "rank two is out today" in str(e)
            assert out["error_caught"]
            try:            # a fetch vouches for the whole tensor, whichever shard it reads
                te.inspect(worse, gpus=1)
                raise AssertionError("expected the failure of rank two")
            except te.RemoteException:
                pass
            still = te.inspect(t.sum(), gpus=1).item()             # the workers carry on
            assert still == 12.0

            # ---- collectives are reductions over named mesh dims
            total = t.reduce("gpus", "sum")                        # all-reduce
            assert te.inspect(total)[0, 0].item() == 10.0
            stacked = t.reduce("gpus", "stack")                    # all-gather: new outer dim
            assert stacked.shape == (4, 2, 3)
            scattered = torch.ones(4, 5).reduce("gpus", "sum", scatter=True)   # reduce-scatter
            assert scattered.shape == (5,) and te.inspect(scattered, gpus=2)[0].item() == 4.0

        # ---- the same devices, reshaped: 2-way data parallel x 2-way pipeline
        grid = mesh.split(gpus=("dp", "pp"), pp=2)
        assert grid.sizes == {"hosts": 1, "dp": 2, "pp": 2}
        with grid.activate():
            r = grid.rank("dp") * 10 + grid.rank("pp")
            out["coords"] = [[te.inspect(r, dp=d, pp=p).item() for p in range(2)] for d in range(2)]
            assert out["coords"] == [[0, 1], [10, 11]]
            dp_sum = (grid.rank("dp") + 1).to(torch.float32).reduce("dp", "sum")
            assert te.inspect(dp_sum, dp=1, pp=1).item() == 3.0    # reduced over dp only

        # ---- pipelining: two stages on two sub-meshes, activations move with to_mesh
        stage0, stage1 = grid.slice(pp=0), grid.slice(pp=1)
        with stage0.activate():
            w0 = torch.full((4, 4), 0.5)
            x = torch.ones(3, 4)
            h = (x @ w0).relu()                                    # lives on stage 0
        h1 = h.to_mesh(stage1)                                     # sent dp-wise to stage 1
        with stage1.activate():
            w1 = torch.full((4, 2), 2.0)
            y = h1 @ w1
            out["pipeline_out"] = te.inspect(y, dp=1)[0, 0].item()
            assert out["pipeline_out"] == 16.0                     # (4*0.5) * 4 * 2

        # ---- remote functions and compiled blocks
        with mesh.activate():
            banner = te.remote(_rank_banner, propagate=lambda t: t)
            b = banner(torch.zeros(2, 5))
            assert te.inspect(b, gpus=2)[0, 0].item() == 10.0

            @te.compile
            def block(a):
                for _ in range(5):
                    a = (a * 2 + 1).clamp(max=100)
                return a.sum()

            first = te.inspect(block(torch.ones(3))).item()
            again = te.inspect(block(torch.ones(3))).item()        # replayed, not re-traced
            out["compiled"] = (first, again)
            assert first == again == 3 * 63.0
    finally:
        mesh.exit()
        procs.stop().get()
    return out


if __name__ == "__main__":
    for k, v in run().items():
        print(f"{k}: {v}")
