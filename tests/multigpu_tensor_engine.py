"""The distributed-tensor engine on N GPUs of one box, driven from this process over an
actor mesh: one proc (one tensor worker, one GPU) per rank.  ``Tensor.reduce`` in all its
forms runs on the package's NVLink kernels; the communicator's buffers are exchanged as CUDA
IPC handles through actor messages, and the workers never initialise ``torch.distributed``
unless an operation outside those kernels' coverage asks for it.

    python tests/multigpu_tensor_engine.py --gpus 2
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _dist_state(_t):
    import torch.distributed as dist
    from monarch_b200.ops import kernels as K
    return {"dist_initialized": dist.is_available() and dist.is_initialized(),
            "launches": K.launch_count, "device": torch.cuda.current_device()}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=2)
    n = ap.parse_args().gpus
    from monarch_b200 import tensor_engine as te
    from monarch_b200.actor import this_host
    pm = this_host().spawn_procs(per_host={"gpus": n})
    dm = te.spawn_tensor_engine(pm, use_cuda=True)
    results = {"gpus": n}
    try:
        tri = n * (n + 1) / 2
        base = torch.arange(1, 7, dtype=torch.float32).reshape(2, 3)      # controller-local
        with dm.activate():
            r = dm.rank("gpus").to(torch.float32).cuda()
            x = (r + 1) * torch.arange(1, 7, dtype=torch.float32, device="cuda").reshape(2, 3)
            y = (r + 1) * torch.ones(n, 5, device="cuda") * \
                torch.arange(1, n + 1, dtype=torch.float32, device="cuda")[:, None]
            big = (r + 1) * torch.ones(24 * 1024 * 1024 // 4 + 3, device="cuda")
            got = {
                "sum": [te.inspect(x.reduce("gpus", "sum"), gpus=g) for g in range(n)],
                "avg": te.inspect(x.reduce("gpus", "avg"), gpus=n - 1),
                "max": te.inspect(x.reduce("gpus", "max"), gpus=0),
                "min": te.inspect(x.reduce("gpus", "min"), gpus=0),
                "bf16": te.inspect(x.to(torch.bfloat16).reduce("gpus", "sum"), gpus=0),
                "stack": te.inspect(x.reduce("gpus", "stack"), gpus=n - 1),
            }
            # reduce-scatter / all-to-all need an outer dim of n
            rs = y.reduce("gpus", "sum", scatter=True)
            a2a = y.reduce("gpus", "stack", scatter=True)
            got["rs"] = [te.inspect(rs, gpus=g) for g in range(n)]
            got["a2a"] = [te.inspect(a2a, gpus=g) for g in range(n)]
            z = x.clone()
            z.reduce_("gpus", "sum")
            got["inplace"] = te.inspect(z, gpus=0)
            # a large tensor: the two-shot path and chunking through the staging area
            s = big.reduce("gpus", "sum")
            got["big"] = te.inspect(torch.stack([s.min(), s.max()]), gpus=n - 1)
            # a collective on a second stream (its own communicator)
            side = te.Stream("side")
            b, borrow = side.borrow(x)
            with side.activate():
                got["side"] = te.inspect(b.reduce("gpus", "sum"), gpus=0)
            borrow.drop()
            state = [te.call_on_shard_and_fetch(_dist_state, x, shard={"gpus": g}).get()
                     for g in range(n)]
        for g in range(n):
            assert torch.equal(got["sum"][g], base * tri), (g, got["sum"][g])
            assert torch.equal(got["rs"][g], torch.full((5,), tri * (g + 1))), (g, got["rs"][g])
            want = torch.stack([torch.full((5,), float((p + 1) * (g + 1))) for p in range(n)])
            assert torch.equal(got["a2a"][g], want), (g, got["a2a"][g])
            assert torch.equal(got["stack"][g], base * (g + 1))
        assert torch.allclose(got["avg"], base * tri / n)
        assert torch.equal(got["max"], base * n) and torch.equal(got["min"], base)
        assert torch.equal(got["bf16"].float(), base * tri)
        assert got["stack"].shape == (n, 2, 3)
        assert torch.equal(got["inplace"], base * tri) and torch.equal(got["side"], base * tri)
        assert got["big"].tolist() == [tri, tri], got["big"]
        assert all(not s["dist_initialized"] for s in state), state
        assert sorted(s["device"] for s in state) == list(range(n)), state
        assert all(s["launches"] > 20 for s in state), state
        results["launches_per_worker"] = [s["launches"] for s in state]
        # an operation outside the kernels' coverage falls back to NCCL, initialised on demand
        with dm.activate():
            bits = (dm.rank("gpus") + 1).to(torch.int32).cuda() * \
                torch.ones(4, dtype=torch.int32, device="cuda")
            bo = te.inspect(bits.reduce("gpus", "bor"), gpus=0)
        want = 0
        for g in range(n):
            want |= g + 1
        assert bo.tolist() == [want] * 4, bo
        print("TENSOR ENGINE MULTIGPU OK " + json.dumps(results))
        return 0
    finally:
        dm.exit()
        pm.stop().get()


if __name__ == "__main__":
    sys.exit(main())
