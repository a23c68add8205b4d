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


def _udf_collectives(x, pg):
    """Worker-side code written against torch.distributed; the group runs on the package's
    NVLink kernels."""
    import torch.distributed as dist
    assert pg.getBackendName() == "mb200"
    out = x.clone()
    dist.all_reduce(out, group=pg)
    parts = [torch.empty_like(x) for _ in range(pg.size())]
    dist.all_gather(parts, x, group=pg)
    rs = torch.empty(x.numel() // pg.size(), device=x.device, dtype=x.dtype)
    dist.reduce_scatter_tensor(rs, x.reshape(-1).contiguous(), group=pg)
    b = x.clone()
    dist.broadcast(b, pg.size() - 1, group=pg)
    dist.barrier(group=pg)
    return out, torch.stack(parts), rs, b


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
            # torch.distributed code inside a remote function, on a group over the kernels
            udf = te.remote(_udf_collectives,
                            propagate=lambda t, pg: (t, torch.stack([t] * pg.size()),
                                                     t.reshape(-1)[: t.numel() // pg.size()], t))
            w = (r + 1) * torch.ones(2 * n, device="cuda")
            u_sum, u_parts, u_rs, u_b = udf(w, dm.process_group("gpus"))
            got["udf"] = [te.inspect((u_sum, u_parts, u_rs, u_b), gpus=g) for g in range(n)]
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
        for g in range(n):
            u_sum, u_parts, u_rs, u_b = got["udf"][g]
            assert torch.equal(u_sum, torch.full((2 * n,), tri)), (g, u_sum)
            assert torch.equal(u_parts, torch.stack([torch.full((2 * n,), float(p + 1))
                                                     for p in range(n)]))
            assert torch.equal(u_rs, torch.full((2,), tri)) and torch.equal(
                u_b, torch.full((2 * n,), float(n)))
        assert torch.allclose(got["avg"], base * tri / n)
        assert torch.equal(got["max"], base * n) and torch.equal(got["min"], base)
        assert torch.equal(got["bf16"].float(), base * tri)
        assert got["stack"].shape == (n, 2, 3)
        assert torch.equal(got["inplace"], base * tri), got["inplace"]
        assert torch.equal(got["side"], base * tri), got["side"]
        assert got["big"].tolist() == [tri, tri], got["big"]
        assert all(not s["dist_initialized"] for s in state), state
        assert sorted(s["device"] for s in state) == list(range(n)), state
        assert all(s["launches"] > 20 for s in state), state
        results["launches_per_worker"] = [s["launches"] for s in state]
        # bitwise reductions of integers run on the kernels too (NCCL has none)
        with dm.activate():
            bits = (dm.rank("gpus") + 1).to(torch.int32).cuda() * \
                torch.ones(4, dtype=torch.int32, device="cuda")
            bo = te.inspect(bits.reduce("gpus", "bor"), gpus=0)
            still = te.call_on_shard_and_fetch(_dist_state, bits, shard={"gpus": 0}).get()
        want = 0
        for g in range(n):
            want |= g + 1
        assert bo.tolist() == [want] * 4, bo
        assert not still["dist_initialized"]
        # a dtype outside the kernels' coverage falls back to NCCL, initialised on demand
        with dm.activate():
            small = (dm.rank("gpus") + 1).to(torch.uint8).cuda() * \
                torch.ones(4, dtype=torch.uint8, device="cuda")
            sm = te.inspect(small.reduce("gpus", "sum"), gpus=0)
            now = te.call_on_shard_and_fetch(_dist_state, small, shard={"gpus": 0}).get()
        assert sm.tolist() == [int(tri)] * 4, sm
        assert now["dist_initialized"]
        print("TENSOR ENGINE MULTIGPU OK " + json.dumps(results))
        return 0
    finally:
        dm.exit()
        pm.stop().get()


if __name__ == "__main__":
    sys.exit(main())
