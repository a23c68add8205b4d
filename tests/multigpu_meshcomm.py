"""Mesh communicator on 2-8 GPUs: every collective against NCCL / fp32 PyTorch.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29512 tests/multigpu_meshcomm.py [--bench]

Two communicators are checked: one whose buffers were exchanged as CUDA IPC handles (the
way the tensor engine bootstraps it over actor messages; here the handles ride
``all_gather_object``), and one on torch's symmetric memory, which adds the NVSwitch
multicast mapping and with it the ``multimem`` paths.  ``--bench`` prints device-timed
all-reduce bus bandwidth (max over ranks) next to NCCL's.
"""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from monarch_b200.ops import ipc  # noqa: E402
from monarch_b200.ops import kernels as K  # noqa: E402
from monarch_b200.parallel.meshcomm import MeshComm  # noqa: E402


def _rel(a, b):
    return ((a.double() - b.double()).norm() / (b.double().norm() + 1e-12)).item()


def _check_comm(comm: MeshComm, rank: int, world: int, dev, tag: str, results: dict) -> None:
    torch.manual_seed(17 + rank)
    worst = 0.0
    for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int32,
                  torch.int64):
        for n in (1, 1000, 65_537, 3_000_000):
            x = (torch.randn(n, device=dev) * 4).to(dtype)
            for op, red in (("sum", dist.ReduceOp.SUM), ("avg", dist.ReduceOp.SUM),
                            ("max", dist.ReduceOp.MAX), ("min", dist.ReduceOp.MIN),
                            ("product", dist.ReduceOp.PRODUCT)):
                if op == "avg" and not dtype.is_floating_point:
                    continue
                if op == "product" and n > 1000:
                    continue
                if op == "product" and dtype.is_floating_point:
                    # factors near one: a product over 8 ranks of values around 4 leaves the
                    # range of fp16
                    x = (1 + 0.1 * torch.randn(n, device=dev)).to(dtype)
                acc = x.clone().double() if dtype.is_floating_point else x.clone()
                dist.all_reduce(acc, op=red)
                if op == "avg":
                    acc = acc / world
                y = comm.all_reduce(x, op)
                torch.cuda.synchronize()
                K.check_status(dev)
                if dtype.is_floating_point:
                    tol = {torch.float32: 1e-6, torch.float64: 1e-12}.get(dtype, 6e-3)
                    r = _rel(y, acc)
                    assert r <= tol, (tag, dtype, n, op, r)
                    worst = max(worst, r) if dtype in (torch.bfloat16, torch.float16) else worst
                else:
                    assert torch.equal(y, acc.to(dtype)), (tag, dtype, n, op)
                # every rank holds the same bits (peer loads are combined in rank order; the
                # switch's own reduction order is not specified, so with multicast only
                # closeness is asserted)
                ref = y.clone()
                dist.broadcast(ref, 0)
                if comm.mc_ptr and dtype.is_floating_point and op in ("sum", "avg"):
                    assert _rel(ref, y) <= 4e-3, (tag, "ranks differ", dtype, n, op)
                else:
                    assert torch.equal(ref, y), (tag, "ranks differ", dtype, n, op)
            if not dtype.is_floating_point:     # bitwise reductions (NCCL has none: fold by hand)
                parts = [torch.empty_like(x) for _ in range(world)]
                dist.all_gather(parts, x)
                for op, f in (("band", torch.bitwise_and), ("bor", torch.bitwise_or),
                              ("bxor", torch.bitwise_xor)):
                    acc = parts[0]
                    for p in parts[1:]:
                        acc = f(acc, p)
                    assert torch.equal(comm.all_reduce(x, op), acc), (tag, dtype, n, op)
    results[f"{tag}_allreduce_16bit_worst_rel"] = worst
    # reduce-scatter, all-gather, all-to-all, broadcast, root reduce; ragged sizes
    for dtype, cols in ((torch.float32, 1001), (torch.bfloat16, 40_003), (torch.float32, 2_500_000)):
        x = torch.randn(world, cols, device=dev).to(dtype)
        acc = x.double()
        dist.all_reduce(acc)
        rs = comm.reduce_scatter(x, "sum")
        tol = 1e-6 if dtype == torch.float32 else 6e-3
        assert _rel(rs, acc[rank]) <= tol, (tag, "reduce_scatter", dtype, cols)
        parts = [torch.empty_like(x[0]) for _ in range(world)]
        dist.all_gather(parts, x[rank].contiguous())
        assert torch.equal(comm.all_gather(x[rank]), torch.stack(parts)), (tag, "all_gather")
        a2a = torch.empty_like(x)
        dist.all_to_all_single(a2a, x.contiguous())
        assert torch.equal(comm.all_to_all(x), a2a), (tag, "all_to_all", dtype, cols)
        root = (world - 1) if cols % 2 else 0
        b = x.clone()
        dist.broadcast(b, root)
        assert torch.equal(comm.broadcast(x, root), b), (tag, "broadcast")
        rr = comm.reduce(x, root, "sum")
        if rank == root:
            assert _rel(rr, acc) <= tol, (tag, "reduce")
        else:
            assert rr is None
        # two root reduces in a row and a copy after them: the staging halves must not be
        # overwritten while the root still reads them
        r2 = comm.reduce(x * 2, root, "max")
        ag = comm.all_gather(x[0])
        torch.cuda.synchronize()
        K.check_status(dev)
        assert ag.shape == (world, cols)
        mx = (x * 2).clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        if rank == root:
            assert torch.equal(r2, mx), (tag, "reduce max")
    comm.barrier()
    torch.cuda.synchronize()
    K.check_status(dev)


def main() -> int:
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    bench = "--bench" in sys.argv
    results: dict = {"world": world}

    # --- buffers exchanged as IPC handles (small capacity: the chunked paths run too)
    cap = 1 << 20
    buf = MeshComm.allocate_local(dev, cap)
    torch.cuda.synchronize()
    exports = [None] * world
    dist.all_gather_object(exports, ipc.export_handle(buf))
    c_ipc = MeshComm.from_exports(rank, exports, buf, dev, cap)
    c_ipc.one_shot_bytes = 1 << 14
    _check_comm(c_ipc, rank, world, dev, "ipc", results)

    # --- symmetric memory (+ multicast where the fabric has it)
    c_sym = MeshComm.from_process_group(None, dev, 8 << 20)
    results["nvls_multicast"] = bool(c_sym.mc_ptr)
    _check_comm(c_sym, rank, world, dev, "symm", results)

    if bench:
        big = MeshComm.from_process_group(None, dev, 256 << 20)
        rows = []
        for nbytes in (8 << 10, 256 << 10, 2 << 20, 32 << 20, 256 << 20):
            x = torch.randn(nbytes // 2, device=dev).to(torch.bfloat16)

            def ours():
                big.all_reduce(x, "sum", out=x)

            def nccl():
                dist.all_reduce(x)

            t = {}
            for name, fn in (("ours", ours), ("nccl", nccl)):
                for _ in range(3):
                    fn()
                    x.mul_(0.01)
                torch.cuda.synchronize()
                dist.barrier()
                iters = 20 if nbytes <= (2 << 20) else 8
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(iters):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                ms = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
                t[name] = float(ms.item())
                x.normal_()
            bus = lambda ms: 2 * (world - 1) / world * nbytes / (ms / 1e3) / 1e9  # noqa: E731
            rows.append({"bytes": nbytes, "ours_us": t["ours"] * 1e3, "nccl_us": t["nccl"] * 1e3,
                         "ours_busbw_gbs": bus(t["ours"]), "nccl_busbw_gbs": bus(t["nccl"])})
        K.check_status(dev)
        results["tensor_allreduce"] = rows

    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print("MESHCOMM OK " + json.dumps(results))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
