#!/usr/bin/env python
"""RDMABuffer bandwidth sweep (GRPO-style weight refresh): trainer actors on the first half
of the GPUs publish bf16 buffers, generator actors on the second half pull them with
``RDMABuffer.read_into``; sizes 4 KB ... 4 GB in powers of 4, values N(0, 0.02).

    python benchmarks/rdma_sweep.py [--gpus 8] [--max-bytes 4294967296] [--out r.json]

Reported per size: GB/s of one trainer->generator pair (device-timed inside the generator
with CUDA events around the copy kernel, max over pairs) next to ``torch`` peer copy
(``dst.copy_(src)`` between the same two devices, cudaMemcpyPeerAsync) measured in the same
run.  With fewer than 2 GPUs the sweep runs host buffers between processes instead.
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200.actor import Actor, current_rank, endpoint, this_host  # noqa: E402
from monarch_b200.tensor_engine import RDMABuffer  # noqa: E402


class Trainer(Actor):
    def __init__(self, use_cuda: bool):
        self.rank = current_rank().rank
        self.dev = torch.device("cuda", self.rank) if use_cuda else torch.device("cpu")
        if use_cuda:
            torch.cuda.set_device(self.dev)
        self.t = None

    @endpoint
    def publish(self, nbytes: int) -> RDMABuffer:
        g = torch.Generator(device=self.dev).manual_seed(self.rank)
        w = torch.empty(nbytes // 2, dtype=torch.bfloat16, device=self.dev)
        w.normal_(0, 0.02, generator=g)
        self.t = w.view(torch.uint8)
        return RDMABuffer(self.t)

    @endpoint
    def checksum(self) -> float:
        return float(self.t.view(torch.bfloat16).float().sum().item())


class Generator(Actor):
    def __init__(self, use_cuda: bool, offset: int):
        self.rank = current_rank().rank
        self.dev = torch.device("cuda", self.rank + offset) if use_cuda else torch.device("cpu")
        if use_cuda:
            torch.cuda.set_device(self.dev)

    @endpoint
    def pull(self, buf: RDMABuffer, nbytes: int, iters: int) -> dict:
        dst = torch.empty(nbytes, dtype=torch.uint8, device=self.dev)
        buf.read_into(dst).get(timeout=120)          # warm-up: maps the peer allocation
        cuda = self.dev.type == "cuda"
        if cuda:
            torch.cuda.synchronize()
        best = 1e30
        for _ in range(iters):
            t0 = time.perf_counter()
            if cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            buf.read_into(dst).get(timeout=120)
            if cuda:
                e1.record()
                torch.cuda.synchronize()
                dt = e0.elapsed_time(e1) / 1e3
            else:
                dt = time.perf_counter() - t0
            best = min(best, dt)
        return {"seconds": best, "checksum": float(dst.view(torch.bfloat16).float().sum().item())}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=torch.cuda.device_count())
    ap.add_argument("--max-bytes", type=int, default=1 << 32)
    ap.add_argument("--out", default=None)
    a = ap.parse_args()
    use_cuda = a.gpus >= 2 and torch.cuda.is_available()
    half = max(1, a.gpus // 2) if use_cuda else 1
    pm_t = this_host().spawn_procs(per_host={"gpus": half})
    pm_g = this_host().spawn_procs(per_host={"gpus": half})
    trainers = pm_t.spawn("trainers", Trainer, use_cuda)
    gens = pm_g.spawn("generators", Generator, use_cuda, half)
    rows = []
    size = 4096
    try:
        while size <= a.max_bytes:
            bufs = trainers.publish.call(size).get(timeout=300)
            iters = 10 if size <= (1 << 26) else 3
            futs = []
            for (p, b) in bufs.items():
                futs.append(gens.slice(gpus=p.rank).pull.call_one(b, size, iters))
            res = [f.get(timeout=600) for f in futs]
            sums = [v for _, v in trainers.checksum.call().get(timeout=120).items()]
            ok = all(abs(r["checksum"] - s) <= 1e-3 * (1 + abs(s)) for r, s in zip(res, sums))
            sec = max(r["seconds"] for r in res)
            row = {"bytes": size, "pairs": half, "seconds": sec, "gbs_per_pair": size / sec / 1e9,
                   "verified": ok}
            if use_cuda:
                src = torch.empty(size, dtype=torch.uint8, device="cuda:0")
                dst = torch.empty(size, dtype=torch.uint8, device=f"cuda:{half}")
                dst.copy_(src)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                with torch.cuda.device(half):
                    e0.record()
                    for _ in range(iters):
                        dst.copy_(src, non_blocking=True)
                    e1.record()
                    torch.cuda.synchronize()
                row["memcpy_peer_gbs"] = size * iters / (e0.elapsed_time(e1) / 1e3) / 1e9
                del src, dst
            rows.append(row)
            print(json.dumps(row), flush=True)
            size *= 4
    finally:
        pm_t.stop().get()
        pm_g.stop().get()
    if a.out:
        with open(a.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
