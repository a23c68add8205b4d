#!/usr/bin/env python
"""Tensor-engine dispatch overhead: the same loop of small tensor ops run locally, dispatched
op by op to a worker, dispatched inside a ``coalescing()`` block, replayed as a ``compile``d
recording, and as one remote function.  Small tensors on purpose: the numbers are the cost of
the controller -> worker path per op, not of the math.

    python benchmarks/dispatch.py [--iters 2000] [--size 100] [--cuda] [--mock] [--null-device]

``--mock`` runs the controller against simulated workers (no processes): the cost of the
front-end alone.  ``--null-device`` runs real worker processes whose tensors are shape-only
(nothing is computed or copied): the cost of the controller -> worker path for a program
written for GPUs, measurable on a box without one.  Parity: python/tests/dispatch_bench.py of the reference (local vs dispatched
vs remote function vs coalesced; the reference publishes the harness, not numbers)."""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200 import tensor_engine as te  # noqa: E402
from monarch_b200.actor import this_host  # noqa: E402


def loop(n: int, x: torch.Tensor) -> torch.Tensor:
    """3 ops per iteration on an [size, size] tensor."""
    for _ in range(n):
        x = x + 1.0
        x = x * 0.5
        x = torch.relu(x)
    return x


def run_loop_remote(n: int, x: torch.Tensor) -> torch.Tensor:
    return loop(n, x)


def timed(fn, repeat=3):
    best = None
    for _ in range(repeat):
        t = time.perf_counter()
        fn()
        dt = time.perf_counter() - t
        best = dt if best is None else min(best, dt)
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=2000)
    ap.add_argument("--size", type=int, default=100)
    ap.add_argument("--cuda", action="store_true")
    ap.add_argument("--mock", action="store_true")
    ap.add_argument("--null-device", action="store_true")
    ap.add_argument("--out")
    a = ap.parse_args()
    n, ops = a.iters, 3 * a.iters
    dev = "cuda" if a.cuda else "cpu"
    out = {"iters": n, "ops": ops, "size": a.size, "device": dev, "mock": a.mock,
           "null_device": a.null_device}

    x0 = torch.ones(a.size, a.size, device=dev)
    t = timed(lambda: (loop(n, x0), torch.cuda.synchronize() if a.cuda else None))
    out["local_us_per_op"] = t / ops * 1e6

    if a.mock:
        from monarch_b200.simulator import mock_mesh
        mesh, _ = mock_mesh(hosts=1, gpus=1)
        pm = None
    else:
        pm = this_host().spawn_procs(per_host={"gpus": 1})
        mesh = te.spawn_tensor_engine(pm, use_cuda=a.cuda, null_device=a.null_device)
    try:
        with mesh.activate():
            x = torch.ones(a.size, a.size)

            def dispatched():
                y = loop(n, x)
                te.fetch_shard(y.sum()).get(timeout=600)

            def coalesced():
                with te.coalescing():
                    y = loop(n, x)
                te.fetch_shard(y.sum()).get(timeout=600)

            out["dispatched_us_per_op"] = timed(dispatched) / ops * 1e6
            out["coalesced_us_per_op"] = timed(coalesced) / ops * 1e6
            if not a.mock:
                compiled = te.compile(lambda t: loop(n, t))
                compiled(x)                      # trace + define the recording

                def replay():
                    y = compiled(x)
                    te.fetch_shard(y.sum()).get(timeout=600)

                out["compiled_us_per_op"] = timed(replay) / ops * 1e6
                rfn = te.remote(run_loop_remote, propagate=lambda k, t: t)

                def remote_fn():
                    y = rfn(n, x)
                    te.fetch_shard(y.sum()).get(timeout=600)

                out["remote_function_us_per_op"] = timed(remote_fn) / ops * 1e6
    finally:
        if pm is not None:
            mesh.exit()
            pm.stop().get()
    print(json.dumps(out))
    if a.out:
        with open(a.out, "w") as f:
            json.dump(out, f)


if __name__ == "__main__":
    main()
