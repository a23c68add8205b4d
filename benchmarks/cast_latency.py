#!/usr/bin/env python
"""Actor-mesh messaging benchmark (CPU only): round-trip latency of ``call()`` on meshes of
1/4/16 procs with a 1 KB payload (p50/p99 in microseconds), fire-and-forget ``broadcast``
rate, and payload throughput for 10 KB ... 100 MB messages to one actor.

    python benchmarks/cast_latency.py [--out r.json]

Parity: python/benches/actor_mesh_benchmark.py:33-187 and hyperactor_mesh/benches/main.rs
(the reference publishes harnesses without numbers)."""
import argparse
import json
import os
import statistics
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200.actor import Actor, endpoint, local_proc_mesh, this_host  # noqa: E402


class Echo(Actor):
    def __init__(self):
        self.n = 0

    @endpoint
    def ping(self, payload: bytes) -> int:
        return len(payload)

    @endpoint
    def bump(self, payload: bytes) -> None:
        self.n += 1

    @endpoint
    def count(self) -> int:
        return self.n


def pct(xs, p):
    xs = sorted(xs)
    return xs[min(len(xs) - 1, int(p * len(xs)))]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--iters", type=int, default=300)
    a = ap.parse_args()
    out = {"call_roundtrip_us": [], "broadcast_msgs_per_s": [], "payload_mb_per_s": []}
    payload = b"x" * 1024
    for kind, n in (("processes", 1), ("processes", 4), ("processes", 16), ("in_process", 64)):
        pm = this_host().spawn_procs(per_host={"gpus": n}) if kind == "processes" \
            else local_proc_mesh(gpus=n)
        try:
            m = pm.spawn("echo", Echo)
            for _ in range(20):
                m.ping.call(payload).get(timeout=60)
            lat = []
            for _ in range(a.iters):
                t0 = time.perf_counter()
                m.ping.call(payload).get(timeout=60)
                lat.append((time.perf_counter() - t0) * 1e6)
            row = {"procs": n, "kind": kind, "p50": statistics.median(lat), "p99": pct(lat, 0.99),
                   "min": min(lat)}
            out["call_roundtrip_us"].append(row)
            print("call", json.dumps(row), flush=True)
            N = 2000
            t0 = time.perf_counter()
            for _ in range(N):
                m.bump.broadcast(payload)
            while min(v for _, v in m.count.call().get(timeout=60).items()) < N:
                time.sleep(0.001)
            dt = time.perf_counter() - t0
            row = {"procs": n, "kind": kind, "msgs_per_s": N / dt, "deliveries_per_s": N * n / dt}
            out["broadcast_msgs_per_s"].append(row)
            print("broadcast", json.dumps(row), flush=True)
        finally:
            pm.stop().get()
    pm = this_host().spawn_procs(per_host={"gpus": 1})
    try:
        m = pm.spawn("echo", Echo)
        for size in (10 << 10, 1 << 20, 10 << 20, 100 << 20):
            data = bytes(size)
            m.ping.call_one(data).get(timeout=120)
            reps = 20 if size <= (1 << 20) else 4
            t0 = time.perf_counter()
            for _ in range(reps):
                m.ping.call_one(data).get(timeout=120)
            dt = time.perf_counter() - t0
            row = {"bytes": size, "mb_per_s": size * reps / dt / 1e6}
            out["payload_mb_per_s"].append(row)
            print("payload", json.dumps(row), flush=True)
    finally:
        pm.stop().get()
    if a.out:
        with open(a.out, "w") as f:
            json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
