"""The benchmark harness end to end on CPU ranks: the launch's processes attach to a proc
mesh, the controller spawns a TrainerActor per proc, times it through endpoint calls and
prints one JSON line with both arms.  (A check of the harness; the numbers mean nothing.)"""
import json
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("n", [1, 2])
def test_bench_flow_on_cpu_ranks(n):
    args = ["bench.py", "--gpus", str(n), "--cpu", "--model", "tiny", "--seq", "64", "--steps", "2",
            "--warmup", "1"]
    if n == 1:
        cmd = [sys.executable, *args]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={n}", "--master-addr", "127.0.0.1", "--master-port",
               str(_free_port()), *args]
    p = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=280)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-3000:]
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, p.stdout
    out = json.loads(lines[0])
    assert out["n_gpus"] == n and out["steps"] == 2 and out["value"] > 0
    assert out["config"]["parallelism"] == ("single" if n == 1 else "fsdp2")
    assert out["e2e"]["value"] > 0 and "step.call" in out["e2e"]["api"]
    assert out["e2e"]["h2d_bytes_per_step"] == 2 * 64 * 8 and out["e2e"]["d2h_bytes_per_step"] == 4
    assert out["baseline"]["value"] > 0
    assert abs(out["vs_baseline"] - out["value"] / out["baseline"]["value"]) < 1e-9
    # both arms trained the same model on the same data: their losses agree roughly
    assert abs(out["loss"] - out["baseline"]["loss"]) < 0.5


def test_reference_arm_says_why_it_is_unavailable():
    p = subprocess.run([sys.executable, "bench.py", "--impl", "reference"], cwd=ROOT,
                       capture_output=True, text=True, timeout=60)
    out = json.loads(p.stdout.strip().splitlines()[-1])
    assert p.returncode == 0 and out["impl"] == "reference" and "unavailable" in out
