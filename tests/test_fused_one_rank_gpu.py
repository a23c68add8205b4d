"""Runs tests/onerank_fused.py: the fused compute+collective kernels (tensor-parallel
gather-GEMM and GEMM-scatter, FSDP in its three gather modes, DDP, MoE dispatch/combine) as a
group of one rank on one GPU, against plain PyTorch and the resident parameter store."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.gpu
def test_fused_kernels_as_a_group_of_one_rank():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29591")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "onerank_fused.py")],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=280)
    assert p.returncode == 0 and "ONERANK FUSED OK" in p.stdout, \
        p.stdout[-2000:] + p.stderr[-3000:]
