"""NVLink kernels and fused FSDP/DDP on >= 2 GPUs: launches one process per GPU running
tests/multigpu_selftest.py (every check compares against NCCL / fp32 PyTorch)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("n", [2, 4, 8])
def test_selftest_n_gpus(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs, have {torch.cuda.device_count()}")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(root, "tests", "multigpu_selftest.py")]
    p = subprocess.run(cmd, env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "SELFTEST OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


def _run(cmd, timeout=600, env_extra=None):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root, **(env_extra or {}))
    return subprocess.run(cmd, env=env, cwd=root, capture_output=True, text=True, timeout=timeout)


def _torchrun(n, script, *args):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
            "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
            os.path.join(root, "tests", script), *args]


@pytest.mark.parametrize("n", [2, 4, 8])
def test_mesh_communicator_n_gpus(n):
    """Every collective of the mesh communicator (IPC-exchanged and symmetric-memory buffers,
    multimem where the fabric has it) against NCCL."""
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs, have {torch.cuda.device_count()}")
    p = _run(_torchrun(n, "multigpu_meshcomm.py"))
    assert p.returncode == 0 and "MESHCOMM OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.parametrize("n", [2, 4, 8])
def test_tensor_engine_n_gpus(n):
    """Tensor.reduce over an actor mesh of GPU workers on the NVLink kernels, no
    torch.distributed on that path."""
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs, have {torch.cuda.device_count()}")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = _run([sys.executable, os.path.join(root, "tests", "multigpu_tensor_engine.py"),
              "--gpus", str(n)])
    assert p.returncode == 0 and "TENSOR ENGINE MULTIGPU OK" in p.stdout, \
        p.stdout[-3000:] + p.stderr[-3000:]


def test_withheld_barrier_times_out_and_recovers_2_gpus():
    """A rank that does not join a device-side barrier costs the other its bounded wait and
    an error status, not a hang; afterwards the barrier works again."""
    p = _run(_torchrun(2, "multigpu_failure.py"), env_extra={"NCCL_NVLS_ENABLE": "0"})
    assert p.returncode == 0 and "FAILURE PATH OK" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
