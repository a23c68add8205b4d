"""RDMABuffer: handles travel in actor messages; read_into / write_from move the bytes.
Host memory paths run on CPU; GPU paths (CUDA IPC mapping + the NVLink copy kernel) need a
device.  Modelled on python/tests/test_rdma.py of the reference."""
import pytest
import torch

from monarch_b200.actor import Actor, endpoint, local_proc_mesh, this_host
from monarch_b200.tensor_engine import RDMABuffer, RDMAError


class Owner(Actor):
    def __init__(self, n, device="cpu"):
        self.data = torch.arange(n, dtype=torch.float32, device=device)
        self.buf = None

    @endpoint
    def export(self) -> RDMABuffer:
        self.buf = RDMABuffer(self.data.view(torch.uint8))
        return self.buf

    @endpoint
    def checksum(self) -> float:
        return float(self.data.double().sum())

    @endpoint
    def drop(self):
        self.buf.drop().get()


class Reader(Actor):
    def __init__(self, device="cpu"):
        self.device = device

    @endpoint
    def pull(self, buf: RDMABuffer, n: int) -> float:
        dst = torch.zeros(n, dtype=torch.float32, device=self.device)
        buf.read_into(dst.view(torch.uint8)).get()
        return float(dst.double().sum())

    @endpoint
    def push(self, buf: RDMABuffer, n: int, value: float) -> None:
        src = torch.full((n,), value, dtype=torch.float32, device=self.device)
        buf.write_from(src.view(torch.uint8)).get()

    @endpoint
    def pull_range(self, buf: RDMABuffer, first: int, count: int):
        dst = torch.zeros(count, dtype=torch.float32, device=self.device)
        buf.read_into(dst.view(torch.uint8), offset=first * 4).get()
        return dst.cpu().tolist()


N = 262144  # 1 MiB of fp32


def _roundtrip(pm, device="cpu"):
    owner = pm.spawn("owner", Owner, N, device).slice(gpus=0)
    reader = pm.spawn("reader", Reader, device).slice(gpus=1)
    buf = owner.export.call_one().get(timeout=30)
    assert buf.nbytes == N * 4
    expect = float(torch.arange(N, dtype=torch.float64).sum())
    assert reader.pull.call_one(buf, N).get(timeout=30) == expect
    assert reader.pull_range.call_one(buf, 10, 4).get(timeout=30) == [10.0, 11.0, 12.0, 13.0]
    reader.push.call_one(buf, N, 2.0).get(timeout=30)
    assert owner.checksum.call_one().get(timeout=30) == 2.0 * N
    return owner, reader, buf


def test_host_buffer_between_in_process_procs():
    pm = local_proc_mesh(gpus=2)
    try:
        _roundtrip(pm)
    finally:
        pm.stop().get()


def test_host_buffer_between_processes_and_errors():
    pm = this_host().spawn_procs(per_host={"gpus": 2})
    try:
        owner, reader, buf = _roundtrip(pm)
        with pytest.raises(Exception, match="outside a buffer"):
            reader.pull_range.call_one(buf, N - 1, 8).get(timeout=30)
        owner.drop.call_one().get(timeout=30)
        with pytest.raises(Exception, match="not registered"):
            reader.pull.call_one(buf, N).get(timeout=30)
    finally:
        pm.stop().get()


def test_client_side_buffer_and_pickle():
    import pickle
    t = torch.arange(1024, dtype=torch.uint8)
    b = RDMABuffer(t)
    b2 = pickle.loads(pickle.dumps(b))
    out = torch.zeros(16, dtype=torch.uint8)
    b2.read_into(out, offset=32).get()
    assert out.tolist() == list(range(32, 48))
    with pytest.raises(RDMAError):
        b2.read_into(torch.zeros(16, dtype=torch.uint8), offset=1020).get()


@pytest.mark.gpu
def test_gpu_buffer_between_processes_uses_peer_copy_kernel():
    """Two processes on one device: the reader maps the owner's allocation through CUDA
    IPC and the copy kernel moves the bytes (same kernel that runs over NVLink between
    two devices)."""
    pm = this_host().spawn_procs(per_host={"gpus": 2}, env={"CUDA_VISIBLE_DEVICES": "0"})
    try:
        _roundtrip(pm, device="cuda")
    finally:
        pm.stop().get()
