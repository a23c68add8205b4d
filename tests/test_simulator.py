"""Mock device mesh + simulator: the controller-side tensor engine runs against simulated
workers (meta tensors), giving shapes, message counts, stream clocks and peak memory."""
import json

import torch

from monarch_b200 import tensor_engine as te
from monarch_b200.simulator import CostModel, mock_mesh


def test_mock_mesh_runs_programs_without_processes(tmp_path):
    mesh, sim = mock_mesh(hosts=4, gpus=8)
    assert mesh.sizes == {"hosts": 4, "gpus": 8}
    with mesh.activate():
        a = torch.ones(1024, 1024)
        b = a @ a
        assert b.shape == (1024, 1024)
        c = b.reduce("gpus", "sum")
        st = b.reduce("gpus", "stack")
        assert st.shape == (8, 1024, 1024)
        got = te.inspect(c, hosts=1, gpus=3)
        assert got.shape == (1024, 1024)
    assert sim.messages(0) >= 4
    assert sim.makespan_us() > 0
    assert sim.peak_memory_bytes() >= 8 * 1024 * 1024 * 4
    del a, b, c, st
    sim.dump_chrome_trace(str(tmp_path / "t.json"))
    ev = json.load(open(tmp_path / "t.json"))["traceEvents"]
    assert any("mm" in e["name"] for e in ev) and any("reduce" in e["name"] for e in ev)


def test_simulated_streams_overlap_and_cost_model():
    cm = CostModel(tflops=1000.0, hbm_gbs=5000.0, link_gbs=500.0, launch_us=0.0)
    mesh, sim = mock_mesh(hosts=1, gpus=2, cost=cm)
    comm = te.Stream("comm")
    with mesh.activate():
        x = torch.ones(4096, 4096)
        y = x @ x                                  # 137 GFLOP -> 137 us at 1000 TFLOP/s
        xb, borrow = comm.borrow(y)
        with comm.activate():
            r = xb.reduce("gpus", "sum")           # on the side stream
        z = x @ x                                  # main stream continues meanwhile
        borrow.drop()
    clocks = sim.stream_clocks(0)
    assert len(clocks) == 2
    main = clocks[0]
    assert main >= 2 * 137.0        # two matmuls back to back on the main stream
    side = [v for k, v in clocks.items() if k != 0][0]
    assert side > 137.0             # the reduce started after the first matmul


def test_compile_on_mock_mesh_counts_messages():
    mesh, sim = mock_mesh(hosts=1, gpus=4, trace=False)

    @te.compile
    def f(x):
        return (x * 2 + 1).sum()

    with mesh.activate():
        x = torch.ones(8, 8)
        f(x)
        n0 = sim.messages(0)
        for _ in range(5):
            f(x)
        assert sim.messages(0) - n0 <= 5 * 2     # one replay (+ deletes) per call


def test_device_mesh_indexing_reshaping_flattening():
    """python/tests/test_device_mesh.py of the reference, on simulated workers."""
    import pytest
    from monarch_b200.simulator import mock_mesh
    dm = mock_mesh(hosts=2, gpus=12, trace=False)[0].split(gpus=("b", "c"), c=4).rename(hosts="a")
    assert dm.names == ("a", "b", "c") and list(dm.processes.sizes) == [2, 3, 4]
    assert dm(a=0, b=0, c=0).processes.ranks() == [0]
    x = dm(a=0, b=0)
    assert x.processes.ranks() == [0, 1, 2, 3] and x.names == ("c",)
    assert dm(c=slice(None, None, 2)).processes.ranks() == list(range(0, 24, 2))
    assert dm(b=2, c=3).processes.ranks() == [11, 23]

    dm = mock_mesh(hosts=60, gpus=24, trace=False)[0].rename(hosts="host", gpus="gpu")
    dm2 = dm.split(host=("dp", "pp"), gpu=("tp",), pp=4)
    assert dm2.names == ("dp", "pp", "tp")
    assert list(dm2.processes.sizes) == [15, 4, 24]
    assert list(dm2.processes.strides) == [4 * 24, 24, 1]
    dm3 = dm.rename(host="dp", gpu="tp")
    assert dm3.names == ("dp", "tp") and list(dm3.processes.strides) == list(dm.processes.strides)
    assert list(dm.split(host=("dp", "pp"), gpu=("tp",), dp=4).processes.sizes) == [4, 15, 24]
    assert list(dm.split(host=("dp", "pp"), dp=60).processes.sizes) == [60, 1, 24]
    assert list(dm.split(host=("dp", "pp"), pp=60).processes.sizes) == [1, 60, 24]
    assert dm.rename(host="dp").names == ("dp", "gpu")
    for kw, msg in (({"host": ("dp", "pp")}, "Cannot infer size"),
                    ({"host": ("dp", "pp"), "pp": 4, "ddp": 3}, "unused size constraints"),
                    ({"host": ("dp", "pp"), "gpu": ("pp",), "dp": 3}, "Duplicate dimension name"),
                    ({"host": ("dp", "pp"), "dp": 7}, "evenly divided")):
        with pytest.raises(ValueError, match=msg):
            dm.split(**kw)

    flat = dm.flatten("gpu")
    assert flat.names == ("gpu",)
    assert list(flat.processes.sizes) == [60 * 24] and list(flat.processes.strides) == [1]
    with pytest.raises(ValueError, match="cannot flatten sparse mesh"):
        dm(gpu=slice(None, None, 2)).flatten("bad_dim")
