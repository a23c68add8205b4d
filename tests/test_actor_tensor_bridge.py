"""Actor endpoints called with distributed tensors: every actor gets its proc's own shard
(`call`), results can stay on the workers (`rref`), constructor arguments may be distributed
tensors.  Scenarios of python/tests/test_tensor_engine.py of the reference
(actor_with_tensors, actor_tensor_ordering, rref_actor) plus error paths."""
import pytest
import torch

from monarch_b200 import tensor_engine as te
from monarch_b200.actor import Actor, ActorError, as_endpoint, current_rank, endpoint, this_host


class AddWithState(Actor):
    def __init__(self, state):
        self.state = state

    @endpoint
    def forward(self, x):
        return x + self.state

    @endpoint
    def kind(self, x) -> str:
        return type(x).__name__


class Counter(Actor):
    def __init__(self):
        self.c = 0

    @endpoint
    def incr(self, x) -> int:
        self.c += 1
        return self.c - 1


class Linear(Actor):
    def __init__(self, n: int, m: int):
        self.weight = torch.zeros((n, m))

    def forward(self, x):
        return x @ self.weight

    @endpoint(propagate="inspect")
    def update(self, w) -> None:
        self.weight += w

    @endpoint
    def scale_in_place(self, t) -> None:
        t.mul_(current_rank().rank + 2)      # the worker's own tensor: the change sticks

    @endpoint
    def broken(self, t) -> None:
        raise ValueError("endpoint says no")


@pytest.fixture(scope="module")
def pm():
    procs = this_host().spawn_procs(per_host={"gpus": 2})
    yield procs
    procs.stop().get()


def test_call_with_distributed_tensors_and_tensor_constructor_args(pm):
    with pm.activate():
        mesh = te.get_active_mesh()
        r = (mesh.rank("gpus") + 1).to(torch.float32)          # 1 on proc 0, 2 on proc 1
        adder = pm.spawn("adder", AddWithState, r * 10)        # each actor keeps its shard
        out = adder.forward.call(r).get(timeout=30)
        assert out.item(gpus=0).item() == 11 and out.item(gpus=1).item() == 22
        assert adder.kind.call(r).get(timeout=30).values() == ["Tensor", "Tensor"]
        # nested containers and plain values travel along
        assert adder.forward.call_one if True else None
        one = adder.slice(gpus=1).forward.call_one(r.slice_mesh(gpus=1)).get(timeout=30)
        assert one.item() == 22


def test_calls_with_and_without_tensors_keep_their_order(pm):
    with pm.activate():
        counter = pm.spawn("ordered", Counter)
        results = []
        for _ in range(5):
            results.append(counter.incr.call(torch.ones(())))      # through the tensor plane
            results.append(counter.incr.call(1))                   # plain message
        assert [f.get(timeout=30).item(gpus=0) for f in results] == list(range(10))


def test_rref_keeps_results_on_the_workers(pm):
    with pm.activate():
        lin = pm.spawn("linear", Linear, 3, 4)
        y = torch.ones((4, 3))
        fwd = as_endpoint(lin.forward, propagate=lambda x: torch.rand(4, 4))
        t = fwd.rref(y)
        assert isinstance(t, te.Tensor) and t.shape == (4, 4)
        assert te.inspect(t.sum()).item() == 0
        lin.update.rref(torch.ones((3, 4)))
        t = fwd.rref(y)
        assert te.inspect(t.sum(), gpus=1).item() == 3 * 4 * 4
        # an endpoint may change the worker's tensor in place
        v = torch.ones(5)
        lin.scale_in_place.call(v).get(timeout=30)
        assert te.inspect(v, gpus=0).tolist() == [2.0] * 5
        assert te.inspect(v, gpus=1).tolist() == [3.0] * 5


def test_failures_on_either_plane_are_reported(pm):
    def _fail_here(t):
        raise RuntimeError("tensor plane broke")

    with pm.activate():
        lin = pm.spawn("linear2", Linear, 2, 2)
        with pytest.raises(ActorError, match="endpoint says no"):
            lin.broken.call(torch.ones(2)).get(timeout=30)
        # a tensor argument that failed on the workers fails the call, not the actor
        bad = te.remote(_fail_here, propagate=lambda t: t)(torch.ones(2))
        with pytest.raises(ActorError, match="tensor plane broke"):
            lin.update.call(bad).get(timeout=30)
        # rref of a raising endpoint poisons the returned tensors
        boom = as_endpoint(lin.broken, propagate=lambda t: t).rref(torch.ones(2))
        with pytest.raises(te.RemoteException, match="endpoint says no"):
            te.inspect(boom)
        lin.update.call(torch.ones((2, 2))).get(timeout=30)           # still alive
    other = this_host().spawn_procs(per_host={"gpus": 2})
    try:
        with other.activate():
            foreign = torch.ones(2)
        with pytest.raises(ValueError, match="own procs"):
            lin.update.call(foreign)
    finally:
        other.stop().get()
