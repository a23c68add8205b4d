"""Library modules on top of the tensor engine: timers, profiler ranges, scalar logging,
RNG state, memory stats, opaque objects/modules -- with and without a device mesh."""
import json
import os

import pytest
import torch

from monarch_b200 import tensor_engine as te
from monarch_b200.actor import this_host


@pytest.fixture(scope="module")
def dm():
    pm = this_host().spawn_procs(per_host={"gpus": 2})
    mesh = te.spawn_tensor_engine(pm, use_cuda=False)
    yield mesh
    mesh.exit()
    pm.stop().get()


def test_execution_timer_statistics():
    from monarch_b200.timer import CudaTimer, ExecutionTimer
    t = CudaTimer("t", use_cuda=False)
    for _ in range(3):
        with t.time():
            sum(range(1000))
    s = t.summary()
    assert s["count"] == 3 and s["min_ms"] <= s["mean_ms"] <= s["max_ms"]
    with pytest.raises(RuntimeError):
        t.stop()
    ExecutionTimer.reset()
    with ExecutionTimer.time("a"):
        pass
    assert ExecutionTimer.summary()["a"]["count"] == 1
    assert ExecutionTimer.get_latest_measurement("a") >= 0


def test_profiler_and_tensorboard_local(tmp_path):
    from monarch_b200.profiler import profile, record_function
    from monarch_b200.tensorboard import Tensorboard
    with profile(out_dir=str(tmp_path / "tr")):
        with record_function("blk"):
            torch.ones(8).sum()
    assert any(f.startswith("trace_rank") for f in os.listdir(tmp_path / "tr"))
    tb = Tensorboard(str(tmp_path / "tb"))
    tb.log("loss", 1, torch.tensor(2.5))
    tb.flush()
    tb.close()
    assert os.listdir(tmp_path / "tb")


def test_remote_libs_on_mesh(dm, tmp_path):
    from monarch_b200 import memory, random as mrandom
    from monarch_b200.tensorboard import Tensorboard
    from monarch_b200.timer import get_latest_timer_measurement
    with dm.activate():
        mrandom.manual_seed(123)
        st = mrandom.get_state()
        a = torch.rand(4)
        mrandom.set_state(st)
        b = torch.rand(4)
        assert torch.equal(te.inspect(a), te.inspect(b))
        assert te.inspect(memory.memory_stats()).shape == (3,)
        te.remote("monarch_b200.timer.execution_timer_start")("k")
        x = torch.ones(64, 64) @ torch.ones(64, 64)
        te.remote("monarch_b200.timer.execution_timer_stop")("k")
        ms = te.remote("monarch_b200.timer.get_latest_timer_measurement",
                       propagate=lambda n: torch.empty((), dtype=torch.float64))("k")
        assert te.inspect(ms).item() >= 0
        tb = Tensorboard(str(tmp_path / "tbm"))
        tb.log("x", 3, x.sum())
        tb.flush()
        te.inspect(x)  # drains the queue
    files = os.listdir(tmp_path / "tbm")
    assert files
    if "scalars.jsonl" in files:
        rec = json.loads(open(tmp_path / "tbm" / "scalars.jsonl").readline())
        assert rec == {"tag": "x", "step": 3, "value": 64.0 * 64 * 64}


def test_opaque_object_and_module(dm):
    from monarch_b200.opaque_module import OpaqueModule
    from monarch_b200.opaque_object import OpaqueObject
    with dm.activate():
        d = OpaqueObject("builtins.dict")
        d.call_method("__setitem__", None, "k", 5)
        got = d.call_method_on_shard_and_fetch("get", "k").get()
        assert got == 5
        torch.manual_seed(0)
        m = OpaqueModule("torch.nn.Linear", 4, 3)
        x = torch.ones(2, 4)
        y = m(x)
        assert y.shape == (2, 3)
        gx = m.backward(torch.ones(2, 3), x)
        assert gx.shape == (2, 4)
        w, b = m.parameters()
        assert torch.allclose(te.inspect(gx), te.inspect(w).sum(0).expand(2, 4))
        gw, gb = m.grads()
        assert te.inspect(gb).tolist() == [2.0, 2.0, 2.0]
        w0 = te.inspect(w).clone()
        m.sgd_step(0.5)
        w1 = te.inspect(m.parameters()[0])
        assert torch.allclose(w1, w0 - 0.5 * te.inspect(gw))


def test_cached_propagation_runs_once():
    from monarch_b200.cached_remote_function import cached_propagation
    calls = []

    def prop(x, k=1):
        calls.append(1)
        return x.new_empty(x.shape[0], k)

    p = cached_propagation(prop)
    assert p(torch.empty(3, 2), k=4).shape == (3, 4)
    assert p(torch.empty(3, 2), k=4).shape == (3, 4)
    assert p(torch.empty(5, 2), k=4).shape == (5, 4)
    assert len(calls) == 2


# ----------------------------------------------------------------------- remote classes --
from monarch_b200.remote_class import ControllerRemoteClass, WorkerRemoteClass  # noqa: E402


class _WorkerAccumulator(WorkerRemoteClass):
    def __init__(self, start):
        self.total = torch.tensor(float(start))

    def add(self, t, scale=1.0):
        self.total = self.total + t.sum() * scale

    def store_into(self, out):
        out.copy_(self.total)


class _Accumulator(ControllerRemoteClass):
    def __init__(self, start):
        super().__init__(_WorkerAccumulator, start)

    @ControllerRemoteClass.remote_method
    def add(self, t, scale=1.0):
        pass

    @ControllerRemoteClass.remote_method
    def store_into(self, out):
        pass


def test_remote_class_runs_methods_on_every_worker(dm):
    with dm.activate():
        acc = _Accumulator(10)
        x = (dm.rank("gpus") + 1).to(torch.float32) * torch.ones(4)
        acc.add(x)
        acc.add(x, scale=0.5)
        out = torch.zeros(())
        acc.store_into(out)
        assert te.inspect(out, gpus=0).item() == 10 + 4 * 1.5
        assert te.inspect(out, gpus=1).item() == 10 + 8 * 1.5
        acc.drop()
        with pytest.raises(Exception):
            _Accumulator.add(acc, x)     # dropped: no mesh to run on


def test_mesh_constructors():
    import monarch_b200 as m
    with m.local_mesh(gpus_per_host=2, use_cuda=False) as mesh:
        assert mesh.sizes == {"hosts": 1, "gpus": 2}
        with mesh.activate():
            x = mesh.rank("gpus").to(torch.float32) + torch.ones(2)
            assert te.inspect(x.reduce("gpus", "sum")).tolist() == [3.0, 3.0]
    sims = m.sim_mesh(n_meshes=2, hosts=1, gpus_per_host=4)
    assert len(sims) == 2 and sims[0].sizes == {"hosts": 1, "gpus": 4}
    with sims[1].activate():
        y = torch.ones(8, 8) @ torch.ones(8, 8)
        assert y.shape == (8, 8)
    assert sims[1].simulator is not None


# ------------------------------------------- objects made and named by worker functions --
class _WorkerFoo:
    def __init__(self, v):
        self.v = v

    def add(self, x):
        return x + self.v


def _make_foo(v):
    return _WorkerFoo(v)


def _setup_state():
    from monarch_b200.opaque_object import OpaqueRef
    torch.manual_seed(0)
    model = torch.nn.Linear(4, 2)
    data = [(torch.randn(8, 4), torch.randn(8, 2)) for _ in range(3)]
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    return [OpaqueRef(model), OpaqueRef(iter(data * 10)), OpaqueRef(torch.nn.MSELoss()),
            OpaqueRef(opt)]


def _iteration(model_ref, data_ref, crit_ref, opt_ref, pg):
    import torch.distributed as dist
    model, opt = model_ref.value, opt_ref.value
    x, y = next(data_ref.value)
    opt.zero_grad()
    loss = crit_ref.value(model(x), y)
    loss.backward()
    for p in model.parameters():
        dist.all_reduce(p.grad, group=pg)
    opt.step()
    return loss.detach().reshape(1)


def _create_ref():
    from monarch_b200.opaque_object import OpaqueRef
    return OpaqueRef(object())


def test_opaque_refs_made_by_worker_functions(dm):
    """python/tests/test_remote_functions.py of the reference: test_opaque_object,
    test_opaqueRef_setup_state_and_iteration, test_opaqueRef_key_deleted."""
    import gc
    from monarch_b200.opaque_object import OpaqueObject, OpaqueRef, opaque_method
    setup_state = te.remote(_setup_state, propagate=lambda: [OpaqueRef(None) for _ in range(4)])
    iteration = te.remote(_iteration, propagate=lambda m, d, c, o, pg: torch.zeros(1))
    create_ref = te.remote(_create_ref, propagate=lambda: OpaqueRef(None))
    alive = te.remote("monarch_b200.opaque_object._keyed_count",
                      propagate=lambda: torch.zeros((), dtype=torch.int64))

    class Foo(OpaqueObject):
        @opaque_method
        def add(self, x):          # the body is the shape rule
            return x + x

    with dm.activate():
        f = Foo(_make_foo, 4.0)
        assert te.inspect(f.add(torch.ones(3, 4))).eq(5.0).all().item()
        f.hi = 4                   # plain attributes stay on the controller object
        assert f.hi == 4

        pg = dm.process_group(tuple(dm._labels))
        model, loader, criterion, optimizer = setup_state()
        losses = [te.inspect(iteration(model, loader, criterion, optimizer, pg)).item()
                  for _ in range(5)]
        assert all(l > 0 for l in losses) and losses[3] < losses[0]
        with pytest.raises(RuntimeError, match="workers only"):
            model.value
        # the wrapped form calls methods of what the worker function made
        w = OpaqueObject(model)
        assert w.call_method_on_shard_and_fetch("extra_repr").get(timeout=30).startswith(
            "in_features=4")
        del model, loader, criterion, optimizer, w
        gc.collect()
        te.inspect(alive())
        base = te.inspect(alive()).item()
        ref = create_ref()
        assert te.inspect(alive()).item() == base + 1
        del ref
        gc.collect()
        assert te.inspect(alive()).item() == base      # the object went with its key


# ------------------------------------------------ an autograd.Function run on the workers --
class _BranchingFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y):
        ctx.save_for_backward(x)
        out0 = x * y if x.requires_grad else x + y
        return out0, y, torch.ones(4), 4

    @staticmethod
    def backward(ctx, dx1, dx2, dx3, dx4):
        return dx1, dx2


class _MultiplyAllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, pg):
        import torch.distributed as dist
        ctx.save_for_backward(x, y)
        ctx.my_property = True
        ctx.pg = pg
        z = x * y
        dist.all_reduce(z, group=pg)
        return z

    @staticmethod
    def backward(ctx, grad_output):
        import torch.distributed as dist
        x, y = ctx.saved_tensors
        assert ctx.my_property
        gx, gy = grad_output * y, grad_output * x
        dist.all_reduce(gx, group=ctx.pg)
        dist.all_reduce(gy, group=ctx.pg)
        return gx, gy, None


def test_remote_autograd_function_from_a_class(dm):
    """python/tests/test_remote_functions.py::test_remote_autograd_function of the reference,
    and its process-group-carrying function."""
    from monarch_b200.cached_remote_function import (RemoteAutogradFunction,
                                                     remote_autograd_function)
    fn = remote_autograd_function(_BranchingFunction)
    assert issubclass(fn, RemoteAutogradFunction) and fn.__name__ == "Remote__BranchingFunction"
    assert remote_autograd_function(fn) is fn
    with pytest.raises(TypeError):
        remote_autograd_function(dict)
    with dm.activate():
        x = torch.ones(1, requires_grad=True)
        y = torch.ones_like(x).requires_grad_(True)
        outs = fn.apply(x, y)
        assert outs[3] == 4 and outs[2].shape == (4,)
        first = te.inspect(outs[0])
        (outs[0] + outs[1]).sum().backward()
        gx, gy = te.inspect(x.grad), te.inspect(y.grad)
        x = x.detach()
        y.grad = None
        outs = fn.apply(x, y)                 # the worker sees that x wants no gradient now
        second = te.inspect(outs[0])
        (outs[0] + outs[1]).sum().backward()
        assert x.grad is None
        gy2 = te.inspect(y.grad)
    assert first.tolist() == [1.0] and second.tolist() == [2.0]
    assert gx.tolist() == [1.0] and gy.tolist() == [1.0] and gy2.tolist() == [1.0]

    mul = remote_autograd_function(_MultiplyAllReduce)
    with dm.activate():
        pg = dm.process_group(tuple(dm._labels))
        a = (torch.ones(3) * 2).requires_grad_(True)
        b = (torch.ones(3) * 3).requires_grad_(True)
        z = mul.apply(a, b, pg)
        z.sum().backward()
        zv, ga, gb = te.inspect(z), te.inspect(a.grad), te.inspect(b.grad)
    n = 2
    assert zv.tolist() == [6.0 * n] * 3
    assert ga.tolist() == [3.0 * n] * 3 and gb.tolist() == [2.0 * n] * 3


def test_opaque_module_in_the_controllers_autograd(dm):
    """python/tests/test_remote_functions.py::test_opaque_module and
    ::test_opaque_module_autograd of the reference."""
    from monarch_b200.opaque_module import OpaqueModule
    with dm.activate():
        linear = OpaqueModule("torch.nn.Linear", 3, 3)
        with torch.no_grad():
            for p in linear.parameters():
                p.zero_()                      # writes the workers' parameters
        out = linear.call_method("forward", lambda x: x.clone(), torch.rand(4, 3))
        assert te.inspect(out.sum()).item() == 0

        inp = torch.rand(3, 3, requires_grad=True)
        lin = OpaqueModule("torch.nn.Linear", 3, 3)
        w, b = lin.parameters()
        assert w.requires_grad and lin.parameters()[0] is w
        lin(inp).sum().backward()
        ig0, wg0, bg0 = te.inspect((inp.grad, w.grad, b.grad))
        inp.grad = w.grad = b.grad = None
        (inp @ w.T + b).sum().backward()       # the same computation written out
        ig1, wg1, bg1 = te.inspect((inp.grad, w.grad, b.grad))
        with torch.no_grad():
            y = lin(inp)                       # no graph is recorded without grad mode
        assert y.grad_fn is None
    assert torch.allclose(ig0, ig1) and torch.allclose(wg0, wg1) and torch.allclose(bg0, bg1)


def test_builtin_remote_functions(dm, tmp_path):
    """python/tests/builtins/test_random.py and test_log.py of the reference."""
    import logging
    from monarch_b200.builtins.log import log_remote, set_logging_level_remote
    from monarch_b200.builtins.random import (get_rng_state_all_cuda_remote,
                                              get_rng_state_remote, manual_seed_all_cuda_remote,
                                              manual_seed_cuda_remote, random_seed_remote,
                                              seed_remote, set_manual_seed_remote,
                                              set_rng_state_remote)
    with dm.activate():
        set_manual_seed_remote(12345)
        t1 = torch.rand(5, 5)
        set_manual_seed_remote(12345)
        t2 = torch.rand(5, 5)
        set_manual_seed_remote(12345, process_idx=1)
        t3 = torch.rand(5, 5)
        set_manual_seed_remote(12345, process_idx=dm.rank(dm._labels[-1]))   # one per worker
        t4 = torch.rand(5, 5)
        a, b, c = te.inspect((t1, t2, t3))
        per_rank = [te.inspect(t4, **{dm._labels[-1]: i}) for i in range(2)]
        assert torch.equal(a, b) and not torch.equal(a, c)
        assert torch.equal(per_rank[0], a) and torch.equal(per_rank[1], c)

        s1, s2 = get_rng_state_remote(), get_rng_state_remote()
        first = torch.rand(3, 3)
        second = torch.rand(3, 3)
        s3 = get_rng_state_remote()
        set_rng_state_remote(s1)
        third = torch.rand(3, 3)
        r = te.inspect((s1, s2, s3, first, second, third))
        assert torch.equal(r[0], r[1]) and not torch.equal(r[0], r[2])
        assert not torch.equal(r[3], r[4]) and torch.equal(r[3], r[5])

        random_seed_remote()
        u1 = torch.rand(5, 5)
        random_seed_remote()
        u2 = torch.rand(5, 5)
        seed_remote()
        u3 = torch.rand(5, 5)
        u = te.inspect((u1, u2, u3))
        assert not torch.equal(u[0], u[1]) and not torch.equal(u[1], u[2])

        manual_seed_cuda_remote(7)              # no CUDA here: these do nothing, and say so
        manual_seed_all_cuda_remote(7)          # by returning without an error
        assert get_rng_state_all_cuda_remote() == []

        set_logging_level_remote(logging.DEBUG)
        log_remote("value %s and %s", 1, "two")
        log_remote("quiet %d", 3, level=logging.DEBUG)
        log_remote("loud", level=logging.ERROR)
        te.inspect(torch.zeros(1))              # everything above has run
