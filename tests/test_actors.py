"""Actor API semantics: endpoints and adverbs, value meshes, ports, ordering, context.
Modelled on python/tests/test_python_actors.py of the reference."""
import asyncio
import pickle
import threading
import time

import pytest

from monarch_b200.actor import (Accumulator, Actor, ActorError, Channel, Future, Point, Port,
                                ValueMesh, as_endpoint, context, current_rank, current_size,
                                endpoint, fake_in_process_host, get_or_spawn_controller,
                                local_proc_mesh, send, this_host, this_proc)


class Counter(Actor):
    def __init__(self, v: int):
        self.v = v

    @endpoint
    def incr(self):
        self.v += 1

    @endpoint
    def value(self) -> int:
        return self.v

    @endpoint
    async def value_async(self) -> int:
        await asyncio.sleep(0)
        return self.v

    def not_an_endpoint(self):
        return self.v * 100

    @endpoint
    def rank_info(self):
        return (current_rank().rank, dict(current_rank()), current_size(),
                context().actor_instance.rank.rank)


class Indirect(Actor):
    @endpoint
    def call_value(self, c: Counter):
        return c.value.choose().get()

    @endpoint
    def fan_in(self, c):
        return sum(v for _, v in c.value.call().get())


@pytest.fixture(scope="module")
def pm():
    m = local_proc_mesh(gpus=4)
    yield m
    m.stop().get()


def test_call_broadcast_choose_call_one(pm):
    c = pm.spawn("counter_a", Counter, 3)
    c.incr.broadcast()
    c.incr.broadcast()
    vm = c.value.call().get()
    assert isinstance(vm, ValueMesh) and vm.values() == [5, 5, 5, 5]
    assert c.value.choose().get() == 5
    assert c.slice(gpus=2).value.call_one().get() == 5
    with pytest.raises(ValueError, match="call_one"):
        c.value.call_one()
    assert c.value_async.call().get().values() == [5] * 4
    assert [f.get() for f in c.value.stream()] == [5] * 4


def test_value_mesh_items_and_points(pm):
    c = pm.spawn("counter_b", Counter, 1)
    vm = c.rank_info.call().get()
    for point, (cast_rank, coords, size, own_rank) in vm.items():
        assert isinstance(point, Point)
        assert point.rank == cast_rank == own_rank
        assert coords == dict(point) and size == {"hosts": 1, "gpus": 4}
    assert vm.item(hosts=0, gpus=3)[0] == 3
    assert str(Point(1, vm.extent)) == "{'hosts': 0/1, 'gpus': 1/4}"
    sub = c.slice(gpus=slice(2, 4)).rank_info.call().get()
    # the rank inside a cast is relative to the slice that was called
    assert [v[0] for v in sub.values()] == [0, 1]
    assert [v[3] for v in sub.values()] == [2, 3]
    assert [v[2] for v in sub.values()] == [{"hosts": 1, "gpus": 2}] * 2


def test_sends_are_ordered_per_sender(pm):
    c = pm.spawn("counter_c", Counter, 0)
    for _ in range(100):
        c.incr.broadcast()
    assert c.value.call().get().values() == [100] * 4
    one = c.slice(gpus=1)
    for _ in range(50):
        one.incr.broadcast()
    c.incr.broadcast()
    assert one.value.call_one().get() == 151


def test_actor_refs_travel_in_messages(pm):
    c = pm.spawn("counter_d", Counter, 7)
    ind = pm.spawn("indirect", Indirect)
    assert ind.call_value.call(c).get().values() == [7] * 4
    assert ind.slice(gpus=0).fan_in.call_one(c).get() == 28


def test_non_endpoint_attribute_and_as_endpoint(pm):
    c = pm.spawn("counter_e", Counter, 2)
    with pytest.raises(RuntimeError, match="not annotated as an endpoint"):
        c.not_an_endpoint.call()
    assert as_endpoint(c.not_an_endpoint).call().get().values() == [200] * 4
    with pytest.raises(TypeError):
        c.value.call(1, 2, 3)  # signature is checked at the call site


def test_ports_and_channels(pm):
    class Producer(Actor):
        @endpoint
        def produce(self, port: Port, n: int):
            for i in range(n):
                port.send((current_rank().rank, i))

        @endpoint(explicit_response_port=True)
        def explicit(self, port, x):
            port.send(x * 2)

    p = pm.spawn("producer", Producer)
    port, rx = Channel.open()
    p.produce.broadcast(port, 3)
    got = sorted(rx.recv().get(timeout=10) for _ in range(12))
    assert got == sorted((r, i) for r in range(4) for i in range(3))
    assert p.explicit.call(21).get().values() == [42] * 4
    port2, rx2 = Channel.open(once=True)
    send(p.explicit, (5,), {}, port=port2, selection="choose")
    assert rx2.recv().get(timeout=10) == 10
    assert pickle.loads(pickle.dumps(port))._port_id == port._port_id


def test_accumulator(pm):
    c = pm.spawn("counter_f", Counter, 10)
    acc = Accumulator(c.value, 0, lambda a, b: a + b)
    assert acc.accumulate().get() == 40


def test_future_timeout_and_await(pm):
    class Slow(Actor):
        @endpoint
        def nap(self, s):
            time.sleep(s)
            return s

    s = pm.spawn("slow", Slow)
    with pytest.raises(TimeoutError):
        s.slice(gpus=0).nap.call_one(0.5).get(timeout=0.05)

    async def main():
        return await s.slice(gpus=1).nap.call_one(0.01)

    assert asyncio.run(main()) == 0.01
    assert Future.ready(3).get() == 3


def test_one_message_at_a_time_but_actors_run_concurrently(pm):
    class Busy(Actor):
        def __init__(self):
            self.active = 0
            self.max_active = 0

        @endpoint
        def work(self):
            self.active += 1
            self.max_active = max(self.max_active, self.active)
            time.sleep(0.02)
            self.active -= 1
            return threading.get_ident()

        @endpoint
        def peak(self):
            return self.max_active

    b = pm.spawn("busy", Busy)
    futs = [b.work.call() for _ in range(3)]
    tids = [set(f.get().values()) for f in futs]
    assert b.peak.call().get().values() == [1] * 4
    assert len(tids[0]) == 4  # four actors, four threads


def test_endpoint_exception_reaches_caller_only(pm):
    class Faulty(Actor):
        @endpoint
        def boom(self):
            raise ValueError("kaboom")

        @endpoint
        def ok(self):
            return "fine"

    f = pm.spawn("faulty", Faulty)
    with pytest.raises(ActorError, match="kaboom") as ei:
        f.boom.call().get()
    assert isinstance(ei.value.exception, ValueError)
    assert "boom" in ei.value.actor_mesh_ref_frames
    assert f.ok.call().get().values() == ["fine"] * 4  # the actor survives


def test_spawn_on_slice_and_after_stop_rejected():
    m = fake_in_process_host().spawn_procs(per_host={"gpus": 2})
    with pytest.raises(NotImplementedError):
        m.slice(gpus=0).spawn("x", Counter, 0)
    with pytest.raises(ValueError):
        fake_in_process_host().spawn_procs(per_host={"hosts": 2})
    m.stop().get()
    with pytest.raises(RuntimeError, match="stopped"):
        m.spawn("y", Counter, 0)


def test_this_proc_and_controllers():
    c = this_proc().spawn("tp_counter", Counter, 9)
    assert c.value.call_one().get() == 9
    a = get_or_spawn_controller("the_one", Counter, 5).get()
    a.incr.broadcast()
    b = get_or_spawn_controller("the_one", Counter, 1000).get()
    assert b.value.call_one().get() == 6  # same singleton, constructor args of the first win


def test_sim_mesh_cast_tree_large():
    from monarch_b200.actor import sim_proc_mesh
    m = sim_proc_mesh(gpus=8, hosts=4, racks=2)
    c = m.spawn("many", Counter, 1)
    assert len(c) == 64 and sum(c.value.call().get().values()) == 64
    assert c.slice(racks=1, hosts=2).value.call().get().values() == [1] * 8
    m.stop().get()


def test_subprocess_mesh_end_to_end():
    m = this_host().spawn_procs(per_host={"gpus": 2})
    try:
        c = m.spawn("counter_proc", Counter, 11)
        c.incr.broadcast()
        vm = c.value.call().get(timeout=30)
        assert vm.values() == [12, 12] and vm.sizes == {"hosts": 1, "gpus": 2}

        class Pid(Actor):
            @endpoint
            def pid(self):
                import os
                return os.getpid()

        pids = m.spawn("pid", Pid).pid.call().get(timeout=30).values()
        import os
        assert len(set(pids)) == 2 and os.getpid() not in pids
    finally:
        m.stop().get()


def test_allocators_and_from_alloc():
    from monarch_b200.actor import ProcMesh
    from monarch_b200.actor.allocator import (AllocConstraints, AllocSpec, LocalAllocator,
                                              ProcessAllocator, RemoteAllocator,
                                              StaticRemoteAllocInitializer)

    class Who(Actor):
        @endpoint
        def pid(self) -> int:
            import os
            return os.getpid()

    import os
    spec = AllocSpec(AllocConstraints(), hosts=1, gpus=2)
    with pytest.raises(ValueError):
        AllocSpec(gpus=0)
    alloc = LocalAllocator().allocate(spec)
    pm = ProcMesh.from_alloc(alloc)
    try:
        assert pm.sizes == {"hosts": 1, "gpus": 2}
        assert set(pm.spawn("who", Who).pid.call().get().values()) == {os.getpid()}
        with pytest.raises(RuntimeError):
            ProcMesh.from_alloc(alloc)             # an alloc is used once
    finally:
        pm.stop().get()
    pm = ProcMesh.from_alloc(ProcessAllocator(env={"MB200_TEST_MARK": "1"}).allocate(spec))
    try:
        pids = pm.spawn("who", Who).pid.call().get(timeout=60).values()
        assert len(set(pids)) == 2 and os.getpid() not in pids
    finally:
        pm.stop().get()
    ra = RemoteAllocator("w", StaticRemoteAllocInitializer("tcp!127.0.0.1:1", "127.0.0.1:2"))
    a = ra.allocate(AllocSpec(hosts=2, gpus=4))
    assert a.params == {"hosts": ["127.0.0.1:1", "127.0.0.1:2"], "procs_per_host": 4}
    with pytest.raises(ValueError):
        ra.allocate(AllocSpec(hosts=3, gpus=1))


def _set_marks_before_anything_else():
    import os
    os.environ["CUDA_CACHE_PATH"] = "/tmp/cuda_cache_test"
    os.environ["CUDA_LAUNCH_BLOCKING"] = "1"


def test_setup_function_runs_in_every_proc_before_actors():
    """python/tests/test_env_before_cuda.py of the reference: ``from_alloc(alloc, setup=...)``
    and ``proc_mesh(setup=...)`` prepare the environment of the procs."""
    from monarch_b200.actor import ProcMesh, proc_mesh
    from monarch_b200.actor.allocator import AllocSpec, ProcessAllocator

    class Env(Actor):
        @endpoint
        def read(self, names):
            import os
            return {n: os.environ.get(n, "NOT_SET") for n in names}

    names = ["CUDA_CACHE_PATH", "CUDA_LAUNCH_BLOCKING"]
    want = {"CUDA_CACHE_PATH": "/tmp/cuda_cache_test", "CUDA_LAUNCH_BLOCKING": "1"}
    pm = ProcMesh.from_alloc(ProcessAllocator().allocate(AllocSpec(hosts=1, gpus=2)),
                             setup=_set_marks_before_anything_else)
    try:
        got = pm.spawn("env", Env).read.call(names).get(timeout=60)
        assert all(v == want for v in got.values()) and len(got) == 2
    finally:
        pm.stop().get()
    pm = proc_mesh(gpus=1, setup=_set_marks_before_anything_else)
    try:
        assert pm.spawn("env", Env).read.call_one(names).get(timeout=60) == want
    finally:
        pm.stop().get()
    pm = proc_mesh(gpus=1, hosts=2)            # two "hosts" laid out on this box
    try:
        assert pm.sizes == {"hosts": 2, "gpus": 1}
        assert len(pm.spawn("env", Env).read.call(names).get(timeout=60)) == 2
    finally:
        pm.stop().get()


def test_mesh_trait_implementor_keeps_its_shape():
    """python/tests/test_mesh_trait.py of the reference: the smallest implementor."""
    from monarch_b200.actor.shape import MeshTrait, Shape, Slice

    class Mesh(MeshTrait):
        def __init__(self, shape, values):
            self._shape = shape
            self._values = values

        def _new_with_shape(self, shape):
            return Mesh(shape, self._values)

        @property
        def _ndslice(self):
            return self._shape.ndslice

        @property
        def _labels(self):
            return self._shape.labels

    mesh = Mesh(Shape(["label0", "label1"], Slice(offset=0, sizes=[2, 3], strides=[3, 1])),
                [1, 2, 3, 4, 5, 6])
    assert len(mesh) == 6
    assert mesh.slice(label0=1)._ndslice.ranks() == [3, 4, 5]
    assert mesh.flatten("all").sizes == {"all": 6}


def test_many_client_threads_call_concurrently():
    """Calls issued from several threads of the client at once (they share the channel to
    every proc: the caller-side send path and the writer thread interleave) all get their
    own answers back."""
    import threading

    class Adder(Actor):
        @endpoint
        def add(self, a: int, b: int) -> int:
            return a + b + current_rank().rank

    pm = this_host().spawn_procs(per_host={"gpus": 4})
    try:
        m = pm.spawn("adders", Adder)
        m.add.call(0, 0).get(timeout=60)
        errors = []

        def worker(t):
            try:
                for i in range(150):
                    got = m.add.call(t * 1000, i).get(timeout=60).values()
                    assert got == [t * 1000 + i + r for r in range(4)], got
                    one = m.slice(gpus=i % 4).add.call_one(t, i).get(timeout=60)
                    assert one == t + i, one    # a slice of one: the rank inside the cast is 0
            except Exception as e:  # noqa: BLE001 - reported by the main thread
                errors.append(repr(e))

        threads = [threading.Thread(target=worker, args=(t,)) for t in range(6)]
        for th in threads:
            th.start()
        for th in threads:
            th.join(120)
        assert not errors, errors[:3]
        assert not any(th.is_alive() for th in threads)
    finally:
        pm.stop().get()


def test_replies_gathered_along_the_cast_tree(monkeypatch):
    """Forced on for a small mesh: results, exceptions and tensor payloads come back through
    the comm actors in batches and look exactly like direct replies."""
    import torch
    from monarch_b200.actor import actor_mesh as am

    class G(Actor):
        @endpoint
        def val(self, k: int):
            r = current_rank().rank
            return {"r": r, "t": torch.full((2000,), float(r + k))}    # 8 KB: travels as a part

        @endpoint
        def flaky(self) -> int:
            if current_rank().rank == 5:
                raise ValueError("rank five says no")
            return 1

        @endpoint(explicit_response_port=True)
        def twice(self, port, x):
            port.send(x)           # explicit ports stay direct: any number of sends is fine

    monkeypatch.setattr(am, "_GATHER_MIN", 2)
    pm = local_proc_mesh(gpus=20)
    try:
        g = pm.spawn("g", G)
        out = g.val.call(3).get(timeout=60)
        vals = out.values()
        assert [v["r"] for v in vals] == list(range(20))
        assert all(v["t"].shape == (2000,) and v["t"][0].item() == v["r"] + 3 for v in vals)
        # a slice: gathered too, ranks renumbered inside the cast
        sub = g.slice(gpus=slice(4, 12)).val.call(0).get(timeout=60).values()
        assert [v["r"] for v in sub] == list(range(8))
        with pytest.raises(ActorError, match="rank five says no"):
            g.flaky.call().get(timeout=60)
        assert g.twice.call(7).get(timeout=60).values() == [7] * 20
        assert g.val.call(1).get(timeout=60).item(gpus=19)["r"] == 19   # still healthy
    finally:
        pm.stop().get()


def test_async_endpoints_give_way_to_later_messages():
    """An async endpoint that is waiting does not block the actor: a later message is
    handled meanwhile (and can end the wait)."""
    class Waiter(Actor):
        def __init__(self):
            self.stop = False
            self.spins = 0

        @endpoint
        async def wait_until_told(self) -> int:
            while not self.stop:
                self.spins += 1
                await asyncio.sleep(0.01)
            return self.spins

        @endpoint
        async def tell(self) -> None:
            self.stop = True

    pm = this_host().spawn_procs(per_host={"gpus": 1})
    try:
        w = pm.spawn("waiter", Waiter)
        pending = w.wait_until_told.call()
        time.sleep(0.1)
        w.tell.call().get(timeout=20)          # goes through while the first call is waiting
        assert pending.get(timeout=20).values()[0] >= 1
    finally:
        pm.stop().get()


def test_sync_and_async_endpoints_share_one_thread():
    """Constructor, sync and async endpoints of an actor see the same thread-local state."""
    import threading

    class TLS(Actor):
        def __init__(self):
            self.local = threading.local()
            self.local.value = 0

        @endpoint
        def increment(self) -> None:
            self.local.value += 1

        @endpoint
        async def increment_async(self) -> None:
            self.local.value += 1

        @endpoint
        def get_value(self) -> int:
            return self.local.value

        @endpoint
        async def get_async(self) -> int:
            return self.local.value

        @endpoint
        async def boom(self) -> None:
            raise ValueError("async boom")

    pm = local_proc_mesh(gpus=1)
    try:
        a = pm.spawn("tls", TLS)
        a.increment.call_one().get(timeout=20)
        a.increment_async.call_one().get(timeout=20)
        a.increment.call_one().get(timeout=20)
        a.increment_async.call_one().get(timeout=20)
        assert a.get_value.call_one().get(timeout=20) == 4
        assert a.get_async.call_one().get(timeout=20) == 4
        with pytest.raises(ActorError, match="async boom"):
            a.boom.call_one().get(timeout=20)
        assert a.get_value.call_one().get(timeout=20) == 4     # still alive
        # without anybody to answer to, an async failure goes up the supervision tree
        mon = pm.monitor()
        a.boom.broadcast()
        ev = mon.get(timeout=20)
        assert ev.kind == "actor_failed" and "async boom" in ev.message
    finally:
        pm.stop().get()


def test_reference_behaviours_rank_strings_duplicates_and_lost_references():
    """Scenarios of the reference's actor test-suite (python/tests/test_python_actors.py:
    rank_size, rank_string, mesh_len, same_actor_twice, this_and_that,
    things_survive_losing_python_reference) on this package's API."""
    import gc
    import operator

    class RunIt(Actor):
        @endpoint
        def run(self, fn):
            return fn()

        @endpoint
        def rank_str(self) -> str:
            return str(current_rank())

    proc = fake_in_process_host().spawn_procs(per_host={"hosts": 1, "gpus": 2})
    r = proc.spawn("runit", RunIt)
    acc = Accumulator(r.run, 0, operator.add)
    assert acc.accumulate(lambda: current_rank()["gpus"]).get() == 1
    assert acc.accumulate(lambda: current_size()["gpus"]).get() == 4
    vm = r.rank_str.call().get().flatten("r")
    assert vm.slice(r=0).item() == "{'hosts': 0/1, 'gpus': 0/2}"
    assert vm.slice(r=1).item() == "{'hosts': 0/1, 'gpus': 1/2}"
    with pytest.raises(ValueError):
        fake_in_process_host().spawn_procs(per_host={"hosts": 2})      # a real conflict
    assert len(fake_in_process_host().spawn_procs(per_host={"gpus": 12}).spawn("s", RunIt)) == 12

    with pytest.raises(RuntimeError, match="an actor with name 'runit' has already been spawned"):
        proc.spawn("runit", RunIt)

    assert this_proc().spawn("counter7", Counter, 7).value.call_one().get() == 7

    kept = this_host().spawn_procs(per_host={"gpus": 1}).spawn("kept", Counter, 3).slice(gpus=0)
    gc.collect()             # the proc mesh object is gone; the actors are not
    assert kept.value.call_one().get(timeout=30) == 3


def test_log_streaming_windows_and_flushes():
    """Log lines of the procs reach the client, similar lines of one window are collapsed,
    a window closes on time by itself, and changing the options flushes what waits
    (python/tests/test_python_actors.py::test_actor_log_streaming,
    ::test_flush_on_disable_aggregation, ::test_adjust_aggregation_window of the reference)."""
    import io
    import time

    class Printer(Actor):
        @endpoint
        def say(self, what: str) -> bool:
            print(what, flush=True)
            return True

    def wait_for(buf, text, secs=10.0):
        deadline = time.time() + secs
        while text not in buf.getvalue() and time.time() < deadline:
            time.sleep(0.05)
        return buf.getvalue()

    pm = this_host().spawn_procs(per_host={"gpus": 2})
    try:
        p = pm.spawn("printer", Printer)
        pm.logging_option(stream_to_client=True, aggregate_window_sec=60).get()
        waiting = io.StringIO()
        pm._owner._log_aggregator.out = waiting
        p.say.call("has print streaming 7").get(timeout=30)
        time.sleep(1.0)
        assert waiting.getvalue() == ""                      # the window is still open
        pm.logging_option(stream_to_client=True, aggregate_window_sec=None).get()
        assert waiting.getvalue() == "[2 similar log lines] has print streaming 7\n"

        direct = io.StringIO()
        pm._owner._log_aggregator.out = direct
        p.say.call("immediate line").get(timeout=30)
        assert wait_for(direct, "immediate line\nimmediate line\n").count("immediate line") == 2

        pm.logging_option(stream_to_client=True, aggregate_window_sec=0.5).get()
        timed = io.StringIO()
        pm._owner._log_aggregator.out = timed
        p.say.call("timed line").get(timeout=30)
        assert "[2 similar log lines] timed line" in wait_for(timed, "timed line")

        pm.logging_option(stream_to_client=False).get()
        assert pm._owner._log_aggregator is None
        p.say.call("nobody listens").get(timeout=30)
    finally:
        pm.stop().get()


def test_stopped_actor_mesh_refuses_calls_and_ports_travel_as_arguments():
    """python/tests/test_python_actors.py::test_actor_mesh_stop,
    ::test_proc_mesh_stop_after_actor_mesh_stop, ::test_port_as_argument of the reference."""
    from monarch_b200.actor import Channel

    class Echo(Actor):
        @endpoint
        def say(self, what: str) -> str:
            return what

        @endpoint
        async def count_into(self, port) -> None:
            for i in range(100):
                port.send(i)

    pm = this_host().spawn_procs(per_host={"gpus": 2})
    try:
        first, second = pm.spawn("echo", Echo), pm.spawn("echo2", Echo)
        assert set(first.say.call("hello 1").get(timeout=30).values()) == {"hello 1"}
        first.stop().get(timeout=30)
        with pytest.raises(RuntimeError, match="has already been stopped"):
            first.say.call("hello again").get(timeout=5)
        with pytest.raises(RuntimeError, match="has already been stopped"):
            first.slice(gpus=0).say.call_one("hello again").get(timeout=5)
        assert set(second.say.call("hello 3").get(timeout=30).values()) == {"hello 3"}

        send, recv = Channel.open()
        second.slice(gpus=1).count_into.broadcast(send)
        assert [recv.recv().get(timeout=30) for _ in range(100)] == list(range(100))
    finally:
        pm.stop().get()              # stopping the procs after one of their actor meshes
