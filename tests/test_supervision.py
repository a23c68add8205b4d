"""Failure detection, all injected on the host: endpoint exceptions without a response
port, procs that exit or are killed, bootstrap failures, undeliverable messages.
Modelled on python/tests/test_actor_error.py of the reference."""
import os
import time

import pytest

from monarch_b200 import _native as N
from monarch_b200.actor import (Actor, ActorError, SupervisionError, endpoint, local_proc_mesh,
                                this_host)


class Worker(Actor):
    def __init__(self):
        self.n = 0

    @endpoint
    def ok(self):
        self.n += 1
        return self.n

    @endpoint
    def fail(self, msg="bad"):
        raise RuntimeError(msg)

    @endpoint
    def exit_now(self, code=3):
        os._exit(code)

    @endpoint
    def hang(self, s):
        time.sleep(s)
        return "woke"

    @endpoint
    def echo(self, x):
        return repr(type(x))


class BadInit(Actor):
    def __init__(self):
        raise ValueError("constructor exploded")

    @endpoint
    def ok(self):
        return 1


def _wait_unhealthy(mesh, timeout=10.0):
    deadline = time.time() + timeout
    while time.time() < deadline:
        try:
            mesh._raise_if_unhealthy()
        except SupervisionError:
            return
        time.sleep(0.01)
    raise AssertionError("mesh did not become unhealthy")


def test_exception_with_port_keeps_actor_alive():
    pm = local_proc_mesh(gpus=2)
    w = pm.spawn("w", Worker)
    with pytest.raises(ActorError, match="bad"):
        w.fail.call().get()
    assert w.ok.call().get().values() == [1, 1]
    pm.stop().get()


def test_broadcast_exception_crashes_actor_and_poisons_mesh():
    pm = local_proc_mesh(gpus=2)
    w = pm.spawn("w", Worker)
    other = pm.spawn("other", Worker)
    mon = pm.monitor()
    w.fail.broadcast("fatal one")
    ev = mon.get(timeout=10)
    assert ev.kind == "actor_failed" and "fatal one" in ev.message and ".w[" in ev.actor_id
    _wait_unhealthy(w)
    with pytest.raises(SupervisionError, match="fatal one"):
        w.ok.call().get()
    # slices inherit the failure of their parent mesh
    with pytest.raises(SupervisionError):
        w.slice(gpus=0).ok.call_one().get()
    # an unrelated actor mesh on the same procs keeps working
    assert other.ok.call().get().values() == [1, 1]
    pm.stop().get()


def test_constructor_failure_surfaces_through_supervision():
    pm = local_proc_mesh(gpus=2)
    b = pm.spawn("bad", BadInit)
    _wait_unhealthy(b)
    with pytest.raises(SupervisionError, match="constructor exploded"):
        b.ok.call().get()
    pm.stop().get()


def test_pending_call_is_woken_by_proc_death():
    pm = this_host().spawn_procs(per_host={"gpus": 2})
    try:
        w = pm.spawn("w", Worker)
        assert w.ok.call().get(timeout=30).values() == [1, 1]
        pending = w.hang.call(30)
        time.sleep(0.2)
        pm._native.kill_rank(1, 9)   # host-side fault: SIGKILL of a CPU-only rank process
        t0 = time.time()
        with pytest.raises(SupervisionError, match="stopped"):
            pending.get(timeout=20)
        assert time.time() - t0 < 10
        with pytest.raises(SupervisionError):
            w.ok.call().get()
    finally:
        pm.stop().get()


def test_proc_exit_is_reported_with_reason():
    pm = this_host().spawn_procs(per_host={"gpus": 2})
    try:
        w = pm.spawn("w", Worker)
        mon = pm.monitor()
        w.slice(gpus=0).exit_now.broadcast(7)
        ev = mon.get(timeout=20)
        assert ev.kind == "proc_stopped" and ev.rank == 0 and "exited(7)" in ev.message
    finally:
        pm.stop().get()


def test_bootstrap_failure_is_an_allocation_error():
    with pytest.raises(RuntimeError, match="during allocation"):
        this_host().spawn_procs(per_host={"gpus": 2},
                                env={"MONARCH_ERROR_DURING_BOOTSTRAP_FOR_TESTING": "1"})


def test_undeliverable_message_fails_the_sender_by_default():
    proc = N.Proc.local("undeliv_test", 0)
    events = []
    sup = proc.attach("sup")
    port_id, rx = sup.open_port()
    proc.set_supervision_coordinator(port_id)

    def handler(inst, env):
        inst.send("undeliv_test[0].nobody[0][0]", b"hello", {}, [])

    a = proc.spawn("sender", handler)
    kick = proc.attach("kick")
    kick.send(a.actor_id + "[0]", b"go", {}, [])
    env = rx.recv(5000)
    assert env is not None and env.headers["kind"] == "supervision"
    assert a.join(2000) and a.status == "failed" and "undeliverable" in a.failure
    proc.stop_all(500)


def test_supervision_bubbles_to_parent_unless_handled():
    proc = N.Proc.local("tree_test", 0)
    sup = proc.attach("sup")
    port_id, rx = sup.open_port()
    proc.set_supervision_coordinator(port_id)
    seen = []

    def parent_handles(inst, actor_id, status, message):
        seen.append((actor_id, message))
        return True

    def crash(inst, env):
        raise RuntimeError("child crashed")

    kick = proc.attach("kick")
    parent = proc.spawn("parent", lambda i, e: None, on_supervision=parent_handles)
    child = proc.spawn("child", crash, parent=parent)
    kick.send(child.actor_id + "[0]", b"x", {}, [])
    assert child.join(2000) and child.status == "failed"
    deadline = time.time() + 2
    while not seen and time.time() < deadline:
        time.sleep(0.01)
    assert seen and "child crashed" in seen[0][1] and parent.status != "failed"
    assert rx.recv(100) is None  # handled: nothing reaches the proc's coordinator

    parent2 = proc.spawn("parent2", lambda i, e: None)  # no handler: failure propagates
    child2 = proc.spawn("child2", crash, parent=parent2)
    kick.send(child2.actor_id + "[0]", b"x", {}, [])
    assert parent2.join(2000) and parent2.status == "failed"
    env = rx.recv(2000)
    assert env is not None and "parent2" in env.sender
    snap = {s["actor_id"]: s for s in proc.ledger_snapshot()}
    assert snap[child2.actor_id]["status"] == "failed"
    assert child2.actor_id in snap[parent2.actor_id]["children"]
    proc.stop_all(500)


class _BrokenPickle:
    def __init__(self, on_get: bool, on_set: bool):
        self.on_get, self.on_set = on_get, on_set

    def __getstate__(self):
        if self.on_get:
            raise RuntimeError("__getstate__ error")
        return {"on_get": self.on_get, "on_set": self.on_set}

    def __setstate__(self, state):
        if state["on_set"]:
            raise RuntimeError("__setstate__ error")
        self.__dict__.update(state)


def test_arguments_that_break_pickling():
    """An argument that cannot be pickled fails the call locally; one that cannot be
    unpickled on the far side comes back as an ActorError, and the actor lives on
    (python/tests/test_actor_error.py test_broken_pickle_class in the reference)."""
    pm = this_host().spawn_procs(per_host={"gpus": 2})
    try:
        w = pm.spawn("w", Worker)
        with pytest.raises(RuntimeError, match="__getstate__ error"):
            w.echo.call(_BrokenPickle(True, False))
        with pytest.raises(ActorError, match="__setstate__ error"):
            w.echo.call(_BrokenPickle(False, True)).get(timeout=30)
        with pytest.raises(ActorError, match="__setstate__ error"):
            w.slice(gpus=1).echo.call_one(_BrokenPickle(False, True)).get(timeout=30)
        assert w.ok.call().get(timeout=30).values() == [1, 1]      # nobody died
    finally:
        pm.stop().get()


def test_base_exceptions_take_the_actor_down():
    """A BaseException (not an Exception) in an endpoint is not an answer: the actor fails
    and the caller sees a supervision error (test_base_exception_handling in the reference)."""
    class Fatal(BaseException):
        pass

    class E(Actor):
        @endpoint
        def die(self):
            raise Fatal("beyond repair")

        @endpoint
        def check(self) -> int:
            return 1

    pm = local_proc_mesh(gpus=1)
    try:
        e = pm.spawn("e", E)
        with pytest.raises(SupervisionError):
            e.die.call_one().get(timeout=30)
        with pytest.raises(SupervisionError):
            e.check.call().get(timeout=30)
    finally:
        pm.stop().get()


def test_slices_without_the_failed_actor_stay_usable():
    """python/tests/test_actor_error.py::test_slice_supervision and
    ::test_mesh_slices_inherit_parent_errors of the reference."""
    import time

    class Fragile(Actor):
        @endpoint
        def fail(self):
            raise RuntimeError("simulated failure")

        @endpoint
        def check(self) -> str:
            return "this is a healthy check"

    class Sturdy(Actor):
        @endpoint
        def check(self) -> str:
            return "this is a healthy check"

    pm = this_host().spawn_procs(per_host={"gpus": 4})
    try:
        sturdy = pm.spawn("sturdy", Sturdy)
        fragile = pm.spawn("fragile", Fragile)
        upper, second, third = (fragile.slice(gpus=slice(2, 4)), fragile.slice(gpus=2),
                                fragile.slice(gpus=3))
        third.fail.broadcast()                  # no reply port: the failure is a crash
        deadline = time.time() + 20
        while time.time() < deadline:
            try:
                third.check.call().get(timeout=5)
                time.sleep(0.05)
            except SupervisionError:
                break
        for mesh in (fragile, third, upper):    # everything that contains the failed actor
            with pytest.raises(SupervisionError, match="unhealthy"):
                mesh.check.call().get(timeout=20)
        for mesh in (second, fragile.slice(gpus=1), sturdy):
            got = mesh.check.call().get(timeout=20)
            assert set(got.values()) == {"this is a healthy check"}
    finally:
        pm.stop().get()
