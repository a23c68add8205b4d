#!/usr/bin/env python
"""A tour of the actor API: actors and endpoints, meshes and adverbs, slicing, references in
messages, ports, supervision, and singleton controllers.  Every step checks what it shows, so
the file doubles as an acceptance test.

    python examples/getting_started.py

Parity: docs/source/examples/getting_started.py of the reference (the same tour, on this
package's API)."""
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200.actor import (Actor, ActorError, Channel, SupervisionError, current_rank,  # noqa: E402
                                endpoint, get_or_spawn_controller, this_host, this_proc)


# ---- 1. an actor is a Python object whose endpoints can be called from elsewhere ---------
class Counter(Actor):
    def __init__(self, initial: int):
        self.value = initial

    @endpoint
    def increment(self) -> None:
        self.value += 1

    @endpoint
    def get_value(self) -> int:
        return self.value


# ---- 2. actors that know about each other ------------------------------------------------
class Trainer(Actor):
    def __init__(self):
        self.rank = current_rank().rank
        self.loader = None
        self.seen = []

    @endpoint
    def attach(self, loaders) -> None:
        """Actor meshes travel in messages; keep the loader of the same rank."""
        self.loader = loaders.slice(gpus=self.rank)

    @endpoint
    def step(self, i: int) -> float:
        batch = self.loader.next_batch.call_one(i).get()
        self.seen.append(batch)
        return float(sum(batch)) / len(batch)


class DataLoader(Actor):
    def __init__(self):
        self.rank = current_rank().rank

    @endpoint
    def next_batch(self, i: int):
        return [self.rank * 100 + i + k for k in range(4)]


# ---- 3. failures ------------------------------------------------------------------------
class Flaky(Actor):
    @endpoint
    def ok(self) -> int:
        return 1

    @endpoint
    def fail(self, msg: str) -> None:
        raise ValueError(msg)


class Registry(Actor):
    """A singleton controller: whoever asks first spawns it, everyone else gets the same."""

    def __init__(self):
        self.names = []

    @endpoint
    def register(self, name: str) -> int:
        self.names.append(name)
        return len(self.names)


def run():
    out = {}

    # in the caller's own process: call_one sends one message and returns a Future
    local = this_proc().spawn("local_counter", Counter, 0)
    local.increment.call_one().get()
    out["local_value"] = local.get_value.call_one().get()
    assert out["local_value"] == 1

    # a mesh of processes, one actor per process; messages go to all of them at once
    procs = this_host().spawn_procs(per_host={"gpus": 4})
    try:
        counters = procs.spawn("counters", Counter, 0)
        counters.increment.broadcast()                       # fire and forget, in send order
        counters.slice(gpus=slice(0, 2)).increment.broadcast()   # only gpus 0 and 1
        values = counters.get_value.call().get()             # a ValueMesh: one value per actor
        out["values"] = [v for _, v in values.items()]
        assert out["values"] == [2, 2, 1, 1]
        assert values.item(gpus=3) == 1
        out["chosen"] = counters.get_value.choose().get()    # any one of them
        out["streamed"] = sorted(f.get() for f in counters.get_value.stream())
        assert out["streamed"] == [1, 1, 2, 2]

        # references in messages: trainers talk to their data loaders directly
        trainers = procs.spawn("trainers", Trainer)
        loaders = procs.spawn("loaders", DataLoader)
        trainers.attach.call(loaders).get()
        means = trainers.step.call(5).get()
        out["means"] = [m for _, m in means.items()]
        assert out["means"] == [r * 100 + 5 + 1.5 for r in range(4)]

        # ports: a stream of values back to whoever holds the receiving end
        port, rx = Channel.open()

        class Reporter(Actor):
            @endpoint
            def report(self, p, n: int) -> None:
                for i in range(n):
                    p.send((current_rank().rank, i))

        procs.spawn("reporters", Reporter).report.broadcast(port, 2)
        out["reports"] = sorted(rx.recv().get(timeout=10) for _ in range(8))
        assert out["reports"] == [(r, i) for r in range(4) for i in range(2)]

        # an exception in a called endpoint goes to the caller; the actor lives on
        flaky = procs.spawn("flaky", Flaky)
        try:
            flaky.fail.call("caller sees this").get()
            raise AssertionError("expected an ActorError")
        except ActorError as e:
            out["caller_error"] = "caller sees this" in str(e)
        assert flaky.ok.call().get().values() == [1] * 4

        # without anybody to answer to, the failure goes up the supervision tree: the actor
        # mesh becomes unhealthy and the proc mesh's monitor reports it
        monitor = procs.monitor()
        flaky.fail.broadcast("nobody to tell")
        event = monitor.get(timeout=20)
        out["supervision_event"] = event.kind
        assert event.kind == "actor_failed" and "nobody to tell" in event.message
        deadline = time.time() + 10
        while True:
            try:
                flaky.ok.call().get(timeout=5)
                assert time.time() < deadline, "the failed mesh still answers"
                time.sleep(0.05)
            except SupervisionError:
                break
        assert counters.get_value.call().get().values() == [2, 2, 1, 1]   # others unaffected

        # singleton controllers by name
        reg = get_or_spawn_controller("registry", Registry).get()
        reg.register.call_one("a").get()
        again = get_or_spawn_controller("registry", Registry).get()
        out["registered"] = again.register.call_one("b").get()
        assert out["registered"] == 2
    finally:
        procs.stop().get()
    return out


if __name__ == "__main__":
    for k, v in run().items():
        print(f"{k}: {v}")
