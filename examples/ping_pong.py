#!/usr/bin/env python
"""Two actor meshes that talk to each other: the classic ping-pong, plus the dining
philosophers problem solved with message passing (a waiter actor grants chopsticks).

    python examples/ping_pong.py

Parity: docs/source/examples/ping_pong.py and hyperactor_mesh/examples/
dining_philosophers.rs of the reference (re-created on this package's actor API)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200.actor import Actor, current_rank, endpoint, local_proc_mesh, this_host  # noqa: E402


class Player(Actor):
    def __init__(self, name: str):
        self.name = name
        self.rank = current_rank().rank
        self.other = None
        self.hits = 0

    @endpoint
    def meet(self, other) -> None:
        self.other = other

    @endpoint
    def hit(self, ball: int, done) -> None:
        """Return the ball (fire and forget: an actor handles one message at a time, so a
        rally cannot be nested blocking calls) to the player of the same rank on the other
        side; the player who receives the ball at 0 reports on ``done``."""
        self.hits += 1
        if ball > 0:
            self.other.slice(gpus=self.rank).hit.broadcast(ball - 1, done)
        else:
            done.send((self.name, self.rank, self.hits))


class Waiter(Actor):
    """Grants both chopsticks or none: no deadlock, no two neighbours eat at once."""

    def __init__(self, n: int):
        self.free = [True] * n
        self.n = n
        self.max_eating = 0

    @endpoint
    def request(self, i: int) -> bool:
        l, r = i, (i + 1) % self.n
        if self.free[l] and self.free[r]:
            self.free[l] = self.free[r] = False
            self.max_eating = max(self.max_eating, sum(1 for f in self.free if not f) // 2)
            return True
        return False

    @endpoint
    def release(self, i: int) -> None:
        self.free[i] = self.free[(i + 1) % self.n] = True

    @endpoint
    def stats(self) -> int:
        return self.max_eating


class Philosopher(Actor):
    def __init__(self):
        self.i = current_rank().rank
        self.meals = 0

    @endpoint
    def dine(self, waiter, meals: int) -> int:
        import time
        while self.meals < meals:
            if waiter.request.call_one(self.i).get(timeout=30):
                self.meals += 1
                waiter.release.call_one(self.i).get(timeout=30)
            else:
                time.sleep(0.001)
        return self.meals


def run(in_process: bool = False, bounces: int = 6, philosophers: int = 5, meals: int = 3):
    mk = (lambda n: local_proc_mesh(gpus=n)) if in_process else \
        (lambda n: this_host().spawn_procs(per_host={"gpus": n}))
    a, b = mk(2), mk(2)
    try:
        ping = a.spawn("ping", Player, "ping")
        pong = b.spawn("pong", Player, "pong")
        ping.meet.call(pong).get(timeout=30)
        pong.meet.call(ping).get(timeout=30)
        from monarch_b200.actor import Channel
        port, rx = Channel.open()
        ping.hit.broadcast(bounces, port)
        ends = sorted(rx.recv().get(timeout=60) for _ in range(2))
        ping_hits = [e[2] for e in ends]
    finally:
        a.stop().get()
        b.stop().get()
    pm = mk(philosophers)
    wm = mk(1)
    try:
        waiter = wm.spawn("waiter", Waiter, philosophers)
        phil = pm.spawn("philosophers", Philosopher)
        ate = [v for _, v in phil.dine.call(waiter, meals).get(timeout=120).items()]
        max_eating = waiter.stats.call_one().get(timeout=30)
    finally:
        pm.stop().get()
        wm.stop().get()
    return {"ping_hits": ping_hits, "meals": ate, "max_eating_at_once": max_eating}


if __name__ == "__main__":
    print(run())
