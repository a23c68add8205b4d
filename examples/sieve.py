#!/usr/bin/env python
"""Sieve of Eratosthenes as a chain of dynamically spawned actors.

Every filter actor holds one prime; a candidate that survives all filters reaches the end of
the chain, which reports it as a new prime and spawns the next filter.  Shows actors spawning
actors at run time and forwarding messages along references they hold.

    python examples/sieve.py [N_PRIMES]

Parity: hyperactor_mesh/examples/sieve.rs of the reference (re-created on this package's
Python actor API)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200.actor import Actor, Channel, endpoint, this_proc  # noqa: E402


class Filter(Actor):
    def __init__(self, prime: int):
        self.prime = prime
        self.next = None

    @endpoint
    def candidate(self, n: int, primes) -> None:
        """Drop multiples of this filter's prime, pass the rest down the chain; at the end
        of the chain the survivor is a prime and gets a filter of its own."""
        if n % self.prime == 0:
            return
        if self.next is None:
            primes.send(n)
            self.next = this_proc().spawn(f"filter_{n}", Filter, n)
        else:
            self.next.candidate.broadcast(n, primes)


def run(n_primes: int = 25):
    port, rx = Channel.open()
    head = this_proc().spawn("filter_2", Filter, 2)
    found = [2]
    n = 3
    while len(found) < n_primes:
        # feed in windows; everything sent is handled in order along the chain
        for c in range(n, n + 32):
            head.candidate.broadcast(c, port)
        n += 32
        while True:
            try:
                found.append(rx.recv().get(timeout=0.5))
            except TimeoutError:
                break
    return {"primes": sorted(found)[:n_primes]}


if __name__ == "__main__":
    out = run(int(sys.argv[1]) if len(sys.argv) > 1 else 25)
    print(out["primes"])
