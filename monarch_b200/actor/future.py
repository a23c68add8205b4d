"""Futures returned by endpoint adverbs.

Parity: python/monarch/_src/actor/future.py (``.get(timeout)`` from synchronous code,
``await`` from coroutines, ``.result()`` / ``.exception()``) over
monarch_hyperactor/src/pytokio.rs (shared tasks, ``with_timeout``, ``select_one``).

A future wraps a blocking ``impl(timeout_seconds | None) -> R`` whose wait happens in native
code with the GIL released, so a simple round trip from synchronous code needs no event
loop (the reference measured the event-loop path at about 4x the direct wait).  From a
coroutine, ``await`` integrates with the running asyncio loop without parking a thread per
pending future where the future knows how to be notified (``arm``: futures of port
receives are woken by the mailbox delivery itself); other futures run on the native task
pool and post their completion to the loop.
"""
from __future__ import annotations

import asyncio
import threading
import time
from typing import Any, Callable, Generic, List, Optional, Sequence, Tuple, TypeVar

R = TypeVar("R")
_UNSET = object()


class Future(Generic[R]):
    """The result (or exception) is computed once and cached; ``impl`` may be entered again
    after a ``TimeoutError`` and must then pick up where it stopped.

    ``arm(wake)``: optional; arranges for ``wake()`` to be called (from any thread) whenever
    progress may have become possible, e.g. a message arrived."""

    def __init__(self, impl: Optional[Callable[[Optional[float]], R]] = None, *,
                 coro=None, arm: Optional[Callable[[Optional[Callable[[], None]]], None]] = None):
        if impl is None and coro is not None:
            def impl(timeout, _coro=coro):  # run a coroutine to completion on a private loop
                async def _with_timeout():
                    return await asyncio.wait_for(_coro, timeout)
                return asyncio.run(_with_timeout())
        self._impl = impl
        self._arm = arm
        self._value: Any = _UNSET
        self._exc: Optional[BaseException] = None
        self._cond = threading.Condition()
        self._running = False

    @staticmethod
    def ready(value: R) -> "Future[R]":
        f: Future[R] = Future(lambda timeout: value)
        f._value = value
        return f

    def _run(self, timeout: Optional[float]) -> None:
        """Compute the result unless it is there already.  One thread at a time is inside
        ``impl``; others wait for it (no lock is held across the blocking wait itself)."""
        deadline = None if timeout is None else time.monotonic() + timeout
        with self._cond:
            while self._running:
                left = None if deadline is None else deadline - time.monotonic()
                if left is not None and left <= 0:
                    raise TimeoutError("timed out waiting for a future another thread is in")
                self._cond.wait(left)
            if self._value is not _UNSET or self._exc is not None:
                return
            self._running = True
        try:
            left = None if deadline is None else max(deadline - time.monotonic(), 0.0)
            value = self._impl(left)
            with self._cond:
                self._value = value
        except TimeoutError:
            raise
        except BaseException as e:  # noqa: BLE001 - cached and re-raised to every waiter
            with self._cond:
                self._exc = e
        finally:
            with self._cond:
                self._running = False
                self._cond.notify_all()

    def get(self, timeout: Optional[float] = None) -> R:
        if self._value is not _UNSET:        # settled: no lock needed to read it
            return self._value
        self._run(timeout)
        if self._exc is not None:
            raise self._exc
        return self._value

    def result(self, timeout: Optional[float] = None) -> R:
        return self.get(timeout)

    def exception(self, timeout: Optional[float] = None) -> Optional[BaseException]:
        try:
            self._run(timeout)
        except TimeoutError:
            raise
        return self._exc

    def done(self) -> bool:
        return self._value is not _UNSET or self._exc is not None

    # ------------------------------------------------------------------------ async
    def __await__(self):
        return self._await().__await__()

    async def _await(self) -> R:
        if self.done():
            return self.get(0)
        loop = asyncio.get_running_loop()
        if self._arm is not None:
            # event driven: poll without blocking, sleep until the producer says something
            # arrived (or a short interval passed: supervision failures surface in the poll)
            try:
                while True:
                    try:
                        return self.get(0)
                    except TimeoutError:
                        pass
                    ev = loop.create_future()

                    def wake(ev=ev):
                        try:
                            loop.call_soon_threadsafe(lambda: ev.done() or ev.set_result(None))
                        except RuntimeError:
                            pass       # the loop is gone
                    self._arm(wake)
                    try:               # something may have arrived before the wake was armed
                        return self.get(0)
                    except TimeoutError:
                        pass
                    try:
                        await asyncio.wait_for(ev, 0.25)
                    except asyncio.TimeoutError:
                        pass
            finally:
                self._arm(None)
        # no notification source: the blocking wait runs on the native task pool and posts
        # its outcome to this loop
        from .. import _native as N
        afut = loop.create_future()
        c = N.task_spawn(lambda: self.get(None))

        def post():
            def settle():
                if afut.done():
                    return
                if c.failed():
                    afut.set_exception(c.value())
                else:
                    afut.set_result(c.value())
            try:
                loop.call_soon_threadsafe(settle)
            except RuntimeError:
                pass
        c.add_done_callback(post)
        return await afut

    # ------------------------------------------------------------------ combinators
    def then(self, fn: Callable[[R], Any]) -> "Future":
        return Future(lambda timeout: fn(self.get(timeout)), arm=self._arm)

    def with_timeout(self, seconds: float) -> "Future[R]":
        """A future that raises ``TimeoutError`` unless this one finishes within ``seconds``
        of the first wait on it."""
        start: List[float] = []

        def impl(timeout):
            if not start:
                start.append(time.monotonic())
            left = seconds - (time.monotonic() - start[0])
            if left <= 0 and not self.done():
                try:
                    return self.get(0)
                except TimeoutError:
                    raise FutureTimeout(f"future did not finish within {seconds} s") from None
            budget = left if timeout is None else min(left, timeout)
            try:
                return self.get(max(budget, 0.0))
            except TimeoutError:
                if timeout is None or left <= timeout:
                    raise FutureTimeout(f"future did not finish within {seconds} s") from None
                raise
        return Future(impl, arm=self._arm)


class FutureTimeout(TimeoutError):
    """A ``with_timeout`` deadline passed."""


def select_one(futures: Sequence[Future], timeout: Optional[float] = None) -> Tuple[Any, int]:
    """Wait for the first of ``futures`` to finish; returns ``(value, index)`` (raises the
    winner's exception if it failed).  Futures that are already done win at once; the rest
    are waited on concurrently on the native task pool."""
    from .. import _native as N
    for i, f in enumerate(futures):
        if f.done():
            return f.get(0), i
    comps = [N.task_spawn(lambda f=f: f.exception(None)) for f in futures]
    idx = N.wait_any(comps, -1 if timeout is None else int(timeout * 1000))
    if idx < 0:
        raise TimeoutError("no future finished in time")
    return futures[idx].get(0), idx
