"""Tasks on the native runtime: ``PythonTask`` (a piece of work that has not started),
``Shared`` (a started one whose result any number of waiters can take), coroutines that
await them without an asyncio loop.

Parity: monarch_hyperactor/src/pytokio.rs:61-295 and its stub
python/monarch/_rust_bindings/monarch_hyperactor/pytokio.pyi (``PythonTask.block_on``,
``spawn``, ``from_coroutine``, ``spawn_blocking``, ``with_timeout``, ``select_one``;
``Shared.block_on`` / ``task``; ``is_tokio_thread``).  The reference schedules Rust
futures on tokio; here work runs on the native task pool (``_native.task_spawn``) and
coroutines are resumed by completion callbacks, so a coroutine that waits parks no thread.
"""
from __future__ import annotations

import threading
from typing import Any, Callable, Coroutine, Generic, Optional, Sequence, Tuple, TypeVar

from .. import _native as N

T = TypeVar("T")


def is_tokio_thread() -> bool:
    """True on a thread of the native task pool (where ``block_on`` would tie up a worker
    that other tasks may need)."""
    return bool(N.is_task_thread())


class Shared(Generic[T]):
    """The result of a spawned task; can be awaited or blocked on any number of times."""

    def __init__(self, completion):
        self._c = completion

    def block_on(self, timeout: Optional[float] = None) -> T:
        if not self._c.wait(-1 if timeout is None else int(timeout * 1000)):
            raise TimeoutError("task did not finish in time")
        if self._c.failed():
            raise self._c.value()
        return self._c.value()

    def done(self) -> bool:
        return self._c.done()

    def task(self) -> "PythonTask[T]":
        """A one-use task that waits for this result (for ``with_timeout`` / ``select_one``)."""
        return PythonTask(_shared=self)

    def __await__(self):
        # awaited from a coroutine driven by PythonTask.from_coroutine: hand the driver the
        # completion to continue from; from asyncio: bridge through the running loop
        if _driving.active:
            value = yield self
            return value
        return (yield from self._await_asyncio().__await__())

    async def _await_asyncio(self) -> T:
        import asyncio
        loop = asyncio.get_running_loop()
        afut = loop.create_future()
        c = self._c

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


class _Driving(threading.local):
    active = False


_driving = _Driving()


class _CoroutineRunner:
    """Steps a coroutine whose awaits yield :class:`Shared` objects: each step runs on the
    task pool, and the next one is scheduled by the awaited completion's callback."""

    def __init__(self, coro: Coroutine, completion):
        self.coro, self.completion = coro, completion

    def start(self) -> None:
        N.task_spawn(lambda: self._step(None, None))

    def _step(self, value, exc) -> None:
        _driving.active = True
        try:
            try:
                awaited = self.coro.throw(exc) if exc is not None else self.coro.send(value)
            except StopIteration as s:
                self.completion.set_result(s.value)
                return
            except BaseException as e:  # noqa: BLE001 - the task's failure
                self.completion.set_exception(e)
                return
        finally:
            _driving.active = False
        if isinstance(awaited, PythonTask):
            awaited = awaited.spawn()
        if not isinstance(awaited, Shared):
            self.completion.set_exception(TypeError(
                f"a pytokio coroutine awaited {type(awaited).__name__}; it may only await "
                "PythonTask / Shared objects"))
            return
        c = awaited._c

        def resume():
            if c.failed():
                N.task_spawn(lambda: self._step(None, c.value()))
            else:
                N.task_spawn(lambda: self._step(c.value(), None))
        c.add_done_callback(resume)


class PythonTask(Generic[T]):
    """Work that runs when it is spawned or blocked on (once)."""

    def __init__(self, fn: Optional[Callable[[], T]] = None, *, _coro=None, _shared=None,
                 _timeout: Optional[float] = None):
        self._fn, self._coro, self._shared, self._timeout = fn, _coro, _shared, _timeout
        self._used = False

    # ---- constructors
    @staticmethod
    def from_coroutine(coro: Coroutine[Any, Any, T]) -> "PythonTask[T]":
        return PythonTask(_coro=coro)

    @staticmethod
    def spawn_blocking(fn: Callable[[], T]) -> Shared[T]:
        """Run ``fn`` on a pool thread of its own (it may block, also on other tasks: the
        pool grows while all its threads are busy)."""
        return Shared(N.task_spawn(fn))

    # ---- running
    def spawn(self) -> Shared[T]:
        if self._used:
            raise RuntimeError("a PythonTask can be consumed once")
        self._used = True
        if self._shared is not None:
            inner = self._shared
        elif self._coro is not None:
            c = N.Completion()
            _CoroutineRunner(self._coro, c).start()
            inner = Shared(c)
        else:
            inner = Shared(N.task_spawn(self._fn))
        if self._timeout is None:
            return inner
        # a watcher completes the outer result with whichever comes first
        outer = N.Completion()
        seconds = self._timeout

        def watch():
            if inner._c.wait(int(seconds * 1000)):
                if inner._c.failed():
                    outer.set_exception(inner._c.value())
                else:
                    outer.set_result(inner._c.value())
            else:
                outer.set_exception(TimeoutError(f"task did not finish within {seconds} s"))
        N.task_spawn(watch)
        return Shared(outer)

    def block_on(self) -> T:
        """Run to completion and return the result (from a thread outside the pool)."""
        return self.spawn().block_on()

    def with_timeout(self, seconds: float) -> "PythonTask[T]":
        if self._used:
            raise RuntimeError("a PythonTask can be consumed once")
        self._used = True
        return PythonTask(self._fn, _coro=self._coro, _shared=self._shared, _timeout=seconds)

    @staticmethod
    def select_one(tasks: "Sequence[PythonTask[T]]") -> "PythonTask[Tuple[T, int]]":
        """A task that runs ``tasks`` concurrently and yields ``(result, index)`` of the
        first to finish."""
        def run():
            shared = [t.spawn() for t in tasks]
            idx = N.wait_any([s._c for s in shared], -1)
            return shared[idx].block_on(), idx
        return PythonTask(run)

    def __await__(self):
        return self.spawn().__await__()
