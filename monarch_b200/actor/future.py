"""Futures returned by endpoint adverbs.

Parity: python/monarch/_src/actor/future.py (``.get(timeout)`` from synchronous code,
``await`` from coroutines, ``.result()`` / ``.exception()``).  The blocking wait happens
in native code with the GIL released, so a simple message round-trip needs no event loop.
"""
from __future__ import annotations

import asyncio
import threading
from typing import Any, Callable, Generic, Optional, TypeVar

R = TypeVar("R")
_UNSET = object()


class Future(Generic[R]):
    """Wraps a blocking ``impl(timeout_seconds | None) -> R``; the result (or exception)
    is computed once and cached."""

    def __init__(self, impl: Optional[Callable[[Optional[float]], R]] = None, *,
                 coro=None):
        if impl is None and coro is not None:
            def impl(timeout, _coro=coro):  # run a coroutine to completion on a private loop
                async def _with_timeout():
                    return await asyncio.wait_for(_coro, timeout)
                return asyncio.run(_with_timeout())
        self._impl = impl
        self._value: Any = _UNSET
        self._exc: Optional[BaseException] = None
        self._lock = threading.Lock()

    @staticmethod
    def ready(value: R) -> "Future[R]":
        f: Future[R] = Future(lambda timeout: value)
        f._value = value
        return f

    def _run(self, timeout: Optional[float]) -> None:
        with self._lock:
            if self._value is not _UNSET or self._exc is not None:
                return
            try:
                self._value = self._impl(timeout)
            except TimeoutError:
                raise
            except BaseException as e:  # noqa: BLE001 - cached and re-raised to every waiter
                self._exc = e

    def get(self, timeout: Optional[float] = None) -> R:
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

    def __await__(self):
        loop = asyncio.get_event_loop()
        return loop.run_in_executor(None, self.get).__await__()

    def then(self, fn: Callable[[R], Any]) -> "Future":
        return Future(lambda timeout: fn(self.get(timeout)))
