"""CUDA-event timers with statistics (see package docstring for parity notes)."""
from __future__ import annotations

import math
import threading
import time
from contextlib import contextmanager
from typing import Dict, List, Optional

import torch


class CudaTimer:
    """One named timer.  ``start()``/``stop()`` record CUDA events on the current stream
    (nothing blocks); elapsed times are read lazily, once the events have completed."""

    def __init__(self, name: str = "default", use_cuda: Optional[bool] = None):
        self.name = name
        self.use_cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        self._pending: List[tuple] = []
        self._times_ms: List[float] = []
        self._t0 = None

    def start(self) -> None:
        if self._t0 is not None:
            raise RuntimeError(f"timer {self.name!r} is already running")
        if self.use_cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._t0 = e
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> None:
        if self._t0 is None:
            raise RuntimeError(f"timer {self.name!r} was not started")
        if self.use_cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._pending.append((self._t0, e))
        else:
            self._times_ms.append((time.perf_counter() - self._t0) * 1e3)
        self._t0 = None

    def _collect(self, block: bool) -> None:
        rest = []
        for a, b in self._pending:
            if block:
                b.synchronize()
            if b.query():
                self._times_ms.append(a.elapsed_time(b))
            else:
                rest.append((a, b))
        self._pending = rest

    def times_ms(self, block: bool = True) -> List[float]:
        self._collect(block)
        return list(self._times_ms)

    def latest_ms(self) -> float:
        t = self.times_ms()
        if not t:
            raise RuntimeError(f"timer {self.name!r} has no measurement")
        return t[-1]

    def summary(self) -> Dict[str, float]:
        t = self.times_ms()
        if not t:
            return {"count": 0}
        mean = sum(t) / len(t)
        var = sum((x - mean) ** 2 for x in t) / len(t)
        return {"count": len(t), "mean_ms": mean, "std_ms": math.sqrt(var), "min_ms": min(t),
                "max_ms": max(t), "total_ms": sum(t)}

    def reset(self) -> None:
        self._pending.clear()
        self._times_ms.clear()
        self._t0 = None

    @contextmanager
    def time(self):
        self.start()
        try:
            yield self
        finally:
            self.stop()


class ExecutionTimer:
    """Process-wide registry of named timers (thread-safe)."""
    _lock = threading.Lock()
    _timers: Dict[str, CudaTimer] = {}

    @classmethod
    def get(cls, name: str = "default") -> CudaTimer:
        with cls._lock:
            t = cls._timers.get(name)
            if t is None:
                t = cls._timers[name] = CudaTimer(name)
            return t

    @classmethod
    def start(cls, name: str = "default") -> None:
        cls.get(name).start()

    @classmethod
    def stop(cls, name: str = "default") -> None:
        cls.get(name).stop()

    @classmethod
    @contextmanager
    def time(cls, name: str = "default"):
        with cls.get(name).time() as t:
            yield t

    @classmethod
    def summary(cls) -> Dict[str, Dict[str, float]]:
        with cls._lock:
            names = list(cls._timers)
        return {n: cls.get(n).summary() for n in names}

    @classmethod
    def get_latest_measurement(cls, name: str = "default") -> float:
        return cls.get(name).latest_ms()

    @classmethod
    def reset(cls, name: Optional[str] = None) -> None:
        with cls._lock:
            if name is None:
                cls._timers.clear()
            else:
                cls._timers.pop(name, None)


# Function forms, usable as remote functions by path on a device mesh
def execution_timer_start(name: str = "default") -> None:
    ExecutionTimer.start(name)


def execution_timer_stop(name: str = "default") -> None:
    ExecutionTimer.stop(name)


def get_latest_timer_measurement(name: str = "default") -> torch.Tensor:
    return torch.tensor(ExecutionTimer.get_latest_measurement(name), dtype=torch.float64)


def get_execution_timer_average_ms(name: str = "default") -> torch.Tensor:
    s = ExecutionTimer.get(name).summary()
    return torch.tensor(s.get("mean_ms", float("nan")), dtype=torch.float64)
