"""Remote profiling: ``torch.profiler`` sessions that run on every worker of the active
device mesh, each writing its own chrome trace, driven from the controller.

Parity: python/monarch/profiler.py:28-160 (``profile`` context manager mirroring
``torch.profiler.profile`` with per-rank trace files; ``record_function`` ranges that are
opened and closed on the workers).  Without an active mesh both degrade to the local
``torch.profiler`` objects.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

_SESSIONS: Dict[int, object] = {}
_RANGES: Dict[int, object] = {}
_NEXT = [0]


# ---- worker-side functions (called by path through the tensor engine) -------------
def _profiler_start(session: int, out_dir: str, record_shapes: bool, with_stack: bool,
                    profile_memory: bool) -> None:
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    p = torch.profiler.profile(activities=acts, record_shapes=record_shapes,
                               with_stack=with_stack, profile_memory=profile_memory)
    p.__enter__()
    _SESSIONS[session] = (p, out_dir)


def _profiler_step(session: int) -> None:
    s = _SESSIONS.get(session)
    if s is not None:
        s[0].step()


def _profiler_stop(session: int, rank_hint: int = -1) -> None:
    s = _SESSIONS.pop(session, None)
    if s is None:
        return
    p, out_dir = s
    p.__exit__(None, None, None)
    os.makedirs(out_dir, exist_ok=True)
    rank = rank_hint if rank_hint >= 0 else int(os.environ.get("RANK", os.getpid()))
    p.export_chrome_trace(os.path.join(out_dir, f"trace_rank{rank}_{os.getpid()}.json"))


def _range_push(rid: int, name: str) -> None:
    r = torch.profiler.record_function(name)
    r.__enter__()
    _RANGES[rid] = r


def _range_pop(rid: int) -> None:
    r = _RANGES.pop(rid, None)
    if r is not None:
        r.__exit__(None, None, None)


def _next_id() -> int:
    _NEXT[0] += 1
    return _NEXT[0]


def _remote(path: str):
    from .tensor_engine import get_active_mesh, remote
    if get_active_mesh() is None:
        return None
    return remote(f"monarch_b200.profiler.{path}", propagate=None)


class profile:
    """``with profile(out_dir="traces"): ...`` -- profiles the workers of the active device
    mesh (or this process when no mesh is active)."""

    def __init__(self, out_dir: str = "monarch_traces", record_shapes: bool = False,
                 with_stack: bool = False, profile_memory: bool = False):
        self.out_dir, self.opts = out_dir, (record_shapes, with_stack, profile_memory)
        self.id = _next_id()
        self._local = False

    def __enter__(self):
        r = _remote("_profiler_start")
        if r is None:
            self._local = True
            _profiler_start(self.id, self.out_dir, *self.opts)
        else:
            r(self.id, self.out_dir, *self.opts)
        return self

    def step(self):
        if self._local:
            _profiler_step(self.id)
        else:
            _remote("_profiler_step")(self.id)

    def __exit__(self, *exc):
        if self._local:
            _profiler_stop(self.id)
        else:
            _remote("_profiler_stop")(self.id)
        return False


class record_function:
    """Named range around work issued to the workers (or local work without a mesh)."""

    def __init__(self, name: str):
        self.name, self.id, self._local = name, _next_id(), False

    def __enter__(self):
        r = _remote("_range_push")
        if r is None:
            self._local = True
            _range_push(self.id, self.name)
        else:
            r(self.id, self.name)
        return self

    def __exit__(self, *exc):
        if self._local:
            _range_pop(self.id)
        else:
            _remote("_range_pop")(self.id)
        return False
