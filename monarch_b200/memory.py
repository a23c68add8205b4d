"""CUDA allocator history and snapshots on the workers of a device mesh.

Parity: python/monarch/memory.py (``record_memory_history``, ``dump_memory_snapshot``:
remote wrappers over ``torch.cuda.memory._record_memory_history`` /
``_dump_snapshot``; one file per rank)."""
from __future__ import annotations

import os

import torch


def _record(enabled: bool = True, max_entries: int = 100000) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(enabled="all" if enabled else None,
                                                 max_entries=max_entries)


def _dump(dir_path: str) -> None:
    os.makedirs(dir_path, exist_ok=True)
    rank = int(os.environ.get("RANK", os.getpid()))
    path = os.path.join(dir_path, f"snapshot_rank{rank}.pickle")
    if torch.cuda.is_available():
        torch.cuda.memory._dump_snapshot(path)
    else:
        import pickle
        with open(path, "wb") as f:
            pickle.dump({"segments": [], "device_traces": [], "note": "no CUDA device"}, f)


def _stats() -> torch.Tensor:
    if not torch.cuda.is_available():
        return torch.zeros(3, dtype=torch.int64)
    return torch.tensor([torch.cuda.memory_allocated(), torch.cuda.memory_reserved(),
                         torch.cuda.max_memory_allocated()], dtype=torch.int64)


def _call(name, *args, propagate=None):
    from .tensor_engine import get_active_mesh, remote
    if get_active_mesh() is None:
        return globals()[name](*args)
    return remote(f"monarch_b200.memory.{name}", propagate=propagate)(*args)


def record_memory_history(enabled: bool = True, max_entries: int = 100000) -> None:
    _call("_record", enabled, max_entries)


def dump_memory_snapshot(dir_path: str = "memory_snapshots") -> None:
    _call("_dump", dir_path)


def memory_stats():
    """[allocated, reserved, peak allocated] bytes per worker (distributed int64 tensor)."""
    return _call("_stats", propagate=lambda: torch.empty(3, dtype=torch.int64))
