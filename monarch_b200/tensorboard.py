"""Remote scalar logging: a writer that lives on one worker of the mesh and receives
scalars computed on the mesh without a controller-side fetch.

Parity: python/monarch/tensorboard.py (``Tensorboard`` remote class whose ``log`` takes
distributed tensors and writes on rank 0).  Uses ``torch.utils.tensorboard`` when the
``tensorboard`` package is importable, else appends JSON lines ``{"tag","step","value"}``
to ``<log_dir>/scalars.jsonl`` (same call surface either way).
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

_WRITERS: Dict[str, object] = {}


class _JsonlWriter:
    def __init__(self, log_dir: str):
        os.makedirs(log_dir, exist_ok=True)
        self._f = open(os.path.join(log_dir, "scalars.jsonl"), "a", buffering=1)

    def add_scalar(self, tag, value, step):
        self._f.write(json.dumps({"tag": tag, "step": int(step), "value": float(value)}) + "\n")

    def flush(self):
        self._f.flush()

    def close(self):
        self._f.close()


def _writer(log_dir: str):
    w = _WRITERS.get(log_dir)
    if w is None:
        try:
            from torch.utils.tensorboard import SummaryWriter
            w = SummaryWriter(log_dir)
        except Exception:  # noqa: BLE001 - tensorboard is optional
            w = _JsonlWriter(log_dir)
        _WRITERS[log_dir] = w
    return w


def _log(log_dir: str, tag: str, step: int, value) -> None:
    """Worker-side: write one scalar (a Python number or a 0-d tensor)."""
    if isinstance(value, torch.Tensor):
        value = value.detach().float().mean().item()
    _writer(log_dir).add_scalar(tag, value, step)


def _flush(log_dir: str) -> None:
    w = _WRITERS.get(log_dir)
    if w is not None:
        w.flush()


def _close(log_dir: str) -> None:
    w = _WRITERS.pop(log_dir, None)
    if w is not None:
        w.close()


class Tensorboard:
    """``tb = Tensorboard("runs/x"); tb.log("loss", step, loss_tensor)``.  With an active
    device mesh the write happens on the first worker of the mesh (the tensor never
    travels to the controller); without one it happens locally."""

    def __init__(self, log_dir: str):
        self.log_dir = log_dir

    def _call(self, fn: str, *args):
        from .tensor_engine import get_active_mesh, remote
        mesh = get_active_mesh()
        if mesh is None:
            return globals()[fn](self.log_dir, *args)
        first = mesh.slice(**{l: 0 for l in mesh._labels})
        moved = [a.slice_mesh(**{l: 0 for l in mesh._labels})
                 if hasattr(a, "slice_mesh") else a for a in args]
        with first.activate():
            remote(f"monarch_b200.tensorboard.{fn}", propagate=None)(self.log_dir, *moved)

    def log(self, tag: str, step: int, value) -> None:
        self._call("_log", tag, step, value)

    def flush(self) -> None:
        self._call("_flush")

    def close(self) -> None:
        self._call("_close")
