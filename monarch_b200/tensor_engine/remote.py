"""Remote functions and fetches for the tensor engine.

Parity: python/monarch/common/remote.py (``remote`` with ``propagate``: a callable run on
fake tensors, ``"inspect"`` to run the function on one shard and copy its metadata,
``"mocked"``/None for tensor-free results), fetch.py (``fetch_shard``, ``inspect``,
``show``), ``call_on_shard_and_fetch``, _coalescing.py (``coalescing``).
"""
from __future__ import annotations

import contextlib
import functools
from typing import Any, Callable, Optional

import torch

from ..actor import Future
from .device_mesh import (DeviceMesh, Tensor, _collect, _mesh_of, _propagation, _send_call,
                          _to_fake, get_active_mesh)
from .worker import Ref


def _resolve_spec(fn) -> tuple:
    if isinstance(fn, str):
        return ("path", fn)
    return ("pickle", fn)


class Remote:
    def __init__(self, fn, propagate=None):
        self._fn = fn
        self._propagate = propagate
        if callable(fn):
            functools.update_wrapper(self, fn)

    def _fake_outputs(self, args, kwargs, mesh: DeviceMesh):
        p = self._propagate
        if callable(p):
            with _propagation():
                return p(*_to_fake(args), **_to_fake(kwargs))
        if p == "inspect":
            # run the real function on one shard and copy the metadata of what comes back
            first = {l: 0 for l in mesh._labels}
            sample = call_on_shard_and_fetch(self, *args, shard=first, _raw=True, **kwargs).get()
            with _propagation():
                return torch.utils._pytree.tree_map(
                    lambda t: torch.empty(t.shape, dtype=t.dtype, device=t.device)
                    if isinstance(t, torch.Tensor) else t, sample)
        if p is None or p == "mocked":
            return None
        raise ValueError(f"unsupported propagate={p!r}")

    def __call__(self, *args, **kwargs):
        ts = []
        _collect(args, ts)
        _collect(kwargs, ts)
        mesh = _mesh_of(ts) if ts else get_active_mesh()
        if mesh is None:
            raise RuntimeError("no active device mesh")
        fake_out = self._fake_outputs(args, kwargs, mesh)
        return _send_call(_resolve_spec(self._fn), args, kwargs, fake_out, mesh)

    def call_on_shard_and_fetch(self, *args, shard=None, **kwargs) -> Future:
        return call_on_shard_and_fetch(self, *args, shard=shard, **kwargs)


def remote(fn=None, *, propagate=None):
    """``@remote(propagate=lambda x: x)`` marks ``fn`` to run on every worker of the mesh of
    its tensor arguments; results are distributed tensors shaped like ``propagate``'s."""
    if fn is None:
        return lambda f: Remote(f, propagate)
    return Remote(fn, propagate)


def _shard_mesh(mesh: DeviceMesh, shard) -> DeviceMesh:
    shard = dict(shard or {})
    for l in mesh._labels:
        shard.setdefault(l, 0)
    return mesh.slice(**shard)


def call_on_shard_and_fetch(rfn, *args, shard=None, _raw=False, **kwargs) -> Future:
    """Run ``rfn`` on a single shard and return its (tensor-containing) result locally."""
    ts = []
    _collect(args, ts)
    _collect(kwargs, ts)
    mesh = _mesh_of(ts) if ts else get_active_mesh()
    if mesh is None:
        raise RuntimeError("no active device mesh")
    sub = _shard_mesh(mesh, shard)
    from .device_mesh import _to_wire
    fn = rfn._fn if isinstance(rfn, Remote) else rfn
    tree = (_to_wire(args), _to_wire(kwargs))
    pre = ("pickle", _Apply(fn))
    f = mesh.client.fetch(sub, tree, pre)
    return Future(lambda t: f.get(t)[0])


class _Apply:
    def __init__(self, fn):
        self.fn = fn

    def __call__(self, tree):
        args, kwargs = tree
        fn = self.fn
        if isinstance(fn, str):
            from .worker import _resolve_function
            fn = _resolve_function(("path", fn))
        return fn(*args, **kwargs)


def fetch_shard(obj, shard=None, **kwargs) -> Future:
    """Fetch the value(s) of distributed tensors in ``obj`` from one shard (default: index
    0 of every dim; pick others with ``fetch_shard(t, host=1, gpu=0)``)."""
    shard = dict(shard or {}, **kwargs)
    return call_on_shard_and_fetch(_identity, obj, shard=shard)


def _identity(x):
    return x


def inspect(obj, shard=None, **kwargs):
    return fetch_shard(obj, shard, **kwargs).get()


def show(obj, shard=None, **kwargs):
    v = inspect(obj, shard, **kwargs)
    print(v)
    return v


@contextlib.contextmanager
def coalescing():
    """Batch every message issued inside the block into one cast per mesh."""
    mesh = get_active_mesh()
    if mesh is None:
        raise RuntimeError("coalescing() needs an active device mesh")
    with mesh.client.coalescing():
        yield
