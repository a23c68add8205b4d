"""Worker-side Python objects addressed from the controller.

Parity: python/monarch/opaque_object.py (``OpaqueObject``: constructed on every worker by
a resolvable constructor, methods called remotely with distributed tensors as
arguments), common/opaque_ref.py (``OpaqueRef``: a picklable handle), remote_class.py
(``ControllerRemoteClass`` / ``WorkerRemoteClass``: a controller proxy paired with a class
instantiated on the workers) and opaque_module.py (``OpaqueModule``).

The object table lives in each worker process; ids are assigned by the controller so all
workers agree on them.
"""
from __future__ import annotations

import importlib
import itertools
from typing import Any, Callable, Dict, Optional

import torch

_TABLE: Dict[int, Any] = {}
_ids = itertools.count(1)


def _resolve(path_or_fn):
    if callable(path_or_fn):
        return path_or_fn
    mod, _, name = path_or_fn.rpartition(".")
    return getattr(importlib.import_module(mod), name)


# ---- worker side ----------------------------------------------------------------------
def _construct(oid: int, ctor, *args, **kwargs) -> None:
    _TABLE[oid] = _resolve(ctor)(*args, **kwargs)


def _call_method(oid: int, method: str, *args, **kwargs):
    return getattr(_TABLE[oid], method)(*args, **kwargs)


def _get_attr(oid: int, name: str):
    return getattr(_TABLE[oid], name)


def _set_attr(oid: int, name: str, value) -> None:
    setattr(_TABLE[oid], name, value)


def _drop(oid: int) -> None:
    _TABLE.pop(oid, None)


def _remote(name: str, propagate=None):
    from .tensor_engine import remote
    return remote(f"monarch_b200.opaque_object.{name}", propagate=propagate)


# ---- controller side --------------------------------------------------------------------
class OpaqueRef:
    """Picklable name of a worker-side object."""

    def __init__(self, oid: Optional[int] = None):
        self.id = next(_ids) if oid is None else oid

    def __reduce__(self):
        return (OpaqueRef, (self.id,))

    def __repr__(self):
        return f"OpaqueRef({self.id})"

    def resolve(self):
        """Worker-side: the object itself."""
        return _TABLE[self.id]


class OpaqueObject:
    """``obj = OpaqueObject("pkg.mod.Class", *args)`` builds the object on every worker of
    the active mesh; ``obj.call_method(name, propagate, *args)`` runs a method there."""

    def __init__(self, constructor, *args, **kwargs):
        self._ref = OpaqueRef()
        from .tensor_engine import get_active_mesh
        self._mesh = get_active_mesh()
        if self._mesh is None:
            _construct(self._ref.id, constructor, *args, **kwargs)
        else:
            _remote("_construct")(self._ref.id, constructor, *args, **kwargs)

    @property
    def ref(self) -> OpaqueRef:
        return self._ref

    def call_method(self, method: str, propagate: Any = None, *args, **kwargs):
        if self._mesh is None:
            return _call_method(self._ref.id, method, *args, **kwargs)
        return _remote("_call_method", propagate)(self._ref.id, method, *args, **kwargs)

    def call_method_on_shard_and_fetch(self, method: str, *args, shard=None, **kwargs):
        from .tensor_engine import call_on_shard_and_fetch
        return call_on_shard_and_fetch("monarch_b200.opaque_object._call_method", self._ref.id,
                                       method, *args, shard=shard, **kwargs)

    def _set(self, name: str, value) -> None:
        if self._mesh is None:
            _set_attr(self._ref.id, name, value)
        else:
            _remote("_set_attr")(self._ref.id, name, value)

    def drop(self) -> None:
        if self._mesh is None:
            _drop(self._ref.id)
        else:
            with self._mesh.activate():
                _remote("_drop")(self._ref.id)


class ControllerRemoteClass:
    """Base of a controller-side proxy: ``super().__init__("pkg.WorkerClass", *args)``
    instantiates the paired worker class on every worker; ``self._remote_method(name,
    propagate)(*args)`` calls it.  Parity: python/monarch/remote_class.py."""

    def __init__(self, worker_class, *args, **kwargs):
        self._obj = OpaqueObject(worker_class, *args, **kwargs)

    @property
    def ref(self) -> OpaqueRef:
        return self._obj.ref

    def _remote_method(self, name: str, propagate: Any = None) -> Callable:
        return lambda *a, **k: self._obj.call_method(name, propagate, *a, **k)


class WorkerRemoteClass:
    """Base of the worker-side half; exists so that worker classes can be recognised and
    can find sibling objects by ref."""

    @staticmethod
    def lookup(ref: OpaqueRef):
        return _TABLE[ref.id]
