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

import functools
import importlib
import itertools
from typing import Any, Callable, Dict, Optional

import torch
from torch.utils.weak import WeakTensorKeyDictionary

_TABLE: Dict[int, Any] = {}
_ids = itertools.count(1)
# objects made by worker functions (``return OpaqueRef(model)``) are named by a key tensor:
# the controller holds it as a distributed tensor, so the name travels and is freed with the
# ordinary tensor references, and the object goes when its key does
_KEYED: WeakTensorKeyDictionary = WeakTensorKeyDictionary()
_key_counter = itertools.count(1)


def _resolve(path_or_fn):
    if callable(path_or_fn):
        return path_or_fn
    mod, _, name = path_or_fn.rpartition(".")
    return getattr(importlib.import_module(mod), name)


def _target(oid):
    return oid.value if isinstance(oid, OpaqueRef) else _TABLE[oid]


# ---- worker side ----------------------------------------------------------------------
def _construct(oid: int, ctor, *args, **kwargs) -> None:
    _TABLE[oid] = _resolve(ctor)(*args, **kwargs)


def _call_method(oid, method: str, *args, **kwargs):
    return getattr(_target(oid), method)(*args, **kwargs)


def _get_attr(oid, name: str):
    return getattr(_target(oid), name)


def _set_attr(oid, name: str, value) -> None:
    setattr(_target(oid), name, value)


def _drop(oid: int) -> None:
    _TABLE.pop(oid, None)


def _keyed_count() -> torch.Tensor:
    """How many worker-made objects are alive on this worker."""
    return torch.tensor(len(_KEYED), dtype=torch.int64)


def _remote(name: str, propagate=None):
    from .tensor_engine import remote
    return remote(f"monarch_b200.opaque_object.{name}", propagate=propagate)


# ---- controller side --------------------------------------------------------------------
class OpaqueRef:
    """Picklable name of a worker-side object.

    ``OpaqueRef(value)`` in a worker function (or in its propagation function, with
    ``None``) names ``value`` by a fresh key tensor; returned from a remote function it
    reaches the controller as an ``OpaqueRef`` whose key is a distributed tensor, and passed
    back into a remote function it gives ``ref.value`` again on the same worker
    (python/monarch/common/opaque_ref.py in the reference).  Refs of objects constructed
    from the controller (:class:`OpaqueObject`) carry a controller-assigned id instead."""

    _holds_tensors = True      # the tensor engine's argument/result walkers look inside

    def __init__(self, value: Any = None):
        self.id: Optional[int] = None
        self._key = torch.tensor(next(_key_counter), dtype=torch.int64)
        _KEYED[self._key] = value

    @classmethod
    def _of_id(cls, oid: int) -> "OpaqueRef":
        r = cls.__new__(cls)
        r.id, r._key = oid, None
        return r

    @classmethod
    def _of_key(cls, key) -> "OpaqueRef":
        r = cls.__new__(cls)
        r.id, r._key = None, key
        return r

    # subclasses degrade to a plain ref when sent to the workers
    def __reduce_ex__(self, protocol):
        if self._key is None:
            return (OpaqueRef._of_id, (self.id,))
        return (OpaqueRef._of_key, (self._key,))

    def __repr__(self):
        return f"OpaqueRef({self.id if self._key is None else self._key!r})"

    def _tensors(self) -> list:
        return [] if self._key is None else [self._key]

    def _rebuild(self, tensors: list) -> "OpaqueRef":
        return OpaqueRef._of_id(self.id) if self._key is None else OpaqueRef._of_key(tensors[0])

    def _local_key(self):
        from torch._subclasses.fake_tensor import FakeTensor
        k = self._key
        if isinstance(k, FakeTensor) or type(k).__name__ == "Ref" or hasattr(k, "mesh"):
            raise RuntimeError("the object behind an OpaqueRef exists on the workers only; use "
                               "it inside a remote function")
        return k

    @property
    def value(self) -> Any:
        """Worker-side: the object itself."""
        if self._key is None:
            return _TABLE[self.id]
        return _KEYED[self._local_key()]

    @value.setter
    def value(self, v: Any) -> None:
        if self._key is None:
            _TABLE[self.id] = v
        else:
            _KEYED[self._local_key()] = v

    def resolve(self):
        return self.value


def opaque_method(fn):
    """Declares a method of the worker object on an :class:`OpaqueObject` subclass; the body
    is the shape propagation rule (python/monarch/opaque_object.py:37-44).

        class Doubler(OpaqueObject):
            @opaque_method
            def add(self, x):
                return x + x
    """
    name = fn.__name__

    @functools.wraps(fn)
    def impl(self, *args, **kwargs):
        return self.call_method(name, lambda *a, **k: fn(self, *a, **k), *args, **kwargs)

    return impl


class OpaqueObject:
    """``obj = OpaqueObject("pkg.mod.Class", *args)`` builds the object on every worker of
    the active mesh; ``obj.call_method(name, propagate, *args)`` runs a method there
    (``propagate(*args)`` gives the shapes of what it returns).  ``OpaqueObject(ref)`` wraps an
    :class:`OpaqueRef` that a remote function returned."""

    def __init__(self, constructor, *args, **kwargs):
        from .tensor_engine import get_active_mesh
        self._mesh = get_active_mesh()
        if isinstance(constructor, OpaqueRef):     # wrap what a remote function returned
            self._ref = constructor
            return
        self._ref = OpaqueRef._of_id(next(_ids))
        if self._mesh is None:
            _construct(self._ref.id, constructor, *args, **kwargs)
        else:
            _remote("_construct")(self._ref.id, constructor, *args, **kwargs)

    @property
    def _handle(self):
        """What the worker functions are sent: the id, or the keyed ref itself."""
        return self._ref if self._ref._key is not None else self._ref.id

    @property
    def ref(self) -> OpaqueRef:
        return self._ref

    def call_method(self, method: str, propagate: Any = None, *args, **kwargs):
        if self._mesh is None:
            return _call_method(self._handle, method, *args, **kwargs)
        prop = propagate
        if callable(propagate):      # the rule sees the method's own arguments
            prop = lambda oid, name, *a, **k: propagate(*a, **k)  # noqa: E731
        return _remote("_call_method", prop)(self._handle, method, *args, **kwargs)

    def call_method_on_shard_and_fetch(self, method: str, *args, shard=None, **kwargs):
        from .tensor_engine import call_on_shard_and_fetch
        return call_on_shard_and_fetch("monarch_b200.opaque_object._call_method", self._handle,
                                       method, *args, shard=shard, **kwargs)

    def _set(self, name: str, value) -> None:
        if self._mesh is None:
            _set_attr(self._handle, name, value)
        else:
            _remote("_set_attr")(self._handle, name, value)

    def drop(self) -> None:
        if self._ref._key is not None:
            self._ref = OpaqueRef._of_id(0)        # the key tensor's release frees the object
        elif self._mesh is None:
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
