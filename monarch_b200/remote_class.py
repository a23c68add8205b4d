"""Controller-side handles of objects that live on every worker of a device mesh.

Parity: python/monarch/remote_class.py:16-121 (``ControllerRemoteClass`` /
``WorkerRemoteClass``).  A controller class names the worker class (dotted path, or the class
itself, which then travels by pickle); constructing the controller object constructs one
worker object per proc of the active mesh, methods marked with ``remote_method`` run on all
of them in program order with the other tensor-engine commands, and dropping the controller
object drops the worker objects.  Methods return nothing; arguments may be distributed
tensors (each worker sees its own shard).

    class WorkerCounter(WorkerRemoteClass):
        def __init__(self, start): self.n = start
        def add(self, t): self.n += int(t.sum())

    class Counter(ControllerRemoteClass):
        def __init__(self, start): super().__init__(WorkerCounter, start)
        @ControllerRemoteClass.remote_method
        def add(self, t): ...
"""
from __future__ import annotations

import importlib
import itertools
import threading
from typing import Any, Dict, Union

from .tensor_engine.device_mesh import get_active_mesh
from .tensor_engine.remote import remote


def _worker_class(cls_ref):
    if isinstance(cls_ref, str):
        mod, _, name = cls_ref.rpartition(".")
        return getattr(importlib.import_module(mod), name)
    return cls_ref


def _remote_class_call(cls_ref, what: str, ident: int, *args, **kwargs) -> None:
    cls = _worker_class(cls_ref)
    if not (isinstance(cls, type) and issubclass(cls, WorkerRemoteClass)):
        raise TypeError(f"{cls_ref!r} is not a WorkerRemoteClass")
    getattr(cls, what)(ident, *args, **kwargs)


_call = remote(_remote_class_call, propagate=lambda *a, **k: None)


class ControllerRemoteClass:
    _idents = itertools.count(1)

    def __init__(self, worker_cls: Union[str, type], *args, **kwargs) -> None:
        mesh = get_active_mesh()
        if mesh is None:
            raise RuntimeError("a remote class is created under `with mesh.activate():`")
        self.ident = next(ControllerRemoteClass._idents)
        self.worker_cls = worker_cls
        self.mesh = mesh
        _call(worker_cls, "remote_init", self.ident, *args, **kwargs)

    @staticmethod
    def remote_method(fn):
        name = fn.__name__

        def call(self, *args, **kwargs) -> None:
            with self.mesh.activate():
                _call(self.worker_cls, "remote_method", self.ident, name, *args, **kwargs)

        call.__name__ = name
        call.__doc__ = fn.__doc__
        return call

    def drop(self) -> None:
        mesh, self.mesh = getattr(self, "mesh", None), None
        if mesh is not None and not mesh.client._closed:
            with mesh.activate():
                _call(self.worker_cls, "remote_del", self.ident)

    def __del__(self) -> None:
        try:
            self.drop()
        except Exception:  # noqa: BLE001 - interpreter or engine shutting down
            pass


class WorkerRemoteClass:
    """Base of the worker-side classes; instances are kept by the ident the controller
    chose."""

    _objects: Dict[int, Any] = {}
    _lock = threading.Lock()

    @classmethod
    def remote_init(cls, ident: int, *args, **kwargs) -> None:
        obj = cls(*args, **kwargs)
        with WorkerRemoteClass._lock:
            WorkerRemoteClass._objects[ident] = obj

    @classmethod
    def remote_del(cls, ident: int) -> None:
        with WorkerRemoteClass._lock:
            WorkerRemoteClass._objects.pop(ident, None)

    @classmethod
    def remote_method(cls, ident: int, method: str, *args, **kwargs) -> None:
        obj = WorkerRemoteClass._objects[ident]
        if type(obj) is not cls:
            raise TypeError(f"object {ident} is a {type(obj).__name__}, not a {cls.__name__}")
        getattr(obj, method)(*args, **kwargs)


__all__ = ["ControllerRemoteClass", "WorkerRemoteClass"]
