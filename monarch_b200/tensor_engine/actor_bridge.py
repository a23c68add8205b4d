"""Actor endpoints called with distributed tensors: the actor sees its proc's local shard.

``actor.ep.call(t)`` with ``t`` a distributed :class:`Tensor` runs the endpoint on every actor
with the *real* tensor its proc's tensor worker holds for ``t``; ``actor.ep.rref(t)`` does the
same but keeps the returned tensors on the workers and hands back distributed tensors (shapes
from the endpoint's ``propagate``).  This is what lets modules be written as actors over
distributed tensors.

Parity: python/monarch/mesh_controller.py:319-447 (``actor_send`` / ``actor_rref``),
monarch_hyperactor/src/local_state_broker.rs:22-66 (the proc-local broker that rendez-vouses
the worker's ``Set(seq, state)`` with the actor's ``Get(seq)``), monarch_tensor_worker
``SendResultOfActorCall`` / ``CallActorMethod`` (stream.rs:1067-1106, 1706-1744).

Two ordered messages leave the controller per call: (a) to the tensor workers, in line with
the tensor commands issued so far -- "resolve these refs and put the tensors under ident I"
(and, for ``rref``, "then wait for the actor's result and store it under these refs");
(b) to the actor mesh, the ordinary cast, with the tensors replaced by placeholders and the
ident in the headers.  Actor and tensor worker of a proc share a process, so the broker is a
table of that process: no bytes are copied, the endpoint works on the worker's own tensors
(in-place changes are seen by later tensor commands).
"""
from __future__ import annotations

import threading
import time
from typing import Any, Dict, List, Optional, Tuple

import torch

from .worker import _seq

_BROKER_TIMEOUT = 120.0


class _Broker:
    """Rendez-vous of a proc's tensor worker and its actors, keyed by (proc, ident)."""

    def __init__(self):
        self._cv = threading.Condition()
        self._items: Dict[Tuple[str, int, str], Any] = {}

    def put(self, proc: str, ident: int, slot: str, value: Any) -> None:
        with self._cv:
            self._items[(proc, ident, slot)] = value
            self._cv.notify_all()

    def take(self, proc: str, ident: int, slot: str, timeout: float = _BROKER_TIMEOUT) -> Any:
        key = (proc, ident, slot)
        deadline = time.monotonic() + timeout
        with self._cv:
            while key not in self._items:
                left = deadline - time.monotonic()
                if left <= 0:
                    raise TimeoutError(f"nothing arrived for call {ident} ({slot}) on {proc} "
                                       f"within {timeout:.0f} s")
                self._cv.wait(left)
            return self._items.pop(key)


BROKER = _Broker()


class BrokerRef:
    """Stands for the ``index``-th tensor of a call in the pickled arguments."""

    def __init__(self, index: int):
        self.index = index

    def __reduce__(self):
        return (BrokerRef, (self.index,))


class CallFailed:
    """Deposited instead of tensors/results when the producing side failed."""

    def __init__(self, text: str):
        self.text = text


def _device_tensor_type():
    from .device_mesh import Tensor
    return Tensor


def has_distributed_tensors(args, kwargs) -> bool:
    T = _device_tensor_type()

    def visit(o) -> bool:
        if isinstance(o, T):
            return True
        if isinstance(o, (list, tuple)):
            return any(visit(x) for x in o)
        if isinstance(o, dict):
            return any(visit(x) for x in o.values())
        return False

    return visit(args) or visit(kwargs)


def _strip(obj, found: List[Any]):
    """Replace distributed tensors by placeholders; collects them in ``found``."""
    T = _device_tensor_type()
    if isinstance(obj, T):
        found.append(obj)
        return BrokerRef(len(found) - 1)
    if isinstance(obj, (list, tuple)):
        return _seq(obj, (_strip(o, found) for o in obj))
    if isinstance(obj, dict):
        return {k: _strip(v, found) for k, v in obj.items()}
    return obj


def substitute(obj, tensors: List[torch.Tensor]):
    """Actor side: placeholders -> the proc's real tensors."""
    if isinstance(obj, BrokerRef):
        return tensors[obj.index]
    if isinstance(obj, (list, tuple)):
        return _seq(obj, (substitute(o, tensors) for o in obj))
    if isinstance(obj, dict):
        return {k: substitute(v, tensors) for k, v in obj.items()}
    return obj


def _check_same_procs(endpoint, tensors) -> Any:
    from .device_mesh import _check_usable, _mesh_of
    mesh = _mesh_of(tensors)
    for t in tensors:
        _check_usable(t)
    amesh = endpoint._mesh
    if amesh._world != mesh.client.proc_mesh.world:
        raise ValueError(f"the tensors live on proc mesh {mesh.client.proc_mesh.world}, the actor "
                         f"mesh '{amesh._name}' on {amesh._world}: an actor can only be handed "
                         "tensors of its own procs")
    if sorted(amesh._shape.ndslice.ranks()) != sorted(mesh._ndslice.ranks()):
        raise ValueError("the tensors and the actors cover different procs of the mesh; slice "
                         "one to match the other (slice_mesh / actor_mesh.slice)")
    return mesh


def actor_send(endpoint, args, kwargs, port, ranks, headers) -> None:
    """``call`` / ``broadcast`` / ... of an endpoint whose arguments contain distributed
    tensors."""
    from .device_mesh import Ref, get_active_stream
    found: List[Any] = []
    s_args, s_kwargs = _strip(args, found), _strip(kwargs, found)
    mesh = _check_same_procs(endpoint, found)
    client = mesh.client
    stream = get_active_stream()
    client._ensure_stream(stream)
    ident = client.new_seq()
    client.send(mesh, ("actor_call_state", ident, [Ref(t.ref) for t in found], stream.id))
    client.flush()
    h = dict(headers or {})
    h["broker_ident"] = str(ident)
    endpoint._mesh._cast(("call", endpoint._name, s_args, s_kwargs, port), ranks, h)


def spawn_state(proc_mesh, args, kwargs):
    """Constructor arguments with distributed tensors: strips them and queues the hand-over
    on the workers.  Returns (args, kwargs, ident) for the spawn parameters."""
    from .device_mesh import Ref, _check_usable, _mesh_of, get_active_stream
    found: List[Any] = []
    s_args, s_kwargs = _strip(args, found), _strip(kwargs, found)
    mesh = _mesh_of(found)
    for t in found:
        _check_usable(t)
    if mesh.client.proc_mesh.world != proc_mesh.world:
        raise ValueError("an actor can only be constructed from tensors of its own proc mesh")
    client = mesh.client
    stream = get_active_stream()
    client._ensure_stream(stream)
    ident = client.new_seq()
    client.send(mesh, ("actor_call_state", ident, [Ref(t.ref) for t in found], stream.id))
    client.flush()
    return s_args, s_kwargs, ident


def endpoint_rref(endpoint, args, kwargs):
    """Run the endpoint on every actor with its proc's shards; the tensors it returns stay on
    the workers and come back as distributed tensors."""
    from .device_mesh import (Ref, _propagation, _to_fake, _wrap_outputs, get_active_mesh,
                              get_active_stream)
    found: List[Any] = []
    s_args, s_kwargs = _strip(args, found), _strip(kwargs, found)
    if found:
        mesh = _check_same_procs(endpoint, found)
    else:
        mesh = get_active_mesh()
        if mesh is None:
            raise RuntimeError("rref needs distributed tensor arguments or an active device mesh")
    endpoint._check_signature(args, kwargs)
    prop = endpoint._propagate
    fake_out = None
    if callable(prop):
        with _propagation():
            fake_out = prop(*_to_fake(args), **_to_fake(kwargs))
    elif prop not in (None, "inspect", "mocked"):
        raise ValueError(f"unsupported propagate={prop!r} for rref")
    client = mesh.client
    stream = get_active_stream()
    client._ensure_stream(stream)
    refs: List[Any] = []
    out = _wrap_outputs(fake_out, mesh, stream, refs)
    ident = client.new_seq()
    client.send(mesh, ("actor_call_rref", ident, [Ref(t.ref) for t in found], refs, stream.id))
    client.flush()
    h = {"broker_ident": str(ident), "broker_rref": "1"}
    endpoint._mesh._cast(("call", endpoint._name, s_args, s_kwargs, None), None, h)
    return out


# ------------------------------------------------------------------------ actor side ----
class BrokerResultPort:
    """Response port of an ``rref`` call: the value goes to the proc's tensor worker."""

    def __init__(self, proc: str, ident: int):
        self._proc, self._ident = proc, ident

    def send(self, obj: Any) -> None:
        BROKER.put(self._proc, self._ident, "result", obj)

    def exception(self, obj: BaseException) -> None:
        BROKER.put(self._proc, self._ident, "result", CallFailed(str(obj)))


def take_state(proc: str, ident: int) -> List[torch.Tensor]:
    state = BROKER.take(proc, ident, "state")
    if isinstance(state, CallFailed):
        raise RuntimeError(f"a tensor argument of this call failed on the worker: {state.text}")
    return state
