"""Actors, endpoints, actor meshes, ports and value meshes.

Parity: python/monarch/_src/actor/actor_mesh.py (Actor, ActorMesh, _Actor.handle dispatch,
Port/PortReceiver/Channel, ValueMesh, Accumulator, ActorError, context()),
python/monarch/_src/actor/endpoint.py (adverbs call / call_one / choose / stream /
broadcast / rref, ``@endpoint``), monarch_hyperactor/src/actor.rs (PythonActor bridge,
PythonMessage kinds).

Every message to an actor mesh -- including single-actor sends -- goes through the native
cast tree (``_native.cast``), so casts and sends from one sender stay in FIFO order.
Replies go straight to the caller's port.
"""
from __future__ import annotations

import asyncio
import collections
import contextvars
import functools
import inspect
import json
import os
import pickle
import random
import struct
import sys
import threading
import time
import traceback
from typing import (Any, Callable, Dict, Generic, Iterator, List, Optional, Tuple, Type,
                    TypeVar)

from .. import _native as N
from .future import Future
from .pickle import flatten, unflatten
from .shape import Extent, MeshTrait, Point, Shape

R = TypeVar("R")
T = TypeVar("T")


# ----------------------------------------------------------------------------- errors --
class ActorError(Exception):
    """An endpoint raised; carries the remote exception and its formatted traceback."""

    def __init__(self, exception: BaseException, message: str = "A remote actor call has failed.",
                 frames: Optional[str] = None):
        self.exception = exception
        self.message = message
        self.actor_mesh_ref_frames = frames if frames is not None else "".join(
            traceback.format_exception(type(exception), exception, exception.__traceback__))
        super().__init__(str(self))

    def __str__(self) -> str:
        return (f"{self.message}\n Traceback of where the remote call failed "
                f"(most recent call last):\n{self.actor_mesh_ref_frames}")

    def __reduce__(self):
        exc = self.exception
        try:
            import cloudpickle
            cloudpickle.dumps(exc)
        except Exception:  # unpicklable exception objects degrade to their text
            exc = RuntimeError(f"{type(self.exception).__name__}: {self.exception}")
        return (ActorError, (exc, self.message, self.actor_mesh_ref_frames))


class SupervisionError(RuntimeError):
    """The actor mesh (or the procs under it) failed; raised on pending and later calls."""


# ---------------------------------------------------------------------------- context --
class ActorInstance:
    """What ``context().actor_instance`` exposes."""

    def __init__(self, native: "N.Instance", proc_mesh=None, rank_point: Optional[Point] = None):
        self._native = native
        self.proc_mesh = proc_mesh
        self._rank_point = rank_point

    @property
    def actor_id(self) -> str:
        return self._native.actor_id

    @property
    def proc_id(self) -> str:
        return self._native.proc_id

    @property
    def rank(self) -> Point:
        return self._rank_point if self._rank_point is not None else Point(0, Extent([], []))

    @property
    def proc(self):
        return self._native.proc

    @property
    def name(self) -> str:
        return self._native.name


class Context:
    def __init__(self, actor_instance: ActorInstance, message_rank: Point):
        self.actor_instance = actor_instance
        self.message_rank = message_rank

    @staticmethod
    def _root() -> "Context":
        return _root_context()


_context: contextvars.ContextVar[Optional[Context]] = contextvars.ContextVar("mb_ctx", default=None)
_tls = threading.local()
_root_lock = threading.Lock()
_root_ctx: Optional[Context] = None


def _root_context() -> Context:
    global _root_ctx
    with _root_lock:
        if _root_ctx is None:
            inst = N.client_proc().attach("root_client")
            _root_ctx = Context(ActorInstance(inst), Point(0, Extent([], [])))
        return _root_ctx


def context() -> Context:
    """The current actor's context, or the root client's outside any actor."""
    c = getattr(_tls, "ctx", None)
    if c is not None:
        return c
    c = _context.get()
    return c if c is not None else _root_context()


def current_rank() -> Point:
    return context().message_rank


def current_size() -> Dict[str, int]:
    r = context().message_rank
    return dict(zip(r.extent.labels, r.extent.sizes))


def current_actor_name() -> str:
    return context().actor_instance.actor_id


# ------------------------------------------------------------------------------ ports --
_KIND_RESULT = "result"
_KIND_EXCEPTION = "exception"


class Port(Generic[R]):
    """Send side of a port; picklable and usable from any actor."""

    def __init__(self, port_id: str, rank: Optional[int] = None, via: Optional[str] = None,
                 key: Optional[str] = None):
        self._port_id = port_id
        self._rank = rank
        # set on the response port of a cast whose replies are gathered along its tree: the
        # reply goes to the comm actor of this proc, which hands one batch per subtree up
        self._via, self._key = via, key

    def _post(self, kind: str, obj: Any) -> None:
        body, parts = flatten((kind, self._rank, obj))
        inst = context().actor_instance._native
        if self._via is not None:
            via, self._via = self._via, None     # exactly one reply travels by the tree
            inst.send(via, body, {"kind": "reduce_part", "no_return": "1", "gather": "1",
                                  "gather_item": "1", "reduce_key": self._key,
                                  "reduce_port": self._port_id, "n": "1"}, parts)
            return
        inst.send(self._port_id, body, {"kind": kind, "no_return": "1"}, parts)

    def send(self, obj: R) -> None:
        self._post(_KIND_RESULT, obj)

    def exception(self, obj: BaseException) -> None:
        if not isinstance(obj, ActorError):
            obj = ActorError(obj)
        self._post(_KIND_EXCEPTION, obj)

    def __reduce__(self):
        return (Port, (self._port_id, self._rank))


class ReducePort(Port):
    """Send side of a native accumulating port: tensors are posted as raw bytes and folded
    by the C++ reducer of the receiving mailbox (no unpickling on the reduce path);
    exceptions go to a separate ordinary port."""

    def __init__(self, port_id: str, error_port_id: str, rank: Optional[int] = None,
                 via: Optional[str] = None, key: Optional[str] = None):
        super().__init__(port_id, rank)
        self._error_port_id = error_port_id
        # when the cast asked for a reduction along its tree: the comm actor of this proc,
        # which folds the subtree's updates before passing one message up
        self._via, self._key = via, key

    def send(self, obj) -> None:
        import numpy as np
        arr = obj.detach().cpu().contiguous().numpy() if hasattr(obj, "detach") else \
            np.ascontiguousarray(obj)
        inst = context().actor_instance._native
        if self._via is not None:
            inst.send(self._via, arr.tobytes(),
                      {"kind": "reduce_part", "no_return": "1", "reduce_key": self._key,
                       "reduce_port": self._port_id, "n": "1"}, [])
            return
        inst.send(self._port_id, arr.tobytes(), {"kind": "reduce", "no_return": "1"}, [])

    def exception(self, obj: BaseException) -> None:
        if not isinstance(obj, ActorError):
            obj = ActorError(obj)
        body, parts = flatten((_KIND_EXCEPTION, self._rank, obj))
        context().actor_instance._native.send(self._error_port_id, body,
                                              {"kind": _KIND_EXCEPTION, "no_return": "1"}, parts)

    def __reduce__(self):
        return (ReducePort, (self._port_id, self._error_port_id, self._rank))


class DroppingPort:
    """Used when the caller did not ask for a response: results vanish, exceptions crash
    the actor (and reach its supervisor)."""

    def send(self, obj: Any) -> None:
        pass

    def exception(self, obj: BaseException) -> None:
        raise obj if not isinstance(obj, ActorError) else obj.exception


class _Health:
    """Failure state of one proc mesh, shared by its actor meshes."""

    def __init__(self):
        self.lock = threading.Lock()
        self.mesh_error: Optional[str] = None
        # actor name -> {proc rank: first failure there}
        self.actor_errors: Dict[str, Dict[int, str]] = {}
        self.stopped = False
        self.stopped_actors: set = set()      # names of actor meshes stopped by their owner

    def error_for(self, actor_name: str, ranks=None) -> Optional[str]:
        """The failure that concerns the actors ``actor_name`` on ``ranks`` (a callable
        giving the set of proc ranks, None for all): a slice that does not contain the failed
        actor stays usable (python/tests/test_actor_error.py ``test_slice_supervision`` in
        the reference).  A failure of the proc mesh itself concerns everyone."""
        with self.lock:
            by_rank = self.actor_errors.get(actor_name)
            if by_rank:
                if ranks is None:
                    return next(iter(by_rank.values()))
                mine = ranks()
                for r, msg in by_rank.items():
                    if r in mine:
                        return msg
            return self.mesh_error


def _recv_checked(receiver, health: Optional[_Health], actor_name: str,
                  deadline: Optional[float], ranks=None):
    """Wait for the next envelope, waking regularly to notice supervision failures."""
    while True:
        slice_ms = 50
        if deadline is not None:   # a poll (deadline now) must not sit out a whole slice
            slice_ms = max(0, min(50, int((deadline - time.monotonic()) * 1000)))
        env = receiver.recv(slice_ms) if slice_ms > 0 else receiver.try_recv()
        if env is not None:
            return env
        if health is not None:
            err = health.error_for(actor_name, ranks)
            if err is not None:
                raise SupervisionError(f"actor mesh '{actor_name}' is unhealthy: {err}")
        if deadline is not None and time.monotonic() > deadline:
            raise TimeoutError("timed out waiting for a reply")


def _unpack_batch(data: bytes, parts: List[bytes]) -> "collections.deque":
    """Replies gathered along a cast tree arrive as one envelope: ``data`` is a sequence of
    records (u32 part count, u64 body length, body), ``parts`` the replies' parts in order."""
    out: "collections.deque" = collections.deque()
    mv = memoryview(data)
    pos, p = 0, 0
    n = len(mv)
    while pos < n:
        n_parts, body_len = struct.unpack_from("<IQ", mv, pos)
        pos += 12
        out.append((bytes(mv[pos:pos + body_len]), parts[p:p + n_parts]))
        pos += body_len
        p += n_parts
    return out


class PortReceiver(Generic[R]):
    def __init__(self, native_receiver, port_id: str, instance, health: Optional[_Health] = None,
                 actor_name: str = "", ranks=None):
        self._rx = native_receiver
        self._port_id = port_id
        self._instance = instance
        self._health = health
        self._actor_name = actor_name
        self._ranks = ranks

    def _next(self, timeout: Optional[float]) -> Tuple[Optional[int], Any]:
        batch = self.__dict__.get("_batch")
        if not batch:
            deadline = None if timeout is None else time.monotonic() + timeout
            env = _recv_checked(self._rx, self._health, self._actor_name, deadline,
                                self._ranks)
            if env.headers.get("kind") != "batch":
                kind, rank, obj = unflatten(env.data, env.parts)
                if kind == _KIND_EXCEPTION:
                    raise obj
                return rank, obj
            batch = self._batch = _unpack_batch(env.data, env.parts)
        data, parts = batch.popleft()
        kind, rank, obj = unflatten(data, parts)
        if kind == _KIND_EXCEPTION:
            raise obj
        return rank, obj

    def _arm(self, wake) -> None:
        """``wake()`` after every delivery to this port (None: stop); lets a coroutine sleep
        until a message is there instead of parking a thread in ``recv``."""
        self._rx.set_notify(wake)

    def recv(self) -> Future[R]:
        return Future(lambda timeout: self._next(timeout)[1], arm=self._arm)

    def ranked(self) -> "RankedPortReceiver[R]":
        return RankedPortReceiver(self)

    def close(self) -> None:
        self._instance.close_port(self._port_id)


class RankedPortReceiver(Generic[R]):
    def __init__(self, inner: PortReceiver):
        self._inner = inner

    def recv(self) -> Future[Tuple[int, R]]:
        return Future(lambda timeout: self._inner._next(timeout), arm=self._inner._arm)


class Channel(Generic[R]):
    @staticmethod
    def open(once: bool = False, _health=None, _actor_name="",
             _ranks=None) -> Tuple[Port, PortReceiver]:
        inst = context().actor_instance._native
        port_id, rx = inst.open_port(once)
        return Port(port_id), PortReceiver(rx, port_id, inst, _health, _actor_name, _ranks)


# ------------------------------------------------------------------------- value mesh --
class ValueMesh(MeshTrait, Generic[R]):
    """The per-actor results of a ``call``, laid out like the mesh that was called."""

    def __init__(self, shape: Shape, values: List[R]):
        self._shape_ = shape
        self._values = values

    @property
    def _ndslice(self):
        return self._shape_.ndslice

    @property
    def _labels(self):
        return tuple(self._shape_.labels)

    def _new_with_shape(self, shape: Shape) -> "ValueMesh[R]":
        base = self._shape_.ndslice
        return ValueMesh(shape_normalised(shape), [self._values[base.index(r)] for r in
                                                   shape.ndslice.ranks()])

    def item(self, **kwargs) -> R:
        sl = self._shape_.ndslice
        unknown = [k for k in kwargs if k not in self._labels]
        missing = [l for l, n in zip(self._labels, sl.sizes) if l not in kwargs and n != 1]
        if unknown or missing:
            raise KeyError(f"expected coordinates for {self._labels}, got {tuple(kwargs)}")
        coords = [kwargs.get(l, 0) for l in self._labels]   # dims of size 1 may be left out
        return self._values[sl.index(sl.nditem(coords))]

    def items(self) -> Iterator[Tuple[Point, R]]:
        ext = self.extent
        for i, v in enumerate(self._values):
            yield Point(i, ext), v

    def values(self) -> List[R]:
        return list(self._values)

    def __iter__(self):
        return self.items()

    def __len__(self) -> int:
        return len(self._values)

    def __repr__(self) -> str:
        return f"ValueMesh({self.extent}, {self._values!r})"


def shape_normalised(shape: Shape) -> Shape:
    """Same labels/sizes, dense row-major ranks 0..n-1 (a ValueMesh owns its values)."""
    return Shape(shape.labels, N.Slice.new_row_major(shape.ndslice.sizes))


# -------------------------------------------------------------------------- endpoints --
def _tracing_on() -> bool:
    return N.events_enabled() or N.trace_enabled()


# Gathering replies along the tree trades one extra (in-process) hop per level for far fewer
# messages at the caller.  Measured on one 8-core box it loses up to 16 procs (call p50
# 1.2 ms against 0.88 ms), so it only switches on for meshes large enough that the caller's
# per-reply cost dominates.
_GATHER_MIN = int(os.environ.get("MB200_GATHER_MIN", "512"))
_signatures: Dict[Any, inspect.Signature] = {}
_bound_ok: set = set()
_cast_points: Dict[Tuple[str, int], "Point"] = {}


def _cast_point(shape_hdr: Optional[str], cast_rank: int) -> "Point":
    """The ``Point`` a cast message is addressed to, from its headers (cached: the same few
    (shape, rank) pairs recur for the life of a mesh)."""
    if not shape_hdr:
        return Point(0, Extent([], []))
    key = (shape_hdr, cast_rank)
    p = _cast_points.get(key)
    if p is None:
        labels, sizes = json.loads(shape_hdr)
        p = Point(cast_rank, Extent(labels, sizes))
        if len(_cast_points) < 65536:
            _cast_points[key] = p
    return p


def _signature_of(fn) -> inspect.Signature:
    """``inspect.signature`` costs tens of microseconds; endpoints are called in loops."""
    sig = _signatures.get(fn)
    if sig is None:
        sig = _signatures[fn] = inspect.signature(fn)
    return sig


class EndpointProperty:
    """What ``@endpoint`` leaves on the class: resolved to an :class:`Endpoint` when read
    from an :class:`ActorMesh`, to the plain bound method when read from the actor."""

    def __init__(self, fn: Callable, propagate=None, explicit_response_port: bool = False):
        self._fn = fn
        self._propagate = propagate
        self._explicit_response_port = explicit_response_port
        functools.update_wrapper(self, fn)

    def __set_name__(self, owner, name):
        self._name = name

    def __get__(self, obj, objtype=None):
        if obj is None:
            return self
        return functools.partial(self._fn, obj)

    def __call__(self, *a, **kw):  # pragma: no cover - guidance only
        raise RuntimeError("an endpoint is invoked through an actor mesh: "
                           "mesh.name.call(...), .call_one(...), .choose(...), .broadcast(...)")


def endpoint(fn: Optional[Callable] = None, *, propagate=None,
             explicit_response_port: bool = False):
    """Mark a method of an :class:`Actor` as remotely callable."""
    if fn is None:
        return lambda f: EndpointProperty(f, propagate, explicit_response_port)
    return EndpointProperty(fn, propagate, explicit_response_port)


class Endpoint(Generic[R]):
    def __init__(self, mesh: "ActorMesh", name: str, fn: Optional[Callable],
                 explicit_response_port: bool = False, propagate=None):
        self._mesh = mesh
        self._name = name
        self._fn = fn
        self._explicit = explicit_response_port
        self._propagate = propagate

    # -- plumbing ---------------------------------------------------------------------
    def _check_signature(self, args, kwargs) -> None:
        if self._fn is None:
            return
        # the outcome depends only on how many positional arguments and which keywords are
        # passed: remember the shapes of calls that bound successfully
        shape = (self._fn, self._explicit, len(args), tuple(kwargs) if kwargs else ())
        if shape in _bound_ok:
            return
        sig = _signature_of(self._fn)
        extra = [None] * (2 if self._explicit else 1)  # self (+ port)
        try:
            sig.bind(*extra, *args, **kwargs)
        except TypeError as e:
            raise TypeError(f"{self._mesh._class_name}.{self._name}: {e}") from None
        if len(_bound_ok) < 4096:
            _bound_ok.add(shape)

    def _send(self, args, kwargs, port: Optional[Port], ranks: Optional[List[int]] = None,
              headers: Optional[Dict[str, str]] = None) -> None:
        self._check_signature(args, kwargs)
        if "monarch_b200.tensor_engine.device_mesh" in sys.modules and \
                not getattr(self._fn, "_wire_messages_only", False):
            from ..tensor_engine import actor_bridge as ab
            if ab.has_distributed_tensors(args, kwargs):
                ab.actor_send(self, args, kwargs, port, ranks, headers)
                return
        self._mesh._cast(("call", self._name, args, kwargs, port), ranks, headers)

    def _open(self, once: bool = False) -> Tuple[Port, PortReceiver]:
        return Channel.open(once, _health=self._mesh._health, _actor_name=self._mesh._name,
                            _ranks=self._mesh._rank_set)

    # -- adverbs ----------------------------------------------------------------------
    def call(self, *args, **kwargs) -> Future[ValueMesh[R]]:
        self._mesh._raise_if_unhealthy()
        port, rx = self._open()
        n = len(self._mesh)
        self._send(args, kwargs, port, headers=self._gather_headers(port, n))
        shape = shape_normalised(self._mesh._shape)

        out: List[Any] = [None] * n
        got = [0]

        def wait(timeout: Optional[float]) -> ValueMesh[R]:
            # resumable: a wait that timed out keeps what has arrived so far
            deadline = None if timeout is None else time.monotonic() + timeout
            try:
                while got[0] < n:
                    left = None if deadline is None else max(deadline - time.monotonic(), 0.0)
                    rank, v = rx._next(left)
                    out[rank] = v
                    got[0] += 1
            except TimeoutError:
                raise
            except BaseException:
                rx.close()
                raise
            rx.close()
            return ValueMesh(shape, out)

        return Future(wait, arm=rx._arm)

    def _gather_headers(self, port: Port, n: int) -> Optional[Dict[str, str]]:
        """Replies of a cast to more than a few actors come back gathered along the cast
        tree: one batch per child of the root instead of one message per actor.  Endpoints
        with an explicit response port answer as often as they like and are left alone."""
        if n <= _GATHER_MIN or self._explicit:
            return None
        return {"reduce_tree": "gather", "reduce_port": port._port_id}

    def call_one(self, *args, **kwargs) -> Future[R]:
        if len(self._mesh) != 1:
            raise ValueError(f"Can only use 'call_one' on a single Actor but this actor has shape "
                             f"{self._mesh._shape}")
        self._mesh._raise_if_unhealthy()
        port, rx = self._open(once=True)
        self._send(args, kwargs, port)
        return Future(lambda timeout: rx._next(timeout)[1], arm=rx._arm)

    def choose(self, *args, **kwargs) -> Future[R]:
        """Load-balanced call to one actor of the mesh, picked by a deterministic PRNG."""
        self._mesh._raise_if_unhealthy()
        port, rx = self._open(once=True)
        ranks = self._mesh._shape.ndslice.ranks()
        self._send(args, kwargs, port, [_choose_rng.choice(ranks)])
        return Future(lambda timeout: rx._next(timeout)[1], arm=rx._arm)

    def stream(self, *args, **kwargs) -> Iterator[Future[R]]:
        self._mesh._raise_if_unhealthy()
        port, rx = self._open()
        n = len(self._mesh)
        self._send(args, kwargs, port)
        for _ in range(n):
            yield Future(lambda timeout: rx._next(timeout)[1], arm=rx._arm)

    def reduce(self, *args, reducer: str = "sum_f32", **kwargs) -> Future:
        """Call every actor and fold the returned tensors element-wise in the native
        mailbox (``sum_f32``, ``sum_f64``, ``max_f64``, ``min_f64``, ``sum_i64``).  The
        future yields the folded values as a 1-D tensor."""
        self._mesh._raise_if_unhealthy()
        inst = context().actor_instance._native
        port_id, acc = inst.open_accum_port(reducer, b"")
        err_port, err_rx = self._open()
        n = len(self._mesh)
        # the updates are folded along the cast tree: every comm actor passes one partial
        # result up, so the caller receives one message per child of the root, not one per actor
        self._send(args, kwargs, ReducePort(port_id, err_port._port_id),
                   headers={"reduce_tree": reducer, "reduce_port": port_id})
        mesh = self._mesh

        def wait(timeout: Optional[float]):
            import numpy as np
            import torch
            deadline = None if timeout is None else time.monotonic() + timeout
            try:
                while not acc.wait_count(n, 20):
                    env = err_rx._rx.try_recv()
                    if env is not None:
                        raise unflatten(env.data, env.parts)[2]
                    mesh._raise_if_unhealthy()
                    if deadline is not None and time.monotonic() > deadline:
                        raise TimeoutError("timed out waiting for the reduction")
            finally:
                inst.close_port(port_id)
                err_rx.close()
            dt = {"f32": np.float32, "f64": np.float64, "i64": np.int64}[reducer.split("_")[-1]]
            return torch.from_numpy(np.frombuffer(acc.state(), dtype=dt).copy())

        return Future(wait)

    def broadcast(self, *args, **kwargs) -> None:
        """Fire and forget; an exception in the endpoint crashes the actor."""
        self._mesh._raise_if_unhealthy()
        self._send(args, kwargs, None)

    def rref(self, *args, **kwargs):
        from ..tensor_engine.actor_bridge import endpoint_rref
        return endpoint_rref(self, args, kwargs)

    def _port_call(self, args, kwargs, port: Port, ranks=None) -> None:
        """``send(endpoint, args, kwargs, port, selection)``: replies go to ``port``."""
        self._send(args, kwargs, port, ranks)


_choose_rng = random.Random(4)


def send(endpoint_: Endpoint, args: Tuple, kwargs: Dict, port: Optional[Port] = None,
         selection: str = "all") -> None:
    """Low-level send: deliver to all actors (``"all"``) or one (``"choose"``)."""
    ranks = None
    if selection == "choose":
        ranks = [_choose_rng.choice(endpoint_._mesh._shape.ndslice.ranks())]
    elif selection != "all":
        raise ValueError(f"invalid selection: {selection}")
    endpoint_._send(args, kwargs, port, ranks)


def as_endpoint(bound_method, *, propagate=None, explicit_response_port=False) -> Endpoint:
    """Treat ``mesh.method`` of an undecorated method as an endpoint."""
    if isinstance(bound_method, Endpoint):
        if propagate is None and not explicit_response_port:
            return bound_method
        e = bound_method
        return Endpoint(e._mesh, e._name, e._fn, explicit_response_port or e._explicit,
                        propagate if propagate is not None else e._propagate)
    if isinstance(bound_method, _NotAnEndpoint):
        return Endpoint(bound_method.mesh, bound_method.name, bound_method.fn,
                        explicit_response_port, propagate)
    raise ValueError("as_endpoint expects an attribute read from an actor mesh")


class _NotAnEndpoint:
    def __init__(self, mesh, name, fn):
        self.mesh, self.name, self.fn = mesh, name, fn

    def _fail(self, *a, **k):
        raise RuntimeError(
            f"Actor {self.mesh._class_name}.{self.name} is not annotated as an endpoint. To call "
            f"it as one, add a @endpoint decorator to it, or wrap it using "
            f"as_endpoint(obj.{self.name})")

    call = call_one = choose = stream = broadcast = rref = __call__ = _fail


class Accumulator(Generic[T, R]):
    """Fold the per-actor results of an endpoint: ``Accumulator(ep, identity,
    combine).accumulate(*args)`` -> Future of the combined value."""

    def __init__(self, endpoint_: Endpoint, identity: T, combine: Callable[[T, R], T]):
        self._endpoint = endpoint_
        self._identity = identity
        self._combine = combine

    def accumulate(self, *args, **kwargs) -> Future[T]:
        gen = self._endpoint.stream(*args, **kwargs)

        def wait(timeout):
            acc = self._identity
            deadline = None if timeout is None else time.monotonic() + timeout
            for f in gen:
                left = None if deadline is None else max(deadline - time.monotonic(), 0.0)
                acc = self._combine(acc, f.get(left))
            return acc

        return Future(wait)


# ------------------------------------------------------------------------------ actor --
class Actor:
    """Base class of user actors.  Methods decorated with :func:`endpoint` are callable
    through the :class:`ActorMesh` returned by ``ProcMesh.spawn``."""

    def _handle_undeliverable_message(self, envelope, reason: str) -> bool:
        """Return True to swallow a returned message; the default fails the actor."""
        return False


class ActorMesh(MeshTrait, Generic[T]):
    def __init__(self, cls: Type[T], name: str, world: str, shape: Shape, proc_mesh=None,
                 health: Optional[_Health] = None, root_slice=None):
        self._class = cls
        self._class_name = getattr(cls, "__name__", str(cls))
        self._name = name
        self._world = world
        self._shape_ = shape
        self._proc_mesh = proc_mesh
        self._health = health
        # the slice the mesh was spawned over: every cast, whatever sub-slice it targets,
        # is routed through this tree so that one sender's messages keep their order
        self._root_slice = root_slice if root_slice is not None else shape.ndslice

    # MeshTrait ------------------------------------------------------------------------
    @property
    def _ndslice(self):
        return self._shape_.ndslice

    @property
    def _labels(self):
        return tuple(self._shape_.labels)

    @property
    def _shape(self) -> Shape:
        return self._shape_

    def _new_with_shape(self, shape: Shape) -> "ActorMesh[T]":
        return ActorMesh(self._class, self._name, self._world, shape, self._proc_mesh,
                         self._health, self._root_slice)

    # endpoints ------------------------------------------------------------------------
    def __getattr__(self, name: str):
        if name.startswith("__") or name in ("_class", "_shape_", "_name"):
            raise AttributeError(name)
        attr = getattr(self._class, name, None)
        if isinstance(attr, EndpointProperty):
            return Endpoint(self, name, attr._fn, attr._explicit_response_port, attr._propagate)
        if attr is None:
            raise AttributeError(f"{self._class_name} has no attribute {name!r}")
        return _NotAnEndpoint(self, name, attr if callable(attr) else None)

    def _rank_set(self) -> frozenset:
        """The proc ranks this (possibly sliced) mesh covers."""
        rs = self.__dict__.get("_rank_set_")
        if rs is None:
            rs = self.__dict__["_rank_set_"] = frozenset(self._shape_.ndslice.ranks())
        return rs

    def _raise_if_unhealthy(self) -> None:
        if self._health is not None:
            if self._name in self._health.stopped_actors:
                raise RuntimeError(f"actor mesh '{self._name}' has already been stopped")
            err = self._health.error_for(self._name, self._rank_set)
            if err is not None:
                raise SupervisionError(f"actor mesh '{self._name}' is unhealthy: {err}")

    def _cast(self, message: Tuple, ranks: Optional[List[int]] = None,
              extra_headers: Optional[Dict[str, str]] = None, plain: bool = False) -> None:
        """``plain``: the caller vouches that the message holds only data that the C pickler
        handles by itself (no functions or classes defined outside importable modules, no
        large tensors worth sending out of band); it is then serialised without the
        per-object Python hooks of the general pickler."""
        if plain:
            body, parts = pickle.dumps(message, protocol=pickle.HIGHEST_PROTOCOL), []
        else:
            body, parts = flatten(message)
        sl = self._shape_.ndslice
        root = self._root_slice
        if ranks is None and sl == root:
            sel = N.Selection.all()
        else:
            sel = N.Selection.of_ranks(root, sl.ranks() if ranks is None else ranks)
        headers = self.__dict__.get("_cast_headers")
        if headers is None:
            headers = self._cast_headers = {
                "cast_shape": json.dumps([self._shape_.labels, list(sl.sizes)])}
        if extra_headers:
            headers = {**headers, **extra_headers}
        port = message[4] if len(message) > 4 else None
        if type(port) is Port:
            # outside the pickle too: a message that cannot be unpickled on the far side can
            # still be answered (with the error) instead of failing the actor
            headers = {**headers, "reply_port": port._port_id}
        inst = context().actor_instance._native
        N.cast(inst, self._world, self._name, root, sel, body, headers, parts, sl)

    def stop(self) -> Future[None]:
        pm = self._proc_mesh
        if pm is None:
            raise NotImplementedError("stopping an actor mesh needs its owning proc mesh")
        def run(timeout):
            if self._health is not None:
                self._health.stopped_actors.add(self._name)   # later calls fail at once
            return pm._native.stop_actor(self._name, int((timeout or 5) * 1000))

        return Future(run)

    def __reduce__(self):
        return (ActorMesh, (self._class, self._name, self._world, self._shape_, None, None,
                            self._root_slice))

    def __repr__(self) -> str:
        return f"ActorMesh({self._class_name}, '{self._name}', {self._shape_})"


# -------------------------------------------------------------- worker-side dispatch ----
class _ActorState:
    """Per-actor state on the hosting proc: the user object, its event loop, dispatch."""

    def __init__(self, proc, name: str, params: bytes):
        self.proc = proc
        self.name = name
        (self.cls, self.args, self.kwargs, self.meta) = unflatten(params, [])
        self.obj: Any = None
        self.loop: Optional[asyncio.AbstractEventLoop] = None
        self._loop_thread: Optional[threading.Thread] = None
        self._has_async: Optional[bool] = None
        self.instance_info: Optional[ActorInstance] = None

    def _ensure(self, instance) -> None:
        if self.instance_info is None:
            labels, sizes = self.meta["labels"], self.meta["sizes"]
            ext = Extent(labels, sizes)
            rank_in_mesh = self.meta["ranks"].index(instance.rank)
            self.instance_info = ActorInstance(instance, proc_mesh=self.meta.get("proc_mesh_ref"),
                                               rank_point=Point(rank_in_mesh, ext))
        if self.obj is None:
            ctx = Context(self.instance_info, self.instance_info.rank)
            _tls.ctx = ctx
            bident = self.meta.get("broker_ident")
            if bident is not None:      # constructor arguments that are distributed tensors
                from ..tensor_engine import actor_bridge as ab
                tensors = ab.take_state(instance.proc_id, int(bident))
                self.args = ab.substitute(self.args, tensors)
                self.kwargs = ab.substitute(self.kwargs, tensors)
                self.meta["broker_ident"] = None
            self.obj = self.cls(*self.args, **self.kwargs)

    def _run(self, fn, args, kwargs):
        r = fn(*args, **kwargs)
        if inspect.iscoroutine(r):
            if self.loop is None:
                self.loop = asyncio.new_event_loop()
            asyncio.set_event_loop(self.loop)
            r = self.loop.run_until_complete(r)
        return r

    def _parse(self, env, instance=None):
        """(kind, method, fn, args, kwargs, response port, explicit, point) of a message."""
        try:
            msg = unflatten(env.data, env.parts, getattr(self, "_extra_load", None))
        except Exception as e:  # noqa: BLE001 - e.g. an argument whose __setstate__ raises
            reply = env.headers.get("reply_port")
            if reply is None or instance is None:
                raise
            body, parts = flatten((_KIND_EXCEPTION, int(env.headers.get("cast_rank", "0")),
                                   ActorError(e)))
            instance.send(reply, body, {"kind": _KIND_EXCEPTION, "no_return": "1"}, parts)
            return "undecodable", None, None, (), {}, None, False, \
                _cast_point(env.headers.get("cast_shape"), int(env.headers.get("cast_rank", "0")))
        kind = msg[0]
        cast_rank = int(env.headers.get("cast_rank", "0"))
        point = _cast_point(env.headers.get("cast_shape"), cast_rank)
        if kind == "init":
            return kind, None, None, (), {}, None, False, point
        _, method, args, kwargs, port = msg
        bident = env.headers.get("broker_ident")
        rref_port = None
        if bident is not None and instance is not None:
            # the call carries distributed tensors: take this proc's real ones from the broker
            # (python/monarch/mesh_controller.py actor_send in the reference)
            from ..tensor_engine import actor_bridge as ab
            if env.headers.get("broker_rref"):
                rref_port = ab.BrokerResultPort(instance.proc_id, int(bident))
            try:
                tensors = ab.take_state(instance.proc_id, int(bident))
                args, kwargs = ab.substitute(args, tensors), ab.substitute(kwargs, tensors)
            except Exception as e:  # noqa: BLE001 - answer with the error, stay alive
                if rref_port is not None:
                    rref_port.exception(ActorError(e))
                elif port is not None:
                    # no actor context yet at this point: post through the instance itself
                    body, parts = flatten((_KIND_EXCEPTION, cast_rank, ActorError(e)))
                    instance.send(port._port_id, body,
                                  {"kind": _KIND_EXCEPTION, "no_return": "1"}, parts)
                else:
                    raise
                return "undecodable", None, None, (), {}, None, False, point
        if isinstance(port, ReducePort):
            port = ReducePort(port._port_id, port._error_port_id, cast_rank,
                              via=env.headers.get("reduce_via"),
                              key=env.headers.get("reduce_key"))
        prop = getattr(self.cls, method, None)
        explicit = isinstance(prop, EndpointProperty) and prop._explicit_response_port
        if port is not None and not isinstance(port, ReducePort):
            via = None if explicit else env.headers.get("reduce_via")
            port = Port(port._port_id, cast_rank, via=via, key=env.headers.get("reduce_key"))
        response = port if port is not None else DroppingPort()
        if rref_port is not None:
            response = rref_port
        fn = prop._fn if isinstance(prop, EndpointProperty) else getattr(self.cls, method)
        return kind, method, fn, args, kwargs, response, explicit, point

    def on_message(self, instance, env) -> None:
        if self._has_async is None:
            self._has_async = any(
                isinstance(v, EndpointProperty) and inspect.iscoroutinefunction(v._fn)
                for klass in self.cls.__mro__ for v in vars(klass).values())
        if self._has_async:
            # an actor with async endpoints lives on its own event-loop thread: constructor,
            # sync and async endpoints all run there (one at a time, except that async
            # endpoints give way to each other and to later messages wherever they await)
            self._start_loop()
            self.loop.call_soon_threadsafe(self._handle_on_loop, instance, env)
            return
        t0 = time.perf_counter()
        kind, method, fn, args, kwargs, response, explicit, point = self._parse(env, instance)
        try:
            self._ensure(instance)
        except BaseException:
            _tls.ctx = None
            raise
        _tls.ctx = Context(self.instance_info, point)
        try:
            if kind == "init" or kind == "undecodable":
                return
            # every endpoint call runs inside a span when somebody is listening (event
            # capture or the chrome trace); otherwise the call pays nothing for it
            span_id = N.span_enter(f"{self.cls.__name__}.{method}", instance.actor_id) \
                if _tracing_on() else 0
            try:
                if explicit:
                    self._run(fn, (self.obj, response, *args), kwargs)
                else:
                    response.send(self._run(fn, (self.obj, *args), kwargs))
            except Exception as e:  # noqa: BLE001
                response.exception(ActorError(e))
            finally:
                if span_id:
                    N.span_exit(span_id)
            N.metrics_counter_add("py_messages_handled", 1)
        finally:
            _tls.ctx = None
            N.metrics_histogram_record("py_endpoint_us", (time.perf_counter() - t0) * 1e6)

    # ---- actors with async endpoints ---------------------------------------------------
    def _start_loop(self) -> None:
        if self.loop is None:
            self.loop = asyncio.new_event_loop()

            def main(loop=self.loop):
                asyncio.set_event_loop(loop)
                loop.run_forever()

            self._loop_thread = threading.Thread(target=main, daemon=True,
                                                 name=f"actor-loop-{self.name}")
            self._loop_thread.start()

    def _handle_on_loop(self, instance, env) -> None:
        """Runs on the actor's loop thread, in message order."""
        try:
            kind, method, fn, args, kwargs, response, explicit, point = self._parse(env, instance)
            try:
                self._ensure(instance)
                ctx = Context(self.instance_info, point)
                if kind == "init" or kind == "undecodable":
                    return
                if inspect.iscoroutinefunction(fn):
                    _tls.ctx = None
                    self.loop.create_task(self._run_async(instance, fn, args, kwargs, response,
                                                          explicit, ctx))
                    return
                _tls.ctx = ctx
                try:
                    if explicit:
                        fn(self.obj, response, *args, **kwargs)
                    else:
                        response.send(fn(self.obj, *args, **kwargs))
                except Exception as e:  # noqa: BLE001
                    response.exception(ActorError(e))
                N.metrics_counter_add("py_messages_handled", 1)
            finally:
                _tls.ctx = None
        except BaseException as e:  # noqa: BLE001 - nobody to answer to: the actor fails
            instance.fail(f"{type(e).__name__}: {e}\n{traceback.format_exc()}")

    async def _run_async(self, instance, fn, args, kwargs, response, explicit, ctx) -> None:
        _context.set(ctx)       # a task has its own copy of the context variables
        try:
            try:
                if explicit:
                    await fn(self.obj, response, *args, **kwargs)
                else:
                    response.send(await fn(self.obj, *args, **kwargs))
            except Exception as e:  # noqa: BLE001
                response.exception(ActorError(e))
            N.metrics_counter_add("py_messages_handled", 1)
        except BaseException as e:  # noqa: BLE001 - e.g. a broadcast endpoint that raised
            instance.fail(f"{type(e).__name__}: {e}\n{traceback.format_exc()}")

    def on_undeliverable(self, instance, env, reason: str) -> bool:
        if self.obj is None:
            return False
        return bool(self.obj._handle_undeliverable_message(env, reason))

    def on_stop(self, instance) -> None:
        if self.loop is not None:
            try:
                if self._loop_thread is not None:
                    self.loop.call_soon_threadsafe(self.loop.stop)
                    self._loop_thread.join(2.0)
                if not self.loop.is_running():
                    self.loop.close()
            except Exception:  # noqa: BLE001
                pass


def _python_actor_factory(proc, name: str, params: bytes):
    st = _ActorState(proc, name, params)
    return (st.on_message, None, st.on_undeliverable, st.on_stop)


N.register_python_actor_type("python", _python_actor_factory)
