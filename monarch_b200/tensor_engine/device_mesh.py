"""Controller side of the tensor engine: distributed ``Tensor``s on a ``DeviceMesh``.

Parity: python/monarch/common/tensor.py (Tensor wrapper subclass whose
``__torch_dispatch__`` turns every torch op into a worker message; ``reduce`` /
``reduce_`` / ``to_mesh`` / ``slice_mesh``), device_mesh.py (DeviceMesh.activate, slice /
split / rename / flatten, ``rank``), remote.py (``remote`` functions with shape
propagation, ``fetch_shard``, ``inspect``, ``call_on_shard_and_fetch``), client.py (seq
numbers, refs, deferred deletes), _coalescing.py (batched sends), stream.py / borrows.py
(streams and borrows), mesh_controller.py (RemoteException).

Shapes are propagated on FakeTensors in the controller; each op allocates result refs
and casts one ``call`` message to the workers of the active mesh (or appends it to the
open coalescing block).  Failures never kill a worker: the failing op's results carry
the error, dependants inherit it, and it surfaces as ``RemoteException`` on fetch.
"""
from __future__ import annotations

import contextlib
import itertools
import os
import socket
import threading
import traceback
import time
import warnings
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
from torch._subclasses.fake_tensor import FakeTensor as _FakeTensor
from torch._subclasses.fake_tensor import FakeTensorMode
from torch.utils._python_dispatch import TorchDispatchMode

from ..actor import Channel, Future
from ..actor.shape import MeshTrait, Shape
from .worker import PGRef, Ref, TensorWorker, _map_refs, _seq

_fake_mode = FakeTensorMode(allow_non_fake_inputs=True)


class RemoteException(Exception):
    """An op failed on a worker; raised when a value depending on it is fetched."""

    def __init__(self, seq: int, rank: int, func: str, exc_text: str, tb: str,
                 dependent_of: Optional[int] = None):
        self.seq, self.rank, self.func = seq, rank, func
        self.exc_text, self.worker_traceback, self.dependent_of = exc_text, tb, dependent_of
        dep = f" (caused by failed op {dependent_of})" if dependent_of is not None else ""
        super().__init__(f"remote function '{func}' failed on rank {rank}{dep}: {exc_text}\n"
                         f"Worker traceback:\n{tb}")


# ---------------------------------------------------------------------------- streams --
class WorkerTimeoutError(RuntimeError):
    """Some workers made no progress within the operation timeout."""

    def __init__(self, msg: str, ranks: List[int]):
        super().__init__(msg)
        self.ranks = ranks


class _ShapeMismatch(TypeError, ValueError):
    """Argument errors that the reference reports as TypeError in some places and ValueError
    in others; callers may catch either."""


class BorrowError(RuntimeError):
    """A tensor was used against the rules of a borrow (written while lent, written through
    a read-only borrow, used after the borrow was dropped).  Not a TypeError as in the
    reference: torch turns a TypeError raised under a binary operator (``x += 1``) into
    Python's "unsupported operand type(s)", which would hide the message."""


class Stream:
    _ids = itertools.count(1)

    def __init__(self, name: str, _default: bool = False):
        self.name = name
        self.id = 0 if _default else next(Stream._ids)
        self._default = _default
        self._created_on: set = set()

    def activate(self):
        return _activate_stream(self)

    def borrow(self, t: "Tensor", mutable: bool = False) -> Tuple["Tensor", "Borrow"]:
        """Make ``t`` usable on this stream.  Until the borrow is dropped the origin stream
        may not write (immutable borrow) or touch (mutable borrow) the tensor."""
        client = t.mesh.client
        client._ensure_stream(self)
        b = Borrow(next(Borrow._ids), t, self, mutable)
        out = Tensor(t._fake, t.mesh, self)
        client.send(t.mesh, ("borrow_create", b.id, Ref(t.ref), t.stream.id, self.id, Ref(out.ref)))
        t._borrowed_by.append(b)
        b._result = out
        out._borrow = b
        return out, b

    def __repr__(self):
        return f"<Stream {self.name!r}>"


_main_stream = Stream("main", _default=True)
_tls = threading.local()


def get_active_stream() -> Stream:
    return getattr(_tls, "stream", _main_stream)


@contextlib.contextmanager
def _activate_stream(s: Stream):
    prev = get_active_stream()
    _tls.stream = s
    try:
        yield
    finally:
        _tls.stream = prev


class Borrow:
    _ids = itertools.count(1)

    def __init__(self, id: int, origin: "Tensor", stream: Stream, mutable: bool):
        self.id, self.origin, self.stream, self.mutable = id, origin, stream, mutable
        self._dropped = False
        self._result: Optional[Tensor] = None

    def drop(self) -> None:
        if self._dropped:
            return
        self._dropped = True
        self.origin.mesh.client.send(self.origin.mesh, ("borrow_drop", self.id))
        if self in self.origin._borrowed_by:
            self.origin._borrowed_by.remove(self)
        if self._result is not None:
            self._result._dropped = True
            # remembered for the message of a later use of the borrowed tensor
            self._result._dropped_at = "".join(traceback.format_stack(limit=6)[:-1])

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.drop()

    def __del__(self):
        if not self._dropped:
            warnings.warn("borrow was never dropped; dropping it now", stacklevel=2)
            try:
                self.drop()
            except Exception:  # noqa: BLE001
                pass


# ----------------------------------------------------------------------------- client --
class Client:
    """Sequencing, ref allocation, batching and fetches for one tensor engine."""

    def __init__(self, proc_mesh, workers, use_cuda: bool):
        self.proc_mesh = proc_mesh
        self.workers = workers
        self.use_cuda = use_cuda
        self._init_history(len(workers))
        self._lock = threading.RLock()
        self._pending_deletes: List[int] = []
        self._coalesce: Optional[List[Tuple[Any, tuple]]] = None
        self._init_batching(int(os.environ.get("MB200_EAGER_BATCH", "16")))
        self.check_all_ranks_on_fetch = os.environ.get("MB200_FETCH_CHECKS_ALL_RANKS", "1") == "1"
        self._recording: Optional[List[tuple]] = None
        self._pg_init = False
        self._comms: set = set()
        self._streams_made: set = {0}
        self.errors: List[tuple] = []
        port, self._err_rx = Channel.open()
        workers.configure.call(port).get(timeout=60)
        self._closed = False
        self._init_watchdog(float(os.environ.get("MB200_OPERATION_TIMEOUT", "120")))

    def _init_history(self, world: int) -> None:
        """Sequence numbers, ref ids, the invocations in flight, the workers' progress and
        what is known to be poisoned live in the native ``ControllerHistory``."""
        from .. import _native as N
        self.history = N.ControllerHistory(world)

    def _init_batching(self, eager_batch: int) -> None:
        """``eager_batch``: how many eager commands may wait for one cast (1 sends each on
        its own)."""
        self.eager_batch = eager_batch
        self._pending: List[Tuple[Any, tuple]] = []
        self._pending_cmds = 0          # commands in _pending (ref deletions do not count)
        self._pending_since = 0.0       # when the oldest of them was queued
        self._plock = threading.RLock()
        self._flusher: Optional[threading.Thread] = None
        self._flush_event = threading.Event()

    def _init_watchdog(self, operation_timeout: float) -> None:
        """Progress watchdog (controller/src/lib.rs:263-336 CheckWorkerProgress): a ping
        rides the command stream; ranks that have not answered it within
        ``operation_timeout`` seconds are stuck behind a command.  0 disables it."""
        self.operation_timeout = operation_timeout
        self.fail_on_worker_timeout = os.environ.get("MB200_FAIL_ON_WORKER_TIMEOUT", "0") == "1"
        self.progress_interval = 5.0
        self.stalls: List[dict] = []
        self._ping: Optional[dict] = None
        self._last_ping = time.monotonic()
        self._failed: Optional[Exception] = None

    def new_seq(self) -> int:
        return self.history.next_seq()

    def new_ref(self) -> int:
        return self.history.next_ref()

    def delete_ref(self, ref: int) -> None:
        with self._lock:
            self._pending_deletes.append(ref)

    def known_failure(self, t: "Tensor") -> Optional["RemoteException"]:
        """The failure that poisons ``t`` as far as the controller has heard (error reports
        arrive asynchronously), without asking the workers; None if it knows of none."""
        self.drain_errors()
        origin = self.history.ref_failed(t.ref)
        if origin < 0:
            return None
        f = self.history.failure(origin)
        if f is None:
            return None
        seq, rank, name, text = f
        return RemoteException(seq, rank, name, text, "", None)

    def _send_deletes(self) -> None:
        """Refs are dropped on every worker, whichever sub-mesh the next message goes to."""
        d = self._flush_deletes(None)
        if d:
            _cast_run(self.root_mesh._workers, d)

    def _flush_deletes(self, mesh) -> List[tuple]:
        with self._lock:
            if not self._pending_deletes:
                return []
            ids, self._pending_deletes = self._pending_deletes, []
        self.history.forget_refs(ids)
        return [("delete", ids)]

    def send(self, mesh: "DeviceMesh", msg: tuple) -> None:
        """Queue ``msg`` for the workers of ``mesh`` (cast now, or at the end of the open
        coalescing block)."""
        if self._closed:
            raise RuntimeError("the tensor engine was shut down")
        if self._coalesce is not None:
            self._coalesce.append((mesh, msg))
            return
        if self.eager_batch <= 1:
            self._watch()
            self._send_deletes()
            _cast_run(mesh._workers, [msg])
            return
        # eager commands are handed to the workers a few at a time: every cast costs the
        # controller a pickle and a trip through the native runtime, and the workers execute
        # asynchronously anyway.  Whatever needs an answer flushes first; a background thread
        # flushes what is left within a millisecond.
        with self._plock:
            if self._pending_deletes and mesh._workers is self.root_mesh._workers:
                # refs dropped before this command was issued are dropped before it runs
                # (joins the run of commands to all workers, so it costs no cast)
                self._pending.extend((mesh, d) for d in self._flush_deletes(None))
            self._pending.append((mesh, msg))
            self._pending_cmds += 1
            if self._pending_cmds >= self.eager_batch:
                self._flush_locked()
            elif self._pending_cmds == 1:
                # the first command of a batch starts the clock; while the program keeps
                # issuing, batches fill up and leave from here, and the flusher only sees to
                # a batch that has been waiting for a millisecond
                self._pending_since = time.monotonic()
                self._kick_flusher()

    def flush(self) -> None:
        """Hand every buffered command to the workers now."""
        with self._plock:
            self._flush_locked()

    def _flush_locked(self) -> None:
        if not self._pending:
            return
        batch, self._pending = self._pending, []
        self._pending_cmds = 0
        self._send_runs(batch)

    def _send_runs(self, batch: List[Tuple[Any, tuple]]) -> None:
        """One cast per run of consecutive messages to the same workers: program order is
        kept across meshes too (a message to a sub-mesh may read what an earlier message to
        the whole mesh wrote, and the other way round)."""
        runs: List[Tuple[Any, List[tuple]]] = []
        for mesh, msg in batch:
            if runs and runs[-1][0]._workers is mesh._workers:
                runs[-1][1].append(msg)
            else:
                runs.append((mesh, [msg]))
        for mesh, msgs in runs:
            _cast_run(mesh._workers, msgs)
        # refs dropped by the controller go last: a buffered command may still name them
        # (a ref that is already dropped cannot appear in any later command)
        self._send_deletes()

    def _kick_flusher(self) -> None:
        if self._flusher is None:
            self._flusher = threading.Thread(target=self._flusher_loop, daemon=True,
                                             name="tensor-engine-flush")
            self._flusher.start()
        self._flush_event.set()

    def _flusher_loop(self) -> None:
        while not self._closed:
            self._flush_event.wait()
            self._flush_event.clear()
            while not self._closed:
                with self._plock:
                    if not self._pending:
                        break
                    age = time.monotonic() - self._pending_since
                    if age >= 0.001:
                        try:
                            self._flush_locked()
                        except Exception as e:  # noqa: BLE001 - surfaces at the next command
                            self._failed = e
                        break
                time.sleep(0.0011 - age)        # let the burst of commands accumulate

    def _watch(self) -> None:
        """Progress watchdog step; called from the command path and from waits, so it needs
        no thread of its own.  Raises :class:`WorkerTimeoutError` once a stall was seen and
        ``fail_on_worker_timeout`` is set."""
        if self._failed is not None:
            raise self._failed
        if self.operation_timeout <= 0 or self._closed:
            return
        now = time.monotonic()
        h = self.history
        if self._ping is not None:
            rx = self._ping
            while True:
                env = rx._rx.try_recv()
                if env is None:
                    break
                from ..actor.pickle import unflatten
                _, rank, last_seq = unflatten(env.data, env.parts)
                if h.ping_answered(rank, last_seq):
                    rx.close()
                    self._ping = None
                    break
            stall = h.stalled(now, self.operation_timeout) if self._ping is not None else None
            if stall is not None:
                self.stalls.append(stall)
                at = h.describe(h.min_completed() + 1)
                msg = (f"tensor workers {stall['ranks']} made no progress for "
                       f"{stall['waited_s']:.1f} s (operation timeout "
                       f"{self.operation_timeout:.1f} s, controller at seq "
                       f"{stall['controller_seq']}"
                       + (f", oldest unfinished command {at[0]}" if at else "") + ")")
                import logging
                logging.getLogger("monarch_b200.tensor_engine").warning(msg)
                if self.fail_on_worker_timeout:
                    self._failed = WorkerTimeoutError(msg, stall["ranks"])
                    raise self._failed
        if self._ping is None and now - self._last_ping >= self.progress_interval:
            self.flush()     # the ping stands behind everything issued so far
            ep = self.root_mesh._workers.progress
            port, rx = ep._open()
            ep._send((), {}, port)
            self._last_ping = now
            self._ping = rx
            h.ping_sent(h.next_seq(), now)

    def _ensure_stream(self, s: Stream) -> None:
        if s.id not in self._streams_made:
            self._streams_made.add(s.id)
            self.send(self.root_mesh, ("create_stream", s.id, s._default))

    @contextlib.contextmanager
    def coalescing(self):
        if self._coalesce is not None:
            yield
            return
        self.flush()
        self._coalesce = []
        try:
            yield
        finally:
            batch, self._coalesce = self._coalesce, None
            with self._plock:
                self._flush_locked()
                self._send_runs(batch)

    def ensure_process_group(self) -> None:
        if self._pg_init:
            return
        self._pg_init = True
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
        s.close()
        ranks = self.root_mesh._ndslice.ranks()
        self.send(self.root_mesh, ("init_pg", "127.0.0.1", port, ranks))

    def _groups_over(self, mesh: "DeviceMesh", dims: Tuple[str, ...]):
        sl = mesh._ndslice
        labels = list(mesh._labels)
        idx = [labels.index(d) for d in dims]
        key = (sl.offset, tuple(sl.sizes), tuple(sl.strides), tuple(idx))
        other = [i for i in range(len(labels)) if i not in idx]
        groups: List[List[int]] = []
        for oc in itertools.product(*[range(sl.sizes[i]) for i in other]):
            ranks = []
            for gc in itertools.product(*[range(sl.sizes[i]) for i in idx]):
                coord = [0] * len(labels)
                for i, c in zip(other, oc):
                    coord[i] = c
                for i, c in zip(idx, gc):
                    coord[i] = c
                ranks.append(sl.nditem(coord))
            groups.append(ranks)
        return key, groups

    def ensure_comm(self, mesh: "DeviceMesh", dims: Tuple[str, ...], stream_id: int = 0,
                    own: bool = False) -> Tuple[int, ...]:
        """Communicators over ``dims`` of ``mesh``: one per combination of the other dims'
        coordinates.  Returns the key workers use to look theirs up.

        ``own=True`` (GPU workers, operations the NVLink kernels cover): every member
        allocates a staging buffer and exports a CUDA IPC handle, the handles come back to
        the controller in the reply and go out again in the next message -- the bootstrap
        rides the actor control plane and needs no ``torch.distributed`` (the reference
        bootstraps NCCL the same way: the unique id travels in a worker message,
        monarch_tensor_worker/src/lib.rs:303-364).  One communicator per (dims, stream):
        collectives of two streams may overlap on the GPU and must not share staging.
        Otherwise: ``torch.distributed`` groups (gloo on CPU workers; NCCL for what the
        kernels do not cover)."""
        key, groups = self._groups_over(mesh, dims)
        if own:
            okey = ("own", key, stream_id)
            hkey = (hash(okey) % (1 << 62),)
            if okey in self._comms:
                return hkey
            self.flush()
            root = self.root_mesh._workers
            exports = root.comm_export.call(hkey, groups).get(timeout=120)
            by_rank = {}
            for point, exp in exports.items():
                if isinstance(exp, dict) and "error" in exp:
                    raise RuntimeError(f"communicator over {dims}: {exp['error']}")
                if exp is not None:
                    by_rank[exp["rank"]] = exp
            for ranks in groups:
                devs = [(by_rank[r]["host"], by_rank[r]["device"]) for r in ranks]
                if len(set(devs)) != len(devs):
                    raise RuntimeError(
                        f"communicator over {dims}: ranks {ranks} share a GPU {devs}; kernels "
                        "that wait on one another need one GPU per rank")
            root.comm_connect.broadcast(hkey, by_rank)
            self._comms.add(okey)
            return hkey
        self.ensure_process_group()
        hkey = (hash(key) % (1 << 62),)
        if key in self._comms:
            return hkey
        self._comms.add(key)
        self.send(self.root_mesh, ("split_comm", hkey, groups))
        return hkey

    def fetch(self, mesh: "DeviceMesh", ref_tree, preprocess=None, timeout: Optional[float] = None):
        seq = self.new_seq()
        self._watch()
        self.flush()
        self._send_deletes()
        ep = mesh._workers.run_and_reply
        if not hasattr(ep, "_open"):      # simulated workers answer synchronously
            vm = ep.call([], (seq, ref_tree, preprocess)).get(timeout)
            return Future(lambda t: [self._unwrap_reply(r) for _, r in vm.items()])
        mesh._workers._raise_if_unhealthy()
        port, rx = ep._open()
        ep._send(([], (seq, ref_tree, preprocess)), {}, port)
        n = len(mesh._workers)

        def wait(t):
            # replies are unpickled into ordinary local tensors: keep the active-mesh
            # dispatch mode out of the way while that happens
            t = t if t is not None else timeout
            deadline = None if t is None else time.monotonic() + t
            prev = getattr(_tls, "propagating", False)
            _tls.propagating = True
            replies: List[Any] = [None] * n
            got = 0
            try:
                while got < n:
                    left = 1.0 if deadline is None else min(1.0, max(deadline - time.monotonic(), 0.0))
                    try:
                        rank, v = rx._next(left)
                    except TimeoutError:
                        self._watch()      # the wait doubles as the watchdog's clock
                        if deadline is not None and time.monotonic() >= deadline:
                            raise
                        continue
                    replies[rank] = v
                    got += 1
            finally:
                _tls.propagating = prev
                rx.close()
            return [self._unwrap_reply(r) for r in replies]

        return Future(wait)

    @staticmethod
    def _unwrap_reply(r):
        if r[0] == "error":
            raise RemoteException(*r[1:])
        return r[1]

    def drain_errors(self) -> List[tuple]:
        while self._err_rx is not None:
            env = self._err_rx._rx.try_recv()
            if env is None:
                break
            from ..actor.pickle import unflatten
            _, _, payload = unflatten(env.data, env.parts)
            self.errors.append(payload)
            if isinstance(payload, tuple) and len(payload) >= 5 and payload[0] == "error":
                # poison, on the controller's books, what the failed command defines and
                # everything issued since that read it
                self.history.fail(int(payload[1]), int(payload[2]), str(payload[3]),
                                  str(payload[4]))
        return self.errors

    def shutdown(self) -> None:
        try:
            self.flush()
        except Exception:  # noqa: BLE001 - the workers may be gone already
            pass
        self._closed = True
        self._flush_event.set()


def _cast_run(workers, msgs: List[tuple]) -> None:
    """``workers.run.broadcast(msgs)``.  Operator calls and deletions hold only refs, numbers,
    strings, dtypes and the like (an ATen operator takes no callables), so batches of those
    skip the general pickler, whose per-object hooks cost more than the cast itself."""
    plain = True
    for m in msgs:
        k = m[0]
        if not (k == "delete" or (k == "call" and m[4][0] == "op")):
            plain = False
            break
    if not plain or not hasattr(workers, "_cast"):      # (simulated workers have no cast)
        workers.run.broadcast(msgs)
        return
    workers._raise_if_unhealthy()
    workers._cast(("call", "run", (msgs,), {}, None), plain=True)


# ----------------------------------------------------------------------------- tensor --
class Tensor(torch.Tensor):
    """A tensor that lives on every proc of a device mesh.  The controller holds only its
    metadata (a FakeTensor); data is named by ``ref`` on the workers."""

    @staticmethod
    def __new__(cls, fake, mesh: "DeviceMesh", stream: Stream):
        if type(fake) is _LazyFake:
            # metadata remembered from an earlier propagation of the same operator: the
            # FakeTensor itself (30 us to build) is made only if something asks for it
            _, shape, stride, dtype, device, req = fake.t
            r = torch.Tensor._make_wrapper_subclass(
                cls, shape, strides=stride, dtype=dtype, device=device, requires_grad=req)
            r._fake_obj = None
            r._tmpl = fake.t
        else:
            r = torch.Tensor._make_wrapper_subclass(
                cls, fake.size(), strides=fake.stride(), storage_offset=fake.storage_offset(),
                dtype=fake.dtype, device=fake.device, layout=fake.layout,
                requires_grad=fake.requires_grad)
            r._fake_obj = fake
            r._tmpl = None
        r.mesh = mesh
        r.stream = stream
        r.ref = mesh.client.new_ref()
        r._dropped = False
        r._borrowed_by = []
        return r

    def __init__(self, *a, **k):
        pass

    @property
    def _fake(self) -> torch.Tensor:
        f = self._fake_obj
        if f is None:
            prev = getattr(_tls, "propagating", False)
            _tls.propagating = True        # the factory call below is not a mesh operation
            try:
                f = self._fake_obj = _from_template(self._tmpl)
            finally:
                _tls.propagating = prev
        return f

    def __repr__(self, *, tensor_contents=None):
        return f"monarch_b200.Tensor(mesh={self.mesh}, ref={self.ref}, fake={self._fake})"

    def __del__(self):
        try:
            if not self._dropped and self.ref is not None:
                self.mesh.client.delete_ref(self.ref)
        except Exception:  # noqa: BLE001 - interpreter teardown
            pass

    def drop(self) -> None:
        if not self._dropped:
            self._dropped = True
            self.mesh.client.delete_ref(self.ref)

    @property
    def dropped(self) -> bool:
        return self._dropped

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        return _dispatch(func, args, kwargs or {})

    # ---- collectives -------------------------------------------------------------------
    def reduce(self, dims, reduction: str = "sum", scatter: bool = False, mesh=None,
               _inplace: bool = False, out: Optional["Tensor"] = None) -> "Tensor":
        """Reduce across mesh dims.  ``reduction`` in {sum, avg, product, min, max, band,
        bor, bxor, stack}; ``scatter=True`` keeps slice i of the outer dim on member i
        (reduce-scatter; with ``"stack"`` an all-to-all); ``"stack"`` alone all-gathers."""
        _check_usable(self)
        if isinstance(dims, str):
            dims = (dims,)
        dims = tuple(dims)
        m = self.mesh
        if not dims:                         # () stands for every dim of the mesh
            dims = tuple(m._labels)
        for d in dims:
            if d not in m._labels:
                raise KeyError(f"{m} has no dimension {d!r}")
        if reduction not in _REDUCTIONS:
            raise ValueError(f"reduction {reduction!r} not in {sorted(_REDUCTIONS)}")
        n = 1
        for d in dims:
            n *= m.size(d)
        if (reduction == "stack" or scatter) and len(dims) != 1:
            what = "stack" if reduction == "stack" else f"{reduction} with scatter"
            raise _ShapeMismatch(f"reduction {what!r} is not valid for multiple dimensions "
                                 f"{dims}: it takes exactly one mesh dim")
        if get_active_stream() is not self.stream:
            raise TypeError(f"WRONG_STREAM: the tensor lives on stream {self.stream.name!r} but "
                            f"{get_active_stream().name!r} is active; borrow it to that stream "
                            "first")
        f = self._fake
        if reduction == "stack":
            if scatter:
                if f.dim() == 0 or f.shape[0] != n:
                    raise _ShapeMismatch(f"When scattering, the outer dimension must equal the "
                                         f"size of the reduced mesh dim ({n}); all-to-all got "
                                         f"{tuple(f.shape)}")
                out_fake = _new_fake(f.shape, f)
            else:
                out_fake = _new_fake((n, *f.shape), f)
        elif scatter:
            if f.dim() == 0 or f.shape[0] != n:
                raise _ShapeMismatch(f"When scattering, the outer dimension must equal the size "
                                     f"of the reduced mesh dim ({n}); reduce-scatter got "
                                     f"{tuple(f.shape)}")
            out_fake = _new_fake(f.shape[1:], f)
        else:
            out_fake = _new_fake(f.shape, f)
        if out is not None and (tuple(out._fake.shape) != tuple(out_fake.shape)
                                or out._fake.dtype != out_fake.dtype):
            raise ValueError(f"Reduce expects the shape to be {out_fake.shape} and the dtype "
                             f"{out_fake.dtype}, but out= has {out._fake.shape} and "
                             f"{out._fake.dtype}")
        if _inplace and tuple(out_fake.shape) != tuple(f.shape):
            raise ValueError("in-place reduce needs matching input and output shapes")
        client = m.client
        if getattr(client, "null_device", False):
            key = ("null", n)              # shape-only workers: no communicator exists
        else:
            own = client.use_cuda and _own_collective(f.dtype, reduction)
            key = client.ensure_comm(m, dims, self.stream.id, own=own)
        seq = client.new_seq()
        if _inplace:
            result = self
            res_ref = Ref(self.ref)
        else:
            result = Tensor(out_fake, m, self.stream)
            res_ref = Ref(result.ref)
        client.history.add_invocation(
            seq, f"reduce.{reduction}",
            [res_ref.id] + ([out.ref] if out is not None else []), [self.ref])
        client.send(m, ("reduce", seq, res_ref, Ref(self.ref), key, reduction, scatter, _inplace,
                        Ref(out.ref) if out is not None else None, self.stream.id,
                        (tuple(f.shape), f.dtype)))
        return out if out is not None else result

    def reduce_(self, dims, reduction: str = "sum", scatter: bool = False, mesh=None) -> "Tensor":
        return self.reduce(dims, reduction, scatter, mesh, _inplace=True)

    def to_mesh(self, mesh: "DeviceMesh", stream: Optional[Stream] = None) -> "Tensor":
        """Move to another mesh (point-to-point sends): rank i of this mesh to rank i of a
        mesh with as many ranks, or -- when ``mesh`` has every dim of this mesh plus others --
        each value to all ranks of ``mesh`` with the same coordinates in the shared dims (a
        broadcast along the other dims, e.g. from ``mesh.slice(host=1)`` to ``mesh``)."""
        _check_usable(self)
        src = self.mesh
        if mesh is src or (mesh._ndslice == src._ndslice):
            # nothing to send, but the result is a value of its own (writing the original
            # afterwards must not show through it)
            return torch.ops.aten.clone.default(self)
        fr, to = src._ndslice.ranks(), mesh._ndslice.ranks()
        if len(fr) != len(to):
            fr = _broadcast_sources(src, mesh)
        client = src.client
        client.ensure_process_group()
        out = Tensor(self._fake, mesh, stream or self.stream)
        seq = client.new_seq()
        root = client.root_mesh
        client.send(root, ("send_meta", Ref(out.ref), tuple(self._fake.shape), self._fake.dtype))
        client.send(root, ("send_tensor", seq, Ref(out.ref), Ref(self.ref), fr, to,
                           self.stream.id, out.stream.id))
        return out

    def slice_mesh(self, **kwargs) -> "Tensor":
        """The same per-proc values viewed on a sub-mesh (no data moves)."""
        sub = self.mesh.slice(**kwargs)
        t = Tensor(self._fake, sub, self.stream)
        sub.client.send(sub, ("call", sub.client.new_seq(), [Ref(t.ref)], [],
                              ("pickle", _identity), (Ref(self.ref),), {}, self.stream.id))
        return t


_REDUCTIONS = {"stack", "sum", "avg", "product", "min", "max", "band", "bor", "bxor"}


def _identity(x):
    return x


@contextlib.contextmanager
def _propagation():
    """Run torch code on FakeTensors for shape inference, with the active-mesh dispatch
    mode standing aside."""
    prev = getattr(_tls, "propagating", False)
    _tls.propagating = True
    try:
        with _fake_mode:
            yield
    finally:
        _tls.propagating = prev


def _new_fake(shape, like) -> torch.Tensor:
    with _propagation():
        return torch.empty(tuple(shape), dtype=like.dtype, device=like.device)


def _check_usable(t: Tensor) -> None:
    if t._dropped:
        at = getattr(t, "_dropped_at", None)
        raise BorrowError(f"tensor {tuple(t.shape)} is dropped at:\n{at}" if at else
                          "this tensor was dropped (or its borrow has ended)")
    for b in t._borrowed_by:
        if b.mutable and get_active_stream() is not b.stream:
            raise RuntimeError("tensor is mutably borrowed by another stream; drop the borrow first")


def _own_collective(dtype, reduction: str) -> bool:
    """Whether GPU workers run this reduce on the package's NVLink kernels (the rest --
    bitwise reductions, dtypes without an arithmetic kernel -- goes to NCCL)."""
    if os.environ.get("MB200_TE_COLLECTIVES", "own") != "own":
        return False
    from ..parallel import meshcomm
    return meshcomm.supports(dtype, None if reduction == "stack" else reduction)


def reduce(tensors, dims, reduction="sum", scatter=False, mesh=None, _inplace=False):
    from torch.utils._pytree import tree_map
    return tree_map(lambda t: t.reduce(dims, reduction, scatter, mesh, _inplace)
                    if isinstance(t, Tensor) else t, tensors)


def reduce_(tensors, dims, reduction="sum", scatter=False, mesh=None):
    return reduce(tensors, dims, reduction, scatter, mesh, _inplace=True)


def to_mesh(tensors, mesh, stream=None):
    from torch.utils._pytree import tree_map
    return tree_map(lambda t: t.to_mesh(mesh, stream) if isinstance(t, Tensor) else t, tensors)


def slice_mesh(tensors, **kwargs):
    from torch.utils._pytree import tree_map
    return tree_map(lambda t: t.slice_mesh(**kwargs) if isinstance(t, Tensor) else t, tensors)


# --------------------------------------------------------------------------- dispatch --
def _collect(obj, out: List[Tensor]) -> None:
    if isinstance(obj, Tensor):
        out.append(obj)
    elif isinstance(obj, (list, tuple)):
        for o in obj:
            _collect(o, out)
    elif isinstance(obj, dict):
        for o in obj.values():
            _collect(o, out)
    elif getattr(type(obj), "_holds_tensors", False):      # e.g. the key of an OpaqueRef
        _collect(obj._tensors(), out)


def _to_fake(obj):
    if isinstance(obj, Tensor):
        return obj._fake
    if isinstance(obj, torch.Tensor):
        return obj
    if isinstance(obj, (list, tuple)):
        return _seq(obj, (_to_fake(o) for o in obj))
    if isinstance(obj, dict):
        return {k: _to_fake(v) for k, v in obj.items()}
    if getattr(type(obj), "_holds_tensors", False):
        return obj._rebuild(_to_fake(obj._tensors()))
    if isinstance(obj, RemoteProcessGroup):
        return shape_only_group(obj.dims, obj.size())
    return obj


def _to_wire(obj):
    if isinstance(obj, Tensor):
        return Ref(obj.ref)
    if isinstance(obj, RemoteProcessGroup):
        return PGRef(obj.key)
    if isinstance(obj, (list, tuple)):
        return _seq(obj, (_to_wire(o) for o in obj))
    if isinstance(obj, dict):
        return {k: _to_wire(v) for k, v in obj.items()}
    if getattr(type(obj), "_holds_tensors", False):
        return obj._rebuild(_to_wire(obj._tensors()))
    return obj


def _wrap_outputs(fake_out, mesh, stream, refs: List[Ref]):
    if type(fake_out) is _LazyFake or isinstance(fake_out, torch.Tensor):
        t = Tensor(fake_out, mesh, stream)
        refs.append(Ref(t.ref))
        return t
    if isinstance(fake_out, (list, tuple)):
        return _seq(fake_out, (_wrap_outputs(o, mesh, stream, refs) for o in fake_out))
    if isinstance(fake_out, dict):
        return {k: _wrap_outputs(v, mesh, stream, refs) for k, v in fake_out.items()}
    if getattr(type(fake_out), "_holds_tensors", False):
        return fake_out._rebuild(_wrap_outputs(fake_out._tensors(), mesh, stream, refs))
    return fake_out


def _send_call(fspec, args, kwargs, fake_out, mesh: "DeviceMesh", mutates: Sequence[Tensor] = (),
               uses: Optional[List[Tensor]] = None):
    stream = get_active_stream()
    client = mesh.client
    client._ensure_stream(stream)
    refs: List[Ref] = []
    out = _wrap_outputs(fake_out, mesh, stream, refs)
    seq = client.new_seq()
    if uses is None:
        uses = []
        _collect(args, uses)
        _collect(kwargs, uses)
    f = fspec[1]
    client.history.add_invocation(
        seq, f if isinstance(f, str) else getattr(f, "__name__", "function"),
        [r.id for r in refs] + [t.ref for t in mutates], [t.ref for t in uses])
    msg = ("call", seq, refs, [Ref(t.ref) for t in mutates], fspec, _to_wire(args),
           _to_wire(kwargs), stream.id)
    if getattr(client, "null_device", False) or getattr(client, "send_metas", False):
        # shape-only workers do not run the function: they need the results' metadata
        flat: List[Tensor] = []
        _collect(out, flat)
        msg += ([(tuple(t.shape), t.dtype) for t in flat],)
    client.send(mesh, msg)
    return out


def _broadcast_sources(src: "DeviceMesh", dst: "DeviceMesh") -> List[int]:
    """For every rank of ``dst`` (in its own order) the rank of ``src`` whose value it gets:
    the one with the same coordinates in the dims that ``src`` has."""
    s_nd, d_nd = src._ndslice, dst._ndslice
    d_labels = list(dst._labels)
    where = []
    for l, n in zip(src._labels, s_nd.sizes):
        if n == 1:
            where.append(None)
            continue
        if l not in d_labels or d_nd.sizes[d_labels.index(l)] != n:
            raise ValueError(f"cannot move between meshes of different sizes: {src} -> {dst} "
                             f"(dim {l!r} of the source has no equal dim in the destination)")
        where.append(d_labels.index(l))
    out = []
    for i in range(len(d_nd.ranks())):
        coords, rest = [], i
        for n in reversed(d_nd.sizes):
            coords.append(rest % n)
            rest //= n
        coords.reverse()
        r = s_nd.offset
        for w, st in zip(where, s_nd.strides):
            if w is not None:
                r += coords[w] * st
        out.append(r)
    return out


def _mesh_of(tensors: List[Tensor]) -> "DeviceMesh":
    m = tensors[0].mesh
    for t in tensors[1:]:
        if t.mesh is not m and t.mesh._ndslice != m._ndslice:
            # a ValueError, not the reference's TypeError: under ``x + y`` torch would
            # turn a TypeError into "unsupported operand type(s)" and lose this message
            raise ValueError(f"WRONG_MESH: tensors live on different meshes ({m} vs "
                             f"{t.mesh}); move one with to_mesh() first")
    return m


# ---- cached shape propagation -------------------------------------------------------------
# Running an operator on FakeTensors costs 100-300 us in this torch (meta kernels and
# decompositions written in Python); the answer depends only on the operator and on the
# metadata of its arguments.  Functional operators (no aliasing or mutation in the schema) are
# therefore propagated once per distinct signature; later calls rebuild the output fakes from
# the remembered shapes, strides and dtypes (python/monarch/common/function_caching.py plays
# this role for remote functions in the reference).
class _Uncacheable(Exception):
    pass


_PLAIN_ARG_TYPES = (int, float, bool, str, type(None), torch.dtype, torch.device, torch.layout,
                    torch.memory_format, complex)
_prop_cache: Dict[tuple, Any] = {}
_cacheable_op: Dict[Any, bool] = {}
_PROP_CACHE_MAX = 4096


def _op_is_functional(func) -> bool:
    r = _cacheable_op.get(func)
    if r is None:
        sch = func._schema
        r = not any(a.alias_info is not None for a in sch.arguments) and \
            not any(x.alias_info is not None for x in sch.returns)
        _cacheable_op[func] = r
    return r


def _arg_sig(o):
    tp = type(o)
    if tp is Tensor:
        f = o._fake_obj
        if f is None:
            return o._tmpl
        return ("T", tuple(f.shape), f.stride(), f.dtype, f.device, f.requires_grad)
    if tp in _PLAIN_ARG_TYPES:
        return (tp, o)
    if tp is list or tp is tuple:
        return (tp, tuple(_arg_sig(x) for x in o))
    if tp is dict:
        return (tp, tuple((k, _arg_sig(v)) for k, v in o.items()))
    if tp is torch.Size:
        return (tp, tuple(o))
    raise _Uncacheable()


def _out_template(o):
    if isinstance(o, torch.Tensor):
        return ("T", tuple(o.shape), tuple(o.stride()), o.dtype, o.device, o.requires_grad)
    if isinstance(o, (list, tuple)):
        return ("S", type(o), [_out_template(x) for x in o])
    if type(o) in _PLAIN_ARG_TYPES:
        return ("V", o)
    raise _Uncacheable()


class _LazyFake:
    """Stands for the FakeTensor that ``_from_template(t)`` would build."""
    __slots__ = ("t",)

    def __init__(self, t):
        self.t = t


def _from_template(t, lazy: bool = False):
    if t[0] == "T":
        if lazy:
            return _LazyFake(t)
        _, shape, stride, dtype, device, req = t
        meta = torch.empty_strided(shape, stride, dtype=dtype, device="meta")
        f = _FakeTensor(_fake_mode, meta, device)
        return f.requires_grad_(True) if req else f
    if t[0] == "S":
        return t[1](_from_template(x, lazy) for x in t[2])
    return t[1]


def _propagate(func, args, kwargs):
    """Output fakes of ``func(*args, **kwargs)`` (``Tensor`` arguments stand for their fakes)."""
    key = None
    if _op_is_functional(func):
        try:
            key = (func, _arg_sig(args), _arg_sig(kwargs) if kwargs else None,
                   torch.is_grad_enabled())
            tmpl = _prop_cache.get(key)
            if tmpl is not None:
                return _from_template(tmpl, lazy=True)
        except (_Uncacheable, TypeError):     # TypeError: an unhashable argument
            key = None
    with _propagation():
        fake_out = func(*_to_fake(args), **_to_fake(kwargs))
    if key is not None:
        try:
            if len(_prop_cache) >= _PROP_CACHE_MAX:
                _prop_cache.clear()
            _prop_cache[key] = _out_template(fake_out)
        except _Uncacheable:
            pass
    return fake_out


# operators whose result is a Python value computed from tensor data: the controller holds no
# data, so these cannot be answered here
_DATA_DEPENDENT = {"_local_scalar_dense", "item", "is_nonzero", "equal", "allclose", "nonzero",
                   "unique", "_unique2", "masked_select"}


_op_info: Dict[Any, tuple] = {}


def _info_of(func) -> tuple:
    """(data dependent?, wire name, [(position, name) of arguments the operator writes])."""
    info = _op_info.get(func)
    if info is None:
        schema = func._schema
        short = schema.name.split("::")[1]
        writes = [(i, a.name) for i, a in enumerate(schema.arguments)
                  if a.alias_info is not None and a.alias_info.is_write]
        info = _op_info[func] = (short in _DATA_DEPENDENT,
                                 f"{func.namespace}.{short}.{func._overloadname}", writes)
    return info


def _dispatch(func, args, kwargs, ts: Optional[List["Tensor"]] = None):
    data_dependent, name, writes = _info_of(func)
    if data_dependent:
        raise RuntimeError(
            f"{func._schema.name} needs the values of a distributed tensor, which live on the "
            "workers.  Bring them to the controller with fetch_shard(t).get() or inspect(t), "
            "or compute on the workers inside a remote function.")
    if ts is None:                      # (the active-mesh mode has collected them already)
        ts = []
        _collect(args, ts)
        _collect(kwargs, ts)
    if ts:
        mesh = _mesh_of(ts)
        for t in ts:
            _check_usable(t)
    else:
        mesh = get_active_mesh()
        if mesh is None:
            raise RuntimeError("no active device mesh")
    fake_out = _propagate(func, args, kwargs)
    # in-place / out= ops return their (already remote) argument: alias, do not re-ref
    mutated: List[Tensor] = []
    if writes:
        for i, arg_name in writes:
            v = args[i] if i < len(args) else kwargs.get(arg_name)
            if isinstance(v, Tensor):
                if v._borrowed_by and any(b.stream is not get_active_stream()
                                          for b in v._borrowed_by):
                    raise BorrowError(f"{name}: the tensor would be mutated while stream "
                                    f"{v._borrowed_by[0].stream.name!r} borrows it; drop the "
                                    "borrow first")
                b = getattr(v, "_borrow", None)
                if b is not None and not b.mutable:
                    raise BorrowError(f"{name}: the tensor would be mutated through a read-only "
                                    "borrow; borrow it with mutable=True")
                mutated.append(v)
    if mutated and isinstance(fake_out, torch.Tensor) and len(mutated) == 1:
        client = mesh.client
        stream = get_active_stream()
        seq = client.new_seq()
        client.history.add_invocation(seq, name, [t.ref for t in mutated], [t.ref for t in ts])
        client.send(mesh, ("call", seq, [], [Ref(t.ref) for t in mutated],
                           ("op", name), _to_wire(args), _to_wire(kwargs), stream.id))
        return mutated[0]
    return _send_call(("op", name), args, kwargs, fake_out, mesh, mutated, ts)


# ------------------------------------------------------------------------ device mesh --
_active: List["DeviceMesh"] = []


def get_active_mesh() -> Optional["DeviceMesh"]:
    return _active[-1] if _active else None


@contextlib.contextmanager
def no_mesh():
    saved = list(_active)
    _active.clear()
    try:
        with _NoDispatch():
            yield
    finally:
        _active.extend(saved)


class _NoDispatch(TorchDispatchMode):
    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        return func(*args, **(kwargs or {}))


class _ActiveMeshMode(TorchDispatchMode):
    """Routes factory functions (no tensor arguments) to the active mesh."""

    @classmethod
    def _should_skip_dynamo(cls) -> bool:
        # torch wraps a mode's __torch_dispatch__ in a "disable dynamo" guard unless this says
        # otherwise: two extra Python frames on every dispatched operator.  Nothing under an
        # active device mesh is compiled by dynamo.
        return False

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if getattr(_tls, "propagating", False):
            return func(*args, **kwargs)
        ts: List[Tensor] = []
        _collect(args, ts)
        _collect(kwargs, ts)
        if not ts and get_active_mesh() is not None and not _has_plain_tensor(args, kwargs):
            return _dispatch(func, args, kwargs, ts)
        if ts:
            return _dispatch(func, args, kwargs, ts)
        return func(*args, **kwargs)


def _has_plain_tensor(args, kwargs) -> bool:
    found = False

    def visit(o):
        nonlocal found
        if isinstance(o, torch.Tensor) and not isinstance(o, Tensor):
            found = True
        elif isinstance(o, (list, tuple)):
            for x in o:
                visit(x)
        elif isinstance(o, dict):
            for x in o.values():
                visit(x)
    visit(args)
    visit(kwargs)
    return found


class RemoteProcessGroup:
    """The controller's handle of the process groups over some dims of a device mesh (one
    group per combination of the other dims' coordinates).  Passed to a remote function it
    arrives as the worker's own ``torch.distributed`` group, for collectives written by hand
    inside the function (python/monarch/common/device_mesh.py:50-95 in the reference)."""

    def __init__(self, dims: Tuple[str, ...], mesh: "DeviceMesh"):
        self.dims = tuple(dims)
        self.device_mesh = mesh
        # GPU workers: a process group over the package's NVLink collectives (no NCCL
        # bootstrap); CPU workers: a gloo group
        own = mesh.client.use_cuda and os.environ.get("MB200_TE_COLLECTIVES", "own") == "own"
        self.key = mesh.client.ensure_comm(mesh, self.dims, stream_id=0, own=own)

    def size(self) -> int:
        n = 1
        for d in self.dims:
            n *= self.device_mesh.sizes[d]
        return n

    def __repr__(self) -> str:
        return f"RemoteProcessGroup({self.dims})"


class _DoneWork:
    def wait(self, timeout=None):
        return True

    def is_completed(self):
        return True


def _done(*args, **kwargs):
    return _DoneWork()


_shape_only_group_cls = None


def shape_only_group(dims: Tuple[str, ...], size: int):
    """What a propagation function gets in place of a :class:`RemoteProcessGroup`: a
    ``torch.distributed`` group of the right size whose collectives do nothing, so worker
    code that calls ``dist.all_reduce(t, group=pg)`` can be run on fakes for its shapes
    (python/monarch/common/remote.py ``DummyProcessGroup`` in the reference)."""
    global _shape_only_group_cls
    if _shape_only_group_cls is None:
        import torch.distributed as dist

        class ShapeOnlyProcessGroup(dist.ProcessGroup):
            def __init__(self, dims, size):
                super().__init__(0, size)
                self.dims = tuple(dims)

        for name in ("allreduce", "allreduce_coalesced", "broadcast", "reduce", "allgather",
                     "_allgather_base", "allgather_coalesced", "allgather_into_tensor_coalesced",
                     "gather", "scatter", "reduce_scatter", "_reduce_scatter_base",
                     "reduce_scatter_tensor_coalesced", "alltoall_base", "alltoall", "send",
                     "recv", "barrier"):
            setattr(ShapeOnlyProcessGroup, name, _done)
        _shape_only_group_cls = ShapeOnlyProcessGroup
    return _shape_only_group_cls(dims, size)


class DeviceMesh(MeshTrait):
    def __init__(self, client: Client, shape: Shape, workers, root: Optional["DeviceMesh"] = None):
        self.client = client
        self._shape_ = shape
        self._workers = workers
        self._root = root
        self._rank_tensors: Dict[str, Tensor] = {}

    def __call__(self, **kwargs) -> "DeviceMesh":
        """``mesh(host=0)`` is ``mesh.slice(host=0)`` (python/monarch/common/device_mesh.py
        ``DeviceMesh.__call__`` in the reference)."""
        return self.slice(**kwargs)

    @property
    def names(self) -> Tuple[str, ...]:
        return tuple(self._labels)

    @property
    def processes(self):
        """The ranks of the mesh as an n-dimensional slice."""
        return self._ndslice

    @property
    def _ndslice(self):
        return self._shape_.ndslice

    @property
    def _labels(self):
        return tuple(self._shape_.labels)

    def _new_with_shape(self, shape: Shape) -> "DeviceMesh":
        root = self._root or self
        sub_workers = root._workers._new_with_shape(Shape(shape.labels, shape.ndslice))
        return DeviceMesh(self.client, shape, sub_workers, root)

    @contextlib.contextmanager
    def activate(self):
        _active.append(self)
        try:
            with _ActiveMeshMode():
                yield self
        finally:
            _active.pop()

    def process_group(self, dims) -> RemoteProcessGroup:
        """Process groups over ``dims`` (a name or a tuple of names) for use inside remote
        functions."""
        if isinstance(dims, str):
            dims = (dims,)
        for d in dims:
            if d not in self._labels:
                raise KeyError(f"mesh has no dim {d!r} (dims: {self._labels})")
        return RemoteProcessGroup(tuple(dims), self)

    def rank(self, dim) -> Tensor:
        """Tensor holding each proc's coordinate along ``dim`` (or the flat index over a
        tuple of dims)."""
        dims = (dim,) if isinstance(dim, str) else tuple(dim)
        # coordinates are those of *this* mesh; the tensor lives on the active mesh when that
        # is a part of this one (``with mesh.slice(host=1).activate(): mesh.rank("host")``
        # gives 1 on every proc of the slice), else on this mesh
        home = self
        active = get_active_mesh()
        if active is not None and active is not self and active.client is self.client and \
                set(active._ndslice.ranks()) <= set(self._ndslice.ranks()):
            home = active
        key = (",".join(dims), id(home) if home is not self else 0)
        if key not in self._rank_tensors:
            labels = list(self._labels)
            sizes = list(self._ndslice.sizes)
            strides = list(self._ndslice.strides)
            offset = self._ndslice.offset
            with _propagation():
                fake = torch.empty((), dtype=torch.int64)
            idx = [labels.index(d) for d in dims]
            spec = ("pickle", _RankFn(offset, sizes, strides, idx))
            t = _send_call(spec, (), {}, fake, home)
            if home is not self:
                return t          # tied to the life of the sub-mesh object: not cached
            self._rank_tensors[key] = t
        return self._rank_tensors[key]

    @property
    def ranks(self) -> Dict[str, Tensor]:
        return {d: self.rank(d) for d in self._labels}

    def exit(self, error: Optional[Exception] = None) -> None:
        self.client.shutdown()

    def __repr__(self) -> str:
        return f"<DeviceMesh {self._shape_}>"


class _RankFn:
    """Computes this proc's coordinate along mesh dims from its global rank."""

    def __init__(self, offset, sizes, strides, idx):
        self.offset, self.sizes, self.strides, self.idx = offset, sizes, strides, idx

    def __call__(self):
        from ..actor import context
        r = context().actor_instance._native.rank - self.offset
        order = sorted(range(len(self.sizes)), key=lambda i: -self.strides[i])
        coord = [0] * len(self.sizes)
        for i in order:
            if self.sizes[i] > 1:
                coord[i] = min(r // self.strides[i], self.sizes[i] - 1)
                r -= coord[i] * self.strides[i]
        flat = 0
        for i in self.idx:
            flat = flat * self.sizes[i] + coord[i]
        return torch.tensor(flat, dtype=torch.int64)


def spawn_tensor_engine(proc_mesh, use_cuda: Optional[bool] = None,
                        null_device: bool = False) -> DeviceMesh:
    """Spawn tensor workers on every proc of ``proc_mesh`` and return its DeviceMesh.
    ``null_device=True``: the workers execute nothing -- every result is a zero tensor of the
    shape the controller computed, nothing is copied or reduced -- so what is left is the
    per-command cost of the controller, the messaging and the workers' hosts."""
    if use_cuda is None:
        use_cuda = torch.cuda.is_available()
    name = f"tensor_engine_workers_{next(_engine_ids)}"
    workers = proc_mesh.spawn(name, TensorWorker, use_cuda and not null_device, null_device)
    client = Client(proc_mesh, workers, use_cuda and not null_device)
    client.null_device = bool(null_device)
    dm = DeviceMesh(client, Shape(list(proc_mesh._labels), proc_mesh._ndslice), workers)
    client.root_mesh = dm
    return dm


_engine_ids = itertools.count()
