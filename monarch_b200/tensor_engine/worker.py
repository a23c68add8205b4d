"""Per-proc executor of the tensor engine.

Parity: monarch_tensor_worker (WorkerActor routing to per-stream executors, the ref ->
tensor/error environment, error poisoning of dependent results, Reduce / SendTensor /
SendValue, borrows as stream events, recordings), monarch_messages/src/worker.rs (the
message set), python/monarch/worker/worker.py (the reduce semantics used as oracle:
all-reduce, reduce-scatter via ``scatter=True``, all-gather via ``"stack"``, all-to-all via
``"stack"`` + scatter).

One worker actor runs per proc.  Ops execute on the proc's device in message order;
named streams map to CUDA streams (side streams are synchronised through borrow events).
Collectives over mesh dims use process groups created on first use; between GPUs of one
box the group's all-reduce / all-gather / reduce-scatter run this package's NVLink
kernels when the tensors live in peer-mapped memory, otherwise torch.distributed.
"""
from __future__ import annotations

import os
import queue
import threading
import traceback
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..actor import Actor, context, current_rank, endpoint
from ..actor.actor_mesh import Port


class Ref:
    """A controller-assigned name of a worker-side value."""
    __slots__ = ("id",)

    def __init__(self, id: int):
        self.id = id

    def __reduce__(self):
        return (Ref, (self.id,))

    def __repr__(self):
        return f"Ref({self.id})"


class PGRef(Ref):
    """Names a process group of the worker (created by ``split_comm``) in the arguments of a
    remote function; the worker passes its ``torch.distributed`` group in its place."""

    def __init__(self, key):
        super().__init__(-1)
        self.key = tuple(key)

    def __reduce__(self):
        return (PGRef, (self.key,))

    def __repr__(self):
        return f"PGRef({self.key})"


class RemoteError:
    """What a failed op leaves in the environment instead of a tensor."""

    def __init__(self, seq: int, rank: int, func: str, exc_text: str, tb: str,
                 dependent_of: Optional[int] = None):
        self.seq, self.rank, self.func = seq, rank, func
        self.exc_text, self.tb, self.dependent_of = exc_text, tb, dependent_of


def _resolve_function(spec):
    kind = spec[0]
    if kind == "op":          # ("op", "aten.add.Tensor")
        ns, name, overload = spec[1].split(".")
        packet = getattr(getattr(torch.ops, ns), name)
        return getattr(packet, overload)
    if kind == "path":        # ("path", "module.sub.fn")
        mod, _, fn = spec[1].rpartition(".")
        import importlib
        return getattr(importlib.import_module(mod), fn)
    if kind == "pickle":      # ("pickle", callable)
        return spec[1]
    raise ValueError(f"bad function spec {spec!r}")


def _seq(like, items):
    """A list/tuple of ``like``'s type from ``items`` (named tuples take them as fields)."""
    return type(like)(*items) if hasattr(like, "_fields") else type(like)(items)


def _map_refs(obj, fn):
    if isinstance(obj, Ref):
        return fn(obj)
    if isinstance(obj, (list, tuple)):
        return _seq(obj, (_map_refs(o, fn) for o in obj))
    if isinstance(obj, dict):
        return {k: _map_refs(v, fn) for k, v in obj.items()}
    if getattr(type(obj), "_holds_tensors", False):       # an OpaqueRef: its key tensor
        return obj._rebuild(_map_refs(obj._tensors(), fn))
    return obj


def _load_core():
    """The native executor core (built in-tree by ``monarch_b200._build``); None when the
    extension is absent or disabled with ``MB200_PY_WORKER=1`` (pure-Python execution)."""
    if os.environ.get("MB200_PY_WORKER") == "1":
        return None
    try:
        from .. import _tensor_worker
        return _tensor_worker
    except ImportError:
        try:
            from .. import _build
            _build.build_tensor_worker()
            from .. import _tensor_worker
            return _tensor_worker
        except Exception:  # noqa: BLE001 - no compiler here: stay on the Python path
            return None


class _Env:
    """dict view of the worker environment.  Integer keys (refs) live in the native core
    when there is one, so operator calls and recordings never leave C++; everything else
    (bookkeeping entries keyed by tuples) stays in a Python dict."""

    def __init__(self, core):
        self._core = core
        self._py: Dict[Any, Any] = {}

    @staticmethod
    def _wrap(v):
        if isinstance(v, tuple) and len(v) == 7 and v[0] == "__remote_error__":
            return RemoteError(v[1], v[2], v[3], v[4], v[5], None if v[6] < 0 else v[6])
        return v

    def __contains__(self, k) -> bool:
        if self._core is not None and isinstance(k, int):
            return self._core.contains(k)
        return k in self._py

    def __getitem__(self, k):
        if self._core is not None and isinstance(k, int):
            return self._wrap(self._core.get(k))
        return self._py[k]

    def get(self, k, default=None):
        return self[k] if k in self else default

    def __setitem__(self, k, v) -> None:
        if self._core is not None and isinstance(k, int):
            if isinstance(v, RemoteError):
                self._core.set_error(k, v.seq, v.rank, v.func, v.exc_text, v.tb,
                                     -1 if v.dependent_of is None else v.dependent_of)
            else:
                self._core.set(k, v)
        else:
            self._py[k] = v

    def pop(self, k, default=None):
        if self._core is not None and isinstance(k, int):
            return self._wrap(self._core.pop(k)) if self._core.contains(k) else default
        return self._py.pop(k, default)

    def __len__(self) -> int:
        return (len(self._core) if self._core is not None else 0) + len(self._py)


class _PipeClosed(Exception):
    pass


class WorkerPipe:
    """Worker end of a pipe: the generator runs on its own thread; its ``send`` blocks while
    ``max_messages`` are waiting (python/monarch/worker/worker.py:573-595, 1158-1191)."""

    def __init__(self, max_messages: int, ranks: Dict[str, int], sizes: Dict[str, int]):
        self._out: "queue.Queue" = queue.Queue(maxsize=max(1, max_messages))
        self._in: "queue.Queue" = queue.Queue(maxsize=max(1, max_messages))
        self.ranks = ranks
        self.sizes = sizes
        self._closed = threading.Event()
        self._thread: Optional[threading.Thread] = None

    # ---- the generator's side
    def _put_out(self, item) -> None:
        while not self._closed.is_set():
            try:
                self._out.put(item, timeout=0.2)
                return
            except queue.Full:
                continue
        raise _PipeClosed()

    def send(self, obj: Any) -> None:
        self._put_out(("value", obj))

    def recv(self) -> Any:
        while not self._closed.is_set():
            try:
                return self._in.get(timeout=0.2)
            except queue.Empty:
                continue
        raise _PipeClosed()

    # ---- the worker's side
    def start(self, fn, args, kwargs) -> None:
        def main():
            try:
                r = fn(self, *args, **kwargs)
                if hasattr(r, "__next__"):
                    for item in r:
                        self.send(item)
                self._put_out(("end", None))
            except _PipeClosed:
                pass
            except Exception as ex:  # noqa: BLE001 - surfaces at the next recv
                self.fail(ex, traceback.format_exc())

        self._thread = threading.Thread(target=main, name="pipe", daemon=True)
        self._thread.start()

    def fail(self, ex, tb: str) -> None:
        try:
            self._put_out(("error", f"{type(ex).__name__}: {ex}\n{tb}"))
        except _PipeClosed:
            pass

    def next_message(self, timeout: float = 600.0) -> Any:
        if getattr(self, "_terminal", None) is not None:
            return self._raise_terminal()
        kind, v = self._out.get(timeout=timeout)
        if kind == "value":
            return v
        self._closed.set()   # terminal: later recvs report the same state
        self._terminal = (kind, v)
        return self._raise_terminal()

    def _raise_terminal(self):
        kind, v = self._terminal
        if kind == "end":
            raise RuntimeError("the remote generator is exhausted")
        raise RuntimeError(f"remote generator failed: {v}")

    def put_inbound(self, v: Any) -> None:
        self._in.put(v, timeout=600.0)

    def close(self) -> None:
        self._closed.set()


class TensorWorker(Actor):
    def __init__(self, use_cuda: bool, null_device: bool = False):
        """``null_device``: operators are not executed -- every result is a zero tensor of the
        shape and dtype the controller computed; copies and collectives move nothing.  What
        remains is the host-side cost per command (controller, messaging, worker routing),
        which is how the dispatch overhead of a program written for GPUs is measured on a box
        without one (the reference patches the CUDA driver's entry points for this,
        python/monarch/common/mock_cuda.cpp:32-100; here it is a switch in the worker)."""
        self.rank = current_rank().rank
        self.world = current_rank().extent.nelements
        self.null_device = bool(null_device)
        self.use_cuda = bool(use_cuda and torch.cuda.is_available()) and not self.null_device
        if self.use_cuda:
            n = torch.cuda.device_count()
            self.device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", self.rank)) % n)
            torch.cuda.set_device(self.device)
        else:
            self.device = torch.device("cpu")
        self.proc_key = context().actor_instance.proc_id   # shared with the proc's actors
        mod = _load_core()
        self.core = mod.WorkerCore(self.rank, Ref) if mod is not None else None
        if self.core is not None and self.use_cuda:
            self.core.set_cuda_index(self.device.index)
        self.env = _Env(self.core)
        self.streams: Dict[int, Any] = {0: None}
        self.groups: Dict[Tuple[int, ...], Any] = {}
        # own NVLink communicators: key -> (MeshComm, ranks); and the buffers exported for
        # communicators whose peers have not been connected yet
        self.comms: Dict[Tuple[int, ...], Any] = {}
        self._comm_pending: Dict[Tuple[int, ...], Any] = {}
        self._own_pgs: Dict[Tuple[int, ...], Any] = {}
        self.borrows: Dict[int, Any] = {}
        self.recordings: Dict[int, List[tuple]] = {}
        self.pipes: Dict[int, WorkerPipe] = {}
        self.pg_ready = False
        self.error_port: Optional[Port] = None
        self.last_seq = -1
        # One OS thread per stream inside the native core (MB200_WORKER_THREADS=0: every
        # command runs on the actor's thread in arrival order, as a single queue).
        self.threaded = self.core is not None and \
            os.environ.get("MB200_WORKER_THREADS", "1") == "1"
        self._borrow_route: Dict[int, Tuple[int, int]] = {}
        if self.threaded:
            self.core.set_report(lambda err: self._report(RemoteError(*err[:5])))
            self.core.set_null_device(self.null_device)
            self._start_stream_thread(0)

    # ---------------------------------------------------------------------- helpers
    def _get(self, ref: Ref, seq: int):
        if isinstance(ref, PGRef):
            own = self.comms.get(ref.key)
            if own is not None:           # a process group over the NVLink collectives
                if isinstance(own[0], Exception):
                    raise own[0]
                pg = self._own_pgs.get(ref.key)
                if pg is None:
                    from ..parallel.mesh_process_group import MeshProcessGroup
                    pg = self._own_pgs[ref.key] = MeshProcessGroup(own[0])
                return pg
            ent = self.groups.get(ref.key)
            if ent is None:
                raise KeyError(f"process group {ref.key} does not include worker {self.rank}")
            return ent[0]
        v = self.env.get(ref.id)
        if v is None and ref.id not in self.env:
            raise KeyError(f"{ref} is not defined on worker {self.rank}")
        return v

    def _poison(self, seq: int, results: List[Ref], err: RemoteError) -> None:
        for r in results:
            self.env[r.id] = err

    def _report(self, err: RemoteError) -> None:
        if self.error_port is not None and err.dependent_of is None:
            self.error_port.send(("error", err.seq, self.rank, err.func, err.exc_text, err.tb))

    def _localize(self, obj):
        """``obj`` with every ``torch.device("cuda", i)`` replaced by this worker's GPU: a
        worker owns one GPU, whatever index the controller's process happened to name."""
        if isinstance(obj, torch.device):
            return self.device if obj.type == "cuda" else obj
        if isinstance(obj, (list, tuple)):
            return _seq(obj, (self._localize(o) for o in obj))
        if isinstance(obj, dict):
            return {key: self._localize(v) for key, v in obj.items()}
        return obj

    def _stream_ctx(self, stream_id: int):
        s = self.streams.get(stream_id)
        if s is None or not self.use_cuda:
            return _Null()
        return torch.cuda.stream(s)

    # ---------------------------------------------------------------- message entry
    @endpoint
    def configure(self, error_port: Port) -> int:
        self.error_port = error_port
        return self.rank

    @endpoint
    def run(self, msgs: List[tuple]) -> None:
        """A batch of worker messages (one for eager dispatch, many under coalescing)."""
        self._route_all(msgs)

    @endpoint
    def run_and_reply(self, msgs: List[tuple], fetch: tuple) -> Any:
        self._route_all(msgs)
        self._drain()
        return self._fetch(*fetch)

    def _route_all(self, msgs: List[tuple]) -> None:
        if self.threaded:
            # operator calls and deletions are decoded and queued by the native core and run
            # on the stream threads without the GIL; the rest comes back to _route in order
            self.core.route_batch(msgs, self._route)
        else:
            for m in msgs:
                self._route(m)

    # ------------------------------------------------------------ per-stream threads
    # position of the stream id in the messages that run on one stream
    _STREAM_ARG = {"call": 7, "reduce": 9, "send_tensor": 6, "pipe_recv": 4, "pipe_send": 4,
                   "actor_call_state": 3, "actor_call_rref": 4}

    def _start_stream_thread(self, stream_id: int) -> None:
        if self.core.has_stream_thread(stream_id):
            return

        def on_start():
            if self.use_cuda:
                torch.cuda.set_device(self.device)
                s = self.streams.get(stream_id)
                if s is not None:
                    torch.cuda.set_stream(s)      # this thread's current stream from now on
        self.core.start_stream_thread(stream_id, on_start)

    def _route(self, m: tuple) -> None:
        """Hand a message to the thread of the stream it belongs to; messages that belong
        to no stream wait for every stream to reach them (deletions without holding the
        streams up, the rest as a barrier across streams)."""
        kind = m[0]
        if not self.threaded:
            getattr(self, "_m_" + kind)(*m[1:])
            return
        from ..actor import actor_mesh as _am
        ctx = context()           # the actor's context of this message, for user functions

        def handler():
            _am._tls.ctx = ctx
            getattr(self, "_m_" + kind)(*m[1:])
        pos = self._STREAM_ARG.get(kind)
        if pos is not None:
            stream = m[pos]
            self._start_stream_thread(stream)
            self.core.submit(stream, handler)
            if kind == "send_tensor" and len(m) > 7 and m[7] is not None and m[7] != stream:
                self._order_after(stream, m[7])    # the result is used on another stream
        elif kind == "create_stream":
            self._m_create_stream(*m[1:])
            self._start_stream_thread(m[1])
        elif kind == "borrow_create":
            self._route_borrow_create(*m[1:])
        elif kind == "borrow_drop":
            self._route_borrow_drop(*m[1:])
        else:
            self.core.fence(handler, kind != "delete")

    def _order_after(self, first: int, then: int) -> None:
        """Everything handed to stream ``then`` from here on runs after what stream ``first``
        has been handed so far (host order by a flag, device order by a CUDA event)."""
        self._start_stream_thread(then)
        issued, box = threading.Event(), {}

        def on_first():
            if self.use_cuda:
                box["ev"] = torch.cuda.Event()
                box["ev"].record(torch.cuda.current_stream())
            issued.set()

        def on_then():
            issued.wait()
            if self.use_cuda:
                torch.cuda.current_stream().wait_event(box["ev"])
        self.core.submit(first, on_first)
        self.core.submit(then, on_then)

    def _route_borrow_create(self, borrow_id, ref, from_stream, to_stream, result) -> None:
        """The borrowing stream may use the value once the producing stream has issued
        everything it was sent before the borrow: a host-side flag carries that, a CUDA
        event the device-side order."""
        self._start_stream_thread(from_stream)
        self._start_stream_thread(to_stream)
        self._borrow_route[borrow_id] = (from_stream, to_stream)
        issued, box = threading.Event(), {}

        def on_from():
            if self.use_cuda:
                box["ev"] = torch.cuda.Event()
                box["ev"].record(torch.cuda.current_stream())
            issued.set()

        def on_to():
            issued.wait()
            if self.use_cuda:
                torch.cuda.current_stream().wait_event(box["ev"])
            self.env[result.id] = self.env.get(ref.id)
            self.borrows[borrow_id] = (from_stream, to_stream)
        self.core.submit(from_stream, on_from)
        self.core.submit(to_stream, on_to)

    def _route_borrow_drop(self, borrow_id) -> None:
        route = self._borrow_route.pop(borrow_id, None)
        if route is None:
            return
        from_stream, to_stream = route
        issued, box = threading.Event(), {}

        def on_to():
            if self.use_cuda:
                box["ev"] = torch.cuda.Event()
                box["ev"].record(torch.cuda.current_stream())
            self.borrows.pop(borrow_id, None)
            issued.set()

        def on_from():
            issued.wait()
            if self.use_cuda:
                torch.cuda.current_stream().wait_event(box["ev"])
        self.core.submit(to_stream, on_to)
        self.core.submit(from_stream, on_from)

    def _drain(self) -> None:
        """Wait until every stream thread has run what it was handed so far."""
        if self.threaded:
            self.core.drain()

    # ------------------------------------------------- own NVLink communicators
    @endpoint
    def comm_export(self, key: Tuple[int, ...], all_groups: List[List[int]]):
        """First half of a communicator's bootstrap: allocate this rank's flag + staging
        buffer and return what its peers need to map it (a CUDA IPC handle and where it
        lives).  The controller hands every member the exports of its group in
        ``comm_connect``.  Ranks outside every group answer None."""
        try:
            mine = next((g for g in all_groups if self.rank in g), None)
            if mine is None:
                return None
            if not self.use_cuda:
                return {"error": f"worker {self.rank} has no GPU"}
            import socket
            from ..ops import ipc
            from ..parallel.meshcomm import MeshComm
            torch.cuda.set_device(self.device)
            local = MeshComm.allocate_local(self.device)
            torch.cuda.synchronize(self.device)      # zeroed before any peer can touch it
            exp = ipc.export_handle(local)
            exp.update(rank=self.rank, host=socket.gethostname())
            self._comm_pending[key] = (local, list(mine))
            return exp
        except Exception as ex:  # noqa: BLE001 - reported to the controller, which raises
            return {"error": f"{type(ex).__name__}: {ex}"}

    @endpoint
    def comm_connect(self, key: Tuple[int, ...], exports: Dict[int, dict]) -> None:
        """Second half: map the peers' buffers.  A failure here surfaces at the first
        collective that asks for the communicator."""
        pend = self._comm_pending.pop(key, None)
        if pend is None:
            return
        local, ranks = pend
        try:
            from ..parallel.meshcomm import MeshComm
            torch.cuda.set_device(self.device)
            comm = MeshComm.from_exports(ranks.index(self.rank), [exports[r] for r in ranks],
                                         local, self.device)
            self.comms[key] = (comm, ranks)
        except Exception as ex:  # noqa: BLE001
            self.comms[key] = (RuntimeError(f"{type(ex).__name__}: {ex}"), ranks)

    def _own_reduce(self, comm, t, reduction, scatter, inplace):
        """One reduce message on the NVLink kernels (current stream)."""
        if reduction == "stack":
            return comm.all_to_all(t) if scatter else comm.all_gather(t)
        if scatter:
            return comm.reduce_scatter(t, reduction)
        return comm.all_reduce(t, reduction, out=t if inplace else None)

    # -------------------------------------------------------------------- messages
    def _m_call(self, seq, results, mutates, fspec, args, kwargs, stream, metas=None) -> None:
        self.last_seq = seq
        if self.null_device and metas is not None:
            # not executed: results of the announced shapes stand in (see __init__)
            for r, (shape, dtype) in zip(results, metas):
                self.env[r.id] = torch.zeros(shape, dtype=dtype)
            return
        fname = fspec[1] if isinstance(fspec[1], str) else getattr(fspec[1], "__name__", "udf")
        if self.core is not None and fspec[0] == "op":
            # ATen operator: resolved, checked for poisoned inputs, dispatched and stored
            # by the native core
            try:
                err = self.core.call_op(seq, [r.id for r in results], [r.id for r in mutates],
                                        fspec[1], tuple(args), dict(kwargs), stream)
            except Exception:  # noqa: BLE001 - argument shapes the core does not take
                err = "python"
            if err is None:
                return
            if err != "python":
                if err[5] < 0:
                    self._report(RemoteError(*err[:5]))
                return
        try:
            dep = None

            def res(r):
                nonlocal dep
                v = self._get(r, seq)
                if isinstance(v, RemoteError) and dep is None:
                    dep = v
                return v

            a = _map_refs(args, res)
            k = _map_refs(kwargs, res)
            if dep is not None:
                e = RemoteError(seq, self.rank, fname, dep.exc_text, dep.tb,
                                dependent_of=dep.seq)
                self._poison(seq, results + mutates, e)
                return
            if self.use_cuda:      # any CUDA device named by the controller is this worker's
                a, k = self._localize(a), self._localize(k)
            fn = _resolve_function(fspec)
            with self._stream_ctx(stream):
                out = fn(*a, **k)
            flat = _flatten_tensors(out)
            if not results and mutates:
                flat = []  # in-place op: its return value aliases an argument
            if len(flat) != len(results):
                raise RuntimeError(f"{fname} returned {len(flat)} tensors, controller expected "
                                   f"{len(results)}")
            for r, t in zip(results, flat):
                self.env[r.id] = t
        except Exception as ex:  # noqa: BLE001 - the worker stays alive; the refs carry it
            e = RemoteError(seq, self.rank, fname, f"{type(ex).__name__}: {ex}",
                            traceback.format_exc())
            self._poison(seq, results + mutates, e)
            self._report(e)

    def _m_delete(self, ids: List[int]) -> None:
        for i in ids:
            self.env.pop(i, None)

    def _m_create_stream(self, stream_id: int, default: bool) -> None:
        if stream_id not in self.streams:
            self.streams[stream_id] = torch.cuda.Stream(device=self.device) \
                if (self.use_cuda and not default) else None
            if self.core is not None:
                # with a thread per stream the thread's current stream is set once, at start
                self.core.create_stream(stream_id,
                                        None if self.threaded else self.streams[stream_id])

    def _m_borrow_create(self, borrow_id, ref, from_stream, to_stream, result) -> None:
        # the borrowing stream waits for the producing stream; the value is aliased
        if self.use_cuda:
            ev = torch.cuda.Event()
            ev.record(self.streams.get(from_stream) or torch.cuda.current_stream())
            (self.streams.get(to_stream) or torch.cuda.current_stream()).wait_event(ev)
        self.env[result.id] = self.env.get(ref.id)
        self.borrows[borrow_id] = (from_stream, to_stream)

    def _m_borrow_drop(self, borrow_id) -> None:
        b = self.borrows.pop(borrow_id, None)
        if b and self.use_cuda:
            ev = torch.cuda.Event()
            ev.record(self.streams.get(b[1]) or torch.cuda.current_stream())
            (self.streams.get(b[0]) or torch.cuda.current_stream()).wait_event(ev)

    def _m_init_pg(self, addr: str, port: int, ranks: List[int]) -> None:
        import torch.distributed as dist
        if self.pg_ready or not dist.is_available():
            return
        if dist.is_initialized():
            self.pg_ready = True
            return
        backend = "nccl" if self.use_cuda else "gloo"
        dist.init_process_group(backend, init_method=f"tcp://{addr}:{port}",
                                rank=ranks.index(self.rank), world_size=len(ranks),
                                **({"device_id": self.device} if self.use_cuda else {}))
        self.pg_ready = True

    def _m_split_comm(self, key: Tuple[int, ...], all_groups: List[List[int]]) -> None:
        import torch.distributed as dist
        if key in self.groups:
            return
        mine = None
        for ranks in all_groups:  # every rank creates every group, in the same order
            g = dist.new_group(ranks)
            if self.rank in ranks:
                mine = (g, ranks)
        self.groups[key] = mine

    def _m_reduce(self, seq, result, ref, key, reduction, scatter, inplace, out_ref, stream,
                  in_meta=None) -> None:
        import torch.distributed as dist
        self.last_seq = seq
        try:
            t = self._get(ref, seq)
            failed = None
            if isinstance(t, RemoteError):
                failed = RemoteError(seq, self.rank, "reduce", t.exc_text, t.tb,
                                     dependent_of=t.seq)
                if in_meta is None:
                    self._poison(seq, [result], failed)
                    return
                # the other ranks of the group do not know that the input failed here and
                # are entering the collective: take part with a stand-in so that they are
                # not left waiting, and keep the failure in this rank's result
                t = torch.zeros(in_meta[0], dtype=in_meta[1], device=self.device)
                inplace, out_ref = False, None
            if self.null_device:      # nothing moves: only the result's shape exists
                n = max(1, int(key[-1])) if isinstance(key, tuple) and len(key) > 1 else 1
                if reduction == "stack":
                    out = torch.empty_like(t) if scatter else \
                        torch.zeros((n, *t.shape), dtype=t.dtype)
                elif scatter:
                    out = torch.zeros(t.shape[1:], dtype=t.dtype)
                else:
                    out = t if inplace else torch.empty_like(t)
                if out_ref is not None:
                    out = self.env[out_ref.id]
                self.env[result.id] = out
                return
            own = self.comms.get(key)
            if own is not None:
                comm, ranks = own
                if isinstance(comm, Exception):
                    raise comm
                with self._stream_ctx(stream):
                    out = self._own_reduce(comm, t, reduction, scatter, inplace)
                    if out_ref is not None:
                        self.env[out_ref.id].copy_(out)
                        out = self.env[out_ref.id]
                self.env[result.id] = out if failed is None else failed
                return
            g, ranks = self.groups[key]
            n = len(ranks)
            with self._stream_ctx(stream):
                if reduction == "stack":
                    if scatter:   # all-to-all: outer dim n in, outer dim n out
                        out = torch.empty_like(t)
                        if dist.get_backend(g) == "nccl":
                            dist.all_to_all_single(out, t.contiguous(), group=g)
                        else:
                            ins = list(t.contiguous().unbind(0))
                            outs = [torch.empty_like(i) for i in ins]
                            _gloo_all_to_all(outs, ins, g, ranks, self.rank)
                            out = torch.stack(outs)
                    else:         # all-gather: adds an outer dim n
                        parts = [torch.empty_like(t) for _ in range(n)]
                        dist.all_gather(parts, t.contiguous(), group=g)
                        out = torch.stack(parts)
                else:
                    op = {"sum": dist.ReduceOp.SUM, "avg": dist.ReduceOp.SUM,
                          "product": dist.ReduceOp.PRODUCT, "prod": dist.ReduceOp.PRODUCT,
                          "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX,
                          "band": dist.ReduceOp.BAND, "bor": dist.ReduceOp.BOR,
                          "bxor": dist.ReduceOp.BXOR}[reduction]
                    work = t if inplace else t.clone()
                    dist.all_reduce(work, op=op, group=g)
                    if reduction == "avg":
                        work = work / n if not inplace else work.div_(n)
                    if scatter:   # reduce-scatter: keep slice i of the outer dim
                        if work.shape[0] != n:
                            raise RuntimeError(f"scatter needs an outer dim of {n}, got "
                                               f"{tuple(work.shape)}")
                        work = work[ranks.index(self.rank)].clone()
                    out = work
                if out_ref is not None:
                    self.env[out_ref.id].copy_(out)
                    out = self.env[out_ref.id]
            self.env[result.id] = out if failed is None else failed
        except Exception as ex:  # noqa: BLE001
            e = RemoteError(seq, self.rank, "reduce", f"{type(ex).__name__}: {ex}",
                            traceback.format_exc())
            self._poison(seq, [result], e)
            self._report(e)

    def _m_send_tensor(self, seq, result, ref, from_ranks, to_ranks, stream,
                       to_stream=None) -> None:
        """Point-to-point move between equally shaped sub-meshes (pipeline activations).
        Runs on the source tensor's stream; ``to_stream`` is the stream the result lives on
        (the router orders that stream behind this transfer)."""
        import torch.distributed as dist
        try:
            pairs = list(zip(from_ranks, to_ranks))
            t = self.env.get(ref.id) if ref is not None and self.rank in from_ranks else None
            for src, dst in pairs:
                if src == dst == self.rank:
                    self.env[result.id] = t
                elif self.rank == src:
                    dist.send(t.contiguous(), dst)
                elif self.rank == dst:
                    meta = self.env.pop(("send_meta", result.id))
                    buf = torch.empty(meta[0], dtype=meta[1], device=self.device)
                    dist.recv(buf, src)
                    self.env[result.id] = buf
        except Exception as ex:  # noqa: BLE001
            e = RemoteError(seq, self.rank, "send_tensor", f"{type(ex).__name__}: {ex}",
                            traceback.format_exc())
            self._poison(seq, [result], e)
            self._report(e)

    def _m_send_meta(self, result, shape, dtype) -> None:
        self.env[("send_meta", result.id)] = (tuple(shape), dtype)

    def _m_define_recording(self, rec_id: int, msgs: List[tuple], temps=()) -> None:
        """``temps``: refs that exist only inside the recording.  Each is dropped right after
        the last message that mentions it, so a replay reuses memory the way eager
        execution does instead of holding every intermediate until the end."""
        last_use: Dict[int, int] = {}
        temp_set = set(temps)
        if temp_set:
            for i, m in enumerate(msgs):
                def note(r, i=i):
                    if r.id in temp_set:
                        last_use[r.id] = i
                    return r
                _map_refs(m, note)
        drop_after: Dict[int, List[int]] = {}
        for rid, i in last_use.items():
            drop_after.setdefault(i, []).append(rid)
        self.recordings[rec_id] = (msgs, drop_after)
        if self.core is not None:
            self.core.define_recording(rec_id, list(msgs), drop_after)

    def _m_call_recording(self, rec_id: int, bind: Dict[int, int]) -> None:
        """Replay a recording with formal ref ids rebound to this call's ids.  Operator calls
        are replayed by the native core in one go; the other messages of the recording come
        back through ``fallback`` in their recorded position."""
        msgs, drop_after = self.recordings[rec_id]

        def run_py(index: int, b: Dict[int, int]) -> None:
            m = msgs[index]
            rb = lambda obj: _map_refs(obj, lambda r: Ref(b.get(r.id, r.id)))  # noqa: E731
            getattr(self, "_m_" + m[0])(*[rb(x) for x in m[1:]])

        if self.core is not None:
            self.core.call_recording(rec_id, dict(bind), run_py,
                                     lambda e: self._report(RemoteError(*e[:5])))
            return
        for i in range(len(msgs)):
            run_py(i, bind)
            for rid in drop_after.get(i, ()):
                self.env.pop(rid, None)

    # ------------------------------------------- actor endpoints called with tensors
    def _resolve_list(self, refs, seq):
        """The tensors behind ``refs``, or the first error among them."""
        out = []
        for r in refs:
            v = self._get(r, seq)
            if isinstance(v, RemoteError):
                return None, v
            out.append(v)
        return out, None

    def _m_actor_call_state(self, ident, refs, stream) -> None:
        """Hand this proc's tensors for ``refs`` to the actor that handles call ``ident``."""
        from .actor_bridge import BROKER, CallFailed
        self.last_seq = ident
        try:
            tensors, err = self._resolve_list(refs, ident)
            if err is not None:
                BROKER.put(self.proc_key, ident, "state", CallFailed(err.exc_text))
                return
            if self.use_cuda:
                with self._stream_ctx(stream):
                    torch.cuda.current_stream().synchronize()   # the actor reads them now
            BROKER.put(self.proc_key, ident, "state", tensors)
        except Exception as ex:  # noqa: BLE001
            BROKER.put(self.proc_key, ident, "state", CallFailed(f"{type(ex).__name__}: {ex}"))

    def _m_actor_call_rref(self, ident, refs, results, stream) -> None:
        """As above, then wait for the actor's return value and keep its tensors under
        ``results``."""
        from .actor_bridge import BROKER, CallFailed
        self._m_actor_call_state(ident, refs, stream)
        try:
            res = BROKER.take(self.proc_key, ident, "result")
            if isinstance(res, CallFailed):
                raise RuntimeError(res.text)
            flat = _flatten_tensors(res)
            if len(flat) != len(results):
                raise RuntimeError(f"the endpoint returned {len(flat)} tensors, its propagate "
                                   f"function promised {len(results)}")
            for r, t in zip(results, flat):
                self.env[r.id] = t.to(self.device)
        except Exception as ex:  # noqa: BLE001 - the result refs carry the failure
            e = RemoteError(ident, self.rank, "actor endpoint (rref)",
                            f"{type(ex).__name__}: {ex}", traceback.format_exc())
            self._poison(ident, list(results), e)
            self._report(e)

    # ----------------------------------------------------------------------- pipes
    def _m_create_pipe(self, pipe_id, fspec, max_messages, args, kwargs, labels, offset, sizes,
                       strides) -> None:
        rem = self.rank - offset
        ranks = {l: ((rem // st) % n if st else 0) for l, n, st in zip(labels, sizes, strides)}
        pipe = WorkerPipe(max_messages, ranks, dict(zip(labels, sizes)))
        self.pipes[pipe_id] = pipe
        try:
            fn = _resolve_function(fspec)
        except Exception as ex:  # noqa: BLE001 - surfaces at the first recv
            pipe.fail(ex, traceback.format_exc())
            return
        pipe.start(fn, args, kwargs)

    def _m_pipe_recv(self, seq, results, pipe_id, stream) -> None:
        self.last_seq = seq
        try:
            out = self.pipes[pipe_id].next_message()
            flat = _flatten_tensors(out)
            if len(flat) != len(results):
                raise RuntimeError(f"pipe produced {len(flat)} tensors, controller expected "
                                   f"{len(results)}")
            with self._stream_ctx(stream):
                for r, t in zip(results, flat):
                    self.env[r.id] = t.to(self.device, non_blocking=True)
        except Exception as ex:  # noqa: BLE001 - the refs carry the failure
            e = RemoteError(seq, self.rank, "pipe.recv", f"{type(ex).__name__}: {ex}",
                            traceback.format_exc())
            self._poison(seq, list(results), e)
            self._report(e)

    def _m_pipe_send(self, seq, pipe_id, obj, stream) -> None:
        self.last_seq = seq
        try:
            dep = None

            def res(r):
                nonlocal dep
                v = self._get(r, seq)
                if isinstance(v, RemoteError) and dep is None:
                    dep = v
                return v

            val = _map_refs(obj, res)
            if dep is not None:
                raise RuntimeError(f"input failed at seq {dep.seq}: {dep.exc_text}")
            if self.use_cuda:
                torch.cuda.synchronize(self.device)   # the generator thread reads the values
            self.pipes[pipe_id].put_inbound(val)
        except Exception as ex:  # noqa: BLE001
            self._report(RemoteError(seq, self.rank, "pipe.send", f"{type(ex).__name__}: {ex}",
                                     traceback.format_exc()))

    def _m_drop_pipe(self, pipe_id) -> None:
        p = self.pipes.pop(pipe_id, None)
        if p is not None:
            p.close()

    # ----------------------------------------------------------------------- fetch
    def _fetch(self, seq, ref_tree, preprocess):
        first_err = None

        def res(r):
            nonlocal first_err
            v = self.env.get(r.id)
            if isinstance(v, RemoteError):
                first_err = first_err or v
                return None
            return v

        vals = _map_refs(ref_tree, res)
        if first_err is not None:
            e = first_err
            return ("error", e.seq, e.rank, e.func, e.exc_text, e.tb, e.dependent_of)
        if preprocess is not None and preprocess[0] == "status":
            return ("ok", None)      # "are these values sound here?": no copy, no device sync
        try:
            if self.use_cuda:
                # the values may come from any named stream; this thread's stream is ordered
                # after none of them, so wait for the device before touching the data
                torch.cuda.synchronize(self.device)
            if preprocess is not None:
                vals = _resolve_function(preprocess)(vals)
            return ("ok", _to_cpu(vals))
        except Exception as ex:  # noqa: BLE001
            return ("error", seq, self.rank, "fetch", f"{type(ex).__name__}: {ex}",
                    traceback.format_exc(), None)

    @endpoint
    def fetch(self, seq, ref_tree, preprocess=None):
        self._drain()
        return self._fetch(seq, ref_tree, preprocess)

    @endpoint
    def progress(self) -> int:
        """Watchdog ping: answered in command order, so a reply means that everything sent
        before it has been executed (not necessarily finished on the GPU)."""
        return self._last_seq()

    @endpoint
    def sync(self) -> int:
        self._drain()
        if self.use_cuda:
            torch.cuda.synchronize(self.device)
        return self._last_seq()

    def _last_seq(self) -> int:
        return max(self.last_seq, self.core.last_seq()) if self.core is not None \
            else self.last_seq


# the worker's endpoints take wire messages (refs, not distributed tensors): casts to them
# skip the scan for distributed tensors that other actors' endpoints need
for _n in ("run", "fetch", "progress", "sync"):
    TensorWorker.__dict__[_n]._fn._wire_messages_only = True


def _flatten_tensors(out) -> List[torch.Tensor]:
    if isinstance(out, torch.Tensor):
        return [out]
    if isinstance(out, (list, tuple)):
        r: List[torch.Tensor] = []
        for o in out:
            r += _flatten_tensors(o)
        return r
    if isinstance(out, dict):
        r = []
        for o in out.values():
            r += _flatten_tensors(o)
        return r
    if getattr(type(out), "_holds_tensors", False):
        return _flatten_tensors(out._tensors())
    return []


def _to_cpu(obj):
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu()
    if isinstance(obj, (list, tuple)):
        return _seq(obj, (_to_cpu(o) for o in obj))
    if isinstance(obj, dict):
        return {k: _to_cpu(v) for k, v in obj.items()}
    return obj


def _gloo_all_to_all(outs, ins, g, ranks, my_rank) -> None:
    import torch.distributed as dist
    me = ranks.index(my_rank)
    for i, src in enumerate(ranks):     # round i: rank i scatters its inputs
        dist.scatter(outs[i], ins if me == i else None, src=src, group=g)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
