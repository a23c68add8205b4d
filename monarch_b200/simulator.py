"""Mock device meshes and a timeline simulator for the tensor engine.

``mock_mesh(hosts, gpus)`` returns a :class:`DeviceMesh` with no processes behind it: the
controller-side machinery (dispatch, shape propagation, refs, borrows, coalescing,
recordings) runs exactly as with real workers, and the messages are consumed by in-process
simulated workers that execute every op on ``meta`` tensors -- shapes and dtypes are real,
data is not.  Each simulated worker keeps a per-stream clock and the bytes held by live
refs, so a program can be "run" on a 1000-GPU mesh on a laptop to see its schedule, its
peak memory and how many messages it sends.

Parity: python/monarch/simulator/mock_controller.py:114 (``MockController``),
python/monarch/_testing.py:203-223 (``mock_mesh``), python/monarch/simulator/simulator.py
(stream timelines, memory tracking, chrome trace), profiling.py (``RuntimeEstimator``),
python/monarch/sim_mesh.py.  The cost model here is a roofline: FLOPs over the measured
bf16 tensor throughput for matmuls, bytes over the measured HBM bandwidth for the rest,
bytes over NVLink bandwidth for collectives.
"""
from __future__ import annotations

import contextlib
import json
from typing import Any, Dict, List, Optional

import torch

from .actor.shape import Shape
from .tensor_engine.worker import Ref, RemoteError, _flatten_tensors, _map_refs, \
    _resolve_function

class CostModel:
    """Roofline estimate of an op's duration in microseconds."""

    def __init__(self, tflops: float = 1432.0, hbm_gbs: float = 6500.0, link_gbs: float = 770.0,
                 launch_us: float = 3.0):
        self.tflops, self.hbm_gbs, self.link_gbs, self.launch_us = tflops, hbm_gbs, link_gbs, launch_us

    @staticmethod
    def _bytes(ts) -> int:
        return sum(t.numel() * t.element_size() for t in ts)

    def op(self, name: str, ins: List[torch.Tensor], outs: List[torch.Tensor]) -> float:
        mem = (self._bytes(ins) + self._bytes(outs)) / (self.hbm_gbs * 1e3)
        flops = 0.0
        if any(k in name for k in ("mm", "matmul", "linear", "einsum")) and len(ins) >= 2 \
                and outs:
            k = ins[0].shape[-1] if ins[0].dim() else 1
            flops = 2.0 * outs[0].numel() * k
        return self.launch_us + max(mem, flops / (self.tflops * 1e6))

    def collective(self, nbytes: int, n: int, kind: str) -> float:
        vol = {"allreduce": 2.0 * (n - 1) / n, "stack": (n - 1), "scatter": (n - 1) / n,
               "p2p": 1.0}.get(kind, 1.0) * nbytes
        return self.launch_us + vol / (self.link_gbs * 1e3)


_META: List[Any] = []


@contextlib.contextmanager
def set_meta(value):
    """Tag every simulated task issued inside the block: the tags show up under ``args.meta``
    of the trace events (nested blocks stack).  Parity: python/monarch/simulator/config.py
    (``set_meta``)."""
    _META.append(value)
    try:
        yield
    finally:
        _META.pop()


class SimWorker:
    """One simulated rank: executes worker messages on meta tensors."""

    def __init__(self, rank: int, cost: CostModel, events: Optional[List[dict]]):
        self.rank, self.cost, self.events = rank, cost, events
        self.env: Dict[int, Any] = {}
        self.clock: Dict[int, float] = {0: 0.0}
        self.live_bytes = 0
        self.peak_bytes = 0
        self.n_messages = 0
        self.recordings: Dict[int, List[tuple]] = {}
        self.groups: Dict[Any, List[int]] = {}
        self.borrows: Dict[int, tuple] = {}

    # ---------------------------------------------------------------- bookkeeping
    def _set(self, rid: int, v) -> None:
        self._drop(rid)
        self.env[rid] = v
        if isinstance(v, torch.Tensor):
            self.live_bytes += v.numel() * v.element_size()
            self.peak_bytes = max(self.peak_bytes, self.live_bytes)

    def _drop(self, rid: int) -> None:
        v = self.env.pop(rid, None)
        if isinstance(v, torch.Tensor):
            self.live_bytes -= v.numel() * v.element_size()

    def _advance(self, stream: int, name: str, dur: float) -> None:
        t0 = self.clock.setdefault(stream, 0.0)
        self.clock[stream] = t0 + dur
        if self.events is not None:
            ev = {"name": name, "ph": "X", "pid": self.rank, "tid": stream, "ts": t0, "dur": dur}
            if _META:
                ev["args"] = {"meta": list(_META)}
            self.events.append(ev)

    # -------------------------------------------------------------------- messages
    def handle(self, msgs: List[tuple]) -> None:
        for m in msgs:
            self.n_messages += 1
            getattr(self, "_m_" + m[0], self._m_other)(*m[1:])

    def _m_other(self, *a) -> None:
        pass

    def _m_call(self, seq, results, mutates, fspec, args, kwargs, stream, metas=None) -> None:
        name = fspec[1] if isinstance(fspec[1], str) else getattr(fspec[1], "__name__", "udf")
        a = _map_refs(args, lambda r: self.env.get(r.id))
        k = _map_refs(kwargs, lambda r: self.env.get(r.id))
        ins = [t for t in _flatten_tensors((a, k))]
        try:
            if metas is not None and len(metas) == len(results) and \
                    not any(isinstance(t, RemoteError) for t in ins):
                # the controller announced the results' shapes (it propagated them already):
                # no need to run the operator on meta tensors a second time
                # (the simulated workers run inside the controller's process: keep the active
                # mesh's dispatch mode from taking these factory calls for mesh operations)
                from .tensor_engine import device_mesh as _dm
                prev = getattr(_dm._tls, "propagating", False)
                _dm._tls.propagating = True
                try:
                    flat = [torch.empty(shape, dtype=dtype, device="meta")
                            for shape, dtype in metas]
                finally:
                    _dm._tls.propagating = prev
            elif fspec[0] == "op":
                with torch.device("meta"):
                    out = _resolve_function(fspec)(*a, **k)
                flat = _flatten_tensors(out)
            else:
                flat = []   # user functions are opaque: results keep no shape
        except Exception as ex:  # noqa: BLE001
            for r in results + mutates:
                self._set(r.id, RemoteError(seq, self.rank, name, str(ex), ""))
            return
        if not results and mutates:
            flat = []
        for r, t in zip(results, flat):
            self._set(r.id, t)
        for r in results[len(flat):]:
            self._set(r.id, None)
        self._advance(stream, name, self.cost.op(name, ins, flat))

    def _m_delete(self, ids) -> None:
        for i in ids:
            self._drop(i)

    def _m_create_stream(self, stream_id, default) -> None:
        self.clock.setdefault(stream_id, 0.0)

    def _m_borrow_create(self, borrow_id, ref, from_stream, to_stream, result) -> None:
        self.clock[to_stream] = max(self.clock.get(to_stream, 0.0), self.clock.get(from_stream, 0.0))
        self.env[result.id] = self.env.get(ref.id)
        self.borrows[borrow_id] = (from_stream, to_stream)

    def _m_borrow_drop(self, borrow_id) -> None:
        b = self.borrows.pop(borrow_id, None)
        if b:
            self.clock[b[0]] = max(self.clock.get(b[0], 0.0), self.clock.get(b[1], 0.0))

    def _m_split_comm(self, key, all_groups) -> None:
        for ranks in all_groups:
            if self.rank in ranks:
                self.groups[key] = ranks

    def _m_reduce(self, seq, result, ref, key, reduction, scatter, inplace, out_ref, stream,
                  in_meta=None) -> None:
        t = self.env.get(ref.id)
        n = len(self.groups.get(key, [0]))
        if not isinstance(t, torch.Tensor):
            self._set(result.id, t)
            return
        nbytes = t.numel() * t.element_size()
        if reduction == "stack":
            out = t if scatter else torch.empty((n,) + tuple(t.shape), dtype=t.dtype, device="meta")
            kind = "scatter" if scatter else "stack"
        else:
            out = torch.empty(t.shape[1:], dtype=t.dtype, device="meta") if scatter else \
                (t if inplace else torch.empty_like(t))
            kind = "scatter" if scatter else "allreduce"
        self._set(result.id, out)
        self._advance(stream, f"reduce[{reduction}{',scatter' if scatter else ''}]",
                      self.cost.collective(nbytes, n, kind))

    def _m_send_meta(self, result, shape, dtype) -> None:
        self.env[("send_meta", result.id)] = (tuple(shape), dtype)

    def _m_send_tensor(self, seq, result, ref, from_ranks, to_ranks, stream) -> None:
        if self.rank in to_ranks:
            meta = self.env.pop(("send_meta", result.id), None)
            src = self.env.get(ref.id) if ref is not None else None
            if meta is not None:
                t = torch.empty(meta[0], dtype=meta[1], device="meta")
            else:
                t = src
            self._set(result.id, t)
            if isinstance(t, torch.Tensor):
                self._advance(stream, "send_tensor",
                              self.cost.collective(t.numel() * t.element_size(), 2, "p2p"))

    def _m_define_recording(self, rec_id, msgs, temps=()) -> None:
        self.recordings[rec_id] = msgs

    def _m_call_recording(self, rec_id, bind) -> None:
        rb = lambda o: _map_refs(o, lambda r: Ref(bind.get(r.id, r.id)))
        for m in self.recordings[rec_id]:
            getattr(self, "_m_" + m[0], self._m_other)(*[rb(x) for x in m[1:]])


class _Done:
    def __init__(self, v):
        self._v = v

    def get(self, timeout=None):
        return self._v


class _VM(list):
    def items(self):
        return iter(self)


class _Endpoint:
    def __init__(self, fn):
        self._fn = fn

    def broadcast(self, *a):
        self._fn(*a)

    def call(self, *a):
        return _Done(self._fn(*a))


class MockWorkers:
    """Stands where an actor mesh of tensor workers would: same endpoints, in process."""

    def __init__(self, ranks: List[int], cost: CostModel, trace: bool, all_workers=None):
        self.events: Optional[List[dict]] = [] if trace else None
        self._all = all_workers if all_workers is not None else \
            {r: SimWorker(r, cost, self.events) for r in ranks}
        self.ranks = ranks
        self.configure = _Endpoint(lambda port: None)
        self.run = _Endpoint(self._run)
        self.run_and_reply = _Endpoint(self._run_and_reply)

    def _run(self, msgs):
        for r in self.ranks:
            self._all[r].handle(msgs)

    def _run_and_reply(self, msgs, fetch):
        self._run(msgs)
        seq, tree, pre = fetch
        out = _VM()
        for r in self.ranks:
            w = self._all[r]
            vals = _map_refs(tree, lambda ref: w.env.get(ref.id))
            vals = torch.utils._pytree.tree_map(
                lambda t: torch.zeros(t.shape, dtype=t.dtype) if isinstance(t, torch.Tensor)
                else t, vals)
            if pre is not None:
                vals = _resolve_function(pre)(vals)
            out.append((r, ("ok", vals)))
        return out

    def _new_with_shape(self, shape) -> "MockWorkers":
        mw = MockWorkers(list(shape.ndslice.ranks()), None, False, all_workers=self._all)
        mw.events = self.events
        return mw


class Simulator:
    """Handle on a mock mesh's simulated workers: timings, memory, message counts."""

    def __init__(self, workers: MockWorkers):
        self._w = workers

    def makespan_us(self) -> float:
        return max(max(w.clock.values()) for w in self._w._all.values())

    def peak_memory_bytes(self) -> int:
        return max(w.peak_bytes for w in self._w._all.values())

    def live_memory_bytes(self, rank: int = 0) -> int:
        return self._w._all[rank].live_bytes

    def messages(self, rank: int = 0) -> int:
        return self._w._all[rank].n_messages

    def stream_clocks(self, rank: int = 0) -> Dict[int, float]:
        return dict(self._w._all[rank].clock)

    def events(self) -> List[dict]:
        """The trace events recorded so far (chrome-trace "X" events; tasks issued under
        :func:`set_meta` carry ``args.meta``)."""
        return list(self._w.events or [])

    def dump_chrome_trace(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"traceEvents": self._w.events or []}, f)


def mock_mesh(hosts: int = 1, gpus: int = 1, cost: Optional[CostModel] = None,
              trace: bool = True):
    """A device mesh ``{hosts, gpus}`` backed by simulated workers.  Returns (mesh, sim)."""
    import itertools
    import threading

    from .tensor_engine.device_mesh import Client, DeviceMesh
    n = hosts * gpus
    workers = MockWorkers(list(range(n)), cost or CostModel(), trace)
    shape = Shape.row_major(hosts=hosts, gpus=gpus)

    class _PM:  # the little of a proc mesh that Client needs
        _labels = ["hosts", "gpus"]

    client = Client.__new__(Client)
    client.proc_mesh = _PM()
    client.workers = workers
    client.use_cuda = False
    client._init_history(n)
    client._lock = threading.RLock()
    client._pending_deletes = []
    client._coalesce = None
    client._init_batching(1)     # simulated workers answer synchronously: nothing to batch
    client._recording = None
    client._pg_init = True      # there are no process groups to create
    client._comms = set()
    client._streams_made = {0}
    client.errors = []
    client._closed = False
    client._err_rx = None
    client._init_watchdog(0.0)   # simulated workers cannot stall
    client.send_metas = True     # results' shapes travel with the calls (see SimWorker._m_call)
    dm = DeviceMesh(client, shape, workers)
    client.root_mesh = dm
    return dm, Simulator(workers)
