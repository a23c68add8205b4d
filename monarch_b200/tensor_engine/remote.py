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


def _string_resolver(fn) -> Optional[tuple]:
    if isinstance(fn, str) and "." in fn:
        return ("path", fn)
    return None


def _torch_op_resolver(fn) -> Optional[tuple]:
    if isinstance(fn, torch._ops.OpOverload):
        return ("op", str(fn))          # e.g. "aten.add.Tensor"
    return None


def _import_path_resolver(fn) -> Optional[tuple]:
    """A module-level function that the workers can import travels as its dotted path (a
    few bytes) instead of a pickle.  Functions of the launching script and of modules loaded
    by a test runner's own import machinery do not qualify: the workers could not find them."""
    mod, name = getattr(fn, "__module__", None), getattr(fn, "__qualname__", "")
    if not callable(fn) or not mod or mod in ("__main__", "__mp_main__") or "<" in name \
            or "." in name:
        return None
    import sys
    m = sys.modules.get(mod)
    if m is None or getattr(m, name, None) is not fn:
        return None
    loader = type(getattr(m, "__loader__", None)).__module__ or ""
    if "pytest" in loader or getattr(m, "__file__", None) is None:
        return None
    return ("path", f"{mod}.{name}")


def _pickle_resolver(fn) -> Optional[tuple]:
    return ("pickle", fn) if callable(fn) else None


# Tried in order; the first that answers decides how a function reaches the workers
# (python/monarch/common/function.py ``resolvers`` in the reference).  Programs may insert
# their own, e.g. to map handles of a registry to paths.
function_resolvers = [_string_resolver, _torch_op_resolver, _import_path_resolver,
                      _pickle_resolver]


def _resolve_spec(fn) -> tuple:
    for r in function_resolvers:
        spec = r(fn)
        if spec is not None:
            return spec
    raise ValueError(f"{fn!r} cannot be sent to the workers as a function")


class _TensorMeta(tuple):
    """(shape, dtype, device) of a tensor a probed call returned."""

    def __new__(cls, *fields):
        return super().__new__(cls, fields)


def _from_meta(meta):
    return torch.utils._pytree.tree_map(
        lambda m: torch.empty(m[0], dtype=m[1], device=m[2]) if isinstance(m, _TensorMeta) else m,
        meta, is_leaf=lambda m: isinstance(m, _TensorMeta))


class Remote:
    def __init__(self, fn, propagate=None):
        self._fn = fn
        self._propagate = propagate
        self._cache: dict = {}
        self.cache_hits = 0
        if callable(fn):
            functools.update_wrapper(self, fn)

    def _fake_outputs(self, args, kwargs, mesh: DeviceMesh):
        p = self._propagate
        if callable(p):
            with _propagation():
                return p(*_to_fake(args), **_to_fake(kwargs))
        if p in ("inspect", "cached"):
            # run the real function on one shard and copy the metadata of what comes back;
            # "cached" does so once per signature of the arguments (shapes, dtypes,
            # requires_grad, plain values) and answers later calls from the table
            # (python/monarch/common/remote.py ``_cached_propagation`` in the reference)
            key = None
            if p == "cached":
                from ..cached_remote_function import _signature
                key = _signature(args, kwargs)
                meta = self._cache.get(key)
                if meta is not None:
                    self.cache_hits += 1
                    with _propagation():
                        return _from_meta(meta)
            first = {l: 0 for l in mesh._labels}
            sample = call_on_shard_and_fetch(self, *args, shard=first, _raw=True, **kwargs).get()
            meta = torch.utils._pytree.tree_map(
                lambda t: _TensorMeta(tuple(t.shape), t.dtype, t.device)
                if isinstance(t, torch.Tensor) else t, sample)
            if key is not None:
                self._cache[key] = meta
            with _propagation():
                return _from_meta(meta)
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
        # a propagation function that changes an argument in place (``t.add_(1)``) says that
        # the worker function does: those tensors are marked as written by the call, so a
        # failure of the function poisons them too (python/monarch/common/remote.py
        # ``dtensor_check`` reads the same from the fakes' version counters)
        before = [t._fake._version for t in ts]
        fake_out = self._fake_outputs(args, kwargs, mesh)
        mutated, seen = [], set()
        for t, v in zip(ts, before):
            if t._fake._version != v and id(t) not in seen:
                seen.add(id(t))
                mutated.append(t)
        return _send_call(_resolve_spec(self._fn), args, kwargs, fake_out, mesh, mutated)

    def call_on_shard_and_fetch(self, *args, shard=None, **kwargs) -> Future:
        return call_on_shard_and_fetch(self, *args, shard=shard, **kwargs)


def remote(fn=None, *, propagate=None):
    """``@remote(propagate=lambda x: x)`` marks ``fn`` to run on every worker of the mesh of
    its tensor arguments; results are distributed tensors shaped like ``propagate``'s.

    ``propagate`` is a function run on fakes (it may be the worker function itself; writing
    an argument in place there marks the argument as written by the call), ``"inspect"``
    (run the real function on the first shard and copy the shapes of what returns),
    ``"cached"`` (the same, once per signature of the arguments), or ``None`` / ``"mocked"``
    for functions that return no tensors."""
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
    # the value comes from one shard, but it stands for the whole distributed tensor: the
    # other ranks are asked whether their shards are sound (a failure on rank 1 is raised
    # by a fetch from rank 0 too, as in the reference's fetch_shard)
    chk = None
    if ts and getattr(mesh.client, "check_all_ranks_on_fetch", False) and len(sub._workers) < len(mesh._workers) \
            and hasattr(mesh._workers.run_and_reply, "_open"):
        chk = mesh.client.fetch(mesh, [Ref(t.ref) for t in ts], ("status",))

    def wait(t):
        v = f.get(t)[0]
        if chk is not None:
            chk.get(t)
        return v

    return Future(wait)


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


# ------------------------------------------------------------------------- recordings --
class _Compiled:
    """Result of :func:`compile`: traces ``fn`` once per input signature, ships the traced
    worker messages as a *recording*, and replays it with one message per later call."""
    _ids = iter(range(1, 1 << 30))

    def __init__(self, fn, verify: bool = False):
        self._fn = fn
        self._verify = verify
        self._cache = {}
        functools.update_wrapper(self, fn)

    @staticmethod
    def _key(args, kwargs, mesh):
        def sig(o):
            if isinstance(o, Tensor):
                return ("T", tuple(o.shape), o.dtype, o.requires_grad)
            if isinstance(o, (list, tuple)):
                return (type(o).__name__,) + tuple(sig(x) for x in o)
            if isinstance(o, dict):
                return tuple(sorted((k, sig(v)) for k, v in o.items()))
            return ("V", repr(o))
        return (sig(args), sig(kwargs), id(mesh._workers))

    def __call__(self, *args, **kwargs):
        from .device_mesh import get_active_stream
        ins: list = []
        _collect(args, ins)
        _collect(kwargs, ins)
        mesh = _mesh_of(ins) if ins else get_active_mesh()
        if mesh is None:
            raise RuntimeError("no active device mesh")
        client = mesh.client
        key = self._key(args, kwargs, mesh)
        rec = self._cache.get(key)
        if rec is None:
            return self._trace(key, mesh, client, ins, args, kwargs)
        rec_id, formals, out_ids, out_meta, out_tree = rec
        bind = {f: t.ref for f, t in zip(formals, ins)}
        by_formal = dict(zip(formals, ins))
        stream = get_active_stream()
        outs = []
        for (shape, dtype), oid in zip(out_meta, out_ids):
            if oid in by_formal:          # the function handed one of its inputs back
                outs.append(by_formal[oid])
                continue
            with _propagation():
                fake = torch.empty(shape, dtype=dtype)
            t = Tensor(fake, mesh, stream)
            bind[oid] = t.ref
            outs.append(t)
        # the recording's temporaries live and die on the workers: nothing to bind or delete
        client.send(mesh, ("call_recording", rec_id, bind))
        it = iter(outs)
        return torch.utils._pytree.tree_map(
            lambda m: next(it) if m == "__tensor__" else m, out_tree)

    def _trace(self, key, mesh, client, ins, args, kwargs):
        if client._coalesce is not None:
            raise RuntimeError("compile() cannot trace inside a coalescing block")
        first_new = client.new_ref()      # every ref allocated from here on is internal
        client._coalesce = []
        try:
            out = self._fn(*args, **kwargs)
        finally:
            batch, client._coalesce = client._coalesce, None
        msgs = []
        for m, msg in batch:
            if m._workers is not mesh._workers and m._ndslice != mesh._ndslice:
                raise RuntimeError("compile() supports functions that stay on one mesh (a "
                                   f"{msg[0]!r} message goes to {m}, the recording to {mesh})")
            msgs.append(msg)
        outs: list = []
        _collect(out, outs)
        internal = set()

        def visit(o):
            if isinstance(o, Ref):
                if o.id > first_new:
                    internal.add(o.id)
            elif isinstance(o, (list, tuple)):
                for x in o:
                    visit(x)
            elif isinstance(o, dict):
                for x in o.values():
                    visit(x)
        visit(msgs)
        rec_id = next(self._ids)
        out_refs = {t.ref for t in outs}
        temps = sorted(i for i in internal if i not in out_refs)
        client.send(mesh, ("define_recording", rec_id, msgs, temps))
        client.send(mesh, ("call_recording", rec_id, {}))
        out_tree = torch.utils._pytree.tree_map(
            lambda t: "__tensor__" if isinstance(t, Tensor) else t, out)
        self._cache[key] = (rec_id, [t.ref for t in ins], [t.ref for t in outs],
                            [(tuple(t.shape), t.dtype) for t in outs], out_tree)
        return out


def compile(fn=None, *, verify: bool = False):
    """``@compile`` -- trace a function of distributed tensors once and replay it on the
    workers with a single message per call (the controller's per-op dispatch and shape
    propagation disappear from the steady state).  A new trace is taken for every new
    combination of input shapes/dtypes and non-tensor argument values.

    Parity: python/monarch/common/_coalescing.py:98-298 (``compile``), worker
    ``DefineRecording`` / ``CallRecording`` (monarch_messages/src/worker.rs:854-905)."""
    if fn is None:
        return lambda f: _Compiled(f, verify)
    return _Compiled(fn, verify)
