"""Remote functions with cached shape propagation, and remote autograd functions.

Parity: python/monarch/cached_remote_function.py (``remote_autograd_function``: a
``torch.autograd.Function`` whose forward/backward run on the workers) and
common/remote.py:344-369 (``_cached_propagation``: propagate once per input signature).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Optional, Tuple

import torch


def _signature(args, kwargs) -> Tuple:
    def sig(o):
        if isinstance(o, torch.Tensor):
            return ("T", tuple(o.shape), o.dtype, o.requires_grad)
        if isinstance(o, (list, tuple)):
            return tuple(sig(x) for x in o)
        if isinstance(o, dict):
            return tuple(sorted((k, sig(v)) for k, v in o.items()))
        return ("V", repr(o))
    return (sig(args), sig(kwargs))


def cached_propagation(fn: Callable) -> Callable:
    """Wrap a propagate function so that it runs once per (shapes, dtypes, values) key and
    later calls reuse the recorded output metadata."""
    cache: Dict[Tuple, Any] = {}

    def prop(*args, **kwargs):
        key = _signature(args, kwargs)
        meta = cache.get(key)
        if meta is None:
            out = fn(*args, **kwargs)
            meta = torch.utils._pytree.tree_map(
                lambda t: ("T", tuple(t.shape), t.dtype) if isinstance(t, torch.Tensor) else t,
                out)
            cache[key] = meta
        return torch.utils._pytree.tree_map(
            lambda m: torch.empty(m[1], dtype=m[2]) if isinstance(m, tuple) and m and m[0] == "T"
            else m, meta, is_leaf=lambda m: isinstance(m, tuple) and bool(m) and m[0] == "T")

    prop.cache = cache
    return prop


def _paths_autograd_function(forward_path: str, backward_path: str, propagate: Callable,
                             backward_propagate: Callable) -> Callable:
    """Differentiable callable from two worker-side functions named by import path:
    ``forward(*tensors) -> tensor`` and ``backward(*tensors, grad) -> grads``."""
    from .tensor_engine import remote
    fwd = remote(forward_path, propagate=cached_propagation(propagate))
    bwd = remote(backward_path, propagate=cached_propagation(backward_propagate))

    class _Fn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *args):
            ctx.save_for_backward(*args)
            return fwd(*args)

        @staticmethod
        def backward(ctx, grad):
            out = bwd(*ctx.saved_tensors, grad)
            return out if isinstance(out, tuple) else (out,)

    return _Fn.apply


# ---- an existing torch.autograd.Function run on the workers --------------------------------
class _WorkerCtx:
    """What the wrapped function's ``forward``/``backward`` get as ``ctx``: it lives on the
    worker between the two (named by an OpaqueRef), so saved tensors, process groups and
    any attribute the function sets never leave the worker."""

    def __init__(self, needs_input_grad):
        self.needs_input_grad = tuple(needs_input_grad)
        self.saved_tensors: tuple = ()
        self.materialize_grads = True

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors

    def mark_non_differentiable(self, *tensors):
        pass

    def mark_dirty(self, *tensors):
        pass

    def set_materialize_grads(self, value: bool):
        self.materialize_grads = bool(value)


def _function_class(target):
    if isinstance(target, str):
        import importlib
        mod, _, name = target.rpartition(".")
        return getattr(importlib.import_module(mod), name)
    return target


def _as_inputs(args, needs):
    """Detached arguments carrying the controller's requires_grad flags (forward bodies
    branch on them)."""
    return [a.detach().requires_grad_(True) if isinstance(a, torch.Tensor) and n else
            (a.detach() if isinstance(a, torch.Tensor) else a) for a, n in zip(args, needs)]


def _detached(out):
    return torch.utils._pytree.tree_map(
        lambda o: o.detach() if isinstance(o, torch.Tensor) else o, out)


def _autograd_forward(target, needs, *args):
    from .opaque_object import OpaqueRef
    ctx = _WorkerCtx(needs)
    with torch.no_grad():
        out = _function_class(target).forward(ctx, *_as_inputs(args, needs))
    return _detached(out), OpaqueRef(ctx)


def _autograd_backward(target, ctx_ref, metas, *grads):
    ctx = ctx_ref.value
    with torch.no_grad():
        g = _function_class(target).backward(ctx, *grads)
    g = g if isinstance(g, tuple) else (g,)
    out = []
    for i, m in enumerate(metas):
        if m is None:
            continue
        gi = g[i] if i < len(g) else None
        if gi is None:
            like = next((t for t in grads if isinstance(t, torch.Tensor)), None)
            gi = torch.zeros(m[0], dtype=m[1], device=like.device if like is not None else None)
        out.append(gi.detach())
    return out


class RemoteAutogradFunction(torch.autograd.Function):
    """Base of the classes :func:`remote_autograd_function` makes."""


def remote_autograd_function(target_class, *rest, name: Optional[str] = None, **kw):
    """``Remote = remote_autograd_function(MyFunction)``: a ``torch.autograd.Function`` whose
    ``Remote.apply(*args)`` runs ``MyFunction.forward`` on every worker of the arguments'
    mesh and, when the controller's autograd reaches it, ``MyFunction.backward`` there too.
    Shapes come from running ``forward`` once on fakes.  ``MyFunction`` may be given by
    import path.  (The older form ``remote_autograd_function(forward_path, backward_path,
    propagate, backward_propagate)`` builds the function from two plain worker functions.)

    Parity: python/monarch/cached_remote_function.py:222-257.  The reference pickles a
    stand-in ctx to the worker and back and keeps its tensors on the controller's ctx as
    distributed tensors; here the ctx stays on the worker under an OpaqueRef that the
    controller's ctx holds, and goes when the graph does."""
    if rest or kw:
        return _paths_autograd_function(target_class, *rest, **kw)
    if isinstance(target_class, type) and issubclass(target_class, RemoteAutogradFunction):
        return target_class
    cls = _function_class(target_class)
    if not (isinstance(cls, type) and issubclass(cls, torch.autograd.Function)):
        raise TypeError(f"{target_class!r} is not a torch.autograd.Function")
    from .opaque_object import OpaqueRef
    from .tensor_engine import remote

    def prop_forward(target, needs, *fake_args):
        out = cls.forward(_WorkerCtx(needs), *_as_inputs(fake_args, needs))
        return _detached(out), OpaqueRef(None)

    def prop_backward(target, ctx_ref, metas, *grads):
        return [torch.empty(m[0], dtype=m[1]) for m in metas if m is not None]

    fwd = remote(_autograd_forward, propagate=prop_forward)
    bwd = remote(_autograd_backward, propagate=prop_backward)

    def forward(ctx, *args):
        needs = tuple(isinstance(a, torch.Tensor) and a.requires_grad for a in args)
        out, ref = fwd(target_class, needs, *args)
        if ctx is not None:
            ctx.worker_ctx = ref
            ctx.metas = tuple((tuple(a.shape), a.dtype) if n else None
                              for a, n in zip(args, needs))
        return out

    def backward(ctx, *grads):
        got = iter(bwd(target_class, ctx.worker_ctx, ctx.metas, *grads))
        return tuple(next(got) if m is not None else None for m in ctx.metas)

    return type(name or f"Remote_{cls.__name__}", (RemoteAutogradFunction,),
                {"forward": staticmethod(forward), "backward": staticmethod(backward)})
