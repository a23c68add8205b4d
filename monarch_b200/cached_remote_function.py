"""Remote functions with cached shape propagation, and remote autograd functions.

Parity: python/monarch/cached_remote_function.py (``remote_autograd_function``: a
``torch.autograd.Function`` whose forward/backward run on the workers) and
common/remote.py:344-369 (``_cached_propagation``: propagate once per input signature).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Tuple

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


def remote_autograd_function(forward_path: str, backward_path: str, propagate: Callable,
                             backward_propagate: Callable) -> Callable:
    """Build a differentiable callable from two worker-side functions named by import
    path.  ``forward(*tensors) -> tensor`` and ``backward(*tensors, grad) -> grads``."""
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
