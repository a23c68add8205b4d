"""Gradients handed out one at a time while the backward pass is still running.

Parity: python/monarch/gradient_generator.py (``grad_generator``, ``GradGenerator``,
``grad_function``, ``gradient_execution_order``) and the C++ executor behind it.  The
autograd engine runs on its own thread; a hook on each tensor publishes its gradient as
soon as it is final, and the generator yields them in the order of ``with_respect_to``
(pass parameters in reverse order of use to receive gradients as early as possible and
overlap their reduction with the rest of backward).  The order in which gradients become
final is computed from the autograd graph by the ``_gradgen`` extension.
"""
from __future__ import annotations

import queue
import threading
from functools import partial
from types import CellType, FunctionType
from typing import Any, List, Optional, Sequence, Union

import torch


def _ext():
    try:
        from . import _gradgen
    except ImportError:
        from . import _build
        _build.build_gradgen()
        from . import _gradgen
    return _gradgen


def gradient_execution_order(roots: Sequence[torch.Tensor],
                             with_respect_to: Sequence[torch.Tensor]) -> List[int]:
    """Indices of ``with_respect_to`` in the order their gradients become available when
    autograd runs on ``roots`` (reverse order of first use in the backward graph)."""
    return list(_ext().execution_order(list(roots), list(with_respect_to)))


class _GradientGenerator:
    def __init__(self, roots, with_respect_to, grad_roots):
        self._wrt = list(with_respect_to)
        self._n = len(self._wrt)
        self._results: List[Any] = [None] * self._n
        self._ready = [threading.Event() for _ in range(self._n)]
        self._error: Optional[BaseException] = None
        self._next = 0
        self._hooks = []
        index = {}
        for i, t in enumerate(self._wrt):
            index.setdefault(id(t), []).append(i)

        def make_hook(ids):
            def hook(g):
                for i in ids:
                    self._results[i] = g
                    self._ready[i].set()
                return g
            return hook

        seen = set()
        for t in self._wrt:
            if id(t) not in seen:
                seen.add(id(t))
                self._hooks.append(t.register_hook(make_hook(index[id(t)])))
        roots = list(roots)
        grads = list(grad_roots) if grad_roots else None

        def run():
            try:
                if self._wrt:
                    torch.autograd.grad(roots, self._wrt, grads, allow_unused=True)
            except BaseException as e:  # noqa: BLE001 - re-raised in the consumer
                self._error = e
            finally:
                for h in self._hooks:
                    h.remove()
                for ev in self._ready:   # unused inputs never fire: they yield None
                    ev.set()

        self._thread = threading.Thread(target=run, daemon=True, name="monarch-backward")
        self._thread.start()

    def __iter__(self):
        return self

    def __next__(self):
        if self._next >= self._n:
            self._thread.join()
            if self._error is not None:
                raise self._error
            raise StopIteration
        i = self._next
        self._next += 1
        self._ready[i].wait()
        if self._error is not None:
            raise self._error
        return self._results[i]


def grad_generator(roots: Union[torch.Tensor, Sequence[torch.Tensor]] = (),
                   with_respect_to: Sequence[torch.Tensor] = (),
                   grad_roots: Sequence[Optional[torch.Tensor]] = ()):
    """Iterator over d(roots)/d(t) for t in ``with_respect_to``, each yielded as soon as it
    is final; ``None`` for tensors the roots do not depend on."""
    if isinstance(roots, torch.Tensor):
        roots = [roots]
    return _GradientGenerator(list(roots), list(with_respect_to), list(grad_roots))


class GradGenerator:
    """Builder form: ``g.root(loss); g.grad(tree)...``; iterating yields one gradient tree
    per ``grad`` call, last registered first."""

    def __init__(self):
        self.roots: List[torch.Tensor] = []
        self.grad_roots: List[Optional[torch.Tensor]] = []
        self.with_respect_to: List[torch.Tensor] = []
        self._groups: List[Any] = []

    def grad(self, tree: Any) -> None:
        from torch.utils._pytree import tree_flatten
        leaves, spec = tree_flatten(tree)
        tensors = [l for l in leaves if isinstance(l, torch.Tensor)]
        self._groups.append((leaves, spec, len(tensors)))
        self.with_respect_to.extend(tensors)

    def root(self, r: torch.Tensor, grad: Optional[torch.Tensor] = None) -> None:
        self.roots.append(r)
        self.grad_roots.append(grad)

    def __iter__(self):
        from torch.utils._pytree import tree_unflatten
        gr = self.grad_roots if any(g is not None for g in self.grad_roots) else []
        gi = grad_generator(self.roots, list(reversed(self.with_respect_to)), gr)
        for leaves, spec, n in reversed(self._groups):
            got = list(reversed([next(gi) for _ in range(n)]))
            it = iter(got)
            yield tree_unflatten([next(it) if isinstance(l, torch.Tensor) else l
                                  for l in leaves], spec)


class _GradFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, *args, **kwargs):
        result, backward_continuation = fn(*args, **kwargs)
        ctx.backward_continuation = backward_continuation
        values = []
        if backward_continuation.__closure__ is not None:
            for cell in backward_continuation.__closure__:
                values.append(cell.cell_contents)
        ctx.n_values = len(values)
        ctx.kinds = [isinstance(v, torch.Tensor) for v in values]
        ctx.others = [None if k else v for k, v in zip(ctx.kinds, values)]
        ctx.save_for_backward(*[v for v in values if isinstance(v, torch.Tensor)])
        return result

    @staticmethod
    def backward(ctx, *grads):
        saved = iter(ctx.saved_tensors)
        vals = [next(saved) if k else o for k, o in zip(ctx.kinds, ctx.others)]
        orig = ctx.backward_continuation
        fn = FunctionType(orig.__code__, orig.__globals__, orig.__name__, orig.__defaults__,
                          tuple(CellType(v) for v in vals))
        out = fn(*grads)
        return (None, *out) if isinstance(out, tuple) else (None, out)


def grad_function(fn):
    """``fn(*args) -> (result, backward_continuation)``: an autograd function whose backward
    is the returned closure (its captured tensors are saved for backward)."""
    return partial(_GradFunction.apply, fn)
