"""``torch.nn.Module`` living on the workers, driven from the controller.

Parity: python/monarch/opaque_module.py (``OpaqueModule``: construct remotely, call
forward with distributed tensors, enumerate parameters as distributed tensors, backward
through a remote autograd function -- cached_remote_function.py's
``remote_autograd_function``)."""
from __future__ import annotations

from typing import Any, Callable, List

import torch

from . import opaque_object as oo


# ---- worker side ----------------------------------------------------------------------
def _forward(oid: int, *args):
    m = oo._TABLE[oid]
    ins = [a.detach().requires_grad_(a.is_floating_point()) if isinstance(a, torch.Tensor)
           else a for a in args]
    with torch.enable_grad():
        out = m(*ins)
    m._mb200_last = (ins, out)
    return out.detach()


def _backward(oid: int, grad_out: torch.Tensor):
    """Accumulates parameter gradients on the worker; returns the input gradients."""
    m = oo._TABLE[oid]
    ins, out = m._mb200_last
    tins = [t for t in ins if isinstance(t, torch.Tensor) and t.requires_grad]
    params = [p for p in m.parameters() if p.requires_grad]
    grads = torch.autograd.grad(out, tins + params, grad_out, allow_unused=True)
    for p, g in zip(params, grads[len(tins):]):
        if g is not None:
            p.grad = g if p.grad is None else p.grad + g
    gi = [g if g is not None else torch.zeros_like(t) for t, g in zip(tins, grads[:len(tins)])]
    return gi[0] if len(gi) == 1 else tuple(gi)


def _parameters(oid: int):
    return [p.detach() for p in oo._TABLE[oid].parameters()]


def _param_grads(oid: int):
    return [p.grad if p.grad is not None else torch.zeros_like(p)
            for p in oo._TABLE[oid].parameters()]


def _sgd_step(oid: int, lr: float) -> None:
    with torch.no_grad():
        for p in oo._TABLE[oid].parameters():
            if p.grad is not None:
                p.add_(p.grad, alpha=-lr)
                p.grad = None


def _forward_graph(oid, needs, n_in: int, *args):
    """Forward that keeps its autograd graph on the worker: returns an OpaqueRef of a
    closure computing the gradients of the inputs and parameters marked in ``needs``, and
    the detached output (python/monarch/opaque_module.py ``_remote_forward`` in the
    reference)."""
    m = oo._target(oid)
    params = list(m.parameters())
    ins = [a.detach().requires_grad_(True) if isinstance(a, torch.Tensor) and n else a
           for a, n in zip(args, needs[:n_in])]
    with torch.enable_grad():
        out = m(*ins)
    outs = [o for o in (out if isinstance(out, (list, tuple)) else [out])
            if isinstance(o, torch.Tensor)]
    wanted = [t for t, n in zip(ins, needs[:n_in]) if n] + \
             [p for p, n in zip(params, needs[n_in:]) if n]

    def backward(grad_outputs):
        live = [(o, g) for o, g in zip(outs, grad_outputs) if o.requires_grad and g is not None]
        with torch.no_grad():
            got = torch.autograd.grad([o for o, _ in live], wanted, [g for _, g in live],
                                      allow_unused=True) if live else [None] * len(wanted)
        return [g if g is not None else torch.zeros_like(w) for g, w in zip(got, wanted)]

    det = [o.detach() for o in outs]
    return oo.OpaqueRef(backward), (det[0] if not isinstance(out, (list, tuple)) else det)


def _backward_graph(closure_ref, grad_outputs):
    return closure_ref.value(grad_outputs)


class _ModuleCall(torch.autograd.Function):
    """The controller's autograd node of one call of an :class:`OpaqueModule`."""

    @staticmethod
    def forward(ctx, module, n_in, *tensors):
        from .tensor_engine import remote
        needs = tuple(isinstance(t, torch.Tensor) and t.requires_grad for t in tensors)
        prop = lambda oid, needs, n, *fa: (oo.OpaqueRef(None), module._out_shape(*fa))  # noqa
        ref, out = remote(_forward_graph, propagate=prop)(module._obj._handle, needs, n_in,
                                                          *tensors[:n_in])
        ctx.closure = ref
        ctx.metas = tuple((tuple(t.shape), t.dtype) if n else None
                          for t, n in zip(tensors, needs))
        return tuple(out) if isinstance(out, list) else out

    @staticmethod
    def backward(ctx, *grads):
        from .tensor_engine import remote
        prop = lambda ref, gs: [torch.empty(m[0], dtype=m[1])  # noqa: E731
                                for m in ctx.metas if m is not None]
        got = iter(remote(_backward_graph, propagate=prop)(ctx.closure, list(grads)))
        return (None, None) + tuple(next(got) if m is not None else None for m in ctx.metas)


class OpaqueModule:
    """``m = OpaqueModule("torch.nn.Linear", 4, 3)`` on the active device mesh.

    ``m(x)`` runs the forward on every worker.  Gradients either stay on the workers
    (``m.backward(grad_out, x)`` returns the input gradient and accumulates ``p.grad`` there;
    ``m.grads()`` / ``m.sgd_step(lr)`` use them), or flow through the controller's autograd
    as for a local module: once ``m.parameters()`` has been taken (leaf tensors that require
    grad, aliasing the workers' parameters) or an input requires grad, ``m(x)`` records an
    autograd node, and ``loss.backward()`` leaves ``x.grad`` and ``p.grad`` on the
    controller as distributed tensors."""

    def __init__(self, constructor, *args, **kwargs):
        self._obj = oo.OpaqueObject(constructor, *args, **kwargs)
        from .tensor_engine import no_mesh
        with no_mesh(), torch.device("meta"):   # shape-only twin used for propagation
            self._fake = oo._resolve(constructor)(*args, **kwargs)
        self._params = None

    def _r(self, name: str, propagate: Any = None) -> Callable:
        from .tensor_engine import get_active_mesh, remote
        if get_active_mesh() is None:
            return globals()[name]
        return remote(f"monarch_b200.opaque_module.{name}", propagate=propagate)

    def _out_shape(self, *fa):
        ins = [torch.empty(a.shape, dtype=a.dtype, device="meta")
               if isinstance(a, torch.Tensor) else a for a in fa]
        with torch.no_grad():
            out = self._fake(*ins)
        like = lambda o: torch.empty(o.shape, dtype=o.dtype)  # noqa: E731
        return [like(o) for o in out] if isinstance(out, (list, tuple)) else like(out)

    def call_method(self, method: str, propagate: Any = None, *args, **kwargs):
        return self._obj.call_method(method, propagate, *args, **kwargs)

    def __call__(self, *args):
        from .tensor_engine import get_active_mesh
        if get_active_mesh() is not None and torch.is_grad_enabled() and (
                self._params is not None
                or any(isinstance(a, torch.Tensor) and a.requires_grad for a in args)):
            params = self._params or []
            return _ModuleCall.apply(self, len(args), *args, *params)
        return self._r("_forward", lambda oid, *fa: self._out_shape(*fa))(self._obj.ref.id, *args)

    def backward(self, grad_out, like_input):
        """Input gradient of the last forward (shaped like ``like_input``)."""
        return self._r("_backward", lambda oid, g: torch.empty_like(like_input))(
            self._obj.ref.id, grad_out)

    def parameters(self) -> List[torch.Tensor]:
        """The workers' parameters as distributed leaf tensors (fetched once): writing them in
        place (under ``torch.no_grad()``) changes the module."""
        if self._params is None:
            shapes = [(tuple(p.shape), p.dtype) for p in self._fake.parameters()]
            ps = self._r("_parameters",
                         lambda oid: [torch.empty(s, dtype=d) for s, d in shapes])(self._obj.ref.id)
            from .tensor_engine import get_active_mesh
            if get_active_mesh() is None:
                return ps
            self._params = [p.requires_grad_(f.requires_grad)
                            for p, f in zip(ps, self._fake.parameters())]
        return self._params

    def grads(self) -> List[torch.Tensor]:
        shapes = [(tuple(p.shape), p.dtype) for p in self._fake.parameters()]
        return self._r("_param_grads", lambda oid: [torch.empty(s, dtype=d) for s, d in shapes])(
            self._obj.ref.id)

    def sgd_step(self, lr: float) -> None:
        self._r("_sgd_step")(self._obj.ref.id, lr)
