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


class OpaqueModule:
    """``m = OpaqueModule("torch.nn.Linear", 4, 3)`` on the active device mesh."""

    def __init__(self, constructor, *args, **kwargs):
        self._obj = oo.OpaqueObject(constructor, *args, **kwargs)
        from .tensor_engine import no_mesh
        with no_mesh(), torch.device("meta"):   # shape-only twin used for propagation
            self._fake = oo._resolve(constructor)(*args, **kwargs)

    def _r(self, name: str, propagate: Any = None) -> Callable:
        from .tensor_engine import get_active_mesh, remote
        if get_active_mesh() is None:
            return globals()[name]
        return remote(f"monarch_b200.opaque_module.{name}", propagate=propagate)

    def __call__(self, *args):
        def prop(oid, *fa):
            ins = [torch.empty(a.shape, dtype=a.dtype, device="meta")
                   if isinstance(a, torch.Tensor) else a for a in fa]
            with torch.no_grad():
                out = self._fake(*ins)
            return torch.empty(out.shape, dtype=out.dtype)
        return self._r("_forward", prop)(self._obj.ref.id, *args)

    def backward(self, grad_out, like_input):
        """Input gradient of the last forward (shaped like ``like_input``)."""
        return self._r("_backward", lambda oid, g: torch.empty_like(like_input))(
            self._obj.ref.id, grad_out)

    def parameters(self) -> List[torch.Tensor]:
        shapes = [(tuple(p.shape), p.dtype) for p in self._fake.parameters()]
        return self._r("_parameters", lambda oid: [torch.empty(s, dtype=d) for s, d in shapes])(
            self._obj.ref.id)

    def grads(self) -> List[torch.Tensor]:
        shapes = [(tuple(p.shape), p.dtype) for p in self._fake.parameters()]
        return self._r("_param_grads", lambda oid: [torch.empty(s, dtype=d) for s, d in shapes])(
            self._obj.ref.id)

    def sgd_step(self, lr: float) -> None:
        self._r("_sgd_step")(self._obj.ref.id, lr)
