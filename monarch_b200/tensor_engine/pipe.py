"""Pipes: worker-side generators (data loaders and the like) feeding distributed tensors.

Parity: python/monarch/common/pipe.py:23-121 (``remote_generator``, ``create_pipe``,
``Pipe.send/recv``) and python/monarch/worker/worker.py:573-595, 1158-1191 (the worker's end
and the pipe process).  The reference runs the generator in a separate process per worker
behind a ZMQ PAIR socket; here it is a thread of the worker proc behind two bounded queues,
which keeps the produced tensors in the address space that consumes them (a GPU batch made
by the generator is handed to the stream without a copy).

    @remote_generator("my_data.loader", max_messages=8)
    def loader(pipe, batch, seq):              # propagation: yields what the worker yields
        while True:
            yield {"x": torch.zeros(batch, seq), "y": torch.zeros(batch)}

    with mesh.activate():
        p = loader(4, 128)
        batch = p.recv()                       # dict of distributed tensors

The worker function ``my_data.loader(pipe, batch, seq)`` either is a generator (its yields
are the messages) or calls ``pipe.send(obj)`` itself; ``pipe.recv()`` on the worker returns
what the controller passed to ``Pipe.send``; ``pipe.ranks`` / ``pipe.sizes`` give the
worker's coordinates in the mesh.
"""
from __future__ import annotations

from collections import deque
from typing import Any

import torch

from .device_mesh import (Tensor, _collect, _propagation, _to_wire, _wrap_outputs,
                          get_active_mesh, get_active_stream)
from .remote import Remote, _resolve_spec
from .worker import Ref


class FakePipe:
    """What the propagation generator sees: ``recv`` replays the fakes of what the
    controller sent (python/monarch/common/pipe.py:136-152)."""

    def __init__(self):
        self._fake_sends: deque = deque()

    def send(self, obj: Any):
        raise RuntimeError("in a propagation function use `yield x`, not pipe.send(x)")

    def recv(self):
        if self._fake_sends:
            return self._fake_sends.popleft()
        raise RuntimeError("propagation asked for a value the controller has not sent")

    @property
    def ranks(self):
        raise ValueError("cannot be accessed on the controller")

    sizes = ranks


class Pipe:
    def __init__(self, fn: Remote, max_messages: int, args, kwargs):
        mesh = get_active_mesh()
        if mesh is None:
            raise ValueError("remote generators require an active device mesh "
                             "(use `with mesh.activate():`)")
        if not isinstance(fn, Remote):
            raise TypeError("expected a remote function")
        ts: list = []
        _collect((args, kwargs), ts)
        if ts:
            raise ValueError("cannot pass distributed tensors to a remote generator")
        if not callable(fn._propagate):
            raise ValueError("a remote generator needs a propagation generator function")
        self.mesh = mesh
        self._fake_pipe = FakePipe()
        with _propagation():
            self._iterator = iter(fn._propagate(self._fake_pipe, *args, **kwargs))
        self.ref = mesh.client.new_ref()
        self._dropped = False
        nd = mesh._ndslice
        mesh.client.send(mesh, ("create_pipe", self.ref, _resolve_spec(fn._fn), int(max_messages),
                                args, kwargs, list(mesh._labels), int(nd.offset),
                                list(nd.sizes), list(nd.strides)))

    def send(self, obj: Any) -> None:
        """Hand ``obj`` (plain values and/or distributed tensors of this mesh) to the
        generator's ``pipe.recv()``."""
        ts: list = []
        _collect(obj, ts)
        for t in ts:
            if t.mesh is not self.mesh and t.mesh._ndslice != self.mesh._ndslice:
                raise ValueError(f"pipe lives on {self.mesh} but a tensor lives on {t.mesh}")
        from .device_mesh import _to_fake
        self._fake_pipe._fake_sends.append(_to_fake(obj))
        client = self.mesh.client
        stream = get_active_stream()
        client._ensure_stream(stream)
        client.send(self.mesh, ("pipe_send", client.new_seq(), self.ref, _to_wire(obj), stream.id))

    def recv(self) -> Any:
        """The generator's next message as distributed tensors (shapes from the
        propagation generator)."""
        with _propagation():
            fake = next(self._iterator)
        client = self.mesh.client
        stream = get_active_stream()
        client._ensure_stream(stream)
        refs: list = []
        out = _wrap_outputs(fake, self.mesh, stream, refs)
        client.send(self.mesh, ("pipe_recv", client.new_seq(), refs, self.ref, stream.id))
        return out

    def drop(self) -> None:
        if not self._dropped:
            self._dropped = True
            try:
                self.mesh.client.send(self.mesh, ("drop_pipe", self.ref))
            except Exception:  # noqa: BLE001 - engine already shut down
                pass

    def __del__(self):
        try:
            self.drop()
        except Exception:  # noqa: BLE001
            pass

    @property
    def ranks(self):
        raise ValueError("cannot be accessed on the controller")

    sizes = ranks


def create_pipe(fn: Remote, *args, max_messages: int = 50, **kwargs) -> Pipe:
    return Pipe(fn, max_messages, args, kwargs)


def remote_generator(path_or_fn, max_messages: int = 50):
    """Decorator: the decorated generator function is the propagation (run on fakes on the
    controller); ``path_or_fn`` names the function that runs on every worker."""
    def wrapper(annotation):
        fn = Remote(path_or_fn, propagate=annotation)
        return lambda *args, **kwargs: create_pipe(fn, *args, max_messages=max_messages, **kwargs)

    return wrapper


__all__ = ["Pipe", "FakePipe", "create_pipe", "remote_generator"]
