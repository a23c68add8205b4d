"""Allocator objects: where the procs of a mesh come from.

Parity: python/monarch/_src/actor/allocator.py (``AllocSpec``, ``AllocConstraints``,
``LocalAllocator``, ``ProcessAllocator``, ``SimAllocator``, ``RemoteAllocator`` with
``StaticRemoteAllocInitializer``) and ``ProcMesh.from_alloc``.  An allocator turns an
``AllocSpec`` (named extents, e.g. ``hosts=1, gpus=8``) into an ``Alloc``; a proc mesh is
built from the alloc.  The native side (``LocalAlloc`` / ``ProcessAlloc`` in C++) does the
work; these classes carry the parameters to it.
"""
from __future__ import annotations

import sys
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence


@dataclass
class AllocConstraints:
    """Placement hints handed to the allocator (``match_labels`` as in the reference)."""
    match_labels: Dict[str, str] = field(default_factory=dict)


class AllocSpec:
    def __init__(self, constraints: Optional[AllocConstraints] = None, **extent: int):
        if not extent:
            raise ValueError("an AllocSpec needs at least one named dimension")
        for k, v in extent.items():
            if int(v) <= 0:
                raise ValueError(f"dimension {k} must be positive, got {v}")
        self.constraints = constraints or AllocConstraints()
        self.extent: Dict[str, int] = {k: int(v) for k, v in extent.items()}

    def __repr__(self) -> str:
        return f"AllocSpec({', '.join(f'{k}={v}' for k, v in self.extent.items())})"


class Alloc:
    """What an allocator hands out: everything needed to build the proc mesh."""

    def __init__(self, spec: AllocSpec, kind: str, **params):
        self.spec = spec
        self.kind = kind
        self.params = params
        self._used = False

    @property
    def extent(self) -> Dict[str, int]:
        return dict(self.spec.extent)

    def __repr__(self) -> str:
        return f"Alloc({self.kind}, {self.spec.extent})"


class _AllocatorBase:
    kind = ""

    def allocate(self, spec: AllocSpec) -> Alloc:
        return Alloc(spec, self.kind, **self._params())

    def _params(self) -> dict:
        return {}


class LocalAllocator(_AllocatorBase):
    """Procs inside the calling process (threads of the client): tests and notebooks."""
    kind = "local"


class SimAllocator(LocalAllocator):
    """In-process procs standing in for a large mesh (cast-tree and API tests at sizes no
    box has); the same mechanism as :class:`LocalAllocator`."""
    kind = "sim"


class ProcessAllocator(_AllocatorBase):
    """One OS process per proc, started with ``cmd args...`` (default: this interpreter
    running the bootstrap entry point) and the extra environment ``env``."""
    kind = "process"

    def __init__(self, cmd: Optional[str] = None, args: Optional[Sequence[str]] = None,
                 env: Optional[Dict[str, str]] = None,
                 bootstrap: Optional[Callable[[], None]] = None):
        self.cmd, self.args, self.env, self.bootstrap = cmd, list(args or []), env, bootstrap

    def _params(self) -> dict:
        argv = None
        if self.cmd is not None:
            argv = [self.cmd] + self.args
        return {"argv": argv, "env": self.env, "bootstrap": self.bootstrap}


class StaticRemoteAllocInitializer:
    """A fixed list of allocator-daemon addresses (``host:port``)."""

    def __init__(self, *addrs: str):
        self.addrs = [a.replace("tcp!", "") for a in addrs]

    def initialize_alloc(self, match_labels: Optional[Dict[str, str]] = None) -> List[str]:
        return list(self.addrs)


class RemoteAllocator(_AllocatorBase):
    """Procs on other hosts, started by the allocator daemon of each host
    (``python -m monarch_b200.tools.process_allocator``)."""
    kind = "remote"

    def __init__(self, world_id: str = "", initializer=None, heartbeat_interval: float = 5.0):
        if initializer is None:
            raise ValueError("a RemoteAllocator needs an initializer that names the hosts")
        self.world_id, self.initializer = world_id, initializer

    def allocate(self, spec: AllocSpec) -> Alloc:
        hosts = self.initializer.initialize_alloc(spec.constraints.match_labels)
        dims = list(spec.extent.items())
        if dims[0][1] != len(hosts):
            raise ValueError(f"the first dimension ({dims[0][0]}={dims[0][1]}) must equal the "
                             f"number of hosts ({len(hosts)})")
        per_host = 1
        for _, n in dims[1:]:
            per_host *= n
        return Alloc(spec, self.kind, hosts=hosts, procs_per_host=per_host)


def _both(first, second):
    if first is None or second is None:
        return first or second

    def run():
        first()
        second()
    return run


def proc_mesh_from_alloc(alloc: Alloc, setup=None):
    """Build the proc mesh an alloc describes (an alloc can be used once).  ``setup`` runs in
    every proc before actors are spawned (after the alloc's own bootstrap function)."""
    from .proc_mesh import _allocate
    if alloc._used:
        raise RuntimeError("this alloc was already turned into a proc mesh")
    alloc._used = True
    dims = alloc.extent
    p = alloc.params
    if alloc.kind in ("local", "sim"):
        if setup is not None:
            setup()           # the procs of these allocs are threads of this process
        return _allocate(dims, in_process=True)
    if alloc.kind == "process":
        boot = _both(p.get("bootstrap"), setup)
        if p.get("argv") is not None:
            return _allocate(dims, in_process=False, env=p.get("env"),
                             bootstrap=boot, argv=p["argv"])
        return _allocate(dims, in_process=False, env=p.get("env"), bootstrap=boot)
    if alloc.kind == "remote":
        if setup is not None:
            raise NotImplementedError("setup= is not carried to remotely allocated procs; set "
                                      "the environment in the allocator's command instead")
        return _allocate(dims, in_process=False, remote_hosts=p["hosts"],
                         procs_per_host=p["procs_per_host"])
    raise ValueError(f"unknown alloc kind {alloc.kind!r}")


__all__ = ["Alloc", "AllocConstraints", "AllocSpec", "LocalAllocator", "ProcessAllocator",
           "RemoteAllocator", "SimAllocator", "StaticRemoteAllocInitializer",
           "proc_mesh_from_alloc"]
