"""One-call constructors of device meshes on this machine, and their simulated twins.

Parity: python/monarch/python_local_mesh.py (``python_local_mesh``), python/monarch/
rust_local_mesh.py (``local_mesh`` / ``local_meshes`` context managers that start the worker
processes and tear them down), python/monarch/sim_mesh.py (``sim_mesh``) and
python/monarch/world_mesh.py.  The reference needs these because its legacy backends start
separate system / controller / worker binaries; here a device mesh is always a proc mesh plus
tensor workers, so the constructors are thin: they exist so that programs written against
those entry points find them.
"""
from __future__ import annotations

import enum

import contextlib
from typing import Iterator, List, Optional


def python_local_mesh(*, gpus: Optional[int] = None, hosts: int = 1, use_cuda: Optional[bool] = None):
    """A ``{hosts, gpus}`` device mesh of worker processes on this machine.  ``mesh.exit()``
    stops the tensor workers and their procs."""
    from .actor import this_host
    from .tensor_engine import spawn_tensor_engine
    if gpus is None:
        try:
            import torch
            gpus = max(torch.cuda.device_count(), 1)
        except Exception:  # noqa: BLE001
            gpus = 1
    if hosts != 1:
        raise NotImplementedError("one machine: hosts must be 1 (use HostMesh.from_allocators "
                                  "for several)")
    pm = this_host().spawn_procs(per_host={"gpus": gpus})
    dm = spawn_tensor_engine(pm, use_cuda=use_cuda)
    inner_exit = dm.exit

    def exit(error: Optional[Exception] = None) -> None:
        try:
            inner_exit(error)
        finally:
            pm.stop().get()

    dm.exit = exit
    return dm


@contextlib.contextmanager
def local_mesh(hosts: int = 1, gpus_per_host: Optional[int] = None,
               use_cuda: Optional[bool] = None) -> Iterator["object"]:
    """``with local_mesh(gpus_per_host=2) as mesh: ...`` -- the mesh is torn down on exit."""
    dm = python_local_mesh(gpus=gpus_per_host, hosts=hosts, use_cuda=use_cuda)
    try:
        yield dm
    finally:
        dm.exit()


@contextlib.contextmanager
def local_meshes(meshes: int = 1, hosts_per_mesh: int = 1, gpus_per_host: Optional[int] = None,
                 use_cuda: Optional[bool] = None) -> Iterator[List["object"]]:
    """Several independent device meshes (e.g. one per pipeline stage)."""
    out = []
    try:
        for _ in range(meshes):
            out.append(python_local_mesh(gpus=gpus_per_host, hosts=hosts_per_mesh,
                                         use_cuda=use_cuda))
        yield out
    finally:
        for dm in out:
            dm.exit()


def sim_mesh(n_meshes: int = 1, hosts: int = 1, gpus_per_host: int = 1, cost=None) -> List["object"]:
    """Simulated device meshes: the same programs run against mock workers that keep shapes
    and a timeline but no data.  Each mesh carries its simulator as ``mesh.simulator``."""
    from .simulator import mock_mesh
    out = []
    for _ in range(n_meshes):
        dm, sim = mock_mesh(hosts=hosts, gpus=gpus_per_host, cost=cost)
        dm.simulator = sim
        out.append(dm)
    return out


def world_mesh(proc_mesh, use_cuda: Optional[bool] = None):
    """The device mesh over every proc of an existing proc mesh."""
    from .tensor_engine import spawn_tensor_engine
    return spawn_tensor_engine(proc_mesh, use_cuda=use_cuda)


__all__ = ["python_local_mesh", "local_mesh", "local_meshes", "sim_mesh", "world_mesh"]


class SocketType(enum.Enum):
    """Transport of a locally spawned mesh (python/monarch/rust_local_mesh.py ``SocketType``);
    both map onto this runtime's channel addresses."""
    TCP = "tcp"
    UNIX = "unix"
