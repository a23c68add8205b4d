"""Proc meshes over processes that something else launched (an SPMD launcher such as
``torchrun``, a batch scheduler): instead of starting its procs, the controller waits for
them to join.

Every process of the launch calls :func:`attach_proc_mesh`.  Rank 0 becomes the
controller: it opens an attach allocation, publishes its address, hosts proc 0 on a
background thread of its own process and gets the :class:`ProcMesh` back.  Every other rank
hosts its proc and gets a :class:`HostedProc`, whose ``join()`` returns when the
controller stops the mesh::

    mesh, hosted = attach_proc_mesh({"gpus": world})
    if mesh is None:
        hosted.join()            # this process now only runs actors
    else:
        trainers = mesh.spawn("trainer", TrainerActor, ...)
        trainers.step.call(0).get()
        mesh.stop().get()

Actors spawned on such a mesh run inside the launcher's processes, so they see the
process group, CUDA context and environment (``RANK``, ``LOCAL_RANK``) that the launcher
set up.  The address travels over ``torch.distributed`` when a process group exists,
otherwise over a ``TCPStore`` at ``MASTER_ADDR``:``MASTER_PORT`` + 1.

Parity: the reference reaches externally started hosts through allocator daemons
(python/monarch/_src/actor/allocator.py RemoteAllocator; hyperactor_mesh
alloc/remoteprocess.rs); attaching to an SPMD launch inside one box is this package's form
of it, used by ``bench.py`` so that the timed training step is driven over the mesh.
"""
from __future__ import annotations

import itertools
import os
import threading
from typing import Dict, Optional, Tuple

from .. import _native as N
from .proc_mesh import ProcMesh, _shape_from_dims

_counter = itertools.count()
_stores: list = []     # rendezvous stores stay up for the life of the process: late ranks read them


class HostedProc:
    """The proc this process hosts for an attached mesh (a thread serving its actors)."""

    def __init__(self, addr: str, index: int):
        self.addr, self.index = addr, index
        self.exit_code: Optional[int] = None
        self._thread = threading.Thread(target=self._run, daemon=True,
                                        name=f"monarch-attached-proc-{index}")
        self._thread.start()

    def _run(self) -> None:
        import monarch_b200.actor  # noqa: F401  (registers the python actor type)
        self.exit_code = N.bootstrap_attach(self.addr, self.index)

    def join(self, timeout: Optional[float] = None) -> Optional[int]:
        """Wait until the controller stops the mesh (or vanishes); the proc's exit code."""
        self._thread.join(timeout)
        return self.exit_code


def _exchange_addr(addr: Optional[str], rank: int, world: int, tag: str) -> str:
    """Rank 0's ``addr`` on every rank."""
    if world == 1:
        return addr
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        box = [addr]
        dist.broadcast_object_list(box, src=0)
        return box[0]
    from datetime import timedelta
    store = dist.TCPStore(os.environ.get("MASTER_ADDR", "127.0.0.1"),
                          int(os.environ.get("MASTER_PORT", "29500")) + 1, world,
                          is_master=(rank == 0), timeout=timedelta(seconds=120))
    _stores.append(store)
    if rank == 0:
        store.set(tag, addr)
        return addr
    return store.get(tag).decode()


def attach_proc_mesh(dims: Optional[Dict[str, int]] = None, *, rank: Optional[int] = None,
                     world: Optional[int] = None, transport: str = "unix",
                     timeout: float = 120.0) -> Tuple[Optional[ProcMesh], HostedProc]:
    """Join (rank > 0) or create and join (rank 0) a proc mesh made of the processes of this
    launch.  ``dims``: the mesh's dimensions (default ``{"gpus": world}``); their product
    must equal ``world``.  ``rank`` / ``world`` default to ``RANK`` / ``WORLD_SIZE``."""
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    world = int(os.environ.get("WORLD_SIZE", "1")) if world is None else world
    dims = dict(dims) if dims else {"gpus": world}
    n = 1
    for v in dims.values():
        n *= int(v)
    if n != world:
        raise ValueError(f"mesh dims {dims} describe {n} procs, the launch has {world}")
    alloc = None
    addr = None
    tag = f"mb200_attach_{next(_counter)}"
    if rank == 0:
        alloc = N.AttachAlloc(f"attached{next(_counter)}_{os.getpid()}", world, transport)
        addr = alloc.bootstrap_addr
    addr = _exchange_addr(addr, rank, world, tag)
    hosted = HostedProc(addr, rank)
    if rank != 0:
        return None, hosted
    native = N.ProcMesh.allocate_attached(alloc, int(timeout * 1000))
    return ProcMesh(native, _shape_from_dims(dims), in_process=False), hosted
