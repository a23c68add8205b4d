"""Actor API: ``Actor`` classes with ``@endpoint`` methods spawned over proc meshes.

Parity: python/monarch/actor/__init__.py (the exported names).
"""
from .actor_mesh import (Accumulator, Actor, ActorError, ActorMesh, Channel, Endpoint, Port,
                         PortReceiver, SupervisionError, ValueMesh, as_endpoint, context,
                         current_actor_name, current_rank, current_size, endpoint, send)
from .future import Future
from .proc_mesh import (HostMesh, ProcEvent, ProcMesh, fake_in_process_host,
                        get_or_spawn_controller, hosts_from_config, local_proc_mesh, proc_mesh,
                        sim_proc_mesh, this_host, this_proc)
from .shape import Extent, Point, Shape
from .attach import HostedProc, attach_proc_mesh


def debug_controller():
    from .debugger import debug_controller as _dc
    return _dc()


__all__ = [
    "Accumulator", "Actor", "ActorError", "ActorMesh", "as_endpoint", "Channel", "context",
    "current_actor_name", "current_rank", "current_size", "Point", "Port", "PortReceiver", "send",
    "ValueMesh", "debug_controller", "endpoint", "Endpoint", "Extent", "Future", "HostMesh",
    "hosts_from_config", "this_host", "this_proc", "get_or_spawn_controller", "local_proc_mesh",
    "proc_mesh", "ProcMesh", "ProcEvent", "Shape", "sim_proc_mesh", "SupervisionError",
    "fake_in_process_host", "attach_proc_mesh", "HostedProc",
]
