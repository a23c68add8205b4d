"""The actor runtime's bindings (monarch_hyperactor crate of the reference).
"""
from . import (actor, actor_mesh, alloc, bootstrap, channel, mailbox, proc, proc_mesh,  # noqa: F401
               pytokio, runtime, selection, shape, supervision, telemetry)
