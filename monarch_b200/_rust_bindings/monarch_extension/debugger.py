"""Remote pdb sessions (monarch_extension/src/debugger.rs).
"""
from ...actor.debugger import DebugController, PdbWrapper, remote_breakpoint  # noqa: F401

PdbActor = DebugController
