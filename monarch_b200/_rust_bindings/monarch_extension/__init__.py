"""Bindings outside the actor runtime (monarch_extension crate of the reference).
"""
from . import (blocking, code_sync, debugger, logging, mesh_controller, panic,  # noqa: F401
               simulation_tools, simulator_client, tensor_worker, trace)
