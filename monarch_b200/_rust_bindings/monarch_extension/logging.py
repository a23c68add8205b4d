"""Log forwarding of a proc mesh (monarch_extension/src/logging.rs).
"""
from ...actor.proc_mesh import LogAggregator  # noqa: F401

LoggingMeshClient = LogAggregator
