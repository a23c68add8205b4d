"""Controller of the tensor engine (monarch_extension/src/mesh_controller.rs:384-861).
"""
from ...tensor_engine.device_mesh import Client as _Controller  # noqa: F401
