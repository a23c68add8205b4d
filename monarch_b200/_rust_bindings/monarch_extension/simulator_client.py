"""Simulated meshes (monarch_extension/src/simulator_client.rs).
"""
from ...simulator import Simulator as SimulatorClient  # noqa: F401
from ...simulator import mock_mesh  # noqa: F401
