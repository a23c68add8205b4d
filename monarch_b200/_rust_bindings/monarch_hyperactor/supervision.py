"""Supervision errors (monarch_hyperactor/src/supervision.rs).
"""
from ...actor.actor_mesh import SupervisionError  # noqa: F401
