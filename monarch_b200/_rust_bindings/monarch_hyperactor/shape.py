"""Slices, shapes, extents and points (ndslice; monarch_hyperactor/src/shape.rs).
"""
from ..._native import Slice  # noqa: F401
from ...actor.shape import Extent, Point, Shape  # noqa: F401
