"""Selections over meshes (ndslice/src/selection).
"""
from ..._native import Selection  # noqa: F401
