"""Message definitions shared between components (monarch_messages crate).
"""
from . import debugger  # noqa: F401
