"""Trace ids (monarch_extension/src/trace.rs).
"""
from ..._native import execution_id


def get_or_create_trace_id() -> str:
    return execution_id()
