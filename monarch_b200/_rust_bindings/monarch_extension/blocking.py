"""A function that blocks in native code with the GIL released (test helper of the reference).
"""
def blocking_function() -> None:
    from ..._native import Completion
    Completion().wait(100)
