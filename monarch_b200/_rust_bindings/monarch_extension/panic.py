"""A function that fails in native code (test helper of the reference).
"""
def panicking_function() -> None:
    from ..._native import parse_actor_id
    parse_actor_id("this is not an actor id")     # raises from C++
