"""Debugger protocol actions (monarch_messages/src/debugger.rs).
"""
from dataclasses import dataclass


class DebuggerAction:
    @dataclass(frozen=True)
    class Paused:
        pass

    @dataclass(frozen=True)
    class Attach:
        pass

    @dataclass(frozen=True)
    class Detach:
        pass

    @dataclass(frozen=True)
    class Write:
        bytes: bytes

    @dataclass(frozen=True)
    class Read:
        requested_size: int
