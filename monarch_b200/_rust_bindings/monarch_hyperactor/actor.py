"""Message envelope of Python actors (monarch_hyperactor/src/actor.rs:200-241).  The wire
format here is a pickled tuple ``("call", method, args, kwargs, port)`` carried as frame
parts; these classes describe it with the reference's vocabulary.
"""
from dataclasses import dataclass, field
from typing import Any, Optional

from ...actor.actor_mesh import Actor, Port  # noqa: F401


class MethodSpecifier:
    """How an endpoint call answers: through a response port created by the caller
    (``ReturnsResponse``), an explicit port argument (``ExplicitPort``), or not at all
    (``Init``: the constructor call)."""

    @dataclass(frozen=True)
    class ReturnsResponse:
        name: str

    @dataclass(frozen=True)
    class ExplicitPort:
        name: str

    @dataclass(frozen=True)
    class Init:
        pass


class PythonMessageKind:
    @dataclass(frozen=True)
    class CallMethod:
        name: Any                      # a MethodSpecifier
        response_port: Optional[Any] = None

    @dataclass(frozen=True)
    class CallMethodIndirect:
        name: Any
        broker_id: Any = None
        id: int = 0
        unflatten_args: tuple = ()

    @dataclass(frozen=True)
    class Result:
        rank: Optional[int] = None

    @dataclass(frozen=True)
    class Exception:
        rank: Optional[int] = None

    @dataclass(frozen=True)
    class Uninit:
        pass


@dataclass
class PythonMessage:
    kind: Any
    message: bytes = b""
    parts: list = field(default_factory=list)


class PanicFlag:
    """Side channel through which a failing endpoint takes its actor down
    (monarch_hyperactor/src/actor.rs:440-455): here a BaseException raised by the endpoint."""

    def __init__(self):
        self.exception = None

    def signal_panic(self, ex: BaseException) -> None:
        self.exception = ex
