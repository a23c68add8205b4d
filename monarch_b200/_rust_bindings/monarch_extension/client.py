"""What a controller's client sees coming back from the workers: results, deterministic
errors, infrastructure failures, log lines (monarch_extension/src/client.rs).

The reference's ``ClientActor`` belongs to its legacy multi-process system (one system actor,
one controller actor per world); this runtime's controller is ``tensor_engine.Client`` over
an actor mesh, so only the value types live here.  They are built from what that client
receives: ``Error.from_remote(RemoteException)``, ``WorkerResponse(seq, result | Error)``.
"""
from __future__ import annotations

import enum
from typing import Any, Dict, Optional


class Exception:  # noqa: A001 - the reference's name for the common base of Error / Failure
    """An exception to commanded execution: :class:`Error` or :class:`Failure`."""


class Error(Exception):
    """A deterministic problem with the user's program on a worker (a failed operator, an
    invariant of the API): invocation ``seq`` failed because invocation ``caused_by_seq``
    did (the same number for the original failure)."""

    def __init__(self, seq: int, caused_by_seq: int, actor_id, backtrace: str):
        self.seq, self.caused_by_seq, self.actor_id, self.backtrace = \
            seq, caused_by_seq, actor_id, backtrace

    @staticmethod
    def new_for_unit_test(seq: int, caused_by_seq: int, actor_id, backtrace: str) -> "Error":
        return Error(seq, caused_by_seq, actor_id, backtrace)

    @staticmethod
    def from_remote(exc) -> "Error":
        """From a ``tensor_engine.RemoteException`` (worker rank in place of an actor id)."""
        cause = exc.dependent_of if exc.dependent_of is not None else exc.seq
        return Error(exc.seq, cause, exc.rank, f"{exc.exc_text}\n{exc.worker_traceback or str()}")

    def __repr__(self) -> str:
        return f"Error(seq={self.seq}, caused_by_seq={self.caused_by_seq}, actor_id={self.actor_id})"


class Failure(Exception):
    """A problem of the worker or its infrastructure rather than of the program (a proc that
    died, a lost device): raised to users as ``SupervisionError``."""

    def __init__(self, actor_id, address: str = "", backtrace: str = ""):
        self.actor_id, self.address, self.backtrace = actor_id, address, backtrace

    @staticmethod
    def new_for_unit_test(actor_id) -> "Failure":
        return Failure(actor_id, "", "")

    def __repr__(self) -> str:
        return f"Failure(actor_id={self.actor_id}, address={self.address!r})"


class WorkerResponse:
    """The outcome of invocation ``seq``: a value or an :class:`Exception`."""

    def __init__(self, seq: int, response: Any):
        self.seq, self._response = seq, response

    @staticmethod
    def new_for_unit_test(*, seq: int, response: Any) -> "WorkerResponse":
        return WorkerResponse(seq, response)

    def is_exception(self) -> bool:
        return isinstance(self._response, Exception)

    def result(self) -> Any:
        return None if self.is_exception() else self._response

    def exception(self) -> Optional[Exception]:
        return self._response if self.is_exception() else None


class LogLevel(enum.Enum):
    INFO = "info"
    WARNING = "warning"
    ERROR = "error"


class LogMessage:
    def __init__(self, level: LogLevel, message: str):
        self.level, self.message = level, message


class DebuggerMessage:
    """A message between the debugger front-end and the actor being debugged."""

    def __init__(self, *, debugger_actor_id, action):
        self.debugger_actor_id, self.action = debugger_actor_id, action


class ProcInfo:
    def __init__(self, labels: Optional[Dict[str, str]] = None):
        self.labels = dict(labels or {})


class WorldState:
    """Labels and procs of one world, as ``ProcMesh.ledger()`` reports them."""

    def __init__(self, labels: Optional[Dict[str, str]] = None,
                 procs: Optional[Dict[str, ProcInfo]] = None):
        self.labels, self.procs = dict(labels or {}), dict(procs or {})


class ClientActor:
    """Not provided: the legacy system's client actor.  Use ``monarch_b200.actor`` proc
    meshes and ``tensor_engine.spawn_tensor_engine``."""

    def __init__(self, *a, **k):
        raise NotImplementedError(
            "ClientActor belongs to the reference's legacy multi-process system; this runtime "
            "drives workers through actor meshes (tensor_engine.spawn_tensor_engine)")
