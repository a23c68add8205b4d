"""Python face of the native telemetry: spans, metric instruments, log forwarding and a
sqlite sink for tests and post-mortems.

Parity: python/monarch/_src/actor/telemetry/__init__.py (``TracingForwarder``, ``Counter``,
``Histogram``, ``UpDownCounter``), monarch_hyperactor/src/telemetry.rs (``PySpan``,
``get_current_span_id``, ``forward_to_tracing``, ``use_sim_clock`` / ``use_real_clock``,
``get_execution_id``, ``PySqliteTracing``) and hyperactor_telemetry/src/sqlite.rs (log events
and span lifecycles as SQL rows).  The instruments write into the C++ registry that the
runtime's own counters use; captured events are drained from the native collector into a
``sqlite3`` database:

    with SqliteTracing(in_memory=True) as t:
        with span("load", actor_id="trainer[0]"):
            logging.getLogger("x").warning("slow batch")
        rows = t.query("select message from log_events where level >= 3")
"""
from __future__ import annotations

import contextlib
import logging
import sqlite3
import tempfile
import threading
from typing import Any, Iterator, List, Optional

from . import _native as N

_LEVELS = {logging.DEBUG: 1, logging.INFO: 2, logging.WARNING: 3, logging.ERROR: 4,
           logging.CRITICAL: 4}


def forward_to_tracing(record: logging.LogRecord) -> None:
    """Hand a Python log record to the native log (file/stderr sinks and event capture),
    keeping its source location and level."""
    level = _LEVELS.get(record.levelno, 2 if record.levelno < logging.WARNING else 4)
    N.log_event(level, record.filename, int(record.lineno), record.getMessage())


class TracingForwarder(logging.Handler):
    """``logging`` handler that forwards to :func:`forward_to_tracing`."""

    def emit(self, record: logging.LogRecord) -> None:
        try:
            forward_to_tracing(record)
        except Exception:  # noqa: BLE001 - logging must not raise
            self.handleError(record)


def get_current_span_id() -> int:
    """Id of the innermost open span on this thread; 0 when none is open."""
    return int(N.current_span_id())


def get_execution_id() -> str:
    return N.execution_id()


def use_sim_clock() -> None:
    N.use_sim_clock()


def use_real_clock() -> None:
    N.use_real_clock()


def advance_sim_clock(seconds: float) -> None:
    N.sim_clock_advance_us(seconds * 1e6)


class Span:
    """An open span; ``exit()`` closes it (and anything still open inside it)."""

    def __init__(self, name: str, actor_id: Optional[str] = None):
        self.name = name
        self.id = int(N.span_enter(name, actor_id or ""))
        self._open = True

    def exit(self) -> None:
        if self._open:
            self._open = False
            N.span_exit(self.id)

    def __enter__(self) -> "Span":
        return self

    def __exit__(self, *exc) -> None:
        self.exit()


@contextlib.contextmanager
def span(name: str, actor_id: Optional[str] = None) -> Iterator[Span]:
    s = Span(name, actor_id)
    try:
        yield s
    finally:
        s.exit()


class Counter:
    def __init__(self, name: str):
        self.name = name

    def add(self, value: int = 1) -> None:
        if value < 0:
            raise ValueError("a counter only goes up; use UpDownCounter")
        N.metrics_counter_add(self.name, int(value))

    def value(self) -> int:
        return int(N.metrics_counter(self.name))


class UpDownCounter(Counter):
    def add(self, value: int = 1) -> None:
        N.metrics_counter_add(self.name, int(value))


class Histogram:
    def __init__(self, name: str):
        self.name = name

    def record(self, value: float) -> None:
        N.metrics_histogram_record(self.name, float(value))

    def snapshot(self) -> Any:
        return N.metrics_histogram(self.name)


class Meter:
    """Factory in the shape of an OpenTelemetry meter (``METER.create_counter(...)``)."""

    def __init__(self, name: str = "monarch"):
        self.name = name

    def create_counter(self, name: str, **_kw) -> Counter:
        return Counter(name)

    def create_up_down_counter(self, name: str, **_kw) -> UpDownCounter:
        return UpDownCounter(name)

    def create_histogram(self, name: str, **_kw) -> Histogram:
        return Histogram(name)


def get_monarch_meter() -> Meter:
    return Meter("monarch")


class SqliteTracing:
    """Capture native and forwarded log events and span lifecycles into a sqlite database.

    Tables: ``log_events(time_us, level, file, line, message, span_id, thread)`` and
    ``spans(id, name, actor_id, parent_id, thread, start_us, end_us)``.  ``in_memory`` keeps
    the database in this process; otherwise a temporary file is used and ``db_path`` names
    it.  Rows appear at ``flush()`` (called by ``query`` and at exit)."""

    _active_lock = threading.Lock()
    _active: Optional["SqliteTracing"] = None

    def __init__(self, in_memory: bool = False, path: Optional[str] = None):
        if in_memory:
            self._path = None
            self.db = sqlite3.connect(":memory:", check_same_thread=False)
        else:
            self._path = path or tempfile.NamedTemporaryFile(prefix="monarch_trace_",
                                                             suffix=".db", delete=False).name
            self.db = sqlite3.connect(self._path, check_same_thread=False)
        self.db.executescript(
            "create table if not exists log_events(time_us real, level integer, file text, "
            "line integer, message text, span_id integer, thread integer);"
            "create table if not exists spans(id integer primary key, name text, actor_id text, "
            "parent_id integer, thread integer, start_us real, end_us real);")
        self._closed = False
        self._lock = threading.Lock()

    def db_path(self) -> Optional[str]:
        return self._path

    def __enter__(self) -> "SqliteTracing":
        with SqliteTracing._active_lock:
            if SqliteTracing._active is not None:
                raise RuntimeError("another SqliteTracing capture is active in this process")
            SqliteTracing._active = self
        N.events_drain()          # start from a clean collector
        N.events_enable(True)
        return self

    def flush(self) -> int:
        rows = N.events_drain()
        with self._lock:
            for kind, t, level, file, line, msg, actor, sid, parent, thread in rows:
                if kind == "event":
                    self.db.execute("insert into log_events values (?,?,?,?,?,?,?)",
                                    (t, level, file, line, msg, sid, thread))
                elif kind == "span_enter":
                    self.db.execute("insert or replace into spans values (?,?,?,?,?,?,null)",
                                    (sid, msg, actor, parent, thread, t))
                else:
                    self.db.execute("update spans set end_us = ? where id = ?", (t, sid))
            self.db.commit()
        return len(rows)

    def query(self, sql: str, params: tuple = ()) -> List[tuple]:
        self.flush()
        with self._lock:
            return list(self.db.execute(sql, params))

    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        with SqliteTracing._active_lock:
            if SqliteTracing._active is self:
                self.flush()
                N.events_enable(False)
                SqliteTracing._active = None
        if self._path is not None:
            self.db.close()       # an in-memory database stays readable after the capture

    def __exit__(self, *exc) -> None:
        self.close()


__all__ = ["Counter", "Histogram", "Meter", "Span", "SqliteTracing", "TracingForwarder",
           "UpDownCounter", "advance_sim_clock", "forward_to_tracing", "get_current_span_id",
           "get_execution_id", "get_monarch_meter", "span", "use_real_clock", "use_sim_clock"]
