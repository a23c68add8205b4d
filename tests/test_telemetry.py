"""Spans, instruments, log forwarding and the sqlite sink (the reference tests its telemetry
through the sqlite layer: python/tests/test_sqlite_tracing.py style queries)."""
import json
import logging
import sqlite3

import pytest

from monarch_b200 import _native as N
from monarch_b200 import telemetry as T
from monarch_b200.actor import Actor, endpoint, local_proc_mesh


def test_spans_nest_and_ids_are_visible():
    assert T.get_current_span_id() == 0
    with T.span("outer", actor_id="a[0]") as o:
        assert T.get_current_span_id() == o.id
        with T.span("inner") as i:
            assert T.get_current_span_id() == i.id != o.id
        assert T.get_current_span_id() == o.id
    assert T.get_current_span_id() == 0
    assert T.get_execution_id() == T.get_execution_id() != ""


def test_sqlite_capture_of_events_and_spans():
    log = logging.getLogger("telemetry_test")
    log.setLevel(logging.DEBUG)
    h = T.TracingForwarder()
    log.addHandler(h)
    try:
        with T.SqliteTracing(in_memory=True) as t:
            with T.span("step", actor_id="trainer[3]") as s:
                log.warning("slow batch %d", 7)
                with T.span("io"):
                    log.info("read shard")
            log.error("outside")
            rows = t.query("select level, message, span_id from log_events order by time_us")
            assert [(r[0], r[1]) for r in rows] == [(3, "slow batch 7"), (2, "read shard"),
                                                   (4, "outside")]
            assert rows[0][2] == s.id and rows[2][2] == 0
            spans = t.query("select name, actor_id, parent_id, end_us >= start_us from spans "
                            "order by id")
            assert spans == [("step", "trainer[3]", 0, 1), ("io", "", s.id, 1)]
            file_row = t.query("select file, line from log_events limit 1")[0]
            assert file_row[0] == "test_telemetry.py" and file_row[1] > 0
            with pytest.raises(RuntimeError):
                T.SqliteTracing(in_memory=True).__enter__()
        # nothing is captured once the sink is closed
        log.warning("after")
        assert N.events_drain() == []
    finally:
        log.removeHandler(h)


def test_sqlite_file_and_runtime_events(tmp_path):
    path = str(tmp_path / "trace.db")

    class A(Actor):
        @endpoint
        def hi(self) -> int:
            with T.span("hi-span"):
                return 1

    with T.SqliteTracing(path=path) as t:
        assert t.db_path() == path
        pm = local_proc_mesh(gpus=2)
        a = pm.spawn("a", A)
        assert a.hi.call().get().values() == [1, 1]
        pm.stop().get()
    db = sqlite3.connect(path)
    assert db.execute("select count(*) from spans where name = 'hi-span'").fetchone()[0] == 2


def test_sim_clock_and_instruments():
    T.use_sim_clock()
    try:
        t0 = N.telemetry_now_us()
        T.advance_sim_clock(2.5)
        assert N.telemetry_now_us() - t0 == pytest.approx(2.5e6)
    finally:
        T.use_real_clock()
    assert N.telemetry_now_us() > 1e15          # wall clock, microseconds since the epoch
    c = T.get_monarch_meter().create_counter("test_py_messages")
    before = c.value()
    c.add(3)
    assert c.value() == before + 3
    with pytest.raises(ValueError):
        c.add(-1)
    u = T.UpDownCounter("test_inflight")
    u.add(2)
    u.add(-2)
    assert u.value() == 0
    hgm = T.Histogram("test_latency_us")
    for v in (1.0, 2.0, 3.0):
        hgm.record(v)
    assert "test_latency_us.count" in json.dumps(N.metrics_snapshot()) or hgm.snapshot()


def test_spans_reach_the_chrome_trace():
    N.trace_clear()
    N.trace_enable(True)
    try:
        with T.span("traced"):
            pass
    finally:
        N.trace_enable(False)
    ev = json.loads(N.trace_json())
    ev = ev["traceEvents"] if isinstance(ev, dict) else ev
    assert any(e.get("name") == "traced" and e.get("ph") == "X" for e in ev)


def test_endpoint_calls_run_in_spans_and_children_share_the_execution_id():
    import os
    from monarch_b200.actor import this_host

    class B(Actor):
        @endpoint
        def exec_id(self) -> str:
            return T.get_execution_id()

        @endpoint
        def work(self) -> int:
            return T.get_current_span_id()

    with T.SqliteTracing(in_memory=True) as t:
        pm = local_proc_mesh(gpus=2)
        b = pm.spawn("b", B)
        ids = b.work.call().get().values()
        assert all(i != 0 for i in ids)          # the handler ran inside its endpoint span
        pm.stop().get()
        rows = t.query("select name, actor_id from spans where name = 'B.work'")
        assert len(rows) == 2 and all(".b[" in r[1] for r in rows)
    # outside a capture no span is opened
    pm = local_proc_mesh(gpus=1)
    b = pm.spawn("b", B)
    assert b.work.call().get().values() == [0]
    pm.stop().get()
    # subprocess children inherit the client's execution id
    pm = this_host().spawn_procs(per_host={"gpus": 1})
    try:
        assert pm.spawn("b", B).exec_id.call().get(timeout=60).values() == [T.get_execution_id()]
    finally:
        pm.stop().get()
