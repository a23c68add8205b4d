"""The native controller history (csrc/tensor/controller_history.{h,cpp}) on its own:
failure propagation in issue order, retirement by the slowest rank, the watchdog's ping
bookkeeping, and concurrent use from several threads.
Modelled on controller/src/history.rs tests of the reference (dependent failures, retirement
once every rank has passed an invocation)."""
import threading

from monarch_b200 import _native as N


def test_failures_reach_dependents_issued_before_and_after_the_report():
    h = N.ControllerHistory(2)
    seqs = [h.next_seq() for _ in range(6)]
    assert seqs == [1, 2, 3, 4, 5, 6]
    h.add_invocation(1, "a", [10], [])          # 10 = a()
    h.add_invocation(2, "b", [11], [10])        # 11 = b(10)
    h.add_invocation(3, "c", [12], [99])        # unrelated
    h.add_invocation(4, "d", [13, 14], [11, 12])  # 13, 14 = d(11, 12)
    assert h.fail(1, 0, "a", "ValueError: x") == [2, 4]
    assert [h.ref_failed(r) for r in (10, 11, 12, 13, 14)] == [1, 1, -1, 1, 1]
    assert h.describe(4) == ("d", 1) and h.describe(3) == ("c", -1)
    assert h.failure(1) == (1, 0, "a", "ValueError: x") and h.failure(2) is None
    # issued after the report: inherits at once, from either input
    assert h.add_invocation(5, "e", [15], [12, 14]) == 1 and h.ref_failed(15) == 1
    assert h.add_invocation(6, "f", [16], [12]) == -1
    # a second report for the same invocation (another rank) changes nothing
    assert h.fail(1, 1, "a", "ValueError: x") == []
    assert h.failure(1)[1] == 0
    # forgetting refs (the controller dropped the tensors) clears their poison only
    h.forget_refs([11, 13])
    assert [h.ref_failed(r) for r in (10, 11, 13, 14)] == [1, -1, -1, 1]


def test_invocations_retire_once_every_rank_has_passed_them():
    h = N.ControllerHistory(3)
    for s in range(1, 11):
        h.add_invocation(s, "op", [100 + s], [])
    assert h.live_invocations() == 10 and h.min_completed() == -1
    h.rank_progress(0, 10)
    h.rank_progress(1, 7)
    assert h.live_invocations() == 10            # rank 2 has reported nothing yet
    h.rank_progress(2, 4)
    assert h.min_completed() == 4 and h.live_invocations() == 6
    h.rank_progress(2, 3)                         # progress never moves backwards
    assert h.min_completed() == 4
    assert h.describe(4) is None and h.describe(5) == ("op", -1)
    # a failure report for a retired invocation has nothing live to poison
    assert h.fail(2, 0, "op", "late") == [] and h.ref_failed(102) == -1
    h.rank_progress(1, 10)
    h.rank_progress(2, 10)
    assert h.live_invocations() == 0


def test_ping_bookkeeping_reports_a_stall_once():
    h = N.ControllerHistory(3)
    assert not h.ping_outstanding() and h.stalled(100.0, 1.0) is None
    h.ping_sent(42, 10.0)
    assert h.ping_outstanding()
    assert not h.ping_answered(0, 40)
    assert h.stalled(10.5, 1.0) is None           # within the timeout
    st = h.stalled(12.0, 1.0)
    assert st["ranks"] == [1, 2] and st["controller_seq"] == 42
    assert st["last_seq_of_responders"] == {0: 40} and abs(st["waited_s"] - 2.0) < 1e-9
    assert h.stalled(13.0, 1.0) is None           # reported once per ping
    assert not h.ping_answered(2, 41)
    assert h.ping_answered(1, 41) and not h.ping_outstanding()
    assert h.min_completed() == 40                # answers carry progress too
    h.ping_sent(43, 20.0)                         # a new ping can stall again
    assert h.stalled(30.0, 1.0)["ranks"] == [0, 1, 2]


def test_concurrent_use_from_several_threads():
    h = N.ControllerHistory(4)
    n, errors = 2000, []

    def issue(base):
        try:
            for i in range(n):
                s = h.next_seq()
                h.add_invocation(s, f"op{base}", [h.next_ref()], [base])
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    def progress(rank):
        try:
            for i in range(0, 4 * n, 7):
                h.rank_progress(rank, i)
                h.min_completed()
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    def failures():
        try:
            for i in range(1, 4 * n, 97):
                h.fail(i, 0, "op", "boom")
                h.ref_failed(i)
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    ts = [threading.Thread(target=issue, args=(b,)) for b in range(4)] + \
         [threading.Thread(target=progress, args=(r,)) for r in range(4)] + \
         [threading.Thread(target=failures)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert not errors
    assert h.next_seq() == 4 * n + 1               # every sequence number handed out once
    for r in range(4):
        h.rank_progress(r, 4 * n)
    assert h.live_invocations() == 0
