"""Distributed pdb: endpoints park at a breakpoint, the client lists the sessions, inspects
variables on each rank, and resumes them (scripted sessions, as in the reference's
test_debugger.py)."""
import io
import time

from monarch_b200.actor import Actor, debug_controller, endpoint, this_host


class Buggy(Actor):
    @endpoint
    def work(self, base: int) -> int:
        from monarch_b200.actor import current_rank
        from monarch_b200.actor.debugger import remote_breakpoint
        x = base + current_rank().rank
        remote_breakpoint()
        return x * 2


def _wait(pred, timeout=30):
    t0 = time.time()
    while time.time() - t0 < timeout:
        v = pred()
        if v:
            return v
        time.sleep(0.1)
    raise AssertionError("timed out")


def test_breakpoint_sessions_can_be_inspected_and_resumed():
    pm = this_host().spawn_procs(per_host={"gpus": 2})
    try:
        ctrl = debug_controller()
        a = pm.spawn("buggy", Buggy)
        fut = a.work.call(10)
        sessions = _wait(lambda: [s for s in ctrl.list.call_one().get()
                                  if s["actor"] == "buggy" and s["active"]]
                         if len(ctrl.list.call_one().get()) >= 2 else None)
        assert sorted(s["rank"] for s in sessions) == [0, 1]
        assert all("work" in s["where"] for s in sessions)
        # inspect a local on each rank
        for r in (0, 1):
            assert ctrl.send.call_one("buggy", r, "p x").get()
            out = _wait(lambda: (lambda t: t if str(10 + r) in t else None)(
                ctrl.read.call_one("buggy", r, False).get()))
            assert str(10 + r) in out
        # change state on rank 1 only, then resume everyone with one cast
        ctrl.send.call_one("buggy", 1, "x = 100").get()
        assert ctrl.cast.call_one("buggy", None, "c").get() == 2
        res = fut.get(timeout=30)
        assert [v for _, v in res.items()] == [20, 200]
        assert not any(s["active"] for s in ctrl.list.call_one().get() if s["actor"] == "buggy")
    finally:
        pm.stop().get()


def test_console_lists_sessions():
    from monarch_b200.debug_cli.__main__ import run_console
    ctrl = debug_controller()
    out = io.StringIO()
    run_console(ctrl, io.StringIO("list\nhelp\nquit\n"), out)
    assert "commands:" in out.getvalue()
