"""Admin endpoint and CLI over the procs' actor ledgers (the reference's `hyper show / procs /
top`, hyper/src/commands/*.rs)."""
import subprocess
import sys

from monarch_b200.actor import Actor, endpoint, this_host
from monarch_b200.tools import admin


class Echo(Actor):
    @endpoint
    def hi(self, x: int) -> int:
        return x + 1


def test_ledger_and_admin_cli(tmp_path):
    pm = this_host().spawn_procs(per_host={"gpus": 2})
    try:
        actors = pm.spawn("echoes", Echo)
        for i in range(5):
            actors.hi.call(i).get(timeout=30)
        led = pm.ledger()
        assert sorted(led) == [0, 1]
        for rank, rows in led.items():
            mine = [a for a in rows if ".echoes[" in a["actor_id"]]
            assert len(mine) == 1 and mine[0]["messages_handled"] >= 5
            assert any(".mesh_agent[" in a["actor_id"] for a in rows)

        addr = pm.serve_admin("unix:" + str(tmp_path / "admin.sock"))
        snap = admin.snapshot(addr)
        assert snap["world"] == pm.world and len(snap["procs"]) == 2
        text = admin.render_show(snap)
        assert "procs: 2 (0 not responding)" in text
        assert "echoes" in admin.render_show(snap, f"{pm.world}[1]")
        actor_id = next(a["actor_id"] for a in snap["procs"][0]["actors"]
                        if ".echoes[" in a["actor_id"])
        assert "messages handled" in admin.render_show(snap, actor_id)
        assert "up" in admin.render_procs(snap)
        actors.hi.call(7).get(timeout=30)
        top = admin.render_top(admin.snapshot(addr), snap, 1.0)
        assert "MSG/S" in top and "echoes" in top

        out = subprocess.run([sys.executable, "-m", "monarch_b200.tools.admin", "procs", addr],
                             capture_output=True, text=True, timeout=60)
        assert out.returncode == 0 and f"{pm.world}[0]" in out.stdout
        out = subprocess.run([sys.executable, "-m", "monarch_b200.tools.admin", "show", addr,
                              "nosuchworld"], capture_output=True, text=True, timeout=60)
        assert out.returncode == 1 and "unknown world" in out.stderr
    finally:
        pm.stop().get()
