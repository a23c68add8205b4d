"""Workspace sync + auto-reload: edit a module on the client, sync, and the procs run the
new code without restarting (modelled on the reference's code_sync/test_auto_reload.py)."""
import os
import sys
import textwrap

from monarch_b200.actor import Actor, endpoint, this_host


class Caller(Actor):
    @endpoint
    def value(self) -> int:
        import ws_mod
        return ws_mod.value()

    @endpoint
    def pid(self) -> int:
        return os.getpid()


def test_sync_and_auto_reload(tmp_path, monkeypatch):
    src = tmp_path / "client_ws"
    dst = tmp_path / "proc_ws"
    src.mkdir()
    (src / "ws_mod.py").write_text("def value():\n    return 1\n")
    (src / "data.txt").write_text("a")
    pm = this_host().spawn_procs(per_host={"gpus": 2}, env={"WORKSPACE_DIR": str(dst)})
    try:
        r = pm.sync_workspace(str(src), auto_reload=True).get(timeout=60)
        assert sorted(r) == [0, 1]
        assert (dst / "ws_mod.py").exists() and (dst / "data.txt").read_text() == "a"
        c = pm.spawn("caller", Caller)
        assert [v for _, v in c.value.call().get(timeout=30).items()] == [1, 1]
        pids = [v for _, v in c.pid.call().get(timeout=30).items()]
        (src / "ws_mod.py").write_text("def value():\n    return 2\n")
        (src / "data.txt").unlink()
        r = pm.sync_workspace(str(src), auto_reload=True).get(timeout=60)
        assert all("ws_mod" in mods for mods in r.values()), r
        assert not (dst / "data.txt").exists()
        assert [v for _, v in c.value.call().get(timeout=30).items()] == [2, 2]
        assert [v for _, v in c.pid.call().get(timeout=30).items()] == pids  # same procs
    finally:
        pm.stop().get()


def test_auto_reloader_local(tmp_path):
    from monarch_b200.actor.code_sync import AutoReloader, manifest
    (tmp_path / "lm_mod.py").write_text("X = 1\n")
    sys.path.insert(0, str(tmp_path))
    try:
        import lm_mod
        ar = AutoReloader(str(tmp_path))
        assert ar.reload_changed() == []
        (tmp_path / "lm_mod.py").write_text("X = 5\n")
        assert ar.reload_changed() == ["lm_mod"] and lm_mod.X == 5
        assert set(manifest(str(tmp_path))) == {"lm_mod.py"}
    finally:
        sys.path.remove(str(tmp_path))
        sys.modules.pop("lm_mod", None)
