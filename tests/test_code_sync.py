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


def test_native_manifest_hashes_contents_and_skips_what_it_should(tmp_path):
    import os
    from monarch_b200.actor.code_sync import _hash_file, manifest
    (tmp_path / "pkg").mkdir()
    (tmp_path / "pkg" / "a.py").write_text("x = 1\n")
    (tmp_path / "pkg" / "b.py").write_bytes(b"y" * (3 << 20))          # several read blocks
    (tmp_path / "pkg" / "b.pyc").write_bytes(b"skip me")
    (tmp_path / "empty.txt").write_bytes(b"")
    (tmp_path / "__pycache__").mkdir()
    (tmp_path / "__pycache__" / "c.py").write_text("skipped dir\n")
    (tmp_path / "other").mkdir()
    (tmp_path / "other" / "d.py").write_text("d\n")
    os.symlink(tmp_path / "other", tmp_path / "pkg" / "link")           # not followed
    m1 = manifest(str(tmp_path))
    assert sorted(m1) == ["empty.txt", "other/d.py", "pkg/a.py", "pkg/b.py"]
    assert all(len(h) == 32 for h in m1.values()) and len(set(m1.values())) == 4
    assert m1["pkg/a.py"] == _hash_file(str(tmp_path / "pkg" / "a.py"))
    # same bytes, same hash; one byte changed (same length), another hash
    assert manifest(str(tmp_path)) == m1
    (tmp_path / "pkg" / "a.py").write_text("x = 2\n")
    big = bytearray(b"y" * (3 << 20))
    big[-1] = ord("z")
    (tmp_path / "pkg" / "b.py").write_bytes(bytes(big))
    m2 = manifest(str(tmp_path))
    assert {k for k in m1 if m1[k] != m2[k]} == {"pkg/a.py", "pkg/b.py"}
    # a file and the same file with a zero byte appended differ (the length is mixed in)
    (tmp_path / "z1").write_bytes(b"abc")
    (tmp_path / "z2").write_bytes(b"abc\0")
    m3 = manifest(str(tmp_path))
    assert m3["z1"] != m3["z2"]
    assert manifest(str(tmp_path / "does-not-exist")) == {}
