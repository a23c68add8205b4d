"""Environment sync (the reference's monarch_conda: diff + sender/receiver protocol with
prefix rewriting)."""
import os
import stat

import pytest

from monarch_b200.actor import this_host
from monarch_b200.actor import env_sync as E


def _make_env(root, prefix_in_files=None):
    p = prefix_in_files or str(root)
    (root / "bin").mkdir(parents=True)
    (root / "lib" / "pkg").mkdir(parents=True)
    (root / "conda-meta").mkdir()
    (root / "conda-meta" / "history").write_text("==> 2024-01-01 <==\n+pkg-1.0\n")
    (root / "bin" / "tool").write_text(f"#!{p}/bin/python\nprint('hi')\n")
    os.chmod(root / "bin" / "tool", 0o755)
    (root / "lib" / "pkg" / "mod.py").write_text("x = 1\n")
    (root / "lib" / "pkg" / "data.bin").write_bytes(
        b"\x7fELF\0\0" + p.encode() + b"/lib\0tail\0" + bytes(range(256)))
    os.symlink("tool", root / "bin" / "tool-link")
    os.symlink(f"{p}/lib/pkg", root / "lib" / "abs-link")
    (root / "big.dat").write_bytes(os.urandom(3 << 20))


def test_rewrite_prefix_text_and_binary():
    assert E.rewrite_prefix(b"#!/a/long/prefix/bin/py\n", b"/a/long/prefix", b"/b") == b"#!/b/bin/py\n"
    data = b"\0\0/a/long/prefix/lib\0rest"
    out = E.rewrite_prefix(data, b"/a/long/prefix", b"/b/x")
    assert len(out) == len(data) and out.startswith(b"\0\0/b/x/lib\0") and out.endswith(b"rest")
    with pytest.raises(ValueError):
        E.rewrite_prefix(data, b"/a/long/prefix", b"/a/much/longer/prefix/than/before")


def test_sync_creates_updates_deletes_and_rewrites(tmp_path, monkeypatch):
    monkeypatch.setattr(E, "_CHUNK", 1 << 20)       # the 3 MB file goes in three pieces
    src, dst = tmp_path / "source_env_long_name", tmp_path / "dst_env"
    _make_env(src)
    st = E.sync_local(str(src), str(dst))
    assert st["sent_files"] == 5 and st["deleted"] == 0
    assert (dst / "bin" / "tool").read_text() == f"#!{dst}/bin/python\nprint('hi')\n"
    assert stat.S_IMODE(os.stat(dst / "bin" / "tool").st_mode) == 0o755
    b = (dst / "lib" / "pkg" / "data.bin").read_bytes()
    assert len(b) == len((src / "lib" / "pkg" / "data.bin").read_bytes())
    assert str(dst).encode() + b"/lib\0" in b and str(src).encode() not in b
    assert os.readlink(dst / "bin" / "tool-link") == "tool"
    assert os.readlink(dst / "lib" / "abs-link") == f"{dst}/lib/pkg"
    assert (dst / "big.dat").read_bytes() == (src / "big.dat").read_bytes()

    # nothing changed: the history digest and the shapes agree, nothing is hashed or sent
    st = E.sync_local(str(src), str(dst))
    assert st.get("in_sync") == 1

    # change one file, add one, remove one, and leave an extra file at the destination
    (src / "lib" / "pkg" / "mod.py").write_text("x = 2222\n")
    (src / "lib" / "pkg" / "new.py").write_text("y = 3\n")
    os.remove(src / "big.dat")
    (dst / "stale.txt").write_text("old")
    st = E.sync_local(str(src), str(dst))
    assert st["sent_files"] == 2 and st["deleted"] == 2
    assert (dst / "lib" / "pkg" / "mod.py").read_text() == "x = 2222\n"
    assert not (dst / "big.dat").exists() and not (dst / "stale.txt").exists()

    # same size, other mtime, same content: compared by hash, not re-sent (without a
    # history file there is no shortcut, every entry is looked at)
    os.remove(src / "conda-meta" / "history")
    os.remove(dst / "conda-meta" / "history")
    os.utime(src / "lib" / "pkg" / "new.py", ns=(1, 1))
    st = E.sync_local(str(src), str(dst))
    assert st["sent_files"] == 0 and st["hashed"] == 1


def test_sync_env_over_a_proc_mesh(tmp_path):
    src, dst = tmp_path / "src_env_with_a_longer_name", tmp_path / "dst"
    _make_env(src)
    pm = this_host().spawn_procs(per_host={"gpus": 1})
    try:
        out = E.sync_env(pm, str(src), str(dst), timeout=60)
        assert out[0]["sent_files"] == 5
        assert (dst / "lib" / "pkg" / "mod.py").read_text() == "x = 1\n"
        assert (dst / "bin" / "tool").read_text().startswith(f"#!{dst}/bin/python")
        out = E.sync_env(pm, str(src), str(dst), timeout=60)
        assert out[0].get("in_sync") == 1
        # a proc that already uses the client's directory is left alone
        out = E.sync_env(pm, str(src), str(src), timeout=60)
        assert out[0].get("shared") == 1
    finally:
        pm.stop().get()
