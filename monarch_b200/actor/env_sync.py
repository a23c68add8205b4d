"""Environment synchronisation: make a destination prefix (a conda or virtualenv tree) equal to
a source prefix by sending only what differs, with the embedded prefix path rewritten.

Parity: monarch_conda (sync.rs: sender/receiver exchanging fingerprints and file contents
over a duplex stream; diff.rs: what changed between two environments; pack_meta_history.rs:
the ``conda-meta/history`` shortcut; hash_utils.rs) and ``sync_workspace(conda=True)`` of
python/monarch/_src/actor/proc_mesh.py.  The protocol is transport-agnostic: ``Sender`` and
``Receiver`` talk through any pair of ``send(obj)`` / ``recv()`` callables (an in-process
queue pair in tests, actor messages in ``EnvSyncActor``).

Protocol (receiver-driven, so the sender never reads the destination's disk):
  receiver -> sender  ("fingerprint", history digest, manifest)
  sender   -> receiver ("in_sync",) | a stream of ("mkdir"|"file"|"symlink"|"delete", ...) then
                       ("done", stats)
Files whose size and mtime match are taken as equal (conda packages are immutable once
extracted); everything else is compared by content hash, computed lazily on both sides.
Text files and symlink targets that embed the source prefix are rewritten to the destination
prefix; in binary files the prefix is replaced in place and padded with NULs, which needs a
destination prefix no longer than the source one (the conda-pack rule).
"""
from __future__ import annotations

import hashlib
import itertools
import os
import stat
from typing import Any, Callable, Dict, List, Optional, Tuple

from .actor_mesh import Actor, endpoint

_ids = itertools.count()
_SKIP = {"__pycache__", ".git", "pkgs"}
# kept by the receiver in its prefix: files whose content was rewritten have another size
# than their source; the index remembers the source size so that the next comparison is
# made on source terms
_INDEX = ".envsync-index.json"
_CHUNK = 8 << 20


def _digest_file(path: str) -> str:
    h = hashlib.blake2b(digest_size=16)
    with open(path, "rb") as f:
        for blk in iter(lambda: f.read(1 << 20), b""):
            h.update(blk)
    return h.hexdigest()


def history_digest(prefix: str) -> str:
    """Digest of ``conda-meta/history`` (the log of every transaction applied to a conda
    environment): equal digests mean that the same packages were installed in the same
    order.  Empty when the tree has no such file."""
    p = os.path.join(prefix, "conda-meta", "history")
    return _digest_file(p) if os.path.isfile(p) else ""


def build_manifest(prefix: str) -> Dict[str, tuple]:
    """{relative path: ("d", mode) | ("l", target) | ("f", size, mtime_ns, mode)}."""
    out: Dict[str, tuple] = {}
    prefix = os.path.abspath(prefix)
    for dirpath, dirnames, filenames in os.walk(prefix):
        dirnames[:] = sorted(d for d in dirnames if d not in _SKIP)
        rel_dir = os.path.relpath(dirpath, prefix)
        for d in list(dirnames):
            full = os.path.join(dirpath, d)
            rel = os.path.normpath(os.path.join(rel_dir, d))
            if os.path.islink(full):
                out[rel] = ("l", os.readlink(full))
                dirnames.remove(d)
            else:
                out[rel] = ("d", stat.S_IMODE(os.lstat(full).st_mode))
        for fn in sorted(filenames):
            full = os.path.join(dirpath, fn)
            rel = os.path.normpath(os.path.join(rel_dir, fn))
            st = os.lstat(full)
            if stat.S_ISLNK(st.st_mode):
                out[rel] = ("l", os.readlink(full))
            elif stat.S_ISREG(st.st_mode):
                out[rel] = ("f", st.st_size, st.st_mtime_ns, stat.S_IMODE(st.st_mode))
    return out


def rewrite_prefix(data: bytes, src: bytes, dst: bytes) -> bytes:
    """Replace the embedded source prefix.  Text: plain replacement.  Binary (contains NUL):
    each NUL-terminated string that contains the prefix keeps its length, the slack filled
    with NULs."""
    if src == dst or src not in data:
        return data
    if b"\0" not in data:
        return data.replace(src, dst)
    if len(dst) > len(src):
        raise ValueError("a binary file embeds the source prefix and the destination prefix is "
                         f"longer ({len(dst)} > {len(src)} bytes): cannot rewrite in place")
    out = bytearray(data)
    pos = 0
    while True:
        i = data.find(src, pos)
        if i < 0:
            break
        end = data.find(b"\0", i)
        if end < 0:
            end = len(data)
        s = data[i:end].replace(src, dst)
        out[i:end] = s + b"\0" * ((end - i) - len(s))
        pos = end
    return bytes(out)


class Sender:
    """Source side: owns the source prefix, answers one receiver."""

    def __init__(self, prefix: str, send: Callable[[Any], None], recv: Callable[[], Any],
                 dst_prefix: Optional[str] = None):
        self.prefix = os.path.abspath(prefix)
        self.dst_prefix = dst_prefix
        self._send, self._recv = send, recv

    def run(self) -> Dict[str, int]:
        kind, dst_prefix, their_history, theirs = self._recv()
        assert kind == "fingerprint"
        dst_prefix = self.dst_prefix or dst_prefix
        src_b, dst_b = self.prefix.encode(), os.path.abspath(dst_prefix).encode()
        mine = build_manifest(self.prefix)
        theirs = {p: e for p, e in theirs.items() if p != _INDEX}
        stats = {"sent_files": 0, "sent_bytes": 0, "deleted": 0, "kept": 0, "hashed": 0}
        hist = history_digest(self.prefix)
        dst_abs = os.path.abspath(dst_prefix)
        expect = {p: (("l", dst_abs + e[1][len(self.prefix):])
                      if e[0] == "l" and e[1].startswith(self.prefix) else e)
                  for p, e in mine.items()}
        if hist and hist == their_history and _same_shape(expect, theirs):
            self._send(("in_sync",))
            stats["kept"] = len(mine)
            return stats
        # ask for content hashes only where size matches but mtime does not
        doubtful = [p for p, e in mine.items()
                    if e[0] == "f" and p in theirs and theirs[p][0] == "f"
                    and theirs[p][1] == e[1] and theirs[p][2] != e[2]]
        their_hashes: Dict[str, str] = {}
        if doubtful:
            self._send(("hashes?", doubtful))
            kind, their_hashes = self._recv()
            assert kind == "hashes"
            stats["hashed"] = len(doubtful)
        for rel in sorted(p for p in theirs if p not in mine):
            self._send(("delete", rel))
            stats["deleted"] += 1
        for rel in sorted(mine):
            e, t = mine[rel], theirs.get(rel)
            full = os.path.join(self.prefix, rel)
            if e[0] == "d":
                if t is None or t[0] != "d":
                    self._send(("mkdir", rel, e[1]))
                continue
            if e[0] == "l":
                target = e[1]
                if target.startswith(self.prefix):
                    target = os.path.abspath(dst_prefix) + target[len(self.prefix):]
                if t != ("l", target):
                    self._send(("symlink", rel, target))
                continue
            same = t is not None and t[0] == "f" and t[1] == e[1] and (
                t[2] == e[2] or their_hashes.get(rel) == _digest_file(full))
            if same:
                stats["kept"] += 1
                if t[3] != e[3]:
                    self._send(("chmod", rel, e[3]))
                continue
            with open(full, "rb") as f:
                data = f.read()
            data = rewrite_prefix(data, src_b, dst_b)
            # large files go in pieces so that no single message holds more than a chunk
            n = max(1, (len(data) + _CHUNK - 1) // _CHUNK)
            for k in range(n):
                self._send(("file", rel, e[3], e[2], k, n, data[k * _CHUNK:(k + 1) * _CHUNK],
                            e[1]))
            stats["sent_files"] += 1
            stats["sent_bytes"] += len(data)
        self._send(("done", stats))
        return stats


def _same_shape(a: Dict[str, tuple], b: Dict[str, tuple]) -> bool:
    if a.keys() != b.keys():
        return False
    return all((e[0], e[1]) == (b[p][0], b[p][1]) for p, e in a.items())


class Receiver:
    """Destination side: owns the destination prefix and applies what the sender streams."""

    def __init__(self, prefix: str, send: Optional[Callable[[Any], None]] = None,
                 recv: Optional[Callable[[], Any]] = None):
        self.prefix = os.path.abspath(prefix)
        self._send, self._recv = send, recv
        self._partial: Dict[str, Any] = {}
        self._index: Dict[str, list] = {}

    def _path(self, rel: str) -> str:
        full = os.path.normpath(os.path.join(self.prefix, rel))
        if not (full + os.sep).startswith(self.prefix + os.sep):
            raise ValueError(f"path escapes the environment: {rel}")
        return full

    def _load_index(self) -> Dict[str, list]:
        import json
        try:
            with open(os.path.join(self.prefix, _INDEX)) as f:
                return json.load(f)
        except (OSError, ValueError):
            return {}

    def _save_index(self) -> None:
        import json
        tmp = os.path.join(self.prefix, _INDEX + f".{os.getpid()}")
        with open(tmp, "w") as f:
            json.dump(self._index, f)
        os.replace(tmp, os.path.join(self.prefix, _INDEX))

    def fingerprint(self) -> tuple:
        os.makedirs(self.prefix, exist_ok=True)
        self._index = self._load_index()
        man = build_manifest(self.prefix)
        man.pop(_INDEX, None)
        for rel, (src_size, dst_size) in list(self._index.items()):
            e = man.get(rel)
            if e is not None and e[0] == "f" and e[1] == dst_size:
                man[rel] = ("f", src_size, e[2], e[3])     # report on the source's terms
            else:
                del self._index[rel]
        return ("fingerprint", self.prefix, history_digest(self.prefix), man)

    def hashes(self, rels: List[str]) -> Dict[str, str]:
        return {rel: _digest_file(self._path(rel)) for rel in rels}

    def apply(self, msg: tuple) -> Optional[Dict[str, int]]:
        """Apply one sender message; returns the final statistics when it ends the stream."""
        import shutil
        kind = msg[0]
        if kind == "in_sync":
            return {"sent_files": 0, "sent_bytes": 0, "deleted": 0, "in_sync": 1}
        if kind == "done":
            self._save_index()
            return dict(msg[1])
        if kind == "delete":
            full = self._path(msg[1])
            if os.path.islink(full) or os.path.isfile(full):
                os.remove(full)
            elif os.path.isdir(full):
                shutil.rmtree(full, ignore_errors=True)
            self._index.pop(msg[1], None)
        elif kind == "mkdir":
            full = self._path(msg[1])
            if os.path.islink(full) or os.path.isfile(full):
                os.remove(full)
            os.makedirs(full, exist_ok=True)
            os.chmod(full, msg[2])
        elif kind == "symlink":
            full = self._path(msg[1])
            if os.path.islink(full) or os.path.isfile(full):
                os.remove(full)
            elif os.path.isdir(full):
                shutil.rmtree(full)
            os.makedirs(os.path.dirname(full), exist_ok=True)
            os.symlink(msg[2], full)
        elif kind == "chmod":
            os.chmod(self._path(msg[1]), msg[2])
        elif kind == "file":
            _, rel, mode, mtime_ns, k, n, data, src_size = msg
            full = self._path(rel)
            tmp = f"{full}.envsync{os.getpid()}"
            if k == 0:
                os.makedirs(os.path.dirname(full), exist_ok=True)
                self._partial[rel] = open(tmp, "wb")
            self._partial[rel].write(data)
            if k == n - 1:
                self._partial.pop(rel).close()
                os.chmod(tmp, mode)
                os.utime(tmp, ns=(mtime_ns, mtime_ns))
                if os.path.isdir(full) and not os.path.islink(full):
                    shutil.rmtree(full)
                os.replace(tmp, full)
                dst_size = os.path.getsize(full)
                if dst_size != src_size:
                    self._index[rel] = [src_size, dst_size]
                else:
                    self._index.pop(rel, None)
        else:
            raise ValueError(f"unknown env-sync message {kind!r}")
        return None

    def run(self) -> Dict[str, int]:
        self._send(self.fingerprint())
        while True:
            msg = self._recv()
            if msg[0] == "hashes?":
                self._send(("hashes", self.hashes(msg[1])))
                continue
            out = self.apply(msg)
            if out is not None:
                return out


def sync_local(src_prefix: str, dst_prefix: str) -> Dict[str, int]:
    """Run both ends in this process (two prefixes on one machine; also the test harness)."""
    import queue
    import threading
    to_sender: "queue.Queue" = queue.Queue()
    to_receiver: "queue.Queue" = queue.Queue(maxsize=8)
    result: Dict[str, Any] = {}

    def sender():
        try:
            result["sender"] = Sender(src_prefix, to_receiver.put, to_sender.get).run()
        except BaseException as ex:  # noqa: BLE001 - surfaced to the caller below
            result["error"] = ex
            to_receiver.put(("done", {"error": 1}))

    t = threading.Thread(target=sender, daemon=True)
    t.start()
    out = Receiver(dst_prefix, to_sender.put, to_receiver.get).run()
    t.join()
    if "error" in result:
        raise result["error"]
    return out


class EnvSyncActor(Actor):
    """One per proc: the receiving end, driven by the client through endpoint calls."""

    def __init__(self, prefix: Optional[str] = None):
        import sys
        self.receiver = Receiver(prefix or os.environ.get("CONDA_PREFIX") or sys.prefix)

    @endpoint
    def fingerprint(self) -> tuple:
        return self.receiver.fingerprint()

    @endpoint
    def hashes(self, rels: List[str]) -> Dict[str, str]:
        return self.receiver.hashes(rels)

    @endpoint
    def apply(self, msgs: List[tuple]) -> Optional[Dict[str, int]]:
        out = None
        for m in msgs:
            r = self.receiver.apply(m)
            out = r if r is not None else out
        return out


_BATCH_BYTES = 32 << 20


def sync_env(proc_mesh, src_prefix: Optional[str] = None, dst_prefix: Optional[str] = None,
             timeout: Optional[float] = None) -> Dict[int, Dict[str, int]]:
    """Make the environment of every proc of ``proc_mesh`` equal to ``src_prefix`` (default:
    the client's active environment).  ``dst_prefix`` defaults to each proc's own active
    environment.  Procs whose prefix is the client's own directory (same box, same path) are
    left alone.  Returns {rank: statistics}."""
    import sys
    src = os.path.abspath(src_prefix or os.environ.get("CONDA_PREFIX") or sys.prefix)
    owner = proc_mesh._owner
    actors = owner.spawn(f"env_sync_{next(_ids)}", EnvSyncActor, dst_prefix)
    out: Dict[int, Dict[str, int]] = {}
    fps = actors.fingerprint.call().get(timeout)
    for point, fp in fps.items():
        rank = point.rank
        one = actors.slice(**{l: c for l, c in zip(owner._labels,
                                                   owner._ndslice.coordinates(rank))})
        if os.path.realpath(fp[1]) == os.path.realpath(src):
            out[rank] = {"sent_files": 0, "sent_bytes": 0, "deleted": 0, "shared": 1}
            continue
        batch: List[tuple] = []
        size = 0
        replies: List[Any] = [fp]
        final: Dict[str, Any] = {}

        def flush():
            nonlocal batch, size
            if batch:
                r = one.apply.call_one(batch).get(timeout)
                if r is not None:
                    final["stats"] = r
                batch, size = [], 0

        def send(msg):
            nonlocal size
            if msg[0] == "hashes?":
                flush()
                replies.append(("hashes", one.hashes.call_one(msg[1]).get(timeout)))
                return
            batch.append(msg)
            size += len(msg[6]) if msg[0] == "file" else 64
            if size >= _BATCH_BYTES or msg[0] in ("done", "in_sync"):
                flush()

        Sender(src, send, lambda: replies.pop(0)).run()
        flush()
        out[rank] = final.get("stats", {})
    return out

