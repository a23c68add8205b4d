"""Workspace synchronisation and module auto-reload for the procs of a mesh.

``proc_mesh.sync_workspace(workspace=dir, auto_reload=True)`` ships the files of ``dir``
that changed since the last sync to every proc (a per-proc ``CodeSyncActor`` writes them
under the proc's workspace root: ``$WORKSPACE_DIR`` or the same path as on the client) and,
with ``auto_reload``, reloads the already imported modules whose source changed, so the
next endpoint call runs the new code without restarting the procs.

Parity: monarch_hyperactor/src/code_sync (manager.rs:71-341 ``CodeSyncManager``, rsync.rs:
the file mover, auto_reload.rs + python/monarch/_src/actor/code_sync/auto_reload.py: the
``AutoReloader`` that snapshots module sources by hash and reloads the changed ones),
python/monarch/_src/actor/proc_mesh.py ``sync_workspace``.  Files travel as message parts
over the actor channels (content-hash manifest computed by the native runtime --
``csrc/mesh/tree_manifest.cpp`` --, only changed files), not through an rsync daemon.  Environment (conda / virtualenv) sync lives in ``env_sync.py``.
"""
from __future__ import annotations

import importlib
import os
import sys
from typing import Dict, List, Optional, Tuple

from .actor_mesh import Actor, endpoint
from .future import Future

_SKIP_DIRS = {".git", "__pycache__", ".pytest_cache", "build", ".hypothesis"}
_MAX_FILE = 64 << 20


_SKIP_SUFFIXES = (".pyc", ".so", ".o")


def _hash_file(path: str) -> str:
    """Content hash of one file: the native 128-bit hash (the one ``manifest`` uses)."""
    from .. import _native as N
    h = N.hash_file_128(path)
    if h is None:
        raise OSError(f"cannot read {path}")
    return h


def manifest(root: str) -> Dict[str, str]:
    """{relative path: content hash} of the regular files under ``root``: the walk and the
    hashing run in the native runtime, on a few threads, without the GIL (a workspace of
    thousands of files is compared on every sync, on the client and on every proc)."""
    from .. import _native as N
    return N.tree_manifest(root, sorted(_SKIP_DIRS), list(_SKIP_SUFFIXES), _MAX_FILE,
                           min(8, os.cpu_count() or 1))


class AutoReloader:
    """Tracks the source hash of every imported module that lives under ``root`` and reloads
    the ones whose file changed (dependencies first is not attempted: modules are reloaded
    in import order, which is how they were first initialised)."""

    def __init__(self, root: str):
        self.root = os.path.realpath(root)
        self._seen: Dict[str, str] = {}
        self.snapshot()

    def _modules(self) -> List[Tuple[str, str]]:
        out = []
        for name, m in list(sys.modules.items()):
            f = getattr(m, "__file__", None)
            if f and f.endswith(".py") and os.path.realpath(f).startswith(self.root + os.sep):
                out.append((name, f))
        return out

    def snapshot(self) -> None:
        for name, f in self._modules():
            try:
                self._seen[name] = _hash_file(f)
            except OSError:
                pass

    def reload_changed(self, touched: Optional[List[str]] = None) -> List[str]:
        """Reload the imported modules whose file changed since the last look, or -- when
        ``touched`` (paths relative to the root) is given -- whose file is in that list,
        whatever their hash (several procs may share one directory, so the file may have
        been rewritten by a neighbour before this proc looked)."""
        importlib.invalidate_caches()
        forced = {os.path.realpath(os.path.join(self.root, t)) for t in (touched or [])}
        changed = []
        for name, f in self._modules():
            try:
                h = _hash_file(f)
            except OSError:
                continue
            if os.path.realpath(f) in forced or self._seen.get(name) not in (None, h):
                importlib.reload(sys.modules[name])
                changed.append(name)
            self._seen[name] = h
        return changed


class CodeSyncActor(Actor):
    """One per proc: owns the proc's copy of the workspace."""

    def __init__(self, root: str):
        self.root = os.environ.get("WORKSPACE_DIR", root)
        os.makedirs(self.root, exist_ok=True)
        if self.root not in sys.path:
            sys.path.insert(0, self.root)
        self.reloader: Optional[AutoReloader] = None

    @endpoint
    def manifest(self) -> Dict[str, str]:
        return manifest(self.root)

    @endpoint
    def enable_auto_reload(self) -> None:
        if self.reloader is None:
            self.reloader = AutoReloader(self.root)

    @endpoint
    def apply(self, files: Dict[str, bytes], deleted: List[str], reload: bool) -> List[str]:
        for rel, data in files.items():
            dst = os.path.join(self.root, rel)
            if not os.path.realpath(dst).startswith(os.path.realpath(self.root)):
                raise ValueError(f"path escapes the workspace: {rel}")
            os.makedirs(os.path.dirname(dst) or self.root, exist_ok=True)
            tmp = f"{dst}.mb200_tmp{os.getpid()}"
            with open(tmp, "wb") as f:
                f.write(data)
            os.replace(tmp, dst)
        for rel in deleted:
            try:
                os.remove(os.path.join(self.root, rel))
            except OSError:
                pass
        if reload and self.reloader is not None:
            return self.reloader.reload_changed(list(files))
        return []


_managers: Dict[str, tuple] = {}


def sync_workspace(proc_mesh, workspace: Optional[str] = None, auto_reload: bool = False) -> Future:
    """See the module docstring.  Returns a Future of {rank: [reloaded modules]}."""
    workspace = os.path.abspath(workspace or os.getcwd())
    owner = proc_mesh._owner
    key = (owner.world, workspace)

    def do(timeout):
        ent = _managers.get(key)
        if ent is None:
            actors = owner.spawn(f"code_sync_{len(_managers)}", CodeSyncActor, workspace)
            remote = {r: m for r, m in ((p.rank, v) for p, v in
                                         actors.manifest.call().get(timeout).items())}
            ent = _managers[key] = (actors, remote)
        actors, remote = ent
        if auto_reload:
            actors.enable_auto_reload.call().get(timeout)
        local = manifest(workspace)
        # every proc receives what differs from *its* copy; procs that share a directory
        # with the client (same box, same path) need nothing
        result = {}
        union_files: Dict[str, bytes] = {}
        need_any = set()
        deleted_any = set()
        for r, rm in remote.items():
            need_any |= {p for p, h in local.items() if rm.get(p) != h}
            deleted_any |= {p for p in rm if p not in local}
        for rel in need_any:
            with open(os.path.join(workspace, rel), "rb") as f:
                union_files[rel] = f.read()
        out = actors.apply.call(union_files, sorted(deleted_any), auto_reload).get(timeout)
        for p, v in out.items():
            result[p.rank] = v
        for r in remote:
            remote[r] = dict(local)
        return result

    return Future(do)
