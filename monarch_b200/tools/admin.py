"""Admin view of a running job: ``show``, ``procs`` and ``top`` over the procs' actor ledgers.

Parity: hyper/src/main.rs:22-48 and hyper/src/commands/{show,procs,top}.rs (the reference's
admin CLI attaches to the legacy system actor and walks world -> proc -> actor snapshots).
Here the job's client process serves its proc mesh's ledger snapshots
(``ProcMesh.serve_admin()``) over a line-delimited JSON socket, and this tool renders them:

    python -m monarch_b200.tools.admin show  ADDR [REFERENCE]   # world, proc or actor
    python -m monarch_b200.tools.admin procs ADDR
    python -m monarch_b200.tools.admin top   ADDR [--interval 1] [--iterations N]

``ADDR`` is ``host:port`` or ``unix:/path``.  ``REFERENCE`` is a world (``mesh0``), a proc
(``mesh0[3]``) or an actor (``mesh0[3].trainers[0]``).
"""
from __future__ import annotations

import argparse
import json
import os
import socket
import socketserver
import sys
import threading
import time
from typing import Dict, List, Optional, Tuple


# ----------------------------------------------------------------------------- server --
class AdminServer:
    def __init__(self, proc_mesh, address: Optional[str] = None):
        self._pm = proc_mesh
        self._t0 = time.time()
        outer = self

        class Handler(socketserver.StreamRequestHandler):
            def handle(self):
                for line in self.rfile:
                    try:
                        req = json.loads(line)
                        resp = outer._answer(req)
                    except Exception as ex:  # noqa: BLE001 - reported to the caller
                        resp = {"error": f"{type(ex).__name__}: {ex}"}
                    self.wfile.write((json.dumps(resp) + "\n").encode())
                    self.wfile.flush()

        if address and address.startswith("unix:"):
            path = address[5:]
            if os.path.exists(path):
                os.unlink(path)

            class Srv(socketserver.ThreadingMixIn, socketserver.UnixStreamServer):
                daemon_threads = True

            self._srv = Srv(path, Handler)
            self.address = "unix:" + path
        else:
            host, port = ("127.0.0.1", 0)
            if address:
                host, _, p = address.rpartition(":")
                port = int(p)

            class Srv(socketserver.ThreadingMixIn, socketserver.TCPServer):
                daemon_threads = True
                allow_reuse_address = True

            self._srv = Srv((host or "127.0.0.1", port), Handler)
            self.address = "%s:%d" % self._srv.server_address[:2]
        self._thread = threading.Thread(target=self._srv.serve_forever, daemon=True,
                                        name="monarch-admin")
        self._thread.start()

    def _answer(self, req: dict) -> dict:
        if req.get("op") != "snapshot":
            return {"error": f"unknown op {req.get('op')!r}"}
        pm = self._pm
        led = pm.ledger(float(req.get("timeout", 5.0)))
        sl = pm._shape_.ndslice
        labels = list(pm._labels)
        procs = []
        for r in sl.ranks():
            procs.append({"rank": r, "coords": dict(zip(labels, sl.coordinates(r))),
                          "responding": r in led, "actors": led.get(r, [])})
        return {"world": pm.world, "labels": labels, "sizes": list(sl.sizes),
                "uptime_s": time.time() - self._t0, "stopped": bool(pm._stopped), "procs": procs}

    def close(self) -> None:
        self._srv.shutdown()
        self._srv.server_close()


# ----------------------------------------------------------------------------- client --
def _connect(addr: str) -> socket.socket:
    if addr.startswith("unix:"):
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        s.connect(addr[5:])
        return s
    host, _, port = addr.rpartition(":")
    return socket.create_connection((host or "127.0.0.1", int(port)), timeout=10)


def snapshot(addr: str, timeout: float = 5.0) -> dict:
    with _connect(addr) as s:
        s.sendall((json.dumps({"op": "snapshot", "timeout": timeout}) + "\n").encode())
        buf = b""
        while not buf.endswith(b"\n"):
            chunk = s.recv(1 << 16)
            if not chunk:
                break
            buf += chunk
    resp = json.loads(buf)
    if "error" in resp:
        raise RuntimeError(resp["error"])
    return resp


def _table(rows: List[List[str]]) -> str:
    widths = [max(len(str(r[i])) for r in rows) for i in range(len(rows[0]))]
    return "\n".join("  ".join(str(c).ljust(w) for c, w in zip(r, widths)).rstrip() for r in rows)


def _parse_reference(ref: str) -> Tuple[str, Optional[int], Optional[str]]:
    """``world``, ``world[rank]`` or ``world[rank].actor[pid]`` -> (world, rank, actor id)."""
    world, rank, actor = ref, None, None
    if "[" in ref:
        world, rest = ref.split("[", 1)
        r, _, tail = rest.partition("]")
        rank = int(r)
        if tail.startswith("."):
            actor = ref
    return world, rank, actor


def render_show(snap: dict, reference: Optional[str] = None) -> str:
    if reference is None:
        n_act = sum(len(p["actors"]) for p in snap["procs"])
        bad = [p["rank"] for p in snap["procs"] if not p["responding"]]
        lines = [f"world: {snap['world']}",
                 f"shape: {dict(zip(snap['labels'], snap['sizes']))}",
                 f"uptime: {snap['uptime_s']:.1f} s",
                 f"procs: {len(snap['procs'])} ({len(bad)} not responding"
                 + (f": {bad}" if bad else "") + ")",
                 f"actors: {n_act}"]
        return "\n".join(lines)
    world, rank, actor = _parse_reference(reference)
    if world != snap["world"]:
        raise KeyError(f"unknown world {world!r} (this job serves {snap['world']!r})")
    if rank is None:
        return render_procs(snap)
    proc = next((p for p in snap["procs"] if p["rank"] == rank), None)
    if proc is None:
        raise KeyError(f"no proc {rank} in {world}")
    if actor is None:
        rows = [["ACTOR", "STATUS", "HANDLED", "CHILDREN", "FAILURE"]]
        for a in proc["actors"]:
            rows.append([a["actor_id"], a["status"], a["messages_handled"], len(a["children"]),
                         a["failure"]])
        head = f"proc {world}[{rank}] {proc['coords']}" + ("" if proc["responding"]
                                                          else "  (not responding)")
        return head + "\n" + _table(rows)
    for a in proc["actors"]:
        if a["actor_id"] == actor:
            return "\n".join([f"actor: {a['actor_id']}", f"status: {a['status']}",
                              f"messages handled: {a['messages_handled']}",
                              f"children: {', '.join(a['children']) or '-'}",
                              f"failure: {a['failure'] or '-'}",
                              f"last event: {a['last_event'] or '-'}"])
    raise KeyError(f"no actor {actor}")


def render_procs(snap: dict) -> str:
    rows = [["PROC", "COORDS", "STATE", "ACTORS", "HANDLED", "FAILED"]]
    for p in snap["procs"]:
        rows.append([f"{snap['world']}[{p['rank']}]",
                     ",".join(f"{k}={v}" for k, v in p["coords"].items()),
                     "up" if p["responding"] else "no-reply", len(p["actors"]),
                     sum(a["messages_handled"] for a in p["actors"]),
                     sum(1 for a in p["actors"] if a["failure"])])
    return _table(rows)


def render_top(snap: dict, prev: Optional[dict], dt: float, limit: int = 20) -> str:
    """Actors by message rate since the previous snapshot (hyper/src/tui/top.rs shows the
    same columns in a TUI; this prints plain frames)."""
    before: Dict[str, int] = {}
    if prev is not None:
        for p in prev["procs"]:
            for a in p["actors"]:
                before[a["actor_id"]] = a["messages_handled"]
    rows = []
    for p in snap["procs"]:
        for a in p["actors"]:
            d = a["messages_handled"] - before.get(a["actor_id"], a["messages_handled"])
            rows.append((d / dt if dt > 0 else 0.0, a))
    rows.sort(key=lambda x: (-x[0], x[1]["actor_id"]))
    out = [["ACTOR", "STATUS", "MSG/S", "HANDLED"]]
    for rate, a in rows[:limit]:
        out.append([a["actor_id"], a["status"], f"{rate:.1f}", a["messages_handled"]])
    return f"{snap['world']}  up {snap['uptime_s']:.0f}s  {len(rows)} actors\n" + _table(out)


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="monarch_b200.tools.admin", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("show")
    p.add_argument("addr")
    p.add_argument("reference", nargs="?")
    p.add_argument("--json", action="store_true")
    p = sub.add_parser("procs")
    p.add_argument("addr")
    p = sub.add_parser("top")
    p.add_argument("addr")
    p.add_argument("--interval", type=float, default=1.0)
    p.add_argument("--iterations", type=int, default=0, help="0 = until interrupted")
    args = ap.parse_args(argv)
    try:
        if args.cmd == "show":
            snap = snapshot(args.addr)
            print(json.dumps(snap, indent=1) if args.json else render_show(snap, args.reference))
        elif args.cmd == "procs":
            print(render_procs(snapshot(args.addr)))
        else:
            prev, t_prev, i = None, time.time(), 0
            while True:
                snap = snapshot(args.addr)
                now = time.time()
                print(render_top(snap, prev, now - t_prev))
                print()
                prev, t_prev, i = snap, now, i + 1
                if args.iterations and i >= args.iterations:
                    break
                time.sleep(args.interval)
    except KeyboardInterrupt:
        return 130
    except (KeyError, RuntimeError, OSError) as ex:
        print(f"error: {ex}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
