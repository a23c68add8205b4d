"""Process-allocator daemon: runs on a host and starts procs there on behalf of remote
clients.

    python -m monarch_b200.tools.process_allocator --addr tcp!127.0.0.1:26600 \
        [--program "python -m monarch_b200.actor.bootstrap_main"]

The daemon decides WHAT runs: its ``--program`` (default: this interpreter running
``monarch_b200.actor.bootstrap_main``), in its own working directory.  A client only asks
for one more instance of it: it connects once per proc (see ``remote_exec``), sends one JSON
line ``{"start": 1, "env": {...}, "token": ...}`` and then receives JSON lines ``{"out": text}`` /
``{"err": text}`` / ``{"exit": code}``.  Of the client's ``env`` only the bootstrap
variables pass (prefixes ``HYPERACTOR_``, ``MONARCH_``, ``MB200_`` and the rank/rendezvous
names in ``ENV_ALLOW``); a request that names a program (``argv``) or a directory (``cwd``)
is refused.  The default bind is the loopback interface; to serve other hosts bind another
address and set ``MB200_ALLOCATOR_TOKEN`` on both sides: with a token configured, requests
without the same token are refused.  It may send ``{"signal": n}``.  ``--native`` runs the
same daemon as a standalone executable (``csrc/tools/process_allocator.cpp``).
Heartbeats ``{"hb": 1}`` flow both ways every ``--heartbeat`` seconds; when the client has
been silent for 3 intervals, or its connection drops, the proc is killed (SIGTERM, then
SIGKILL): a host never keeps orphans of a vanished client.

Parity: monarch_hyperactor/src/bin/process_allocator (the daemon; the program is fixed by
its ``--program`` option, common.rs:41), hyperactor_mesh
alloc/remoteprocess.rs:73-108 (RemoteProcessAllocator), :940-1085 (heartbeats and the host
watchdog); Python address syntax ``tcp!host:port`` (python/monarch/_src/actor/allocator.py
:104-113).
"""
from __future__ import annotations

import argparse
import hmac
import json
import os
import shlex
import signal
import socket
import subprocess
import sys
import threading
import time


def parse_addr(addr: str):
    """``tcp!host:port`` (or ``host:port``) -> (host, port)."""
    if addr.startswith("tcp!"):
        addr = addr[4:]
    host, _, port = addr.rpartition(":")
    return host or "127.0.0.1", int(port)


#: environment a client may set for the procs it asks for (prefixes and exact names)
ENV_ALLOW_PREFIX = ("HYPERACTOR_", "MONARCH_", "MB200_", "MASTER_")
# PYTHONPATH passes because the procs must import the client's actor classes; like the
# bootstrap function it lets an accepted client choose code, which is what an actor
# client does anyway -- who may be a client is decided by the bind address and the token.
ENV_ALLOW = ("CUDA_VISIBLE_DEVICES", "LOCAL_RANK", "RANK", "WORLD_SIZE", "PYTHONPATH")
#: never taken from a client, whatever its prefix
ENV_DENY = ("MB200_ALLOCATOR_TOKEN",)


def default_program() -> list:
    return [sys.executable, "-m", "monarch_b200.actor.bootstrap_main"]


def filter_env(env: dict) -> dict:
    """The part of a client's environment request that the daemon honours."""
    return {str(k): str(v) for k, v in (env or {}).items()
            if (k.startswith(ENV_ALLOW_PREFIX) or k in ENV_ALLOW) and k not in ENV_DENY}


class _Session(threading.Thread):
    def __init__(self, conn: socket.socket, peer, heartbeat: float, registry: set,
                 program: list, token: str = ""):
        super().__init__(daemon=True)
        self.conn, self.peer, self.hb, self.registry = conn, peer, heartbeat, registry
        self.program, self.token = list(program), token
        self.proc: subprocess.Popen | None = None
        self._wlock = threading.Lock()
        self._last_seen = time.monotonic()
        self._closed = False

    def _send(self, obj) -> bool:
        data = (json.dumps(obj) + "\n").encode()
        with self._wlock:
            try:
                self.conn.sendall(data)
                return True
            except OSError:
                return False

    def _pump(self, stream, key) -> None:
        for line in iter(stream.readline, b""):
            if not self._send({key: line.decode(errors="replace")}):
                break
        stream.close()

    def _kill(self) -> None:
        p = self.proc
        if p is None or p.poll() is not None:
            return
        try:
            os.killpg(p.pid, signal.SIGTERM)
        except OSError:
            pass
        for _ in range(30):
            if p.poll() is not None:
                return
            time.sleep(0.1)
        try:
            os.killpg(p.pid, signal.SIGKILL)
        except OSError:
            pass

    def _watch(self) -> None:
        while not self._closed:
            time.sleep(self.hb)
            self._send({"hb": 1})
            if time.monotonic() - self._last_seen > 3 * self.hb + 1.0:
                self._kill()   # the client vanished without closing the connection
                return

    def run(self) -> None:
        self.registry.add(self)
        f = self.conn.makefile("rb")
        try:
            try:
                req = json.loads(f.readline() or b"{}")
            except ValueError:
                req = None
            if not isinstance(req, dict) or not req.get("start"):
                self._send({"exit": 126, "error": "malformed request"})   # or a port probe
                return
            if self.token and not hmac.compare_digest(str(req.get("token") or ""), self.token):
                self._send({"exit": 126, "error": "bad or missing allocator token"})
                return
            if req.get("argv") or req.get("cwd"):
                self._send({"exit": 126, "error": "this daemon runs its own --program; a "
                            "request may not name a program or a working directory"})
                return
            env = dict(os.environ)
            env.pop("MB200_ALLOCATOR_TOKEN", None)
            env.update(filter_env(req.get("env")))
            try:
                self.proc = subprocess.Popen(self.program, env=env,
                                             stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                                             start_new_session=True)
            except OSError as e:
                self._send({"exit": 127, "error": str(e)})
                return
            self._send({"pid": self.proc.pid, "host": socket.gethostname()})
            pumps = [threading.Thread(target=self._pump, args=(self.proc.stdout, "out"), daemon=True),
                     threading.Thread(target=self._pump, args=(self.proc.stderr, "err"), daemon=True)]
            for t in pumps:
                t.start()
            threading.Thread(target=self._watch, daemon=True).start()

            def reader():
                for line in iter(f.readline, b""):
                    self._last_seen = time.monotonic()
                    try:
                        msg = json.loads(line)
                    except ValueError:
                        continue
                    if "signal" in msg and self.proc and self.proc.poll() is None:
                        try:
                            os.killpg(self.proc.pid, int(msg["signal"]))
                        except OSError:
                            pass
                self._kill()   # connection closed by the client
            threading.Thread(target=reader, daemon=True).start()
            code = self.proc.wait()
            for t in pumps:
                t.join(2)
            self._send({"exit": code})
        finally:
            self._closed = True
            self._kill()
            try:
                self.conn.close()
            except OSError:
                pass
            self.registry.discard(self)


def serve(addr: str, heartbeat: float = 5.0, ready=None, program=None, token=None) -> None:
    host, port = parse_addr(addr)
    program = list(program) if program else default_program()
    token = os.environ.get("MB200_ALLOCATOR_TOKEN", "") if token is None else token
    srv = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    srv.bind((host, port))
    srv.listen(256)
    sessions: set = set()
    if ready is not None:
        ready(srv.getsockname()[1])
    print(f"process_allocator listening on tcp!{host}:{srv.getsockname()[1]}", flush=True)

    def stop(*_):
        for s in list(sessions):
            s._kill()
        os._exit(0)
    try:
        signal.signal(signal.SIGTERM, stop)
        signal.signal(signal.SIGINT, stop)
    except ValueError:
        pass   # not the main thread (tests run the daemon in a thread)
    while True:
        conn, peer = srv.accept()
        conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        _Session(conn, peer, heartbeat, sessions, program, token).start()


def native_daemon() -> str | None:
    """Path of the native daemon (``csrc/tools/process_allocator.cpp``, the same protocol in
    a standalone executable), built on demand; None where no compiler is available."""
    try:
        from .. import _build
        return str(_build.build_allocator())
    except Exception:  # noqa: BLE001 - no compiler on this host: the Python daemon serves
        return None


def native_command(addr: str, heartbeat: float = 5.0, program=None) -> list | None:
    """Command line that runs the native daemon with this module's defaults."""
    exe = native_daemon()
    if exe is None:
        return None
    return [exe, "--addr", addr, "--heartbeat", str(heartbeat), "--program",
            shlex.join(list(program) if program else default_program())]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--addr", default="tcp!127.0.0.1:26600")
    ap.add_argument("--heartbeat", type=float, default=5.0)
    ap.add_argument("--program", default=None,
                    help="command line of the proc this daemon starts for its clients "
                         "(default: this interpreter -m monarch_b200.actor.bootstrap_main)")
    ap.add_argument("--native", action="store_true",
                    help="run the native daemon (same protocol, no Python in the serving path)")
    a = ap.parse_args(argv)
    program = shlex.split(a.program) if a.program else None
    if a.native:
        cmd = native_command(a.addr, a.heartbeat, program)
        if cmd is None:
            print("process_allocator: the native daemon could not be built here", file=sys.stderr)
            return 2
        os.execv(cmd[0], cmd)
    serve(a.addr, a.heartbeat, program=program)
    return 0


if __name__ == "__main__":
    sys.exit(main())
