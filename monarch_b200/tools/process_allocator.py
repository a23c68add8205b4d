"""Process-allocator daemon: runs on a host and starts procs there on behalf of remote
clients.

    python -m monarch_b200.tools.process_allocator --addr tcp!0.0.0.0:26600

A client that wants procs on this host connects once per proc (see ``remote_exec``), sends
one JSON line ``{"argv": [...], "env": {...}, "cwd": ...}`` and then receives JSON lines
``{"out": text}`` / ``{"err": text}`` / ``{"exit": code}``.  It may send ``{"signal": n}``.
Heartbeats ``{"hb": 1}`` flow both ways every ``--heartbeat`` seconds; when the client has
been silent for 3 intervals, or its connection drops, the proc is killed (SIGTERM, then
SIGKILL): a host never keeps orphans of a vanished client.

Parity: monarch_hyperactor/src/bin/process_allocator (the daemon), hyperactor_mesh
alloc/remoteprocess.rs:73-108 (RemoteProcessAllocator), :940-1085 (heartbeats and the host
watchdog); Python address syntax ``tcp!host:port`` (python/monarch/_src/actor/allocator.py
:104-113).
"""
from __future__ import annotations

import argparse
import json
import os
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


class _Session(threading.Thread):
    def __init__(self, conn: socket.socket, peer, heartbeat: float, registry: set):
        super().__init__(daemon=True)
        self.conn, self.peer, self.hb, self.registry = conn, peer, heartbeat, registry
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
            req = json.loads(f.readline() or b"{}")
            argv = req.get("argv")
            if not argv:
                self._send({"exit": 127, "error": "no argv"})
                return
            env = dict(os.environ)
            env.update(req.get("env") or {})
            try:
                self.proc = subprocess.Popen(argv, env=env, cwd=req.get("cwd") or None,
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


def serve(addr: str, heartbeat: float = 5.0, ready=None) -> None:
    host, port = parse_addr(addr)
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
        _Session(conn, peer, heartbeat, sessions).start()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--addr", default="tcp!0.0.0.0:26600")
    ap.add_argument("--heartbeat", type=float, default=5.0)
    a = ap.parse_args(argv)
    serve(a.addr, a.heartbeat)
    return 0


if __name__ == "__main__":
    sys.exit(main())
