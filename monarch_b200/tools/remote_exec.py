"""Local stand-in of a proc that runs on another host's process-allocator daemon (the
Python form; ``csrc/tools/remote_exec.cpp`` is the same program as a native executable and is
what the process allocator starts where it can be built).

The process allocator of the client starts one of these per remote proc:

    python -m monarch_b200.tools.remote_exec

It picks the daemon from ``MB200_REMOTE_HOSTS`` (comma-separated ``tcp!host:port``) by the
proc's rank (``HYPERACTOR_MESH_INDEX`` // ``MB200_PROCS_PER_HOST``), forwards the bootstrap
environment (the daemon starts its own program; clients cannot name one) and the shared
``MB200_ALLOCATOR_TOKEN`` when one is set, relays the remote stdout/stderr to its own (where the
allocator's log tailer reads them), forwards SIGTERM/SIGINT, sends heartbeats, and exits
with the remote exit code.  Killing it kills the remote proc (the daemon sees the
connection drop)."""
from __future__ import annotations

import json
import os
import signal
import socket
import sys
import threading
import time

from .process_allocator import filter_env, parse_addr


def main(argv=None) -> int:
    hosts = [h for h in os.environ.get("MB200_REMOTE_HOSTS", "").split(",") if h]
    if not hosts:
        print("remote_exec: MB200_REMOTE_HOSTS is empty", file=sys.stderr)
        return 2
    rank = int(os.environ.get("HYPERACTOR_MESH_INDEX", "0"))
    per_host = max(1, int(os.environ.get("MB200_PROCS_PER_HOST", "1")))
    host, port = parse_addr(hosts[min(rank // per_host, len(hosts) - 1)])
    env = filter_env(dict(os.environ))
    env["MB200_LOCAL_INDEX"] = str(rank % per_host)
    hb = float(os.environ.get("MB200_ALLOCATOR_HEARTBEAT", "5"))
    try:
        conn = socket.create_connection((host, port), timeout=10)
    except OSError as e:
        print(f"remote_exec: cannot reach allocator {host}:{port}: {e}", file=sys.stderr)
        return 111
    conn.settimeout(None)
    wlock = threading.Lock()

    def send(obj):
        with wlock:
            try:
                conn.sendall((json.dumps(obj) + "\n").encode())
            except OSError:
                pass

    send({"start": 1, "env": env, "token": os.environ.get("MB200_ALLOCATOR_TOKEN", "")})
    for s in (signal.SIGTERM, signal.SIGINT):
        signal.signal(s, lambda n, _f: send({"signal": n}))

    def beat():
        while True:
            time.sleep(hb)
            send({"hb": 1})
    threading.Thread(target=beat, daemon=True).start()
    code = 1
    for line in conn.makefile("rb"):
        try:
            msg = json.loads(line)
        except ValueError:
            continue
        if "out" in msg:
            sys.stdout.write(msg["out"])
            sys.stdout.flush()
        elif "err" in msg:
            sys.stderr.write(msg["err"])
            sys.stderr.flush()
        elif "exit" in msg:
            code = int(msg["exit"])
            if msg.get("error"):
                print(f"remote_exec: {msg['error']}", file=sys.stderr)
            break
    return code if code >= 0 else 128 - code


if __name__ == "__main__":
    sys.exit(main())
