"""Job CLI: start, inspect and stop sets of process-allocator daemons ("jobs") that host
meshes can be built on.

    python -m monarch_b200.tools.cli create --name dev --hosts 2      # two local daemons
    python -m monarch_b200.tools.cli info dev
    python -m monarch_b200.tools.cli bounce dev                        # restart the daemons
    python -m monarch_b200.tools.cli stop dev   |  kill dev

A job is a JSON file ``<jobs dir>/<name>.json`` = {"name", "allocators": ["tcp!h:p", ...],
"pids": [...], "created"}; ``hosts_from_config(name)`` turns it into a HostMesh.  ``create
--remote tcp!h:p ...`` registers daemons that were started elsewhere (other boxes) instead
of starting local ones.

Parity: python/monarch/tools/cli.py:42-169 (create/info/kill/bounce/stop), commands.py,
mesh_spec.py (the job description); the reference drives TorchX schedulers, this tool
drives local or pre-started daemons.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import socket
import subprocess
import sys
import time
from typing import List


def jobs_dir() -> str:
    d = os.environ.get("MB200_JOBS_DIR", os.path.expanduser("~/.monarch_b200/jobs"))
    os.makedirs(d, exist_ok=True)
    return d


def _path(name: str) -> str:
    return os.path.join(jobs_dir(), f"{name}.json")


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
        return True
    except OSError:
        return False


def _reachable(addr: str) -> bool:
    from .process_allocator import parse_addr
    try:
        socket.create_connection(parse_addr(addr), timeout=1.0).close()
        return True
    except OSError:
        return False


def _daemon_command(addr: str) -> list:
    """The allocator daemon for ``addr``: the native executable where it can be built
    (``MB200_ALLOCATOR_DAEMON=python`` forces the Python one; both speak one protocol)."""
    if os.environ.get("MB200_ALLOCATOR_DAEMON", "native") != "python":
        from .process_allocator import native_command
        cmd = native_command(addr)
        if cmd is not None:
            return cmd
    return [sys.executable, "-m", "monarch_b200.tools.process_allocator", "--addr", addr]


def _start_local(n: int) -> tuple:
    addrs, pids = [], []
    for _ in range(n):
        port = _free_port()
        addr = f"tcp!127.0.0.1:{port}"
        p = subprocess.Popen(_daemon_command(addr), stdout=subprocess.DEVNULL,
                             stderr=subprocess.DEVNULL, start_new_session=True)
        addrs.append(addr)
        pids.append(p.pid)
    deadline = time.time() + 20
    while time.time() < deadline and not all(_reachable(a) for a in addrs):
        time.sleep(0.1)
    return addrs, pids


def create(name: str, hosts: int = 1, remote: List[str] | None = None) -> dict:
    if os.path.exists(_path(name)):
        raise SystemExit(f"job {name!r} already exists (stop it first)")
    if remote:
        addrs, pids = list(remote), []
    else:
        addrs, pids = _start_local(hosts)
    job = {"name": name, "allocators": addrs, "pids": pids, "created": time.time()}
    with open(_path(name), "w") as f:
        json.dump(job, f, indent=1)
    return job


def load(name: str) -> dict:
    if not os.path.exists(_path(name)):
        raise SystemExit(f"no job named {name!r}")
    with open(_path(name)) as f:
        return json.load(f)


def info(name: str) -> dict:
    job = load(name)
    job["state"] = [{"allocator": a, "reachable": _reachable(a)} for a in job["allocators"]]
    job["running"] = all(s["reachable"] for s in job["state"])
    return job


def stop(name: str, sig: int = signal.SIGTERM) -> None:
    job = load(name)
    for pid in job.get("pids", []):
        if _alive(pid):
            try:
                os.killpg(pid, sig)
            except OSError:
                pass
    os.remove(_path(name))


def bounce(name: str) -> dict:
    job = load(name)
    n = len(job["allocators"])
    if not job.get("pids"):
        raise SystemExit("only locally started jobs can be bounced")
    stop(name)
    return create(name, n)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="monarch_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("create")
    c.add_argument("--name", required=True)
    c.add_argument("--hosts", type=int, default=1)
    c.add_argument("--remote", nargs="*", help="addresses of daemons started elsewhere")
    for n in ("info", "stop", "kill", "bounce"):
        sub.add_parser(n).add_argument("name")
    sub.add_parser("list")
    a = ap.parse_args(argv)
    if a.cmd == "create":
        print(json.dumps(create(a.name, a.hosts, a.remote), indent=1))
    elif a.cmd == "info":
        print(json.dumps(info(a.name), indent=1))
    elif a.cmd == "stop":
        stop(a.name)
    elif a.cmd == "kill":
        stop(a.name, signal.SIGKILL)
    elif a.cmd == "bounce":
        print(json.dumps(bounce(a.name), indent=1))
    elif a.cmd == "list":
        for f in sorted(os.listdir(jobs_dir())):
            if f.endswith(".json"):
                print(f[:-5])
    return 0


if __name__ == "__main__":
    sys.exit(main())
