"""Remote process allocation: procs started by process-allocator daemons ("hosts" here are
daemons on localhost ports, as in the reference's allocator tests), driven through the job
CLI and ``hosts_from_config``; a vanished client leaves no orphan procs."""
import os
import subprocess
import sys
import time

import pytest

from monarch_b200.actor import Actor, endpoint, hosts_from_config
from monarch_b200.tools import cli


class Where(Actor):
    @endpoint
    def pid(self) -> int:
        return os.getpid()

    @endpoint
    def env(self, k: str):
        return os.environ.get(k)


@pytest.fixture(params=["native", "python"])
def job(tmp_path, monkeypatch, request):
    monkeypatch.setenv("MB200_JOBS_DIR", str(tmp_path))
    monkeypatch.setenv("MB200_ALLOCATOR_DAEMON", request.param)
    monkeypatch.setenv("MB200_REMOTE_EXEC", request.param)   # the client-side stub likewise
    if request.param == "native":
        from monarch_b200.tools.process_allocator import native_daemon
        if native_daemon() is None:
            pytest.skip("no compiler for the native daemon")
    j = cli.create("t", hosts=2)
    exe = open(f"/proc/{j['pids'][0]}/cmdline", "rb").read().split(b"\0")[0].decode()
    assert exe.endswith("process_allocator_native") == (request.param == "native"), exe
    yield j
    try:
        cli.stop("t")
    except SystemExit:
        pass


def _children_of(pid):
    out = []
    for d in os.listdir("/proc"):
        if d.isdigit():
            try:
                if int(open(f"/proc/{d}/stat").read().split(")")[1].split()[1]) == pid:
                    out.append(int(d))
            except (OSError, ValueError, IndexError):
                pass
    return out


def test_procs_run_under_the_daemons(job):
    assert cli.info("t")["running"]
    hosts = hosts_from_config("t")
    assert hosts.sizes == {"hosts": 2}
    pm = hosts.spawn_procs(per_host={"gpus": 2})
    assert pm.sizes == {"hosts": 2, "gpus": 2}
    stubs = [open(f"/proc/{c}/cmdline", "rb").read().split(b"\0")[0].decode()
             for c in _children_of(os.getpid())]
    native_stub = any(x.endswith("remote_exec_native") for x in stubs)
    assert native_stub == (os.environ["MB200_REMOTE_EXEC"] == "native"), stubs
    a = pm.spawn("w", Where)
    pids = [v for _, v in a.pid.call().get(timeout=60).items()]
    assert len(set(pids)) == 4 and os.getpid() not in pids
    idx = [v for _, v in a.env.call("MB200_LOCAL_INDEX").get(timeout=30).items()]
    assert idx == ["0", "1", "0", "1"]
    # each proc is a child of a daemon, not of this client
    daemon_pids = set(job["pids"])
    for p in pids:
        ppid = int(open(f"/proc/{p}/stat").read().split(")")[1].split()[1])
        assert ppid in daemon_pids, (p, ppid, daemon_pids)
    pm.stop().get()
    deadline = time.time() + 15
    while time.time() < deadline and any(os.path.exists(f"/proc/{p}") for p in pids):
        time.sleep(0.2)
    assert not any(os.path.exists(f"/proc/{p}") for p in pids)


def test_cli_roundtrip(tmp_path, monkeypatch):
    monkeypatch.setenv("MB200_JOBS_DIR", str(tmp_path))
    env = dict(os.environ, MB200_JOBS_DIR=str(tmp_path))
    run = lambda *a: subprocess.run([sys.executable, "-m", "monarch_b200.tools.cli", *a],
                                    env=env, capture_output=True, text=True, timeout=60)
    r = run("create", "--name", "x", "--hosts", "1")
    assert r.returncode == 0, r.stderr
    assert "x" in run("list").stdout
    assert '"running": true' in run("info", "x").stdout
    assert run("bounce", "x").returncode == 0
    assert run("stop", "x").returncode == 0
    assert "x" not in run("list").stdout


def _ask(port, req):
    import json
    import socket
    c = socket.create_connection(("127.0.0.1", port), timeout=10)
    c.sendall((json.dumps(req) + "\n").encode())
    f = c.makefile("rb")
    for line in f:
        msg = json.loads(line)
        if "exit" in msg or "pid" in msg:
            c.close()
            return msg
    c.close()
    return {}


@pytest.mark.parametrize("daemon", ["native", "python"])
def test_daemon_runs_only_its_own_program_and_checks_the_token(daemon):
    """A client cannot name the program, the working directory or arbitrary environment, and
    with a token configured a request without it is refused."""
    import threading
    from monarch_b200.tools import process_allocator as pa
    prog = [sys.executable, "-c", "import os,sys; print(os.environ.get('MB200_X'), "
            "os.environ.get('LD_PRELOAD'), os.environ.get('MB200_ALLOCATOR_TOKEN')); sys.exit(7)"]
    if daemon == "native":
        cmd = pa.native_command("tcp!127.0.0.1:0", 1.0, prog)
        if cmd is None:
            pytest.skip("no compiler for the native daemon")
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, text=True,
                                env=dict(os.environ, MB200_ALLOCATOR_TOKEN="s3cret"))
        try:
            line = proc.stdout.readline()            # "... listening on tcp!127.0.0.1:PORT"
            port = int(line.rsplit(":", 1)[1])
            _check_daemon_policy(port, pa)
        finally:
            proc.terminate()
            proc.wait(10)
        return
    ports = []
    started = threading.Event()
    threading.Thread(target=pa.serve, args=("tcp!127.0.0.1:0",), daemon=True,
                     kwargs=dict(heartbeat=1.0, ready=lambda p: (ports.append(p), started.set()),
                                 program=prog, token="s3cret")).start()
    assert started.wait(10)
    _check_daemon_policy(ports[0], pa)


def _check_daemon_policy(port, pa):
    assert _ask(port, {"start": 1, "env": {}})["exit"] == 126                 # no token
    assert _ask(port, {"start": 1, "token": "wrong"})["exit"] == 126
    r = _ask(port, {"start": 1, "token": "s3cret", "argv": ["/bin/sh", "-c", "id"]})
    assert r["exit"] == 126 and "own --program" in r["error"]
    assert _ask(port, {"start": 1, "token": "s3cret", "cwd": "/tmp"})["exit"] == 126
    assert _ask(port, {})["exit"] == 126                                        # a port probe
    assert pa.filter_env({"MB200_X": "1", "LD_PRELOAD": "x", "PATH": "y", "HOME": "/",
                          "MB200_ALLOCATOR_TOKEN": "t", "RANK": "3"}) == {"MB200_X": "1",
                                                                          "RANK": "3"}
    # a well-formed request starts the daemon's program with the filtered environment
    import json
    import socket
    c = socket.create_connection(("127.0.0.1", port), timeout=10)
    c.sendall((json.dumps({"start": 1, "token": "s3cret",
                           "env": {"MB200_X": "hello", "LD_PRELOAD": "evil.so"}}) + "\n").encode())
    out, code = "", None
    for line in c.makefile("rb"):
        msg = json.loads(line)
        out += msg.get("out", "")
        if "exit" in msg:
            code = msg["exit"]
            break
    c.close()
    assert code == 7 and out.split() == ["hello", "None", "None"], (code, out)


@pytest.mark.parametrize("daemon", ["native", "python"])
@pytest.mark.parametrize("how", ["close", "silence"])
def test_a_vanished_client_leaves_no_orphan(daemon, how):
    """The proc of a client that closes its connection, or stays connected but goes silent
    for three heartbeat intervals, is killed by the daemon (its whole process group)."""
    import json
    import socket
    import threading
    from monarch_b200.tools import process_allocator as pa
    prog = [sys.executable, "-c", "import time; print('up', flush=True); time.sleep(600)"]
    proc = None
    if daemon == "native":
        cmd = pa.native_command("tcp!127.0.0.1:0", 0.5, prog)
        if cmd is None:
            pytest.skip("no compiler for the native daemon")
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, text=True)
        port = int(proc.stdout.readline().rsplit(":", 1)[1])
    else:
        ports, started = [], threading.Event()
        threading.Thread(target=pa.serve, args=("tcp!127.0.0.1:0",), daemon=True,
                         kwargs=dict(heartbeat=0.5, program=prog, token="",
                                     ready=lambda p: (ports.append(p), started.set()))).start()
        assert started.wait(10)
        port = ports[0]
    try:
        c = socket.create_connection(("127.0.0.1", port), timeout=10)
        c.sendall((json.dumps({"start": 1, "env": {}}) + "\n").encode())
        f = c.makefile("rb")
        pid = None
        for line in f:
            msg = json.loads(line)
            if "pid" in msg:
                pid = msg["pid"]
            if msg.get("out", "").startswith("up"):
                break
        assert pid and os.path.exists(f"/proc/{pid}")
        if how == "close":
            c.close()
        # "silence": the connection stays open and nothing (no heartbeat) is sent any more
        deadline = time.time() + 15
        while time.time() < deadline and os.path.exists(f"/proc/{pid}") and \
                open(f"/proc/{pid}/stat").read().split(")")[1].split()[0] != "Z":
            time.sleep(0.1)
        gone = not os.path.exists(f"/proc/{pid}") or \
            open(f"/proc/{pid}/stat").read().split(")")[1].split()[0] == "Z"
        assert gone, f"proc {pid} outlived its client ({how})"
        if how == "silence":
            c.close()
    finally:
        if proc is not None:
            proc.terminate()
            proc.wait(10)
