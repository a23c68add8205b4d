"""Proc meshes attached to an SPMD launch: the processes exist already (here: three
``multiprocessing`` children standing in for torchrun ranks), rank 0 is the controller and
every rank hosts one proc of the mesh in-process."""
import os
import socket

import torch.multiprocessing as mp

from monarch_b200.actor import Actor, current_rank, endpoint


class Where(Actor):
    def __init__(self, tag: str):
        self.tag = tag

    @endpoint
    def report(self, x: int):
        # actors of an attached mesh live inside the launcher's processes and see their state
        return (self.tag, current_rank().rank, os.getpid(), os.environ["RANK"], x * 2)


def _rank_main(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from monarch_b200.actor.attach import attach_proc_mesh
    mesh, hosted = attach_proc_mesh({"gpus": world})
    if mesh is None:
        code = hosted.join(timeout=120)
        q.put(("joined", rank, os.getpid(), code))
        return
    assert mesh.sizes == {"gpus": world}
    actors = mesh.spawn("where", Where, "t")
    vm = actors.report.call(21).get(timeout=60)
    got = sorted(v for _, v in vm.items())
    one = actors.slice(gpus=2).report.call_one(5).get(timeout=60)
    mesh.stop().get()
    code = hosted.join(timeout=60)
    q.put(("controller", got, one, os.getpid(), code))


def test_attached_mesh_spans_the_launchers_processes():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    world = 3
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    msgs = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    ctl = next(m for m in msgs if m[0] == "controller")
    joined = {m[1]: m for m in msgs if m[0] == "joined"}
    _, got, one, ctl_pid, ctl_code = ctl
    assert [g[1] for g in got] == [0, 1, 2] and all(g[0] == "t" and g[4] == 42 for g in got)
    # rank r's actor ran inside launcher process r
    pids = {0: ctl_pid, 1: joined[1][2], 2: joined[2][2]}
    for g in got:
        assert g[2] == pids[g[1]] and g[3] == str(g[1]), (g, pids)
    assert one[2] == pids[2] and one[3] == "2" and one[4] == 10
    # the hosts came back from join() with an orderly stop
    assert ctl_code == 0 and joined[1][3] == 0 and joined[2][3] == 0
