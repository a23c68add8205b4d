"""Write-ahead message log + durable sender, checkpoint files, and the preemptible
reader/writer lock (hyperactor's DurableMailboxSender / Checkpointable / preempt_rwlock)."""
import os
import threading
import time

from monarch_b200 import _native as N
from monarch_b200.actor import context


def _client_port():
    inst = context().actor_instance._native
    port_id, rx = inst.open_port(False)
    return inst, port_id, rx


def test_durable_sender_logs_before_forwarding_and_replays(tmp_path):
    inst, port_id, rx = _client_port()
    me = inst.actor_id
    path = str(tmp_path / "wal.log")
    log = N.MessageLog(path)
    d = N.DurableSender(log, N.client_proc())
    for i in range(3):
        d.post(me, port_id, b"m%d" % i, {"k": str(i)}, [b"part%d" % i])
    got = [rx.recv(2000) for _ in range(3)]
    assert [bytes(e.data) for e in got] == [b"m0", b"m1", b"m2"]
    assert got[1].headers["k"] == "1" and bytes(got[2].parts[0]) == b"part2"
    assert log.next_seq == 3
    recs = log.read(1)
    assert [s for s, _ in recs] == [1, 2] and bytes(recs[0][1].data) == b"m1"

    # a receiver that lost its state asks for everything from seq 1 again
    assert d.replay(1) == 2
    assert [bytes(rx.recv(2000).data) for _ in range(2)] == [b"m1", b"m2"]

    # reopening continues the sequence; a torn tail is cut off
    del d, log
    with open(path, "ab") as f:
        f.write(b"\x07\x00\x00\x00\x00\x00\x00\x00\x10\x00")      # half a record
    log2 = N.MessageLog(path)
    assert log2.next_seq == 3 and len(log2.read()) == 3
    log2.append(me, port_id, b"m3")
    log2.flush()
    assert [s for s, _ in N.MessageLog(path).read(3)] == [3]
    inst.close_port(port_id)


def test_checkpoint_files_are_replaced_atomically(tmp_path):
    p = str(tmp_path / "actor.ckpt")
    assert N.read_checkpoint(p) is None
    N.write_checkpoint(p, b"state-1")
    N.write_checkpoint(p, b"state-2" * 1000)
    assert N.read_checkpoint(p) == b"state-2" * 1000
    assert os.listdir(tmp_path) == ["actor.ckpt"]          # no temp files left behind


def test_readers_see_a_waiting_writer():
    lock = N.PreemptibleRwLock()
    r1 = lock.read_acquire()
    r2 = lock.read_acquire()
    assert lock.readers == 2 and not lock.preempted(r1)
    order = []

    def writer():
        lock.write_acquire()
        order.append("writer in")
        time.sleep(0.05)
        lock.write_release()

    t = threading.Thread(target=writer)
    t.start()
    deadline = time.time() + 5
    while not lock.preempted(r1) and time.time() < deadline:
        time.sleep(0.005)
    assert lock.preempted(r1) and lock.preempted(r2) and lock.writers_waiting == 1
    assert lock.read_acquire(20) is None        # new readers queue behind the writer
    assert order == []                          # the writer waits for the readers
    lock.read_release(r1)
    lock.read_release(r2)
    t.join(5)
    assert order == ["writer in"]
    r3 = lock.read_acquire(1000)
    assert r3 is not None and not lock.preempted(r3)
    lock.read_release(r3)
