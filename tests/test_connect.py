"""Duplex byte streams between actors (hyperactor_mesh/src/connect.rs in the reference): a
stream opened from the client to an actor in another process, large transfers under the flow
control window, EOF, and a file-sync protocol running over it."""
import hashlib
import os

import pytest

from monarch_b200.actor import Actor, endpoint, this_host
from monarch_b200.actor.connect import ConnectionClosed, connect, listen


class Echo(Actor):
    @endpoint
    def open(self):
        self.port, self.listener = listen()
        return self.port

    @endpoint
    def serve_upper(self) -> int:
        """Accept one connection; send back everything upper-cased until EOF."""
        conn = self.listener.accept(timeout=30)
        total = 0
        while True:
            chunk = conn.read(1 << 20, timeout=30)
            if not chunk:
                break
            total += len(chunk)
            conn.write(chunk.upper())
        conn.close()
        return total

    @endpoint
    def serve_digest(self) -> str:
        """Accept one connection; read to EOF without answering, then send the digest."""
        conn = self.listener.accept(timeout=30)
        h = hashlib.sha256()
        while True:
            chunk = conn.read(-1, timeout=60)
            if not chunk:
                break
            h.update(chunk)
        conn.write(h.hexdigest().encode())
        conn.close()
        return h.hexdigest()


@pytest.fixture(scope="module")
def echo():
    pm = this_host().spawn_procs(per_host={"gpus": 1})
    yield pm.spawn("echo", Echo)
    pm.stop().get()


def test_stream_round_trip_and_eof(echo):
    port = echo.open.call_one().get(timeout=30)
    served = echo.serve_upper.call_one()
    conn = connect(port)
    msgs = [b"hello ", b"actor ", b"streams", os.urandom(3 << 20).hex().encode()]
    for m in msgs:
        conn.write(m)
        assert conn.readexactly(len(m), timeout=30) == m.upper()
    conn.close()
    assert conn.read(timeout=30) == b""                      # the peer closed after our EOF
    assert served.get(timeout=30) == sum(len(m) for m in msgs)
    with pytest.raises(ConnectionClosed):
        conn.write(b"late")


def test_one_way_bulk_transfer_respects_the_window(echo):
    port = echo.open.call_one().get(timeout=30)
    served = echo.serve_digest.call_one()
    conn = connect(port, window=1 << 20)                     # far smaller than the payload
    data = os.urandom(24 << 20)
    conn.write(data, timeout=60)
    assert conn._sent == len(data) and conn._sent - conn._acked <= (1 << 20) + (4 << 20)
    conn.close()
    want = hashlib.sha256(data).hexdigest()
    assert conn.readexactly(64, timeout=60).decode() == want
    assert served.get(timeout=60) == want
