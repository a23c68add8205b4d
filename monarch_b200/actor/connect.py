"""Duplex byte streams between actors, carried by actor messages.

One side listens (``listen()`` gives a picklable :class:`Port` to hand out and a
:class:`ConnectionListener`), the other connects to that port; both ends then hold an
:class:`ActorConnection` with ``write`` / ``read`` / ``readexactly`` / ``close`` -- a pipe
that works wherever actor messages do (across procs and hosts, through the same channels,
ordered and reliable), for protocols that want a stream rather than messages: file
synchronisation, log shipping, a debugger's terminal.

Data travels as out-of-band frame parts (no pickling of the payload).  Flow control is a
byte window: a writer blocks once ``window`` bytes are unacknowledged, the reader
acknowledges what the application has consumed.

Parity: hyperactor_mesh/src/connect.rs (``ActorConnection`` as AsyncRead + AsyncWrite over
ports, ``Connect`` / accept handshake, EOF by closing the write half).
"""
from __future__ import annotations

import collections
import itertools
import threading
import time
from typing import Deque, Optional, Tuple

from .actor_mesh import Channel, Port, PortReceiver

_ids = itertools.count(1)
DEFAULT_WINDOW = 32 << 20
MAX_FRAME = 4 << 20


class ConnectionClosed(EOFError):
    pass


class ActorConnection:
    """One end of a duplex stream.  Thread-safe for one reader and one writer."""

    def __init__(self, tx: Port, rx: PortReceiver, window: int = DEFAULT_WINDOW):
        self._tx, self._rx = tx, rx
        self._window = window
        self._buf: Deque[bytes] = collections.deque()
        self._buffered = 0
        self._eof = False
        self._closed = False
        self._sent = 0            # bytes written
        self._acked = 0           # bytes the peer says it consumed
        self._consumed = 0        # bytes handed to our application
        self._ack_sent = 0
        self._lock = threading.Lock()       # serialises pumping the receive port

    # --------------------------------------------------------------------- receiving
    def _pump(self, timeout: Optional[float]) -> bool:
        """Take one message off the port (data, ack or eof).  False on timeout."""
        with self._lock:
            try:
                _, msg = self._rx._next(timeout)
            except TimeoutError:
                return False
            kind = msg[0]
            if kind == "data":
                self._buf.append(bytes(msg[1]))
                self._buffered += len(msg[1])
            elif kind == "ack":
                self._acked = max(self._acked, msg[1])
            elif kind == "eof":
                self._eof = True
            return True

    def _maybe_ack(self) -> None:
        if self._consumed - self._ack_sent >= max(1, self._window // 4) or \
                (self._buffered == 0 and self._consumed > self._ack_sent):
            self._ack_sent = self._consumed
            try:
                self._tx.send(("ack", self._consumed))
            except Exception:  # noqa: BLE001 - the peer is gone; reads still drain the buffer
                pass

    def read(self, n: int = -1, timeout: Optional[float] = None) -> bytes:
        """Up to ``n`` bytes (all that is buffered if ``n`` < 0); blocks until at least one
        byte is available; ``b""`` at end of stream."""
        deadline = None if timeout is None else time.monotonic() + timeout
        while self._buffered == 0 and not self._eof:
            left = None if deadline is None else max(deadline - time.monotonic(), 0.0)
            if not self._pump(left) and deadline is not None and time.monotonic() >= deadline:
                raise TimeoutError("no data on the connection")
        out = bytearray()
        while self._buf and (n < 0 or len(out) < n):
            head = self._buf[0]
            take = len(head) if n < 0 else min(len(head), n - len(out))
            out += head[:take]
            if take == len(head):
                self._buf.popleft()
            else:
                self._buf[0] = head[take:]
            self._buffered -= take
        self._consumed += len(out)
        self._maybe_ack()
        return bytes(out)

    def readexactly(self, n: int, timeout: Optional[float] = None) -> bytes:
        deadline = None if timeout is None else time.monotonic() + timeout
        out = bytearray()
        while len(out) < n:
            left = None if deadline is None else max(deadline - time.monotonic(), 0.0)
            chunk = self.read(n - len(out), left)
            if not chunk:
                raise ConnectionClosed(f"stream ended after {len(out)} of {n} bytes")
            out += chunk
        return bytes(out)

    # ----------------------------------------------------------------------- sending
    def write(self, data, timeout: Optional[float] = None) -> int:
        """Send all of ``data`` (bytes-like); blocks while the window is full."""
        if self._closed:
            raise ConnectionClosed("write on a closed connection")
        mv = memoryview(data).cast("B")
        deadline = None if timeout is None else time.monotonic() + timeout
        pos = 0
        while pos < len(mv):
            while self._sent - self._acked >= self._window:
                left = None if deadline is None else max(deadline - time.monotonic(), 0.0)
                if not self._pump(left if left is not None else 0.25) and deadline is not None \
                        and time.monotonic() >= deadline:
                    raise TimeoutError("the peer does not drain the connection")
                if self._eof and self._sent - self._acked >= self._window:
                    raise ConnectionClosed("the peer closed the connection")
            n = min(MAX_FRAME, len(mv) - pos)
            self._tx.send(("data", bytes(mv[pos: pos + n])))
            pos += n
            self._sent += n
        return pos

    def close(self) -> None:
        """Close the write half (the peer reads EOF after the data) and stop reading."""
        if self._closed:
            return
        self._closed = True
        try:
            self._tx.send(("eof",))
        except Exception:  # noqa: BLE001
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()
        return False


class ConnectionListener:
    def __init__(self, rx: PortReceiver):
        self._rx = rx

    def accept(self, timeout: Optional[float] = None) -> ActorConnection:
        """Wait for a ``connect`` and complete the handshake."""
        _, msg = self._rx._next(timeout)
        assert msg[0] == "connect", msg
        _, peer_port, window = msg
        my_port, my_rx = Channel.open()
        peer_port.send(("accept", my_port))
        return ActorConnection(peer_port, my_rx, window)

    def close(self) -> None:
        self._rx.close()


def listen() -> Tuple[Port, ConnectionListener]:
    """A port to hand to peers (it is picklable: return it from an endpoint, put it in a
    message) and the listener that accepts their connections."""
    port, rx = Channel.open()
    return port, ConnectionListener(rx)


def connect(dest: Port, timeout: Optional[float] = 30.0,
            window: int = DEFAULT_WINDOW) -> ActorConnection:
    """Open a stream to whoever listens on ``dest``."""
    my_port, my_rx = Channel.open()
    dest.send(("connect", my_port, window))
    _, msg = my_rx._next(timeout)
    assert msg[0] == "accept", msg
    return ActorConnection(msg[1], my_rx, window)
