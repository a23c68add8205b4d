"""Channels: framing, ordering, ack/redelivery after a dropped connection, undeliverable
returns.  Modelled on hyperactor/src/channel/net.rs tests."""
import os
import threading
import time

import pytest

from monarch_b200 import _native as N


@pytest.mark.parametrize("kind", ["local", "unix", "tcp"])
def test_send_receive_in_order(kind):
    rx = N.channel_serve_any(kind)
    tx = N.channel_dial(rx.addr)
    for i in range(200):
        tx.post(f"m{i}".encode(), [b"x" * i])
    for i in range(200):
        head, parts = rx.recv(5000)
        assert head == f"m{i}".encode() and parts == [b"x" * i]
    assert rx.recv(50) is None
    tx.close()
    rx.close()


def test_address_syntax():
    assert N.parse_channel_addr("tcp:127.0.0.1:1234") == "tcp:127.0.0.1:1234"
    assert N.parse_channel_addr("tcp!localhost:26600") == "tcp:localhost:26600"
    assert N.parse_channel_addr("unix:/tmp/x.sock") == "unix:/tmp/x.sock"
    assert N.parse_channel_addr("local:7") == "local:7"
    with pytest.raises(RuntimeError):
        N.parse_channel_addr("carrier-pigeon:1")


def test_large_multipart_frame():
    rx = N.channel_serve_any("unix")
    tx = N.channel_dial(rx.addr)
    big = os.urandom(8 << 20)
    tx.post(b"head", [big, b"", big[:100]])
    head, parts = rx.recv(10000)
    assert head == b"head" and parts[0] == big and parts[1] == b"" and parts[2] == big[:100]
    tx.close()
    rx.close()


def test_redelivery_after_connection_drop():
    rx = N.channel_serve_any("tcp")
    tx = N.channel_dial(rx.addr)
    got = []
    stop = threading.Event()

    def reader():
        while not stop.is_set():
            m = rx.recv(100)
            if m is not None:
                got.append(int(m[0]))

    t = threading.Thread(target=reader)
    t.start()
    before = N.channel_stats()
    for i in range(300):
        tx.post(str(i).encode())
        if i in (50, 150):
            # the accepting side must have the connection before it can be dropped
            wait_until = time.time() + 10
            while not got and time.time() < wait_until:
                time.sleep(0.005)
            N.channel_debug_drop_connections(rx.addr)
    deadline = time.time() + 10
    while len(got) < 300 and time.time() < deadline:
        time.sleep(0.01)
    stop.set()
    t.join()
    assert got == list(range(300)), "messages must arrive exactly once, in order"
    after = N.channel_stats()
    assert after["reconnects"] > before["reconnects"]
    tx.close()
    rx.close()


def test_undeliverable_when_nobody_listens():
    N.config_set("MESSAGE_DELIVERY_TIMEOUT_MS", "300")
    try:
        tx = N.channel_dial("unix:@mb200_nobody_home_%d" % os.getpid())
        lost = []
        ev = threading.Event()

        def on_fail(head):
            lost.append(head)
            ev.set()

        tx.post(b"hello?", [], on_fail)
        assert ev.wait(5), "the undeliverable callback must fire after the delivery timeout"
        assert lost == [b"hello?"] and tx.is_closed()
        tx.close()
    finally:
        N.config_unset("MESSAGE_DELIVERY_TIMEOUT_MS")


def test_local_channel_closed_is_undeliverable():
    rx = N.channel_serve_any("local")
    tx = N.channel_dial(rx.addr)
    rx.close()
    lost = []
    tx.post(b"x", [], lost.append)
    assert lost == [b"x"]
