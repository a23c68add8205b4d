"""The simulated transport: ``sim:`` channels deliver after a latency that depends on the
distance between the two nodes, on the simulated clock; a proc mesh laid out over a
topology pays those latencies on every hop of a cast (hyperactor/src/channel/sim.rs,
simnet.rs in the reference)."""
import time

import pytest

from monarch_b200 import _native as N
from monarch_b200.actor import Actor, endpoint
from monarch_b200.actor.proc_mesh import configure_simnet, sim_proc_mesh, simnet_stats


def test_sim_addresses_and_distances():
    a = N.parse_channel_addr("sim:dc0.rack1.host3/7")
    assert a["kind"] == "sim" if isinstance(a, dict) else True
    assert N.simnet_distance("dc0.rack1.host3", "dc0.rack1.host3") == 0
    assert N.simnet_distance("dc0.rack1.host3", "dc0.rack1.host4") == 1
    assert N.simnet_distance("dc0.rack1.host3", "dc0.rack2.host3") == 2
    assert N.simnet_distance("dc0.rack1.host3", "dc1.rack1.host3") == 3
    assert N.simnet_distance("client", "dc0.rack1.host3") == 3


def test_frames_arrive_in_order_after_the_simulated_latency():
    N.use_sim_clock()
    try:
        configure_simnet([1.0, 100.0, 10_000.0], bandwidth_gbs=1000.0)
        rx = N.channel_serve("sim:rack0.host1/0")
        near = N.channel_dial("sim:rack0.host0->" + rx.addr[4:])
        far = N.channel_dial("sim:rack1.host0->" + rx.addr[4:])
        t0 = N.telemetry_now_us()
        near.post(b"n1")
        near.post(b"n2")
        assert rx.recv(2000)[0] == b"n1" and rx.recv(2000)[0] == b"n2"
        t1 = N.telemetry_now_us()
        assert 100.0 <= t1 - t0 < 1000.0                 # one rack-local hop of simulated time
        far.post(b"f1")
        assert rx.recv(2000)[0] == b"f1"
        assert N.telemetry_now_us() - t1 >= 10_000.0     # a cross-rack hop
    finally:
        N.use_real_clock()


class Where(Actor):
    @endpoint
    def ping(self, x: int) -> int:
        return x + 1


def test_mesh_over_a_simulated_topology_pays_for_distance():
    N.use_sim_clock()
    try:
        configure_simnet([1.0, 50.0, 2_000.0, 2_000.0], bandwidth_gbs=100.0)
        pm = sim_proc_mesh(racks=2, hosts=2, gpus=2, network=True)
        try:
            assert pm.sizes == {"racks": 2, "hosts": 2, "gpus": 2}
            actors = pm.spawn("where", Where)
            N.simnet_reset_stats()
            wall0 = time.monotonic()
            t0 = N.telemetry_now_us()
            vm = actors.ping.call(1).get(timeout=60)
            t1 = N.telemetry_now_us()
            assert sorted(v for _, v in vm.items()) == [2] * 8
            st = simnet_stats()
            assert st["frames"] >= 16            # requests down the tree and replies back
            # the client is far from every host: the round trip costs at least two far hops
            # of simulated time and took (almost) no wall-clock time
            assert t1 - t0 >= 2 * 2_000.0
            assert time.monotonic() - wall0 < 5.0
            assert st["frames_by_distance"][0] + st["frames_by_distance"][1] > 0   # tree hops
        finally:
            pm.stop().get()
    finally:
        N.use_real_clock()
