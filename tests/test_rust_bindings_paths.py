"""Programs written against the reference import its native extension's submodules by
path (``monarch._rust_bindings.monarch_hyperactor.pytokio`` ...).  The paths resolve here
and name working objects of this runtime."""
import importlib

import pytest

PATHS = {
    "monarch_hyperactor.actor": ["PythonMessage", "PythonMessageKind", "MethodSpecifier", "PanicFlag"],
    "monarch_hyperactor.actor_mesh": ["PythonActorMesh", "ActorSupervisionEvent"],
    "monarch_hyperactor.alloc": ["Alloc", "AllocSpec", "AllocConstraints", "LocalAllocatorBase",
                                 "ProcessAllocatorBase", "SimAllocatorBase", "RemoteAllocatorBase"],
    "monarch_hyperactor.bootstrap": ["bootstrap_main"],
    "monarch_hyperactor.channel": ["ChannelAddr", "ChannelTransport"],
    "monarch_hyperactor.mailbox": ["Mailbox", "PortId", "PortHandle", "PortRef", "PortReceiver",
                                   "OncePortHandle", "OncePortRef", "OncePortReceiver",
                                   "UndeliverableMessageEnvelope"],
    "monarch_hyperactor.proc": ["ActorId", "Proc", "Serialized", "init_proc"],
    "monarch_hyperactor.proc_mesh": ["ProcMesh", "ProcMeshMonitor", "ProcEvent"],
    "monarch_hyperactor.pytokio": ["PythonTask", "Shared", "is_tokio_thread"],
    "monarch_hyperactor.runtime": ["sleep_indefinitely_for_unit_tests"],
    "monarch_hyperactor.selection": ["Selection"],
    "monarch_hyperactor.shape": ["Slice", "Shape", "Extent", "Point"],
    "monarch_hyperactor.supervision": ["SupervisionError"],
    "monarch_hyperactor.telemetry": ["forward_to_tracing", "get_current_span_id", "PySpan",
                                     "use_sim_clock", "use_real_clock", "get_execution_id"],
    "monarch_extension.mesh_controller": ["_Controller"],
    "monarch_extension.tensor_worker": ["Ref", "CallFunction", "Reduce", "SendTensor",
                                        "BorrowCreate", "DefineRecording", "CallRecording"],
    "monarch_extension.client": ["Error", "Failure", "WorkerResponse", "LogMessage", "LogLevel",
                                 "DebuggerMessage", "WorldState"],
    "monarch_extension.controller": ["Node", "Send"],
    "monarch_extension.code_sync": ["CodeSyncMeshClient"],
    "monarch_extension.debugger": ["PdbActor"],
    "monarch_extension.logging": ["LoggingMeshClient"],
    "monarch_extension.simulation_tools": ["sleep", "start_event_loop", "is_simulator_active"],
    "monarch_extension.simulator_client": ["SimulatorClient"],
    "monarch_extension.trace": ["get_or_create_trace_id"],
    "monarch_extension.blocking": ["blocking_function"],
    "monarch_extension.panic": ["panicking_function"],
    "monarch_messages.debugger": ["DebuggerAction"],
    "rdma": ["_RdmaBuffer", "_RdmaManager"],
}


@pytest.mark.parametrize("prefix", ["monarch._rust_bindings", "monarch_b200._rust_bindings"])
def test_every_path_imports_and_has_its_names(prefix):
    for sub, names in PATHS.items():
        mod = importlib.import_module(f"{prefix}.{sub}")
        for n in names:
            assert hasattr(mod, n), f"{prefix}.{sub}.{n}"


def test_the_names_are_the_runtimes_own_objects():
    from monarch._rust_bindings.monarch_hyperactor.proc import ActorId, Serialized
    from monarch._rust_bindings.monarch_hyperactor.pytokio import PythonTask
    from monarch._rust_bindings.monarch_hyperactor.shape import Shape, Slice
    from monarch._rust_bindings.monarch_extension.tensor_worker import CallFunction
    from monarch_b200.actor.shape import Shape as S2
    assert Shape is S2
    assert PythonTask(lambda: 3).block_on() == 3
    a = ActorId.from_string("world[3].trainer[0]")
    assert (a.world_name, a.rank, a.actor_name, a.pid) == ("world", 3, "trainer", 0)
    assert Serialized({"k": [1, 2]}).decode() == {"k": [1, 2]}
    assert Slice.new_row_major([2, 3]).ranks() == list(range(6))
    m = CallFunction(1, [], [], ("op", "aten.add.Tensor"), (), {}, 0)
    assert m[0] == "call" and len(m) == 8
    with pytest.raises(TypeError):
        CallFunction(1, [])
    from monarch._rust_bindings.monarch_extension.panic import panicking_function
    with pytest.raises(Exception):
        panicking_function()
    from monarch._rust_bindings.monarch_extension import simulation_tools as st
    st.start_event_loop()
    assert st.is_simulator_active()
    st.sleep(5.0)
    st.stop()


def test_client_and_controller_value_types():
    from monarch._rust_bindings.monarch_extension.client import Error, Failure, WorkerResponse
    from monarch._rust_bindings.monarch_extension.controller import Node, Send
    from monarch_b200 import _native as N
    from monarch_b200.tensor_engine import RemoteException
    e = Error.from_remote(RemoteException(7, 2, "aten.add", "RuntimeError: boom", "tb", 5))
    assert (e.seq, e.caused_by_seq, e.actor_id) == (7, 5, 2) and "boom" in e.backtrace
    r = WorkerResponse.new_for_unit_test(seq=7, response=e)
    assert r.is_exception() and r.exception() is e and r.result() is None
    assert WorkerResponse(8, 41).result() == 41 and not WorkerResponse(8, 41).is_exception()
    assert isinstance(Failure.new_for_unit_test("w[0]"), type(e).__mro__[1])
    n = Node.from_serialized(Node(seq=3, defs=[10], uses=[1, 2]).serialize())
    h = N.ControllerHistory(1)
    assert n.record(h) == -1 and h.describe(3) == ("node", -1)
    s = Send.from_serialized(Send(ranks=[0, 1], message=("delete", [10])).serialize())
    assert s.ranks == [0, 1] and s.message == ("delete", [10])


def test_top_level_names_of_the_reference():
    import monarch_b200 as m
    assert m.SocketType.TCP.value == "tcp" and m.SocketType.UNIX.value == "unix"
    from monarch_b200.simulator import mock_mesh
    import torch
    mesh, sim = mock_mesh(hosts=1, gpus=1)
    with mesh.activate():
        x = torch.ones(4, 4)
        with m.set_meta("phase-1"):
            y = x + 1
        z = y * 2
    tagged = [e for e in sim.events() if e.get("args", {}).get("meta") == ["phase-1"]]
    assert tagged and len(tagged) < len(sim.events())
