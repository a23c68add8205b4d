"""monarch_b200: a B200-native actor-mesh execution engine for PyTorch.

Sub-packages: ``actor`` (actor meshes, endpoints, supervision), ``ops`` (sm_100a
kernels), ``models``, ``parallel`` (DDP/FSDP/TP/PP/EP over NVLink), ``tensor_engine``
(distributed tensors, RDMABuffer), ``tools`` (allocator daemon, job CLI), ``utils``.

The names a single-controller program needs are also available at the top level, resolved
lazily so that ``import monarch_b200`` stays cheap (same idea as the lazy public API of the
reference's top-level package, python/monarch/__init__.py:74-122):

    from monarch_b200 import DeviceMesh, Tensor, remote, coalescing, fetch_shard, Stream
"""
__version__ = "0.1.0"

_LAZY = {
    # distributed tensors
    "Tensor": ("tensor_engine", "Tensor"), "DeviceMesh": ("tensor_engine", "DeviceMesh"),
    "Stream": ("tensor_engine", "Stream"), "Borrow": ("tensor_engine", "Borrow"),
    "RemoteException": ("tensor_engine", "RemoteException"),
    "RemoteProcessGroup": ("tensor_engine", "RemoteProcessGroup"),
    "function_resolvers": ("tensor_engine", "function_resolvers"),
    "get_active_mesh": ("tensor_engine", "get_active_mesh"),
    "get_active_stream": ("tensor_engine", "get_active_stream"),
    "no_mesh": ("tensor_engine", "no_mesh"), "reduce": ("tensor_engine", "reduce"),
    "reduce_": ("tensor_engine", "reduce_"), "to_mesh": ("tensor_engine", "to_mesh"),
    "slice_mesh": ("tensor_engine", "slice_mesh"), "remote": ("tensor_engine", "remote"),
    "Pipe": ("tensor_engine", "Pipe"), "create_pipe": ("tensor_engine", "create_pipe"),
    "remote_generator": ("tensor_engine", "remote_generator"),
    "coalescing": ("tensor_engine", "coalescing"), "compile": ("tensor_engine", "compile"),
    "call_on_shard_and_fetch": ("tensor_engine", "call_on_shard_and_fetch"),
    "fetch_shard": ("tensor_engine", "fetch_shard"), "inspect": ("tensor_engine", "inspect"),
    "show": ("tensor_engine", "show"), "RDMABuffer": ("tensor_engine", "RDMABuffer"),
    "spawn_tensor_engine": ("tensor_engine", "spawn_tensor_engine"),
    # autograd helpers
    "grad_generator": ("gradient_generator", "grad_generator"),
    "grad_function": ("gradient_generator", "grad_function"),
    # geometry
    "Shape": ("actor.shape", "Shape"), "Point": ("actor.shape", "Point"),
    "Extent": ("actor.shape", "Extent"),
    # meshes and simulation
    "Future": ("actor", "Future"), "ProcMesh": ("actor", "ProcMesh"),
    "local_proc_mesh": ("actor", "local_proc_mesh"), "proc_mesh": ("actor", "proc_mesh"),
    "sim_proc_mesh": ("actor", "sim_proc_mesh"),
    "mock_mesh": ("simulator", "mock_mesh"), "Simulator": ("simulator", "Simulator"),
    "python_local_mesh": ("mesh_constructors", "python_local_mesh"),
    "local_mesh": ("mesh_constructors", "local_mesh"),
    "local_meshes": ("mesh_constructors", "local_meshes"),
    "sim_mesh": ("mesh_constructors", "sim_mesh"),
    "world_mesh": ("mesh_constructors", "world_mesh"),
    "SocketType": ("mesh_constructors", "SocketType"),
    "set_meta": ("simulator", "set_meta"),
    "ControllerRemoteClass": ("remote_class", "ControllerRemoteClass"),
    "WorkerRemoteClass": ("remote_class", "WorkerRemoteClass"),
    "ProcessAllocator": ("actor.allocator", "ProcessAllocator"),
    "LocalAllocator": ("actor.allocator", "LocalAllocator"),
    "SimAllocator": ("actor.allocator", "SimAllocator"),
    "RemoteAllocator": ("actor.allocator", "RemoteAllocator"),
    "AllocSpec": ("actor.allocator", "AllocSpec"),
    "NDSlice": ("actor.shape", "NDSlice"), "Selection": ("_native", "Selection"),
    "ActorFuture": ("actor", "Future"),
    # opaque objects
    "OpaqueRef": ("opaque_object", "OpaqueRef"), "OpaqueObject": ("opaque_object", "OpaqueObject"),
    "OpaqueModule": ("opaque_module", "OpaqueModule"),
}


def __getattr__(name):
    ent = _LAZY.get(name)
    if ent is None:
        if name in ("timer", "profiler", "random", "memory", "tensorboard", "builtins", "telemetry",
                    "remote_class", "mesh_constructors"):
            import importlib
            return importlib.import_module(f"{__name__}.{name}")
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    import importlib
    v = getattr(importlib.import_module(f"{__name__}.{ent[0]}"), ent[1])
    globals()[name] = v
    return v


def __dir__():
    return sorted(list(globals()) + list(_LAZY))
