"""Distributed tensors and one-sided buffers.

Parity: python/monarch/tensor_engine/__init__.py (RDMABuffer, is_available)."""
from .rdma import RDMABuffer, RDMAError, is_available

__all__ = ["RDMABuffer", "RDMAError", "is_available"]

from .device_mesh import (Borrow, BorrowError, DeviceMesh, RemoteException, Stream, Tensor,  # noqa: E402
                          WorkerTimeoutError, RemoteProcessGroup,
                          get_active_mesh, get_active_stream, no_mesh, reduce, reduce_,
                          slice_mesh, spawn_tensor_engine, to_mesh)
from .remote import (Remote, call_on_shard_and_fetch, coalescing, compile, fetch_shard,  # noqa: E402
                     inspect, remote, show, function_resolvers)

__all__ += ["BorrowError", "WorkerTimeoutError", "RemoteProcessGroup", "Borrow", "DeviceMesh", "RemoteException", "Stream", "Tensor", "get_active_mesh",
            "get_active_stream", "no_mesh", "reduce", "reduce_", "slice_mesh",
            "spawn_tensor_engine", "to_mesh", "Remote", "call_on_shard_and_fetch", "coalescing",
            "compile", "fetch_shard", "inspect", "remote", "show", "function_resolvers"]

from .pipe import Pipe, create_pipe, remote_generator  # noqa: E402

__all__ += ["Pipe", "create_pipe", "remote_generator"]
