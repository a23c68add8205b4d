"""Proc meshes (monarch_hyperactor/src/proc_mesh.rs:55-513).
"""
from ...actor.proc_mesh import ProcEvent, ProcMesh  # noqa: F401


class ProcMeshMonitor:
    """Async iterator over a proc mesh's lifecycle events (``ProcMesh.monitor()``)."""

    def __init__(self, mesh: ProcMesh):
        self._it = mesh.monitor()

    def __aiter__(self):
        return self

    async def __anext__(self) -> ProcEvent:
        from ...actor.future import Future
        return await Future(lambda timeout: next(self._it))
