"""Actor meshes (monarch_hyperactor/src/actor_mesh.rs:60-280).
"""
from ...actor.actor_mesh import ActorMesh as PythonActorMesh  # noqa: F401
from ...actor.actor_mesh import ActorMesh as PythonActorMeshImpl  # noqa: F401
from ...actor.proc_mesh import ProcEvent as ActorSupervisionEvent  # noqa: F401
