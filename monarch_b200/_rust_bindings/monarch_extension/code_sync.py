"""Workspace synchronisation (monarch_hyperactor/src/code_sync; monarch_extension/src/code_sync.rs).
"""
from ...actor.code_sync import AutoReloader, CodeSyncActor, manifest, sync_workspace  # noqa: F401

CodeSyncMeshClient = CodeSyncActor
