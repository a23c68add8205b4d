"""Procs and actor ids (monarch_hyperactor/src/proc.rs).
"""
from ..._native import Proc, client_proc, parse_actor_id  # noqa: F401


class ActorId:
    """``world[rank].name[pid]``."""

    def __init__(self, text: str):
        self.text = text
        self.world_name, self.rank, self.actor_name, self.pid = parse_actor_id(text)

    @staticmethod
    def from_string(text: str) -> "ActorId":
        return ActorId(text)

    def __str__(self) -> str:
        return self.text


class Serialized:
    """A pickled payload with its out-of-band parts (actor/pickle.py)."""

    def __init__(self, obj=None, *, data: bytes = b"", parts=None):
        from ...actor.pickle import flatten
        if obj is not None:
            data, parts = flatten(obj)
        self.data, self.parts = data, list(parts or [])

    def decode(self):
        from ...actor.pickle import unflatten
        return unflatten(self.data, self.parts)


def init_proc(*, proc_id: str = "", **_ignored):
    """The calling process's client proc (a proc per process is created lazily)."""
    return client_proc()
