"""Messages of the (legacy) controller actor: a node of the invocation graph and a send of a
worker message to ranks (monarch_extension/src/controller.rs).

This runtime keeps the invocation graph in ``_native.ControllerHistory`` (``add_invocation``
takes the same seq / defs / uses triple) and sends worker messages by casting to the worker
actor mesh; ``Node`` and ``Send`` are the value forms of the two.
"""
from __future__ import annotations

import pickle
from typing import Any, List, Sequence


class Node:
    """Invocation ``seq`` defines the refs ``defs`` and reads the refs ``uses``."""

    def __init__(self, *, seq: int, defs: Sequence[Any], uses: Sequence[Any]):
        self.seq, self.defs, self.uses = seq, list(defs), list(uses)

    def serialize(self) -> bytes:
        return pickle.dumps(("node", self.seq, self.defs, self.uses))

    @staticmethod
    def from_serialized(serialized: bytes) -> "Node":
        tag, seq, defs, uses = pickle.loads(serialized)
        if tag != "node":
            raise ValueError("not a serialized Node")
        return Node(seq=seq, defs=defs, uses=uses)

    def record(self, history, name: str = "node") -> int:
        """Enter the node into a ``ControllerHistory``."""
        ids = lambda refs: [getattr(r, "id", r) for r in refs]
        return history.add_invocation(self.seq, name, ids(self.defs), ids(self.uses))


class Send:
    """Worker message ``message`` for the ranks in ``ranks`` (slices of the world)."""

    def __init__(self, *, ranks: List[Any], message: Any):
        self.ranks, self.message = list(ranks), message

    def serialize(self) -> bytes:
        return pickle.dumps(("send", self.ranks, self.message))

    @staticmethod
    def from_serialized(serialized: bytes) -> "Send":
        tag, ranks, message = pickle.loads(serialized)
        if tag != "send":
            raise ValueError("not a serialized Send")
        return Send(ranks=ranks, message=message)
