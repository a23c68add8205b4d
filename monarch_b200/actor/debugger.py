"""Distributed pdb: actors that hit ``breakpoint()`` (or ``remote_breakpoint()``) park in
a pdb session whose input and output travel through a singleton ``DebugController`` actor;
a user attaches to any session from the client or from ``python -m monarch_b200.debug_cli``.

Parity: python/monarch/_src/actor/debugger/debugger.py:520-737 (``DebugController``:
session registry, ``list``/``attach``/``cast`` commands), pdb_wrapper.py:44-181
(``PdbWrapper``: pdb with its stdin/stdout replaced by message queues), bootstrap_main.py:
``sys.breakpointhook``; monarch_messages/src/debugger.rs (the actions).

The controller never blocks: sessions poll it for input (one small message per 50 ms while
parked), and output is pushed to it line by line.
"""
from __future__ import annotations

import os
import pdb
import sys
import threading
import time
from typing import Dict, List, Optional, Tuple

from .actor_mesh import Actor, context, endpoint

_POLL_S = 0.05


class DebugController(Actor):
    """Registry of parked sessions: (actor name, rank) -> input queue + output log."""

    def __init__(self):
        self.sessions: Dict[Tuple[str, int], dict] = {}

    @endpoint
    def register(self, actor: str, rank: int, where: str, pid: int, host: str) -> None:
        self.sessions[(actor, rank)] = {"where": where, "pid": pid, "host": host, "in": [],
                                        "out": [], "active": True}

    @endpoint
    def finish(self, actor: str, rank: int) -> None:
        s = self.sessions.get((actor, rank))
        if s:
            s["active"] = False

    @endpoint
    def output(self, actor: str, rank: int, text: str) -> None:
        s = self.sessions.get((actor, rank))
        if s is not None:
            s["out"].append(text)

    @endpoint
    def next_input(self, actor: str, rank: int) -> Optional[str]:
        s = self.sessions.get((actor, rank))
        if s and s["in"]:
            return s["in"].pop(0)
        return None

    # ---- user side
    @endpoint
    def list(self) -> List[dict]:
        return [{"actor": a, "rank": r, "where": s["where"], "pid": s["pid"], "host": s["host"],
                 "active": s["active"]} for (a, r), s in sorted(self.sessions.items())]

    @endpoint
    def send(self, actor: str, rank: int, line: str) -> bool:
        s = self.sessions.get((actor, rank))
        if not s or not s["active"]:
            return False
        s["in"].append(line)
        return True

    @endpoint
    def cast(self, actor: str, ranks: Optional[List[int]], line: str) -> int:
        """Send one pdb command to several sessions of an actor mesh (all when ``ranks`` is
        None); returns how many received it."""
        n = 0
        for (a, r), s in self.sessions.items():
            if a == actor and s["active"] and (ranks is None or r in ranks):
                s["in"].append(line)
                n += 1
        return n

    @endpoint
    def read(self, actor: str, rank: int, clear: bool = True) -> str:
        s = self.sessions.get((actor, rank))
        if not s:
            return ""
        text = "".join(s["out"])
        if clear:
            s["out"].clear()
        return text


def debug_controller():
    """The singleton debug controller (spawned on first use)."""
    from .proc_mesh import get_or_spawn_controller
    return get_or_spawn_controller("debug_controller", DebugController).get()


class _Out:
    def __init__(self, push):
        self._push = push

    def write(self, s: str) -> int:
        if s:
            self._push(s)
        return len(s)

    def flush(self) -> None:
        pass


class _In:
    def __init__(self, pull):
        self._pull = pull

    def readline(self) -> str:
        while True:
            line = self._pull()
            if line is not None:
                return line if line.endswith("\n") else line + "\n"
            time.sleep(_POLL_S)


class PdbWrapper(pdb.Pdb):
    """pdb whose console is the debug controller."""

    def __init__(self, ctrl, actor: str, rank: int):
        self._ctrl, self._actor, self._rank = ctrl, actor, rank
        super().__init__(stdin=_In(self._pull), stdout=_Out(self._push), readrc=False)
        self.use_rawinput = False
        self.prompt = "(mb200-pdb) "

    def _push(self, text: str) -> None:
        self._ctrl.output.call_one(self._actor, self._rank, text).get()

    def _pull(self) -> Optional[str]:
        return self._ctrl.next_input.call_one(self._actor, self._rank).get()

    def set_trace(self, frame=None):
        import socket
        frame = frame or sys._getframe().f_back
        where = f"{frame.f_code.co_filename}:{frame.f_lineno} in {frame.f_code.co_name}"
        self._ctrl.register.call_one(self._actor, self._rank, where, os.getpid(),
                                     socket.gethostname()).get()
        super().set_trace(frame)

    def set_continue(self):
        super().set_continue()
        self._done()

    def set_quit(self):
        super().set_quit()
        self._done()

    def _done(self):
        try:
            self._ctrl.finish.call_one(self._actor, self._rank).get()
        except Exception:  # noqa: BLE001 - the controller may already be gone
            pass


def remote_breakpoint() -> None:
    """Park the calling actor endpoint in a remote pdb session at the caller's frame."""
    try:
        ctx = context()
        name = ctx.actor_instance.actor_id.split(".")[-1].split("[")[0]
        rank = int(ctx.message_rank.rank) if hasattr(ctx.message_rank, "rank") else 0
    except Exception:  # noqa: BLE001 - outside an actor: plain pdb
        pdb.Pdb().set_trace(sys._getframe().f_back)
        return
    PdbWrapper(debug_controller(), name, rank).set_trace(sys._getframe().f_back)


def install_breakpoint_hook() -> None:
    """Make the builtin ``breakpoint()`` open a remote session inside actors."""
    def hook(*a, **k):
        frame = sys._getframe().f_back
        try:
            ctx = context()
            name = ctx.actor_instance.actor_id.split(".")[-1].split("[")[0]
            rank = int(getattr(ctx.message_rank, "rank", 0))
            PdbWrapper(debug_controller(), name, rank).set_trace(frame)
        except Exception:  # noqa: BLE001
            pdb.Pdb().set_trace(frame)
    sys.breakpointhook = hook
