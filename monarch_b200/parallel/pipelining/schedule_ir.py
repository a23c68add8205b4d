"""Pipeline-schedule IR: per-rank lists of actions, schedule generators, comm insertion,
a dependency-respecting simulator and a chrome-trace dump.

An action is ``(kind, stage, microbatch)`` with kind one of

    F  forward            B  backward (input + weight gradient)
    BI backward, input gradient only      W  weight gradient only   (zero-bubble split)
    SEND_F / RECV_F  activation to / from the next / previous stage
    SEND_B / RECV_B  gradient to / from the previous / next stage

Parity: python/monarch/parallel/pipelining/schedule_ir.py:21-110 (action vocabulary),
:275-445 (schedule construction), :445-626 (comm insertion and simulation), :626-661
(chrome trace) in the reference.  The generators here are written from the published
schedules (GPipe, 1F1B, interleaved 1F1B, ZB-H1), not from that code.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

COMPUTE = ("F", "B", "BI", "W")
COMM = ("SEND_F", "RECV_F", "SEND_B", "RECV_B")


@dataclass(frozen=True)
class Action:
    kind: str
    stage: int
    mb: int

    def __str__(self) -> str:
        return f"{self.stage}{self.kind}{self.mb}"

    @staticmethod
    def parse(s: str) -> "Action":
        i = 0
        while s[i].isdigit():
            i += 1
        j = len(s)
        while s[j - 1].isdigit():
            j -= 1
        return Action(s[i:j], int(s[:i]), int(s[j:]))


Schedule = Dict[int, List[Action]]  # rank -> ordered actions


def stage_to_rank(stage: int, n_ranks: int) -> int:
    """Looped placement: virtual stage s lives on rank s % n_ranks."""
    return stage % n_ranks


# ------------------------------------------------------------------------ generators
def gpipe(n_ranks: int, n_mb: int) -> Schedule:
    return {r: [Action("F", r, m) for m in range(n_mb)] +
               [Action("B", r, m) for m in range(n_mb)] for r in range(n_ranks)}


def one_f_one_b(n_ranks: int, n_mb: int) -> Schedule:
    """Non-interleaved 1F1B: rank r runs min(P-r-1, M) warm-up forwards, then alternates
    one forward with one backward, then drains the remaining backwards."""
    out: Schedule = {}
    for r in range(n_ranks):
        warm = min(n_ranks - r - 1, n_mb)
        acts = [Action("F", r, m) for m in range(warm)]
        f, b = warm, 0
        while f < n_mb:
            acts.append(Action("F", r, f))
            f += 1
            acts.append(Action("B", r, b))
            b += 1
        while b < n_mb:
            acts.append(Action("B", r, b))
            b += 1
        out[r] = acts
    return out


def interleaved_1f1b(n_ranks: int, n_mb: int, n_virtual: int) -> Schedule:
    """Interleaved (looped, depth-first) 1F1B with ``n_virtual`` model chunks per rank;
    micro-batches advance in groups of ``n_ranks``."""
    if n_mb % n_ranks:
        raise ValueError("interleaved 1F1B needs n_mb to be a multiple of the rank count")
    total = n_mb * n_virtual
    out: Schedule = {}
    for r in range(n_ranks):
        def fwd(k):  # k-th forward of this rank -> (stage, mb)
            grp, pos = divmod(k, n_ranks * n_virtual)
            v, i = divmod(pos, n_ranks)
            return v * n_ranks + r, grp * n_ranks + i

        def bwd(k):
            grp, pos = divmod(k, n_ranks * n_virtual)
            v, i = divmod(pos, n_ranks)
            return (n_virtual - 1 - v) * n_ranks + r, grp * n_ranks + i

        warm = min((n_ranks - r - 1) * 2 + (n_virtual - 1) * n_ranks, total)
        acts = [Action("F", *fwd(k)) for k in range(warm)]
        f, b = warm, 0
        while f < total:
            acts.append(Action("F", *fwd(f)))
            f += 1
            acts.append(Action("B", *bwd(b)))
            b += 1
        while b < total:
            acts.append(Action("B", *bwd(b)))
            b += 1
        out[r] = acts
    return out


def zero_bubble_h1(n_ranks: int, n_mb: int) -> Schedule:
    """ZB-H1: 1F1B with the backward split into BI (input gradient, on the critical path)
    and W (weight gradient), the W's filling the drain bubble."""
    out: Schedule = {}
    for r in range(n_ranks):
        warm = min(n_ranks - r - 1, n_mb)
        acts = [Action("F", r, m) for m in range(warm)]
        f, b, w = warm, 0, 0
        while f < n_mb:
            acts.append(Action("F", r, f))
            f += 1
            acts.append(Action("BI", r, b))
            b += 1
            if b - w > r:  # defer up to r weight gradients (they fill this rank's bubble)
                acts.append(Action("W", r, w))
                w += 1
        while b < n_mb:
            acts.append(Action("BI", r, b))
            b += 1
            if w < b and b - w > r:
                acts.append(Action("W", r, w))
                w += 1
        while w < n_mb:
            acts.append(Action("W", r, w))
            w += 1
        out[r] = acts
    return out


GENERATORS = {"gpipe": gpipe, "1f1b": one_f_one_b, "zb-h1": zero_bubble_h1}


# -------------------------------------------------------------------- comm insertion
def add_communication(sched: Schedule, n_stages: int, n_ranks: Optional[int] = None) -> Schedule:
    """Insert SEND/RECV around compute actions whose neighbour stage lives on another
    rank.  Receives are placed directly before the consumer, sends directly after the
    producer."""
    n_ranks = n_ranks or len(sched)
    out: Schedule = {}
    for r, acts in sched.items():
        seq: List[Action] = []
        for a in acts:
            if a.kind == "F":
                if a.stage > 0 and stage_to_rank(a.stage - 1, n_ranks) != r:
                    seq.append(Action("RECV_F", a.stage, a.mb))
                seq.append(a)
                if a.stage < n_stages - 1 and stage_to_rank(a.stage + 1, n_ranks) != r:
                    seq.append(Action("SEND_F", a.stage, a.mb))
            elif a.kind in ("B", "BI"):
                if a.stage < n_stages - 1 and stage_to_rank(a.stage + 1, n_ranks) != r:
                    seq.append(Action("RECV_B", a.stage, a.mb))
                seq.append(a)
                if a.stage > 0 and stage_to_rank(a.stage - 1, n_ranks) != r:
                    seq.append(Action("SEND_B", a.stage, a.mb))
            else:
                seq.append(a)
        out[r] = seq
    return out


# ------------------------------------------------------------------------- validation
def validate(sched: Schedule, n_stages: int, n_mb: int) -> None:
    """Every (stage, mb) is forwarded once and fully backwarded once, forward first."""
    seen_f, seen_b, seen_w = set(), set(), set()
    for r, acts in sched.items():
        for a in acts:
            key = (a.stage, a.mb)
            if a.kind == "F":
                assert key not in seen_f, f"duplicate {a}"
                seen_f.add(key)
            elif a.kind == "B":
                assert key in seen_f and key not in seen_b, f"bad order at {a}"
                seen_b.add(key)
                seen_w.add(key)
            elif a.kind == "BI":
                assert key in seen_f and key not in seen_b, f"bad order at {a}"
                seen_b.add(key)
            elif a.kind == "W":
                assert key in seen_b and key not in seen_w, f"bad order at {a}"
                seen_w.add(key)
    want = {(s, m) for s in range(n_stages) for m in range(n_mb)}
    assert seen_f == want and seen_b == want and seen_w == want, "schedule is incomplete"


# -------------------------------------------------------------------------- simulation
def simulate(sched: Schedule, n_stages: int, cost: Optional[Dict[str, float]] = None,
             comm_latency: float = 0.0) -> Tuple[float, List[dict]]:
    """Earliest-start simulation honouring rank order and cross-stage dependencies.
    Returns (makespan, events); events are dicts with rank, action, start, end."""
    cost = dict({"F": 1.0, "B": 2.0, "BI": 1.0, "W": 1.0}, **(cost or {}))
    n_ranks = len(sched)
    pos = {r: 0 for r in sched}
    clock = {r: 0.0 for r in sched}
    done: Dict[Tuple[str, int, int], float] = {}
    events: List[dict] = []
    remaining = sum(len(a) for a in sched.values())
    while remaining:
        progressed = False
        for r in sched:
            while pos[r] < len(sched[r]):
                a = sched[r][pos[r]]
                if a.kind in COMM:
                    pos[r] += 1
                    remaining -= 1
                    progressed = True
                    continue
                dep = None
                if a.kind == "F" and a.stage > 0:
                    dep = ("F", a.stage - 1, a.mb)
                elif a.kind in ("B", "BI") and a.stage < n_stages - 1:
                    dep = ("B", a.stage + 1, a.mb)
                ready = clock[r]
                if dep is not None:
                    if dep not in done:
                        break
                    remote = stage_to_rank(dep[1], n_ranks) != r
                    ready = max(ready, done[dep] + (comm_latency if remote else 0.0))
                end = ready + cost[a.kind]
                events.append({"rank": r, "action": str(a), "start": ready, "end": end})
                clock[r] = end
                done[("B" if a.kind == "BI" else a.kind, a.stage, a.mb)] = end
                pos[r] += 1
                remaining -= 1
                progressed = True
        if not progressed:
            stuck = {r: str(sched[r][pos[r]]) for r in sched if pos[r] < len(sched[r])}
            raise RuntimeError(f"schedule deadlocks at {stuck}")
    return max(clock.values()), events


def bubble_fraction(sched: Schedule, n_stages: int, **kw) -> float:
    span, events = simulate(sched, n_stages, **kw)
    busy = sum(e["end"] - e["start"] for e in events)
    return 1.0 - busy / (span * len(sched))


def dump_chrome_trace(events: Iterable[dict], path: str, unit_us: float = 1000.0) -> None:
    trace = [{"name": e["action"], "ph": "X", "pid": 0, "tid": e["rank"],
              "ts": e["start"] * unit_us, "dur": (e["end"] - e["start"]) * unit_us}
             for e in events]
    with open(path, "w") as f:
        json.dump({"traceEvents": trace}, f)
