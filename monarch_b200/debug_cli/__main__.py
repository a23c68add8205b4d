"""Interactive console over a DebugController (same process as the client program, e.g.
started from a notebook cell or a signal handler with ``run_console(debug_controller())``).

Commands:  list | attach <actor> <rank> | cast <actor> <rank,rank|*> <pdb command> |
           continue | quit.   While attached, every line is a pdb command ("detach" leaves).

Parity: python/monarch/_src/debug_cli/debug_cli.py and the controller commands of
python/monarch/_src/actor/debugger/debugger.py.
"""
import sys
import time


def run_console(ctrl, stdin=sys.stdin, stdout=sys.stdout) -> None:
    def p(*a):
        print(*a, file=stdout, flush=True)

    attached = None
    while True:
        stdout.write("(attached) " if attached else "mb200_dbg> ")
        stdout.flush()
        line = stdin.readline()
        if not line:
            return
        line = line.strip()
        if attached:
            if line == "detach":
                attached = None
                continue
            ctrl.send.call_one(attached[0], attached[1], line).get()
            time.sleep(0.2)
            p(ctrl.read.call_one(attached[0], attached[1]).get(), end="")
            if line in ("c", "continue", "q", "quit"):
                attached = None
            continue
        if line == "list":
            for s in ctrl.list.call_one().get():
                p(f"{s['actor']}[{s['rank']}] pid {s['pid']}@{s['host']} "
                  f"{'parked' if s['active'] else 'done'} at {s['where']}")
        elif line.startswith("attach "):
            _, a, r = line.split()
            attached = (a, int(r))
            p(ctrl.read.call_one(a, int(r), False).get(), end="")
        elif line.startswith("cast "):
            _, a, ranks, cmd = line.split(" ", 3)
            rs = None if ranks == "*" else [int(x) for x in ranks.split(",")]
            p(f"sent to {ctrl.cast.call_one(a, rs, cmd).get()} sessions")
        elif line == "continue":
            for s in ctrl.list.call_one().get():
                if s["active"]:
                    ctrl.send.call_one(s["actor"], s["rank"], "c").get()
        elif line in ("quit", "exit"):
            return
        elif line:
            p("commands: list | attach <actor> <rank> | cast <actor> <ranks|*> <cmd> | "
              "continue | quit")


if __name__ == "__main__":
    from monarch_b200.actor import debug_controller
    run_console(debug_controller())
