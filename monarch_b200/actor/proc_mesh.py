"""Proc meshes, hosts and named controllers.

Parity: python/monarch/_src/actor/proc_mesh.py (ProcMesh.spawn / stop / monitor /
activate / rank_tensor(s) / logging_option / sync_workspace, proc_mesh(),
local_proc_mesh(), sim_proc_mesh(), get_or_spawn_controller), host_mesh.py (HostMesh,
this_host, this_proc, fake_in_process_host, hosts_from_config), allocator.py
(LocalAllocator / ProcessAllocator wrappers), hyperactor_mesh/src/proc_mesh.rs.
"""
from __future__ import annotations

import atexit
import itertools
import os
import sys
import threading
import warnings
import weakref
from typing import Any, Callable, Dict, List, Optional, Type, TypeVar

from .. import _native as N
from .actor_mesh import (Actor, ActorMesh, SupervisionError, _Health, context, endpoint)
from .future import Future
from .pickle import flatten
from .shape import MeshTrait, Shape

T = TypeVar("T")
_world_counter = itertools.count()
_live_meshes: "weakref.WeakSet[ProcMesh]" = weakref.WeakSet()


class ProcEvent:
    """A crash delivered by ``ProcMesh.monitor()``."""

    def __init__(self, kind: str, rank: int, actor_id: str, message: str):
        self.kind, self.rank, self.actor_id, self.message = kind, rank, actor_id, message

    def __repr__(self) -> str:
        return f"ProcEvent({self.kind}, rank={self.rank}, actor={self.actor_id!r}, {self.message!r})"


class LogAggregator:
    """Collapses similar log lines from many procs within a time window into one line
    prefixed ``[N similar log lines]`` (digits are normalised before comparing)."""

    def __init__(self, window_sec: float = 5.0, out=None):
        import re
        self._re = re.compile(r"\d+")
        self.window = window_sec
        self.out = out or sys.stdout
        self._lock = threading.Lock()
        self._groups: Dict[str, List] = {}
        self._t0 = None
        self._timer: Optional[threading.Timer] = None

    def add(self, rank: int, is_err: bool, line: str) -> None:
        import time
        key = self._re.sub("#", line)
        with self._lock:
            now = time.monotonic()
            if self._t0 is None:
                self._t0 = now
            g = self._groups.setdefault(key, [0, line])
            g[0] += 1
            if now - self._t0 >= self.window:
                self._flush_locked()
            elif self._timer is None:
                # the window closes on time even if no further line arrives
                self._timer = threading.Timer(self.window - (now - self._t0), self.flush)
                self._timer.daemon = True
                self._timer.start()

    def _flush_locked(self) -> None:
        for count, line in self._groups.values():
            prefix = f"[{count} similar log lines] " if count > 1 else ""
            print(prefix + line, file=self.out)
        self._groups.clear()
        self._t0 = None
        if self._timer is not None:
            self._timer.cancel()
            self._timer = None

    def flush(self) -> None:
        with self._lock:
            self._flush_locked()


class ProcMesh(MeshTrait):
    """A mesh of OS processes (or in-process procs) on which actors are spawned."""

    def __init__(self, native: "N.ProcMesh", shape: Shape, *, in_process: bool,
                 _root: Optional["ProcMesh"] = None):
        self._native = native
        self._shape_ = shape
        self._in_process = in_process
        self._root = _root
        if _root is None:
            self._health = _Health()
            self._monitor_taken = False
            self._monitor_events: List[ProcEvent] = []
            self._monitor_cv = threading.Condition()
            self._stopped = False
            self._actor_names: set = set()
            self._log_aggregator: Optional[LogAggregator] = None
            self._device_mesh = None
            self._thread = threading.Thread(target=self._monitor_loop, daemon=True,
                                            name=f"monarch-monitor-{native.world}")
            self._thread.start()
            _live_meshes.add(self)
        self.initialized: Future = Future.ready(True)

    # MeshTrait ------------------------------------------------------------------------
    @property
    def _ndslice(self):
        return self._shape_.ndslice

    @property
    def _labels(self):
        return tuple(self._shape_.labels)

    def _new_with_shape(self, shape: Shape) -> "ProcMesh":
        return ProcMesh(self._native, shape, in_process=self._in_process,
                        _root=self._root or self)

    @property
    def _owner(self) -> "ProcMesh":
        return self._root or self

    @property
    def world(self) -> str:
        return self._native.world

    # supervision ----------------------------------------------------------------------
    def _monitor_loop(self) -> None:
        native = self._native
        while not self._stopped:
            try:
                ev = native.next_event(200)
            except Exception:  # noqa: BLE001
                break
            if ev is None:
                if native.stopped:
                    break
                continue
            if self._stopped:
                break
            if ev["kind"] == "supervision":
                actor_id = ev["actor_id"]
                name = N.parse_actor_id(actor_id)[2]
                msg = f"actor {actor_id} failed: {ev['message']}"
                with self._health.lock:
                    if name in self._actor_names:
                        self._health.actor_errors.setdefault(name, {}).setdefault(
                            int(ev["rank"]), msg)
                    else:
                        self._health.mesh_error = self._health.mesh_error or msg
                pe = ProcEvent("actor_failed", ev["rank"], actor_id, ev["message"])
            else:
                msg = f"proc {self.world}[{ev['rank']}] is stopped: {ev['reason']}"
                with self._health.lock:
                    self._health.mesh_error = self._health.mesh_error or msg
                pe = ProcEvent("proc_stopped", ev["rank"], "", ev["reason"])
            with self._monitor_cv:
                self._monitor_events.append(pe)
                self._monitor_cv.notify_all()
            if not self._monitor_taken:
                N.log(4, f"unhandled crash on proc mesh {self.world}: {msg} "
                         "(use proc_mesh.monitor() to handle crashes)")

    def monitor(self) -> Future[ProcEvent]:
        """Future of the next crash on this mesh.  Taking it marks crashes as handled by
        the caller (they are no longer logged as unhandled)."""
        owner = self._owner
        owner._monitor_taken = True

        def wait(timeout):
            with owner._monitor_cv:
                if not owner._monitor_cv.wait_for(lambda: owner._monitor_events, timeout):
                    raise TimeoutError("no crash within the timeout")
                return owner._monitor_events.pop(0)

        return Future(wait)

    # spawning -------------------------------------------------------------------------
    def spawn(self, name: str, cls: Type[T], *args: Any, **kwargs: Any) -> ActorMesh[T]:
        if self._root is not None:
            raise NotImplementedError("cannot spawn on a slice of a proc mesh; spawn on the "
                                      "whole mesh and slice the actor mesh")
        if self._stopped:
            raise RuntimeError("`ProcMesh` has already been stopped")
        if not (isinstance(cls, type) and issubclass(cls, Actor)):
            raise ValueError(f"{cls} must subclass monarch_b200.actor.Actor to be spawned")
        sl = self._shape_.ndslice
        meta = {"labels": self._shape_.labels, "sizes": list(sl.sizes), "ranks": sl.ranks(),
                "world": self.world, "proc_mesh_ref": ProcMeshRef(self.world, self._shape_)}
        if "monarch_b200.tensor_engine.device_mesh" in sys.modules:
            # constructor arguments may be distributed tensors: every actor is built with its
            # proc's own shard (taken from the proc's tensor worker when the actor starts)
            from ..tensor_engine import actor_bridge as ab
            if ab.has_distributed_tensors(args, kwargs):
                args, kwargs, meta["broker_ident"] = ab.spawn_state(self, args, kwargs)
        params, parts = flatten((cls, args, kwargs, meta))
        if parts:
            raise ValueError("large tensors cannot be passed as spawn arguments; send them "
                             "through an endpoint after spawning")
        if name in self._actor_names:
            raise RuntimeError(f"gspawn failed: an actor with name '{name}' has already been "
                               "spawned on this proc mesh")
        results = self._native.spawn(name, "python", params)
        bad = [r for r in results if not r[1]]
        if bad:
            raise RuntimeError(f"spawn of '{name}' failed on rank {bad[0][0]}: {bad[0][2]}")
        self._actor_names.add(name)
        mesh = ActorMesh(cls, name, self.world, self._shape_, self, self._health)
        # Construct the user objects now so constructor errors surface through supervision
        # rather than on some later, unrelated call.
        mesh._cast(("init",), None)
        return mesh

    def __getstate__(self):
        raise RuntimeError("ProcMesh objects stay in the client that owns them; pass actor "
                           "meshes (or ProcMeshRef) to other actors instead")

    # tensor engine ----------------------------------------------------------------------
    def activate(self):
        return self._device_mesh_or_create().activate()

    def _device_mesh_or_create(self):
        owner = self._owner
        if owner._device_mesh is None:
            from ..tensor_engine.device_mesh import spawn_tensor_engine
            owner._device_mesh = spawn_tensor_engine(owner)
        return owner._device_mesh

    def rank_tensor(self, dim):
        return self._device_mesh_or_create().rank(dim)

    def rank_tensors(self):
        return self._device_mesh_or_create().ranks

    def to_table(self) -> str:
        rows = ["rank\t" + "\t".join(self._labels)]
        sl = self._shape_.ndslice
        for r in sl.ranks():
            rows.append(f"{r}\t" + "\t".join(str(c) for c in sl.coordinates(r)))
        return "\n".join(rows)

    @staticmethod
    def from_alloc(alloc, setup: Optional[Callable[[], None]] = None) -> "ProcMesh":
        """The proc mesh described by an :class:`~monarch_b200.actor.allocator.Alloc`.
        ``setup`` runs in every proc before any actor is spawned there (environment
        variables that must be in place before CUDA is initialised, for instance)."""
        from .allocator import proc_mesh_from_alloc
        return proc_mesh_from_alloc(alloc, setup=setup)

    def ledger(self, timeout: float = 5.0) -> Dict[int, List[dict]]:
        """Actor-tree snapshot of every proc of the mesh (hyperactor/src/proc.rs:139-315
        ``ledger_snapshot``): rank -> list of ``{actor_id, status, messages_handled, failure,
        children, last_event}``.  Procs that do not answer in time are absent."""
        out: Dict[int, List[dict]] = {}
        for rank, text in self._owner._native.ledger(int(timeout * 1000)):
            rows = []
            for line in text.splitlines():
                f = (line.split("\t") + [""] * 6)[:6]
                rows.append({"actor_id": f[0], "status": f[1], "messages_handled": int(f[2] or 0),
                             "failure": f[3], "children": [c for c in f[4].split(",") if c],
                             "last_event": f[5]})
            out[int(rank)] = rows
        return out

    def serve_admin(self, address: Optional[str] = None) -> str:
        """Start the admin endpoint of this job (``python -m monarch_b200.tools.admin`` talks
        to it) and return its address."""
        from ..tools.admin import AdminServer
        owner = self._owner
        if getattr(owner, "_admin", None) is None:
            owner._admin = AdminServer(owner, address)
        return owner._admin.address

    # ops --------------------------------------------------------------------------------
    def logging_option(self, stream_to_client: bool = True, aggregate_window_sec: Optional[float] = 5,
                       level: int = 20) -> Future[None]:
        owner = self._owner
        if owner._log_aggregator is not None:
            owner._log_aggregator.flush()      # nothing waits in a window that is going away
        if not stream_to_client:
            owner._log_aggregator = None
            _log_sinks.pop(owner.world, None)
        else:
            agg = LogAggregator(aggregate_window_sec or 0.0)
            owner._log_aggregator = agg
            _log_sinks[owner.world] = agg.add
        return Future.ready(None)

    def sync_workspace(self, workspace: Optional[str] = None, conda: bool = False,
                       auto_reload: bool = False) -> Future[None]:
        from .code_sync import sync_workspace
        fut = sync_workspace(self, workspace, auto_reload)
        if not conda:
            return fut
        # also bring the procs' Python environment (conda prefix or virtualenv) in line with
        # the client's; procs that share the client's directory need nothing
        from .env_sync import sync_env

        def both(timeout):
            out = fut.get(timeout)
            sync_env(self, timeout=timeout)
            return out

        return Future(both)

    def stop(self) -> Future[None]:
        owner = self._owner

        def do(timeout):
            if owner._stopped:
                return None
            owner._stopped = True
            with owner._health.lock:
                owner._health.stopped = True
                owner._health.mesh_error = owner._health.mesh_error or "the proc mesh was stopped"
            owner._native.stop()
            if owner._log_aggregator is not None:
                owner._log_aggregator.flush()
            return None

        return Future(do)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop().get()

    async def __aenter__(self):
        return self

    async def __aexit__(self, *exc):
        await self.stop()

    def __del__(self):
        if self._root is None and not getattr(self, "_stopped", True):
            warnings.warn(f"unstopped ProcMesh {self.world!r}: call .stop() or use it as a "
                          "context manager", ResourceWarning, stacklevel=2)
            try:
                self._stopped = True
                self._native.stop()
            except Exception:  # noqa: BLE001
                pass

    def __repr__(self) -> str:
        return f"ProcMesh({self.world!r}, {self._shape_})"


class ProcMeshRef:
    """Inert, picklable description of a proc mesh (what remote actors see)."""

    def __init__(self, world: str, shape: Shape):
        self.world, self.shape = world, shape

    def __repr__(self) -> str:
        return f"ProcMeshRef({self.world!r}, {self.shape})"


_log_sinks: Dict[str, Callable[[int, bool, str], None]] = {}


def _make_log_sink(world: str):
    def sink(rank: int, is_err: bool, line: str) -> None:
        fn = _log_sinks.get(world)
        if fn is not None:
            fn(rank, is_err, line)
        else:
            print(f"[{world}[{rank}]] {line}", file=sys.stderr if is_err else sys.stdout,
                  flush=True)
    return sink


def _child_env(extra: Optional[Dict[str, str]]) -> Dict[str, str]:
    env = dict(extra or {})
    paths = [p for p in sys.path if p]
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if root not in paths:
        paths.insert(0, root)
    env.setdefault("PYTHONPATH", os.pathsep.join(paths))
    # A proc whose first ``import torch`` happens on one of the runtime's actor threads (while
    # a message carrying tensors is being unpickled) crashed on its next tensor allocation;
    # importing it on the proc's main thread before any actor runs does not.  So when this
    # process uses torch, tell the children to import it at start-up.
    if "torch" in sys.modules:
        env.setdefault("MB200_PREIMPORT", "torch")
    main = sys.modules.get("__main__")
    main_file = getattr(main, "__file__", None)
    if main_file:
        env.setdefault("MB200_MAIN_FILE", os.path.abspath(main_file))
    # one execution id for the whole job: logs, spans and traces of every proc carry it
    # (hyperactor_mesh/src/bootstrap.rs MONARCH_CLIENT_TRACE_ID in the reference)
    env.setdefault("HYPERACTOR_EXECUTION_ID", N.execution_id())
    env.setdefault("MONARCH_CLIENT_TRACE_ID", N.execution_id())
    return env


def _shape_from_dims(dims: Dict[str, int]) -> Shape:
    return Shape(list(dims), N.Slice.new_row_major([int(v) for v in dims.values()]))


def _allocate(dims: Dict[str, int], *, in_process: bool, env: Optional[Dict[str, str]] = None,
              bootstrap: Optional[Callable[[], None]] = None, gpu_env: bool = False,
              transport: str = "unix", remote_hosts: Optional[List[str]] = None,
              procs_per_host: int = 1, argv: Optional[List[str]] = None) -> ProcMesh:
    n = 1
    for v in dims.values():
        n *= int(v)
    world = f"mesh{next(_world_counter)}_{os.getpid()}"
    if in_process:
        native = N.ProcMesh.allocate_local(world, n)
    else:
        argv = list(argv) if argv else [sys.executable, "-m", "monarch_b200.actor.bootstrap_main"]
        # the job-wide controller registry must exist before children are started: they
        # find it through MB200_CONTROLLER_REF in their environment
        _controller_controller()
        e = _child_env(env)
        e.setdefault("MB200_CONTROLLER_REF", os.environ.get("MB200_CONTROLLER_REF", ""))
        if remote_hosts:
            # every proc is started by the allocator daemon of its host; a local stub per
            # proc relays its output and lifetime: the native executable
            # (csrc/tools/remote_exec.cpp) where it can be built, else tools/remote_exec.py
            # (the daemon runs its own program: nothing of `argv` travels)
            argv = _remote_stub_command()
            e["MB200_REMOTE_HOSTS"] = ",".join(remote_hosts)
            e["MB200_PROCS_PER_HOST"] = str(procs_per_host)
            transport = "tcp"
        if bootstrap is not None:
            import base64
            import cloudpickle
            e["MB200_BOOTSTRAP_FN"] = base64.b64encode(cloudpickle.dumps(bootstrap)).decode()
        native = N.ProcMesh.allocate_process(world, n, argv, e, gpu_env, _make_log_sink(world),
                                             transport)
    return ProcMesh(native, _shape_from_dims(dims), in_process=in_process)


def _remote_stub_command() -> List[str]:
    if os.environ.get("MB200_REMOTE_EXEC", "native") != "python":
        try:
            from .. import _build
            return [str(_build.build_remote_exec())]
        except Exception:  # noqa: BLE001 - no compiler on this host
            pass
    return [sys.executable, "-m", "monarch_b200.tools.remote_exec"]


# ---------------------------------------------------------------------------- hosts ----
class HostMesh(MeshTrait):
    """A mesh of hosts on which procs are spawned.  One box = one host; ``in_process``
    hosts create procs inside the client (fast API tests)."""

    def __init__(self, shape: Shape, in_process: bool = False,
                 allocators: Optional[List[str]] = None):
        self._shape_ = shape
        self._in_process = in_process
        # addresses (``tcp!host:port``) of the process-allocator daemons, one per host
        self._allocators = list(allocators) if allocators else None

    @property
    def _ndslice(self):
        return self._shape_.ndslice

    @property
    def _labels(self):
        return tuple(self._shape_.labels)

    def _new_with_shape(self, shape: Shape) -> "HostMesh":
        al = None
        if self._allocators:
            al = [self._allocators[r] for r in shape.ndslice.ranks()]
        return HostMesh(shape, self._in_process, al)

    def spawn_procs(self, per_host: Optional[Dict[str, int]] = None,
                    bootstrap: Optional[Callable[[], None]] = None,
                    env: Optional[Dict[str, str]] = None) -> ProcMesh:
        per_host = dict(per_host or {})
        have = dict(zip(self._labels, self._shape_.ndslice.sizes))
        # naming a host dim again is only accepted when it says what is already true
        # (``per_host={"hosts": 1, "gpus": 2}`` on a one-host mesh)
        for k in [k for k in per_host if k in have and int(per_host[k]) == have[k]]:
            del per_host[k]
        clash = set(per_host) & set(self._labels)
        if clash:
            raise ValueError(f"host mesh already has dims {sorted(clash)}")
        dims = {**dict(zip(self._labels, self._shape_.ndslice.sizes)), **per_host}
        if self._allocators:
            n_per = 1
            for v in per_host.values():
                n_per *= int(v)
            hosts = list(self._allocators)
            return _allocate(dims, in_process=False, env=env, bootstrap=bootstrap,
                             remote_hosts=hosts, procs_per_host=n_per)
        if len(self._shape_.ndslice) != 1 and not self._in_process:
            raise NotImplementedError("a multi-host mesh needs process-allocator daemons: build "
                                      "it with hosts_from_config() or HostMesh.from_allocators()")
        return _allocate(dims, in_process=self._in_process, env=env, bootstrap=bootstrap,
                         gpu_env="gpus" in per_host or "gpu" in per_host)

    @staticmethod
    def from_allocators(addresses: List[str], dim: str = "hosts") -> "HostMesh":
        """A host mesh whose procs are started by the process-allocator daemons listening at
        ``addresses`` (``tcp!host:port``, see ``monarch_b200.tools.process_allocator``)."""
        return HostMesh(Shape([dim], N.Slice.new_row_major([len(addresses)])),
                        allocators=list(addresses))


def this_host() -> HostMesh:
    """The host the calling actor (or client) runs on."""
    return HostMesh(Shape(["hosts"], N.Slice.new_row_major([1])))


def fake_in_process_host() -> HostMesh:
    """A host whose procs live inside this process (no subprocesses)."""
    return HostMesh(Shape(["hosts"], N.Slice.new_row_major([1])), in_process=True)


def hosts_from_config(name: str) -> HostMesh:
    """Host mesh named ``name`` in the job file written by ``monarch_b200.tools.cli create``
    (``$MB200_JOBS_DIR`` or ``~/.monarch_b200/jobs``): a JSON list of allocator addresses."""
    import json
    d = os.environ.get("MB200_JOBS_DIR", os.path.expanduser("~/.monarch_b200/jobs"))
    path = os.path.join(d, f"{name}.json")
    if not os.path.exists(path):
        raise KeyError(f"no host configuration {name!r} in {d}")
    with open(path) as f:
        job = json.load(f)
    return HostMesh.from_allocators(job["allocators"])


_this_proc: Optional[ProcMesh] = None


def this_proc() -> ProcMesh:
    """A singleton in-process proc mesh for actors that should live with the caller."""
    global _this_proc
    if _this_proc is None or _this_proc._stopped:
        _this_proc = _allocate({}, in_process=True)
    return _this_proc


def proc_mesh(*, gpus: Optional[int] = None, hosts: int = 1, env: Optional[Dict[str, str]] = None,
              setup: Optional[Callable[[], None]] = None) -> ProcMesh:
    """Subprocess proc mesh with dims {hosts, gpus} on this box (``hosts`` > 1 lays that many
    groups of procs out on the same box, as the reference's local ``proc_mesh`` does; real
    hosts come from ``HostMesh.from_allocators``)."""
    if hosts < 1:
        raise ValueError("hosts must be at least 1")
    if gpus is None:
        try:
            import torch
            gpus = max(torch.cuda.device_count(), 1)
        except Exception:  # noqa: BLE001
            gpus = 1
    return _allocate({"hosts": hosts, "gpus": gpus}, in_process=False, env=env, bootstrap=setup,
                     gpu_env=True)


def local_proc_mesh(*, gpus: Optional[int] = None, hosts: int = 1) -> ProcMesh:
    """In-process proc mesh (procs are threads of the client): for tests and notebooks."""
    return _allocate({"hosts": hosts, "gpus": gpus or 1}, in_process=True)


def sim_proc_mesh(*, gpus: int = 1, hosts: int = 1, racks: int = 1, zones: int = 1, dcs: int = 1,
                  regions: int = 1, network: bool = False) -> ProcMesh:
    """A large in-process mesh with topology dims, for exercising casts without hardware.

    ``network=True``: the procs talk through ``sim:`` channels -- every message crosses a
    simulated network and pays the latency of the distance between the two procs' hosts
    (same host, same rack, same zone, ...; ``configure_simnet``), on the simulated clock
    when ``telemetry.use_sim_clock()`` is on, so cast trees and protocols can be costed
    against a topology.  (hyperactor/src/channel/sim.rs, simnet.rs in the reference.)"""
    named = [(k, v) for k, v in (("regions", regions), ("dcs", dcs), ("zones", zones),
                                 ("racks", racks), ("hosts", hosts), ("gpus", gpus))]
    dims = {k: v for k, v in named if v > 1}
    if not network:
        return _allocate(dims or {"gpus": 1}, in_process=True)
    dims = dims or {"gpus": 1}
    import itertools as _it
    nodes = []
    for coord in _it.product(*[range(v) for v in dims.values()]):
        # the node is the proc's host: every topology level above "gpus"
        parts = [f"{k}{c}" for k, c in zip(dims, coord) if k != "gpus"]
        nodes.append(".".join(parts) or "host0")
    world = f"sim{next(_world_counter)}_{os.getpid()}"
    native = N.ProcMesh.allocate_sim(world, nodes)
    return ProcMesh(native, _shape_from_dims(dims), in_process=True)


def configure_simnet(latency_us, bandwidth_gbs: float = 0.0) -> None:
    """Latencies (microseconds) of the simulated network by node distance: index 0 within a
    host, 1 between hosts of a rack, 2 between racks, ...; optionally the link bandwidth."""
    N.simnet_configure([float(x) for x in latency_us], float(bandwidth_gbs))


def simnet_stats() -> dict:
    """Frames, bytes and summed simulated latency that crossed the simulated network."""
    return N.simnet_stats()


# ---------------------------------------------------------------------- controllers ----
class _ControllerController(Actor):
    """Hosts named singleton actors for the whole job (in the root client)."""

    def __init__(self):
        self._controllers: Dict[str, ActorMesh] = {}

    @endpoint
    def get_or_spawn(self, name: str, cls: type, args: tuple, kwargs: dict) -> ActorMesh:
        if name not in self._controllers:
            self._controllers[name] = _controller_procs().spawn(name, cls, *args, **kwargs)
        m = self._controllers[name]
        return ActorMesh(m._class, m._name, m._world, m._shape_, None, None, m._root_slice)


_cc_lock = threading.Lock()
_cc_mesh: Optional[ActorMesh] = None
_cc_procs: Optional[ProcMesh] = None


def _controller_procs() -> ProcMesh:
    global _cc_procs
    if _cc_procs is None or _cc_procs._stopped:
        _cc_procs = _allocate({}, in_process=True)
    return _cc_procs


def _controller_controller() -> ActorMesh:
    global _cc_mesh
    with _cc_lock:
        ref = os.environ.get("MB200_CONTROLLER_REF")
        if _cc_mesh is None and ref:
            import base64
            import pickle
            _cc_mesh = pickle.loads(base64.b64decode(ref))
        if _cc_mesh is None:
            _cc_mesh = _controller_procs().spawn("controller_controller", _ControllerController)
            import base64
            import pickle
            os.environ["MB200_CONTROLLER_REF"] = base64.b64encode(pickle.dumps(
                ActorMesh(_cc_mesh._class, _cc_mesh._name, _cc_mesh._world, _cc_mesh._shape_, None,
                          None, _cc_mesh._root_slice))).decode()
        return _cc_mesh


def get_or_spawn_controller(name: str, cls: Type[T], *args: Any, **kwargs: Any) -> Future[ActorMesh[T]]:
    """Named singleton actor shared by every proc of the job."""
    cc = _controller_controller()
    return cc.get_or_spawn.call_one(name, cls, args, kwargs)


@atexit.register
def _shutdown() -> None:
    for pm in list(_live_meshes):
        try:
            if not pm._stopped:
                pm._stopped = True
                pm._native.stop()
        except Exception:  # noqa: BLE001
            pass
