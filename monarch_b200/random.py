"""Random-number state of every worker of a device mesh, driven from the controller.

Parity: python/monarch/random.py:26-61 and python/monarch/builtins/random.py
(``manual_seed``, ``get_state``/``set_state`` returning/accepting distributed tensors,
``new_state``).  ``get_rng_state_all``/``set_rng_state_all`` cover CPU and every visible
CUDA generator so a checkpoint restores the streams exactly."""
from __future__ import annotations

from typing import Any, List, NamedTuple

import torch


# ---- worker-side (called by path) ---------------------------------------------------
def _manual_seed(seed: int, per_rank: bool = False) -> None:
    import os
    rank = os.environ.get("RANK", os.environ.get("HYPERACTOR_MESH_INDEX", "0"))
    s = int(seed) + (int(rank) if per_rank else 0)
    torch.manual_seed(s)


def _get_state() -> torch.Tensor:
    return torch.get_rng_state()


def _set_state(state: torch.Tensor) -> None:
    torch.set_rng_state(state.cpu().to(torch.uint8))


def _get_state_cuda() -> torch.Tensor:
    if not torch.cuda.is_available():
        return torch.zeros(0, dtype=torch.uint8)
    return torch.cuda.get_rng_state()


def _set_state_cuda(state: torch.Tensor) -> None:
    if torch.cuda.is_available() and state.numel():
        torch.cuda.set_rng_state(state.cpu().to(torch.uint8))


def _remote(name: str, propagate=None):
    from .tensor_engine import remote
    return remote(f"monarch_b200.random.{name}", propagate=propagate)


def _state_like():
    return torch.empty(torch.get_rng_state().shape, dtype=torch.uint8)


# ---- controller-side ------------------------------------------------------------------
def manual_seed(seed: int, per_rank: bool = False) -> None:
    """Seed the default generator of every worker of the active mesh (``per_rank=True``
    adds the worker's rank so data-parallel ranks draw different numbers)."""
    from .tensor_engine import get_active_mesh
    if get_active_mesh() is None:
        _manual_seed(seed, per_rank)
    else:
        _remote("_manual_seed")(seed, per_rank)


class State(NamedTuple):
    """Generator states of every worker: CPU and current CUDA device (empty without CUDA)."""
    cpu: Any
    cuda: Any


def _get_states():
    return _get_state(), _get_state_cuda()


def _set_states(cpu, cuda) -> None:
    _set_state(cpu)
    _set_state_cuda(cuda)


def _seed_from(seed) -> None:
    torch.manual_seed(int(seed.item()) if isinstance(seed, torch.Tensor) else int(seed))


def _make_deterministic() -> None:
    import os
    torch.use_deterministic_algorithms(True)
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False
    os.environ["CUBLAS_WORKSPACE_CONFIG"] = ":4096:8"     # deterministic cuBLAS workspaces


def _cuda_state_like():
    n = torch.cuda.get_rng_state().numel() if torch.cuda.is_available() else 0
    return torch.empty(n, dtype=torch.uint8)


def get_state() -> State:
    """The generator states of every worker as distributed uint8 tensors."""
    from .tensor_engine import get_active_mesh
    if get_active_mesh() is None:
        return State(*_get_states())
    mesh = get_active_mesh()
    if getattr(mesh.client, "use_cuda", None) is False:
        cuda_like = lambda: torch.empty(0, dtype=torch.uint8)  # noqa: E731
    else:
        cuda_like = _cuda_state_like_remote(mesh)
    return State(*_remote("_get_states", propagate=lambda: (_state_like(), cuda_like()))())


_cuda_state_len: dict = {}


def _cuda_state_like_remote(mesh):
    """The length of the workers' CUDA generator state (asked once per client: the
    controller may have no GPU to ask)."""
    key = id(mesh.client)
    if key not in _cuda_state_len:
        from .tensor_engine import call_on_shard_and_fetch
        _cuda_state_len[key] = int(call_on_shard_and_fetch(
            "monarch_b200.random._cuda_state_numel").get(timeout=60))
    n = _cuda_state_len[key]
    return lambda: torch.empty(n, dtype=torch.uint8)


def _cuda_state_numel() -> int:
    return int(_get_state_cuda().numel())


def set_state(state) -> None:
    """Restore what :func:`get_state` / :func:`new_state` returned (a lone tensor is taken
    as the CPU state)."""
    from .tensor_engine import get_active_mesh
    if isinstance(state, (tuple, list)):
        cpu, cuda = state
    else:
        cpu, cuda = state, None
    if get_active_mesh() is None:
        _set_state(cpu)
        if cuda is not None:
            _set_state_cuda(cuda)
    elif cuda is None:
        _remote("_set_state")(cpu)
    else:
        _remote("_set_states")(cpu, cuda)


def new_state(seed) -> State:
    """The states a generator seeded with ``seed`` starts from, without disturbing the
    current ones.  ``seed`` may be a distributed tensor (``mesh.rank(...) + 4``) to give
    every worker its own."""
    from .tensor_engine import get_active_mesh
    orig = get_state()
    if get_active_mesh() is None:
        _seed_from(seed)
    else:
        _remote("_seed_from")(seed)
    mine = get_state()
    set_state(orig)
    return mine


def make_deterministic() -> None:
    """Deterministic algorithms on every worker of the active mesh."""
    from .tensor_engine import get_active_mesh
    if get_active_mesh() is None:
        _make_deterministic()
    else:
        _remote("_make_deterministic")()


def get_rng_state_all() -> List[torch.Tensor]:
    """Local helper for checkpoints: [cpu_state, cuda_state_dev0, ...]."""
    out = [torch.get_rng_state()]
    if torch.cuda.is_available():
        out += list(torch.cuda.get_rng_state_all())
    return out


def set_rng_state_all(states: List[torch.Tensor]) -> None:
    torch.set_rng_state(states[0])
    if torch.cuda.is_available() and len(states) > 1:
        torch.cuda.set_rng_state_all(states[1:])
