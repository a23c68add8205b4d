"""Random-number state of every worker of a device mesh, driven from the controller.

Parity: python/monarch/random.py:26-61 and python/monarch/builtins/random.py
(``manual_seed``, ``get_state``/``set_state`` returning/accepting distributed tensors,
``new_state``).  ``get_rng_state_all``/``set_rng_state_all`` cover CPU and every visible
CUDA generator so a checkpoint restores the streams exactly."""
from __future__ import annotations

from typing import List

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


def get_state():
    """The CPU generator state of every worker as a distributed uint8 tensor."""
    from .tensor_engine import get_active_mesh
    if get_active_mesh() is None:
        return _get_state()
    return _remote("_get_state", propagate=lambda: _state_like())()


def set_state(state) -> None:
    from .tensor_engine import get_active_mesh
    if get_active_mesh() is None:
        _set_state(state)
    else:
        _remote("_set_state")(state)


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
