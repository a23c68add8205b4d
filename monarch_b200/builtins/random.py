"""Generator helpers as remote functions on the active device mesh.

Parity: python/monarch/builtins/random.py (``set_manual_seed_remote(seed, process_idx)``,
``get_rng_state_remote``, ``set_rng_state_remote``, ``seed_remote``, ``random_seed_remote``,
the ``*_cuda_remote`` family).  The plain names (``set_manual_seed`` ...) are the worker-side
functions; richer state handling lives in :mod:`monarch_b200.random`."""
from __future__ import annotations

from typing import List

import torch

from ..random import _get_state as get_rng_state, _set_state as set_rng_state  # noqa: F401


# ---- worker side ------------------------------------------------------------------------
def set_manual_seed(seed: int, process_idx=0) -> None:
    idx = int(process_idx.item()) if isinstance(process_idx, torch.Tensor) else int(process_idx)
    torch.manual_seed(int(seed) ^ idx)


def _seed() -> None:
    torch.seed()


def _manual_seed_cuda(seed: int) -> None:
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)


def _manual_seed_all_cuda(seed: int) -> None:
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def _get_rng_state_all_cuda() -> List[torch.Tensor]:
    return list(torch.cuda.get_rng_state_all()) if torch.cuda.is_available() else []


def _set_rng_state_all_cuda(states: List[torch.Tensor]) -> None:
    if torch.cuda.is_available():
        torch.cuda.set_rng_state_all([s.cpu() for s in states])


# ---- controller side ----------------------------------------------------------------------
def _r(name: str, propagate=None):
    from ..tensor_engine import remote
    return remote(f"monarch_b200.builtins.random.{name}", propagate=propagate)


def set_manual_seed_remote(seed: int, process_idx=0) -> None:
    """Seed every worker's default generator with ``seed ^ process_idx``; ``process_idx`` may
    be a distributed tensor (``mesh.rank("gpu")``) to give each worker its own stream."""
    _r("set_manual_seed")(seed, process_idx)


def get_rng_state_remote():
    return _r("get_rng_state", propagate=lambda: torch.empty(torch.get_rng_state().shape,
                                                             dtype=torch.uint8))()


def set_rng_state_remote(new_state) -> None:
    _r("set_rng_state")(new_state)


def seed_remote() -> None:
    """A fresh non-deterministic seed on every worker."""
    _r("_seed")()


random_seed_remote = seed_remote


def manual_seed_cuda_remote(seed: int) -> None:
    _r("_manual_seed_cuda")(seed)


def manual_seed_all_cuda_remote(seed: int) -> None:
    _r("_manual_seed_all_cuda")(seed)


def get_rng_state_all_cuda_remote():
    """The states of every CUDA generator each worker sees (shapes probed on one shard)."""
    return _r("_get_rng_state_all_cuda", propagate="cached")()


def set_rng_state_all_cuda_remote(states) -> None:
    _r("_set_rng_state_all_cuda")(states)
