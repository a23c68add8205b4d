"""ctypes binding of the sm_100a kernel library (``_mb200_kernels.so``).

The library is built in-tree by :mod:`monarch_b200._build`.  On a machine with a GPU a
missing or unloadable library is an error (never a silent PyTorch fallback); without a
GPU the pure-PyTorch reference implementations in :mod:`monarch_b200.ops.reference`
are used so that the host-side logic stays testable.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch

#: MB200_KERNEL_LIB=checked loads the build whose collectives bounds-check every peer access
CHECKED = os.environ.get("MB200_KERNEL_LIB", "") == "checked"
_SO = Path(__file__).resolve().parent / ("_mb200_kernels_checked.so" if CHECKED
                                         else "_mb200_kernels.so")
_lib: Optional[ctypes.CDLL] = None
_status: dict[int, torch.Tensor] = {}

#: number of kernels of this library launched since import (bench.py reports the delta)
launch_count = 0


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _SO.exists():
            if os.environ.get("MB200_NO_AUTOBUILD") != "1":
                from .. import _build
                _build.build_kernels(checked=CHECKED)
        if not _SO.exists():
            raise KernelError(f"{_SO} is missing: run `python -m monarch_b200._build kernels`")
        _lib = ctypes.CDLL(str(_SO))
        _declare(_lib)
        if os.environ.get("MB200_GEMM_IMPL"):
            _lib.mb200_gemm_set_impl(int(os.environ["MB200_GEMM_IMPL"]))
    return _lib


def available() -> bool:
    """True when the CUDA kernels can run (GPU present).  Raises if a GPU is present
    but the library cannot be loaded."""
    if not torch.cuda.is_available():
        return False
    lib()
    return True


_vp, _i, _f, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_int64


def _declare(l: ctypes.CDLL) -> None:
    l.mb200_gemm_bf16.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp,
                                  _vp]
    l.mb200_rmsnorm_fwd.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _f, _vp]
    l.mb200_rmsnorm_bwd_blocks.argtypes = [_i]
    l.mb200_rmsnorm_bwd.argtypes = [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]
    l.mb200_rope_inplace.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp]
    l.mb200_swiglu_fwd.argtypes = [_vp, _vp, _i, _i, _vp]
    l.mb200_swiglu_bwd.argtypes = [_vp, _vp, _vp, _i, _i, _vp]
    l.mb200_cross_entropy_fwd_bwd.argtypes = [_vp, _vp, _vp, _i, _i, _i, _f, _vp]
    l.mb200_adamw.argtypes = [_vp, _vp, _vp, _vp, _vp, _i64, _i, _f, _f, _f, _f, _f, _i, _f, _vp]
    l.mb200_embedding_fwd.argtypes = [_vp, _vp, _vp, _i, _i, _vp]
    l.mb200_embedding_bwd.argtypes = [_vp, _vp, _vp, _i, _i, _vp]
    l.mb200_sumsq.argtypes = [_vp, _i64, _i, _vp, _vp]
    for n in ("mb200_gemm_bf16", "mb200_rmsnorm_fwd", "mb200_rmsnorm_bwd_blocks",
              "mb200_rmsnorm_bwd", "mb200_rope_inplace", "mb200_swiglu_fwd", "mb200_swiglu_bwd",
              "mb200_cross_entropy_fwd_bwd", "mb200_adamw", "mb200_embedding_fwd",
              "mb200_embedding_bwd", "mb200_sumsq"):
        getattr(l, n).restype = _i
    for n, args in _OPTIONAL.items():
        if hasattr(l, n):
            getattr(l, n).argtypes = args
            getattr(l, n).restype = _i


_OPTIONAL: dict[str, list] = {
    "mb200_attn_fwd": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp],
    "mb200_attn_bwd": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                       _i, _i, _f, _vp, _vp],
    "mb200_barrier": [_vp, _i, _i, _i, ctypes.c_uint32, _vp, _vp],
    "mb200_wait_flags": [_vp, _i, _i, ctypes.c_uint32, _vp, _vp],
    "mb200_allgather_pull": [_vp, _vp, _i64, _i, _i, _vp, _i, ctypes.c_uint32, _vp, _i64,
                             ctypes.c_uint32, _i, _vp, _vp],
    "mb200_rs_adamw": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i, ctypes.c_uint32, _f, _f,
                       _f, _f, _f, _i, _f, _vp, _i, _vp, _vp],
    "mb200_allreduce_scale_cast": [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _f, _i, ctypes.c_uint32, _vp,
                                   _i, _vp, _vp],
    "mb200_peer_copy": [_vp, _vp, _i64, _vp, ctypes.c_uint32, _vp, _i, _vp],
    "mb200_peer_copy_sync": [_vp, _vp, _i64, _i, _vp],
    "mb200_memcpy_d2d_async": [_vp, _vp, _i64, _vp],
    "mb200_memset_d32_async": [_vp, ctypes.c_uint32, _i64, _vp],
    "mb200_enable_peer_access": [_i, _i],
    "mb200_ipc_export": [_vp, _vp, _vp, _vp],
    "mb200_ipc_open": [_vp, _i, _vp],
    "mb200_ipc_close": [_vp],
    "mb200_wait_flag": [_vp, ctypes.c_uint32, _i, _vp, _vp],
    "mb200_ag_gemm": [_vp, _i, _i, _i, _i, _vp, ctypes.c_longlong, _i, _vp, _i, _vp, _i, _vp,
                      ctypes.c_longlong, _i, _i, ctypes.c_longlong, ctypes.c_longlong,
                      ctypes.c_longlong, _vp, ctypes.c_uint32, _vp, _i, ctypes.c_uint32, _i, _vp,
                      _vp],
    "mb200_gemm_set_impl": [_i],
    "mb200_gemm_get_impl": [],
    "mb200_ag_a_gemm": [_vp, _vp, ctypes.c_longlong, _i, _i, _i, _i, _vp, _i, _i, _i, _vp, _i, _vp,
                        _i, ctypes.c_longlong, _vp, ctypes.c_uint32, _vp, _i, ctypes.c_uint32, _i,
                        _vp, _vp],
    "mb200_gemm_rs": [_vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _i, _i, _i, _i, _vp, _vp],
    "mb200_rs_finish": [_vp, _i, _i, _i, _i, _vp, _i, _vp, _i, _vp],
    "mb200_rs_finish_sync": [_vp, _i, _i, _i, _i, _vp, _i, _vp, _i, _vp, _i, _i, ctypes.c_uint32,
                             _vp, _vp],
    "mb200_moe_route": [_vp, _i, _i, _i, _vp, _vp, _vp],
    "mb200_moe_gather_gemm": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp,
                              _vp, ctypes.c_uint32, _vp, _i, _i, _i, _vp, _i, _i, _vp, _vp],
    "mb200_gemm_bf16_ex": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp,
                           _vp, _i, _i, _i, _vp, _vp],
    "mb200_moe_swiglu_fwd": [_vp, _vp, _vp, _vp, _i, _i, _vp],
    "mb200_moe_swiglu_bwd": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
    "mb200_moe_combine": [_vp, _i, _i, _i, _vp, _i, _vp, _i, _vp],
    "mb200_pingpong": [_vp, _vp, _vp, _vp, ctypes.c_longlong, _i, ctypes.c_uint32, _i, _vp, _vp,
                       _vp],
    "mb200_coll_stage": [_vp, _vp, _i64, _vp, _i, _i, _i, ctypes.c_uint32, _vp, _i, _vp],
    "mb200_coll_reduce": [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i, _i, _f, _i, _vp, _i, _i,
                          _i, _i, ctypes.c_uint32, _vp, _i, _vp, _vp, _vp, _vp, _i64, _vp],
    "mb200_coll_gather": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, ctypes.c_uint32, _i, _vp, _vp],
    "mb200_bounds_enabled": [],
    "mb200_bounds_reset": [_vp],
    "mb200_bounds_register": [_vp, _i64],
    "mb200_gather_chunks": [_vp, _vp, ctypes.c_longlong, _i, _i, ctypes.c_longlong,
                            ctypes.c_longlong, ctypes.c_longlong, _vp, ctypes.c_uint32, _vp, _i,
                            ctypes.c_uint32, _i, _vp, _vp],
}


_bounds_ready: set = set()


def bounds_register(ptr: int, nbytes: int, device=None) -> None:
    """In a checked build: allow the collectives of ``device`` to touch ``[ptr, ptr+nbytes)``
    (a local buffer, a peer mapping or a multicast mapping).  A no-op in the regular build."""
    l = lib()
    if not l.mb200_bounds_enabled():
        return
    idx = status_word(device).device.index
    with torch.cuda.device(idx):
        if idx not in _bounds_ready:
            check(l.mb200_bounds_reset(status_word(idx).data_ptr()), "bounds_reset", 0)
            _bounds_ready.add(idx)
        check(l.mb200_bounds_register(ptr, nbytes), "bounds_register", 0)


def set_gemm_impl(impl: int) -> None:
    """Select the GEMM kernel behind :func:`monarch_b200.ops.gemm`: 1 = single-CTA
    128x256 tiles, 2 = CTA-pair (``cta_group::2``) 256x256 tiles."""
    rc = lib().mb200_gemm_set_impl(int(impl))
    if rc:
        raise KernelError(f"unknown GEMM implementation {impl}")


def gemm_impl() -> int:
    return int(lib().mb200_gemm_get_impl())


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 status word written by kernels whose bounded waits ran out."""
    idx = None if device is None else (device if isinstance(device, int)
                                       else torch.device(device).index)
    if idx is None:     # no device given, or an index-less "cuda": the current device
        idx = torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
        _status[idx] = t
    return t


_STATUS_TEXT = {1: "mbarrier wait timed out inside a kernel",
                2: "wait on a peer/ready flag timed out inside a kernel",
                3: "kernel rejected its arguments",
                4: "a kernel's bounds check refused an access"}


def status_text(v: int) -> str:
    return _STATUS_TEXT.get(int(v), f"kernel status {int(v)}")


def raise_status(v: int, device=None) -> None:
    """Raise :class:`KernelError` for a non-zero status value already read from the device
    (and clear the sticky word so that later kernels wait normally again)."""
    if int(v) != 0:
        status_word(device).zero_()
        raise KernelError(status_text(v))


def check_status(device=None) -> None:
    """Synchronising check of the status word; raises KernelError on a recorded timeout."""
    raise_status(int(status_word(device)[0].item()), device)


class StatusWatch:
    """Reads a device's status word without stalling the stream: ``post()`` queues a copy
    into pinned host memory behind the work issued so far, ``poll()`` raises once such a
    copy has landed with a non-zero value.  A training loop that never synchronises still
    learns of a timed-out device-side wait one step later instead of never."""

    def __init__(self, device):
        self.device = torch.device(device)
        self._host = torch.zeros(4, dtype=torch.int32).pin_memory()
        self._event: Optional[torch.cuda.Event] = None

    def post(self) -> None:
        self._host.copy_(status_word(self.device), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self._event = ev

    def poll(self, wait: bool = False) -> None:
        ev = self._event
        if ev is None:
            return
        if wait:
            ev.synchronize()
        elif not ev.query():
            return
        self._event = None
        raise_status(int(self._host[0]), self.device)


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str, n_launch: int = 1) -> None:
    global launch_count
    if rc != 0:
        msg = f"{what}: error {rc}"
        if rc < 1000:
            msg += f" ({torch.cuda.cudart().cudaGetErrorString(rc) if hasattr(torch.cuda.cudart(), 'cudaGetErrorString') else 'cuda error'})"
        raise KernelError(msg)
    launch_count += n_launch
