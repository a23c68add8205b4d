"""CUDA IPC plumbing shared by RDMABuffer and the mesh communicators: export a device
buffer as a 64-byte handle that travels in an ordinary actor message, map a peer's handle
for kernels of a given device, and switch peer access on.

The reference has no counterpart (its GPU buffers are registered with the NIC:
monarch_rdma/src/ibverbs_primitives.rs); the role is the same as its memory-region
registration -- make a buffer addressable by a remote party.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Tuple

import torch

from . import kernels as K

_ipc_open: Dict[Tuple[bytes, int], int] = {}   # (handle, reader device) -> mapped base address
_peer_enabled: set = set()


class PeerAccessError(RuntimeError):
    pass


def ensure_peer_access(dev: int, other: int) -> None:
    """A kernel on ``dev`` is about to dereference memory of device ``other`` (an IPC mapping
    of another process's buffer is opened on the owner's device): peer access must be on in
    that direction, or the first access faults."""
    if dev == other or (dev, other) in _peer_enabled:
        return
    rc = K.lib().mb200_enable_peer_access(dev, other)
    if rc == 1003:
        raise PeerAccessError(f"GPU {dev} has no peer path to GPU {other}")
    K.check(rc, "enable_peer_access", 0)
    _peer_enabled.add((dev, other))


def export_handle(t: torch.Tensor) -> dict:
    """What a peer needs to map ``t`` (a contiguous CUDA tensor): the IPC handle of the
    allocation that holds it, its offset inside that allocation, size, owning device and
    process.  The caller keeps ``t`` alive for as long as peers may touch it."""
    raw = t.reshape(-1).view(torch.uint8)
    h = ctypes.create_string_buffer(64)
    off, size = ctypes.c_int64(0), ctypes.c_int64(0)
    K.check(K.lib().mb200_ipc_export(raw.data_ptr(), h, ctypes.byref(off), ctypes.byref(size)),
            "ipc_export", 0)
    return {"handle": bytes(h.raw), "offset": int(off.value), "nbytes": raw.numel(),
            "device": raw.device.index or 0, "pid": os.getpid(), "ptr": raw.data_ptr()}


def open_ipc(handle: bytes, reader_device: int) -> int:
    """Map another process's allocation for kernels of ``reader_device`` (once per handle and
    device; CUDA refuses to open the same handle twice in one process)."""
    key = (handle, reader_device)
    base = _ipc_open.get(key)
    if base is None:
        torch.cuda.init()
        with torch.cuda.device(reader_device):
            torch.cuda.current_stream()          # makes sure the device's context exists
            out = ctypes.c_void_p(0)
            K.check(K.lib().mb200_ipc_open(handle, reader_device, ctypes.byref(out)),
                    "ipc_open", 0)
        base = int(out.value)
        _ipc_open[key] = base
    return base


def map_export(exp: dict, reader_device: int) -> int:
    """Address of byte 0 of an exported buffer, valid for kernels of ``reader_device`` in
    this process: the pointer itself when this process owns the buffer, else an IPC mapping."""
    if exp["pid"] == os.getpid():
        ensure_peer_access(reader_device, exp["device"])
        return exp["ptr"]
    return open_ipc(exp["handle"], reader_device) + exp["offset"]
