"""RDMABuffer: one-sided reads and writes of another actor's memory.

Parity: python/monarch/_src/tensor_engine/rdma.py (RDMABuffer.read_into / write_from /
drop, picklable handles that travel in ordinary actor messages, default timeout 3 s),
monarch_rdma (per-proc manager actor, buffer registry).  The reference moves bytes with
ibverbs queue pairs and bounces GPU tensors through the host; here

* GPU buffers are first class: the owner exports a CUDA IPC handle, the peer maps it and a
  hand-written copy kernel moves the bytes with in-kernel NVLink loads/stores
  (``peer_copy``), publishing a completion flag; no host bounce;
* host buffers in the same process are copied directly; between processes of one box they
  are read and written in place with ``process_vm_readv`` / ``process_vm_writev`` (one copy);
  otherwise the owner's manager actor -- a native actor, ``csrc/rdma/rdma_manager.cpp`` --
  serves the bytes as out-of-band frame parts over the actor channels (no ibverbs device
  exists on this class of box).
"""
from __future__ import annotations

import itertools
import os
import threading
import time
import warnings
from typing import Any, Dict, Optional, Tuple

import torch

from ..actor.actor_mesh import context
from ..actor.future import Future
from ..actor.pickle import flatten, unflatten

_MANAGER_NAME = "rdma_manager"
_lock = threading.Lock()
_managers: Dict[str, "_Manager"] = {}   # proc id -> manager (this process)
_ids = itertools.count(1)


class RDMAError(RuntimeError):
    pass


def is_available() -> bool:
    return True


class _Manager:
    """The proc's RDMA manager: a native actor (``_native.RdmaManager``) owns the registry and
    answers remote handles without entering Python; this object registers buffers with it and
    keeps the tensors alive while they are exported."""

    def __init__(self, proc):
        from .. import _native as N
        self.proc = proc
        self.proc_id = proc.proc_id
        self.buffers: Dict[int, torch.Tensor] = {}
        self.native = N.RdmaManager(proc, _MANAGER_NAME, self._serve_cuda_bytes)
        self.actor_id = self.native.actor_id

    def register(self, t: torch.Tensor) -> dict:
        """Export ``t`` (1-D uint8 view of a contiguous tensor); returns what a handle carries."""
        import socket
        info = {"nbytes": t.numel(), "cuda": t.is_cuda, "device": t.device.index if t.is_cuda
                else -1, "addr": t.data_ptr(), "pid": os.getpid(), "host": socket.gethostname(),
                "ipc_handle": b"", "ipc_offset": 0}
        if t.is_cuda:
            from ..ops import ipc
            exp = ipc.export_handle(t)
            info["ipc_handle"], info["ipc_offset"] = exp["handle"], exp["offset"]
        bid = self.native.register(info["addr"], info["nbytes"], info["cuda"], info["device"],
                                   info["ipc_handle"], info["ipc_offset"], info["host"])
        self.buffers[bid] = t        # the owner must not free it while peers may touch it
        info["id"] = bid
        info["valid_addr"] = self.native.get(bid)["valid_addr"]
        return info

    def drop(self, bid: int) -> None:
        self.native.drop(bid)
        self.buffers.pop(bid, None)

    def _serve_cuda_bytes(self, info: dict, op: str, off: int, n: int, payload):
        """GPU bytes over messages, for requesters that cannot map the buffer (no peer path,
        a host-side destination): called by the native manager actor."""
        t = self.buffers.get(info["id"])
        if t is None:
            raise RDMAError(f"buffer {info['id']} is not registered (dropped?)")
        raw = _as_bytes(t)
        if op == "read":
            return raw[off: off + n].cpu().numpy().tobytes()
        data = torch.frombuffer(bytearray(payload), dtype=torch.uint8)
        raw[off: off + data.numel()].copy_(data)
        return None


_hostname: Optional[str] = None
_DONE: Future = Future.ready(None)


def _as_bytes(t: torch.Tensor) -> torch.Tensor:
    if not t.is_contiguous():
        raise ValueError("RDMABuffer needs a contiguous tensor")
    return t.reshape(-1).view(torch.uint8)


def _check_range(raw: torch.Tensor, off: int, n: int) -> None:
    if off < 0 or n < 0 or off + n > raw.numel():
        raise RDMAError(f"range [{off}, {off + n}) outside a buffer of {raw.numel()} bytes")


def _manager_for_current_proc() -> _Manager:
    proc = context().actor_instance.proc
    with _lock:
        m = _managers.get(proc.proc_id)
        if m is None:
            m = _Manager(proc)
            _managers[proc.proc_id] = m
        return m


_peer_cache: Dict[tuple, int] = {}


def _ensure_peer_access(dev: int, other: int) -> None:
    from ..ops import ipc
    try:
        ipc.ensure_peer_access(dev, other)
    except ipc.PeerAccessError as e:
        raise RDMAError(str(e)) from None


def _device_copy_ptr(dst_ptr: int, src_ptr: int, nbytes: int, dev_index: int) -> None:
    """nbytes from src_ptr to dst_ptr with the peer-copy kernel running on ``dev_index``
    (either pointer may be a mapping of another process's / GPU's memory), queued on the
    caller's current stream of that device behind whatever produced the source.  Returns when
    the bytes have landed: waiting for the stream is waiting for the transfer, so no
    completion flag has to be zeroed, published and read back per call."""
    from ..ops import kernels as K
    if torch.cuda.current_device() == dev_index:       # the usual case: no device switch
        K.check(K.lib().mb200_peer_copy_sync(dst_ptr, src_ptr, nbytes, 0, K.stream_ptr()),
                "peer_copy")
        return
    with torch.cuda.device(dev_index):
        K.check(K.lib().mb200_peer_copy_sync(dst_ptr, src_ptr, nbytes, 0, K.stream_ptr()),
                "peer_copy")


def _device_copy(dst: torch.Tensor, src: torch.Tensor) -> None:
    """dst <- src between tensors of this process (same or different GPUs)."""
    dev = dst.device if dst.is_cuda else src.device
    idx = dev.index or 0
    for t in (dst, src):
        if t.is_cuda and (t.device.index or 0) != idx:
            _ensure_peer_access(idx, t.device.index or 0)
    _device_copy_ptr(dst.data_ptr(), src.data_ptr(), dst.numel(), idx)


def _open_ipc(handle: bytes, reader_device: int) -> int:
    from ..ops import ipc
    return ipc.open_ipc(handle, reader_device)


class RDMABuffer:
    """A handle to ``data``'s memory that other actors can read from and write into."""

    def __init__(self, data: torch.Tensor):
        if data.dim() != 1 or data.dtype != torch.uint8:
            data = data.reshape(-1).view(torch.uint8) if data.is_contiguous() else None
            if data is None:
                raise ValueError("RDMABuffer needs a contiguous tensor (viewed as 1-D uint8)")
        mgr = _manager_for_current_proc()
        self._owner = mgr.actor_id
        self._owner_proc = mgr.proc_id
        self._info = mgr.register(data)

    # handles travel by value; the memory stays with the owner
    def __reduce__(self):
        return (_rebuild, (self._owner, self._owner_proc, self._info))

    @property
    def nbytes(self) -> int:
        return self._info["nbytes"]

    @property
    def _id(self) -> int:
        return self._info["id"]

    @property
    def _cuda(self) -> bool:
        return self._info["cuda"]

    # ------------------------------------------------------------------------------
    def _local_tensor(self) -> Optional[torch.Tensor]:
        m = _managers.get(self._owner_proc)
        if m is not None and self._id in m.buffers:
            return _as_bytes(m.buffers[self._id])
        return None

    def _request(self, op: str, timeout: float, offset: int = 0, length: int = 0,
                 payload: Optional[bytes] = None):
        """One round trip to the owner's manager actor; returns the reply envelope."""
        inst = context().actor_instance._native
        port, rx = inst.open_port(True)
        headers = {"kind": "rdma", "rdma_op": op, "rdma_id": str(self._id),
                   "rdma_offset": str(offset), "rdma_len": str(length), "rdma_reply": port}
        inst.send(self._owner + "[0]", b"", headers, [payload] if payload is not None else [])
        env = rx.recv(int(timeout * 1000))
        if env is None:
            inst.close_port(port)
            raise TimeoutError(f"RDMA operation on {self._owner} timed out after {timeout} s")
        if env.headers.get("rdma_status") != "ok":
            raise RDMAError(bytes(env.data).decode(errors="replace"))
        return env

    def _fast_ok(self) -> bool:
        """The buffer lives on a GPU of this box and in another process (a buffer of this
        very process is copied from its tensor directly)."""
        ok = self.__dict__.get("_fast")
        if ok is None:
            ok = self._fast = self._same_host() and self._local_tensor() is None
        return ok

    def _same_host(self) -> bool:
        global _hostname
        if _hostname is None:
            import socket
            _hostname = socket.gethostname()
        return self._info["host"] == _hostname

    def _peer_pointer(self, reader_device: int) -> int:
        """Address, valid for kernels of ``reader_device`` in this process, of byte 0 of the
        owner's GPU buffer (the handle carries the IPC export, so no round trip is needed)."""
        key = (self._owner, self._id, reader_device)
        p = _peer_cache.get(key)
        if p is None:
            self._request("info", 3)          # refuses a handle whose buffer was dropped
            _ensure_peer_access(reader_device, self._info["device"])
            p = _open_ipc(self._info["ipc_handle"], reader_device) + self._info["ipc_offset"]
            _peer_cache[key] = p
        return p

    def _check(self, offset: int, n: int) -> None:
        if offset < 0 or offset + n > self.nbytes:
            raise RDMAError(f"range [{offset}, {offset + n}) outside a buffer of "
                            f"{self.nbytes} bytes")

    def read_into(self, dst: torch.Tensor, offset: int = 0, timeout: float = 3) -> Future[None]:
        """Copy ``dst.nbytes`` bytes starting at ``offset`` of the remote buffer into ``dst``."""
        if self._cuda and dst.is_cuda and dst.is_contiguous() and self._fast_ok():
            # GPU to GPU on one box: launch and wait right here (the bytes have landed when
            # this returns; the future is already settled) -- the whole call is a few host
            # microseconds around one kernel
            n = dst.numel() * dst.element_size()
            self._check(offset, n)
            idx = dst.device.index or 0
            _device_copy_ptr(dst.data_ptr(), self._peer_pointer(idx) + offset, n, idx)
            return _DONE
        d = _as_bytes(dst)

        def run(_t):
            from .. import _native as N
            n = d.numel()
            self._check(offset, n)
            local = self._local_tensor()
            if local is not None:
                src = local[offset: offset + n]
                if src.is_cuda and d.is_cuda:
                    _device_copy(d, src)
                else:
                    d.copy_(src)
                return None
            if self._cuda and d.is_cuda and self._same_host():
                idx = d.device.index or 0
                _device_copy_ptr(d.data_ptr(), self._peer_pointer(idx) + offset, n, idx)
                return None
            if not self._cuda and self._same_host():
                # one copy, straight out of the owner's address space
                host = d if not d.is_cuda else torch.empty(n, dtype=torch.uint8).pin_memory()
                rc = N.rdma_host_read(self._info["pid"], self._info["addr"] + offset,
                                      host.data_ptr(), n, self._info["valid_addr"], self._id)
                if rc == 0:
                    if host is not d:
                        d.copy_(host)
                    return None
                if rc == -2:
                    raise RDMAError(f"buffer {self._id} is not registered on {self._owner} "
                                    "(dropped?)")
            env = self._request("read", timeout, offset, n)
            d.copy_(torch.frombuffer(bytearray(env.parts[0]), dtype=torch.uint8))
            return None

        return Future(run)

    def write_from(self, src: torch.Tensor, offset: int = 0, timeout: float = 3) -> Future[None]:
        """Copy ``src`` into the remote buffer starting at ``offset``."""
        if self._cuda and src.is_cuda and src.is_contiguous() and self._fast_ok():
            n = src.numel() * src.element_size()
            self._check(offset, n)
            idx = src.device.index or 0
            _device_copy_ptr(self._peer_pointer(idx) + offset, src.data_ptr(), n, idx)
            return _DONE
        s = _as_bytes(src)

        def run(_t):
            from .. import _native as N
            n = s.numel()
            self._check(offset, n)
            local = self._local_tensor()
            if local is not None:
                dst = local[offset: offset + n]
                if dst.is_cuda and s.is_cuda:
                    _device_copy(dst, s)
                else:
                    dst.copy_(s)
                return None
            if self._cuda and s.is_cuda and self._same_host():
                idx = s.device.index or 0
                _device_copy_ptr(self._peer_pointer(idx) + offset, s.data_ptr(), n, idx)
                return None
            if not self._cuda and self._same_host():
                host = s if not s.is_cuda else s.cpu()
                rc = N.rdma_host_write(self._info["pid"], self._info["addr"] + offset,
                                       host.data_ptr(), n, self._info["valid_addr"], self._id)
                if rc == 0:
                    return None
                if rc == -2:
                    raise RDMAError(f"buffer {self._id} is not registered on {self._owner} "
                                    "(dropped?)")
            self._request("write", timeout, offset, n, s.cpu().numpy().tobytes())
            return None

        return Future(run)

    def drop(self) -> Future[None]:
        def run(_t):
            m = _managers.get(self._owner_proc)
            if m is not None:
                m.drop(self._id)
            else:
                self._request("drop", 3)
            for k in [k for k in _peer_cache if k[:2] == (self._owner, self._id)]:
                _peer_cache.pop(k, None)
            return None
        return Future(run)


def _rebuild(owner, owner_proc, info) -> RDMABuffer:
    b = RDMABuffer.__new__(RDMABuffer)
    b._owner, b._owner_proc, b._info = owner, owner_proc, dict(info)
    return b
