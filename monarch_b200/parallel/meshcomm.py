"""Mesh communicator: collectives on ordinary CUDA tensors through this package's own
NVLink kernels (``csrc/kernels/collectives.cu``), for one group of GPUs in a box.

Every rank owns one device buffer -- a small flag array followed by a double-buffered
staging area -- that all ranks of the group have mapped.  How the mapping came about does
not matter to the collectives:

* :meth:`MeshComm.from_exports`: each rank allocates its buffer, exports a CUDA IPC handle
  (:func:`monarch_b200.ops.ipc.export_handle`), the handles travel over any control plane
  (the tensor engine sends them through actor messages) and every rank maps its peers'.
  No ``torch.distributed`` is involved.
* :meth:`MeshComm.from_process_group`: torch's symmetric-memory allocator does allocation
  and exchange over an existing process group and also yields an NVSwitch multicast
  mapping, which switches sums of f32/bf16/f16 to ``multimem.ld_reduce`` / ``multimem.st``.

Operations: ``all_reduce`` (sum, avg, product, min, max; band, bor, bxor on int32/int64),
``reduce_scatter``,
``all_gather``, ``all_to_all``, ``broadcast``, ``reduce`` (to a root), ``barrier``.  They
are asynchronous on the current CUDA stream; every rank of the group must issue the same
sequence.  Tensors larger than the staging capacity are moved in chunks.

Parity: the communicator of the reference's tensor worker (NCCL behind
monarch_tensor_worker/src/comm.rs; torch-sys-cuda/src/nccl.rs:464-835 all_reduce,
broadcast, reduce, all_gather, all_gather_into_tensor, reduce_scatter_tensor,
all_to_all_single, barrier).
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence

import torch

from ..ops import kernels as K

MAX_RANKS = 8
FLAG_BYTES = 4096            # 4 slots x 8 ranks x u32 used; a page keeps staging aligned
SLOT_STAGED, SLOT_RESULT, SLOT_BARRIER = 0, 1, 2

_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2, torch.float64: 3, torch.int32: 4,
       torch.int64: 5}
_OP = {"sum": 0, "avg": 0, "product": 1, "prod": 1, "min": 2, "max": 3, "band": 4, "bor": 5,
       "bxor": 6}
_BITWISE = ("band", "bor", "bxor")


def default_capacity() -> int:
    return int(os.environ.get("MB200_COMM_STAGE_MB", "32")) << 20


def supports(dtype: torch.dtype, reduction: Optional[str] = None) -> bool:
    """Whether a tensor of ``dtype`` can go through these kernels (copy-type collectives
    take any dtype; reductions the six arithmetic ones)."""
    if reduction is None:
        return True
    if reduction in _BITWISE:
        return dtype in (torch.int32, torch.int64)
    return dtype in _DT and reduction in _OP


def _ptr_array(ptrs: Sequence[int]):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def _i64_array(vals: Sequence[int]):
    return (ctypes.c_int64 * len(vals))(*vals)


def plan_chunks(nbytes: int, cap: int, align: int = 16) -> List[tuple]:
    """[(offset, size)] covering ``nbytes`` in pieces of at most ``cap`` bytes whose offsets
    are multiples of ``align``."""
    if nbytes <= 0:
        return [(0, 0)]
    step = max(align, cap // align * align)
    return [(o, min(step, nbytes - o)) for o in range(0, nbytes, step)]


class MeshComm:
    def __init__(self, rank: int, world: int, device, local: torch.Tensor, ptrs: Sequence[int],
                 mc_ptr: int = 0, cap: Optional[int] = None, keepalive=None):
        if world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks per NVLink domain")
        self.rank, self.world = rank, world
        self.device = torch.device(device)
        self.local = local                      # this rank's buffer (kept alive here)
        self.ptrs = [int(p) for p in ptrs]      # every rank's buffer, as seen from this GPU
        self.mc_ptr = int(mc_ptr or 0)
        self.cap = cap or default_capacity()
        if local.numel() < self.buffer_bytes(self.cap):
            raise ValueError("communicator buffer is smaller than its capacity needs")
        self._keepalive = keepalive
        for p in self.ptrs:                     # checked builds: the ranges kernels may touch
            K.bounds_register(p, self.buffer_bytes(self.cap), self.device)
        if self.mc_ptr:
            K.bounds_register(self.mc_ptr, self.buffer_bytes(self.cap), self.device)
        self._flag_ptrs = _ptr_array(self.ptrs)
        self._counter = torch.zeros(8, dtype=torch.int32, device=self.device)
        self._counter_p = self._counter.data_ptr()
        self._status_p = K.status_word(self.device).data_ptr()
        self._at_cache: dict = {}
        self.epoch = 0
        self._barrier_epoch = 0
        # below this many bytes an all-reduce is one pass in which every rank combines the
        # whole tensor; above, each rank combines 1/world and writes it to everyone
        self.one_shot_bytes = int(os.environ.get("MB200_COMM_ONE_SHOT_KB",
                                                 "1024" if self.mc_ptr else "256")) << 10
        self.launches = 0

    # --------------------------------------------------------------- construction
    @staticmethod
    def buffer_bytes(cap: int) -> int:
        return FLAG_BYTES + 4 * cap             # 2 halves x (input + result region)

    @classmethod
    def allocate_local(cls, device, cap: Optional[int] = None) -> torch.Tensor:
        cap = cap or default_capacity()
        return torch.zeros(cls.buffer_bytes(cap), dtype=torch.uint8, device=device)

    @classmethod
    def from_exports(cls, rank: int, exports: Sequence[dict], local: torch.Tensor, device,
                     cap: Optional[int] = None) -> "MeshComm":
        """``exports[p]``: what rank p's :func:`export_handle` returned for its buffer."""
        from ..ops import ipc
        dev = torch.device(device)
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        devs = [e["device"] for e in exports]
        if len(set((e["pid"], e["device"]) for e in exports)) != len(exports) or \
                len(set(devs)) != len(devs):
            # kernels of two ranks that wait on one another must run on different GPUs
            raise RuntimeError("the ranks of a communicator must sit on distinct GPUs: "
                               f"devices {devs}")
        ptrs = []
        for p, e in enumerate(exports):
            if p == rank:
                ptrs.append(local.data_ptr())
            else:
                ipc.ensure_peer_access(idx, e["device"])
                ptrs.append(ipc.map_export(e, idx))
        return cls(rank, len(exports), dev, local, ptrs, 0, cap)

    @classmethod
    def from_process_group(cls, group=None, device=None, cap: Optional[int] = None) -> "MeshComm":
        from .symm import SymmBuffer
        import torch.distributed as dist
        cap = cap or default_capacity()
        group = group or dist.group.WORLD
        dev = torch.device(device) if device is not None else \
            torch.device("cuda", torch.cuda.current_device())
        sb = SymmBuffer(cls.buffer_bytes(cap), torch.uint8, dev, group, zero=True)
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)
        return cls(sb.rank, sb.world, dev, sb.tensor, sb.ptrs, sb.multicast_ptr, cap,
                   keepalive=sb)

    # ------------------------------------------------------------------- plumbing
    def _status(self) -> int:
        return K.status_word(self.device).data_ptr()

    def _next(self):
        """A new collective: its epoch and the byte offsets of its input and result regions
        inside every rank's buffer."""
        self.epoch += 1
        base = FLAG_BYTES + (self.epoch & 1) * 2 * self.cap
        return self.epoch, base, base + self.cap

    def _at(self, off: int):
        arr = self._at_cache.get(off)
        if arr is None:          # the offsets are the few region starts of the two halves
            arr = _ptr_array([p + off for p in self.ptrs])
            if len(self._at_cache) < 1024:
                self._at_cache[off] = arr
        return arr

    def _stage(self, src_ptr: int, nbytes: int, in_off: int, epoch: int) -> None:
        K.check(K.lib().mb200_coll_stage(self.ptrs[self.rank] + in_off, src_ptr, nbytes,
                                         self._flag_ptrs, self.rank, self.world, SLOT_STAGED,
                                         epoch, self._counter_p, 0, K.stream_ptr()),
                "coll_stage")
        self.launches += 1

    def _reduce(self, in_off, out_off, out_local, lo, hi, valid, dt, op, scale, epoch,
                to_peers: bool, stage_src: Optional[int] = None, stage_bytes: int = 0) -> None:
        """``stage_src``: the kernel stages that many bytes itself before it combines (one
        launch instead of two; for tensors small enough that its grid is co-resident)."""
        mc_ok = self.mc_ptr and op == 0 and dt in (0, 1, 2)
        K.check(K.lib().mb200_coll_reduce(
            self._at(in_off), (self.mc_ptr + in_off) if mc_ok else None,
            self._at(out_off) if to_peers else None,
            (self.mc_ptr + out_off) if (to_peers and self.mc_ptr) else None,
            out_local, lo, hi, valid, dt, op, float(scale if scale is not None else 1.0),
            0 if scale is None else 1, self._flag_ptrs, self.rank, self.world, SLOT_STAGED,
            SLOT_RESULT if to_peers else -1, epoch, self._counter_p + 4, 0,
            self._status_p, K.stream_ptr(), stage_src,
            (self.ptrs[self.rank] + in_off) if stage_src is not None else None, stage_bytes,
            self._counter_p if stage_src is not None else None), "coll_reduce")
        self.launches += 1

    def _gather(self, src_off: Sequence[int], dst_off: Sequence[int], nbytes: Sequence[int],
                out_ptr: int, wait_slot: int, epoch: int) -> None:
        K.check(K.lib().mb200_coll_gather(_ptr_array(self.ptrs), _i64_array(src_off),
                                          _i64_array(dst_off), _i64_array(nbytes), out_ptr,
                                          self.ptrs[self.rank], self.rank, self.world, wait_slot,
                                          epoch, 0, self._status(), K.stream_ptr()),
                "coll_gather")
        self.launches += 1

    def _check(self, t: torch.Tensor) -> torch.Tensor:
        if not t.is_cuda or t.device != self.device:
            raise ValueError(f"tensor on {t.device}, communicator on {self.device}")
        t = t.contiguous()
        if t.data_ptr() % 16:
            t = t.clone()
        return t

    # ---------------------------------------------------------------- collectives
    def all_reduce(self, t: torch.Tensor, op: str = "sum", out: Optional[torch.Tensor] = None,
                   scale: Optional[float] = None) -> torch.Tensor:
        """Element-wise ``op`` over the ranks; every rank gets the result (bit-identical on
        all ranks).  ``avg`` is a sum scaled by 1/world.  ``out`` may be ``t`` itself."""
        if not supports(t.dtype, op):
            raise TypeError(f"all_reduce: unsupported {t.dtype} / {op!r}")
        src = self._check(t)
        if op == "avg":
            scale = (scale if scale is not None else 1.0) / self.world
        res = out if (out is not None and out.is_contiguous() and out.data_ptr() % 16 == 0) \
            else torch.empty_like(src)
        dt, opc = _DT[t.dtype], _OP[op]
        sp, rp = src.data_ptr(), res.data_ptr()
        for off, nb in plan_chunks(src.numel() * src.element_size(), self.cap):
            epoch, in_off, out_off = self._next()
            nvec = (nb + 15) // 16
            if nb <= self.one_shot_bytes or self.world == 1:
                # one launch: stage, publish, wait for the peers, combine everything
                self._reduce(in_off, out_off, rp + off, 0, nvec, nb, dt, opc, scale, epoch, False,
                             stage_src=sp + off, stage_bytes=nb)
            else:
                self._stage(sp + off, nb, in_off, epoch)
                per = (nvec + self.world - 1) // self.world
                lo = min(nvec, per * self.rank)
                self._reduce(in_off, out_off, None, lo, min(nvec, lo + per), 0, dt, opc, scale,
                             epoch, True)
                z = [0] * self.world
                nbs = list(z)
                so = list(z)
                nbs[self.rank], so[self.rank] = nb, out_off
                self._gather(so, z, nbs, rp + off, SLOT_RESULT, epoch)
        if out is not None:
            if res is not out:
                out.copy_(res.view_as(out))
            return out
        return res.view_as(t)

    def reduce_scatter(self, t: torch.Tensor, op: str = "sum",
                       scale: Optional[float] = None) -> torch.Tensor:
        """``t``: [world, ...]; rank r gets ``op`` over the ranks of slice r."""
        if not supports(t.dtype, op):
            raise TypeError(f"reduce_scatter: unsupported {t.dtype} / {op!r}")
        if t.dim() == 0 or t.shape[0] != self.world:
            raise ValueError(f"reduce_scatter needs an outer dim of {self.world}, got "
                             f"{tuple(t.shape)}")
        if op == "avg":
            scale = (scale if scale is not None else 1.0) / self.world
        W, es = self.world, t.element_size()
        flat = self._check(t).view(W, -1)
        cols = flat.shape[1]
        out = torch.empty(cols, dtype=t.dtype, device=self.device)
        # columns per pass: a multiple of 16 bytes, and world x that within the capacity
        step = max(16 // es, (self.cap // W) // 16 * 16 // es)
        dt, opc = _DT[t.dtype], _OP[op]
        for c0 in range(0, max(cols, 1), step):
            c1 = min(cols, c0 + step)
            nbr = (c1 - c0) * es                       # bytes per rank slice in this pass
            pad = (nbr + 15) // 16 * 16
            if c0 == 0 and c1 == cols and nbr == pad:
                piece = flat
            else:                                        # strided or ragged: repack, padded
                piece = torch.zeros(W, pad // es, dtype=t.dtype, device=self.device)
                piece[:, : c1 - c0] = flat[:, c0:c1]
            epoch, in_off, out_off = self._next()
            self._stage(piece.data_ptr(), W * pad, in_off, epoch)
            lo = self.rank * (pad // 16)
            self._reduce(in_off, out_off, out.data_ptr() + c0 * es, lo, lo + pad // 16, nbr, dt,
                         opc, scale, epoch, False)
        return out.view(t.shape[1:])

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[world, *t.shape]: slice p is rank p's ``t``."""
        src = self._check(t)
        nb_all = src.numel() * src.element_size()
        out = torch.empty((self.world, *t.shape), dtype=t.dtype, device=self.device)
        for off, nb in plan_chunks(nb_all, self.cap):
            epoch, in_off, _ = self._next()
            self._stage(src.data_ptr() + off, nb, in_off, epoch)
            self._gather([in_off] * self.world, [p * nb_all + off for p in range(self.world)],
                         [nb] * self.world, out.data_ptr(), SLOT_STAGED, epoch)
        return out

    def all_to_all(self, t: torch.Tensor) -> torch.Tensor:
        """``t``: [world, ...]; result slice p is slice ``rank`` of rank p's ``t``."""
        if t.dim() == 0 or t.shape[0] != self.world:
            raise ValueError(f"all_to_all needs an outer dim of {self.world}, got "
                             f"{tuple(t.shape)}")
        W = self.world
        flat = self._check(t).view(W, -1).view(torch.uint8)
        cb = flat.shape[1]
        out = torch.empty_like(flat)
        step = max(16, (self.cap // W) // 16 * 16)
        for c0 in range(0, max(cb, 1), step):
            c1 = min(cb, c0 + step)
            n = c1 - c0
            piece = flat if (c0 == 0 and c1 == cb) else flat[:, c0:c1].contiguous()
            epoch, in_off, _ = self._next()
            self._stage(piece.data_ptr(), W * n, in_off, epoch)
            self._gather([in_off + self.rank * n] * W, [p * cb + c0 for p in range(W)], [n] * W,
                         out.data_ptr(), SLOT_STAGED, epoch)
        return out.view(t.dtype).view(t.shape)

    def broadcast(self, t: torch.Tensor, root: int) -> torch.Tensor:
        """Every rank gets the root's ``t`` (same shape and dtype everywhere)."""
        src = self._check(t)
        nb_all = src.numel() * src.element_size()
        out = torch.empty_like(src)
        for off, nb in plan_chunks(nb_all, self.cap):
            epoch, in_off, _ = self._next()
            self._stage(src.data_ptr() + off, nb if self.rank == root else 0, in_off, epoch)
            nbs = [0] * self.world
            nbs[root] = nb
            self._gather([in_off] * self.world, [off] * self.world, nbs, out.data_ptr(),
                         SLOT_STAGED, epoch)
        return out.view_as(t)

    def reduce(self, t: torch.Tensor, root: int, op: str = "sum",
               scale: Optional[float] = None) -> Optional[torch.Tensor]:
        """``op`` over the ranks, delivered to ``root`` only (other ranks get None)."""
        if not supports(t.dtype, op):
            raise TypeError(f"reduce: unsupported {t.dtype} / {op!r}")
        src = self._check(t)
        if op == "avg":
            scale = (scale if scale is not None else 1.0) / self.world
        res = torch.empty_like(src) if self.rank == root else None
        dt, opc = _DT[t.dtype], _OP[op]
        for off, nb in plan_chunks(src.numel() * src.element_size(), self.cap):
            epoch, in_off, out_off = self._next()
            self._stage(src.data_ptr() + off, nb, in_off, epoch)
            nvec = (nb + 15) // 16 if self.rank == root else 0   # the others only wait
            self._reduce(in_off, out_off, res.data_ptr() + off if res is not None else None, 0,
                         nvec, nb, dt, opc, scale, epoch, False)
        return res.view_as(t) if res is not None else None

    def barrier(self) -> None:
        """Device-side flag barrier on the current stream (bounded wait)."""
        self._barrier_epoch += 1
        K.check(K.lib().mb200_barrier(self._flag_ptrs, self.rank, self.world, SLOT_BARRIER,
                                      self._barrier_epoch, self._status(), K.stream_ptr()),
                "barrier")
        self.launches += 1
