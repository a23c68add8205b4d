"""Data-parallel parameter store: replicated parameters, bucketed gradient all-reduce
overlapped with backward.

``comm="fused"``: gradients live in peer-mapped memory and each bucket (25 MB by default)
is reduced by the two-shot ``allreduce_scale_cast`` kernel -- all-reduce, 1/N scale and
bf16 cast in one pass over NVLink -- on a side stream as soon as the backward of the unit
that owns it has finished.  ``comm="nccl"``: ``dist.all_reduce`` + a separate scale (the
library baseline; runs under gloo on CPU).

Parity: the reference's single-controller DDP reduces each parameter's gradient with
``grad.reduce_("dp", "sum")`` on a comms stream while backward continues
(docs/source/examples/distributed_tensors.py:258-342).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..models.llama import LocalParamStore, ParamLayout
from ..ops import kernels as K

bf16 = torch.bfloat16


class DDPParamStore(LocalParamStore):
    def __init__(self, layout: ParamLayout, device, seed: int = 0, init_std: float = 0.02,
                 comm: str = "fused", group: Optional[dist.ProcessGroup] = None,
                 bucket_bytes: int = 25 * 1024 * 1024):
        super().__init__(layout, device, seed=seed, init_std=init_std)
        self.group = group or dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.device.type != "cuda" and comm == "fused":
            comm = "nccl"
        self.comm = comm
        gran = 8 * self.world
        self.bucket_elems = max(gran, (bucket_bytes // 2) // gran * gran)
        self._epoch = 0
        self.reduce_scale = 1.0 / self.world   # gradient all-reduce computes the mean
        if comm == "fused":
            from .symm import FlagArray, SymmBuffer
            self._grads_sym = SymmBuffer(layout.total, bf16, self.device, self.group)
            self.grads = self._grads_sym.tensor
            self._flags = FlagArray(4, self.device, self.group)
        self._comm_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" \
            else None
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def _reduced_extent(self, ui: int) -> int:
        """Elements of unit ``ui`` (from its start) that are replicated across the group
        and therefore all-reduced; the rest (none here) is rank-private."""
        return self.layout.units[ui].size

    def _buckets(self, ui: int) -> List[Tuple[int, int]]:
        u = self.layout.units[ui]
        out = []
        off = u.offset
        end = u.offset + self._reduced_extent(ui)
        while off < end:
            n = min(self.bucket_elems, end - off)
            out.append((off, n))
            off += n
        return out

    def post_backward(self, ui: int) -> None:
        cuda = self.device.type == "cuda"
        if cuda:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self._comm_stream.wait_event(ev)
        ctx = torch.cuda.stream(self._comm_stream) if cuda else _Null()
        with ctx:
            for off, n in self._buckets(ui):
                if self.comm == "fused":
                    self._epoch += 1
                    K.check(K.lib().mb200_allreduce_scale_cast(
                        self._grads_sym.ptrs_at(off), self._grads_sym.ptrs_at(off),
                        self._grads_sym.mc_at(off), self._grads_sym.mc_at(off),
                        self._flags.ptrs, n, 0, self.rank, self.world, self.reduce_scale, 0,
                        self._epoch, self._flags.counter.data_ptr(), 0,
                        K.status_word(self.device).data_ptr(), K.stream_ptr()),
                        "allreduce_scale_cast")
                else:
                    g = self.grads[off: off + n]
                    if g.dtype == bf16 and dist.get_backend(self.group) != "nccl":
                        t = g.float()
                        dist.all_reduce(t, group=self.group)
                        g.copy_(t * self.reduce_scale)
                    else:
                        dist.all_reduce(g, group=self.group)
                        if self.reduce_scale != 1.0:
                            g.mul_(self.reduce_scale)
            if self._updating:
                # hyper-parameters known before backward (set_hyper): the unit's AdamW update
                # follows its all-reduce on the comm stream, under the rest of the backward
                u = self.layout.units[ui]
                lo, hi = u.offset, u.offset + u.size
                ops.adamw_(self.master[lo:hi], self.m[lo:hi], self.v[lo:hi], self.grads[lo:hi],
                           self.params[lo:hi], step=self.step_count + 1, **self._hyper)
                self._updated_units += 1

    def optimizer_step(self, lr, **kw):
        if self._comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self._comm_stream)
        super().optimizer_step(lr, **kw)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
