"""Fully-sharded data parallel parameter store (ZeRO-3 style) over one NVLink domain.

Parameters, gradients' reduction and the AdamW state are sharded along the mesh dim of
the process group: rank r owns slice r of every *unit* (embedding, each decoder layer,
head) of the flat parameter layout.

``comm="fused"`` (GPU): this package's own kernels over peer-mapped memory --
  * the bf16 shards of a unit are brought from all ranks into a local buffer on a side
    stream, one unit ahead of compute: by the copy engines (``gather="dma"``, the default:
    a bounded wait for the peers' "shard updated" flags, then one asynchronous copy per
    peer out of its mapped shard -- no SM is taken from the GEMMs of the compute stream),
    by the ``allgather_pull`` kernel (``gather="prefetch"``), or, with ``gather="gemm"``,
    by the layer's own QKV and gate/up GEMM launches: the fused all-gather->GEMM kernel
    pulls the chunks while its tensor-core CTAs multiply;
  * after a unit's backward, ``rs_adamw`` reads that unit's gradient slice from every
    rank, reduces it in fp32, applies AdamW to the rank's fp32 master/moment shard and
    writes the updated bf16 shard -- reduce-scatter, cast and optimizer in one kernel,
    overlapped with the backward of the next unit.
  Cross-rank ordering is carried by epoch flags (one "gradients ready" and one "shard
  updated" slot per unit); every device-side wait is bounded.

``comm="nccl"``: the same schedule with ``torch.distributed`` collectives and a separate
AdamW kernel -- the library baseline, and the path that runs under gloo on CPU.

The reference has no FSDP; the primitives it offers are ``reduce(scatter=True)`` and
``reduce("stack")`` (python/monarch/common/tensor.py:234-249).
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from .. import ops
from ..models.llama import ParamLayout, init_params_
from ..ops import kernels as K

bf16 = torch.bfloat16


class _DeferredUnit(dict):
    """Parameter views of a unit whose gather rides on its GEMMs.  ``gemm(a, name)`` runs
    the fused gather+GEMM kernel when ``name`` lies beyond the gather frontier; plain item
    access pulls whatever the item still lacks with the copy-only kernel first, so code
    that knows nothing of the deferral stays correct."""

    def __init__(self, views, store, ui, b):
        super().__init__(views)
        self._store, self._ui, self._b = store, ui, b

    def _live(self) -> bool:
        st = self._store
        return st._buf_unit[self._b] == self._ui and st._frontier[self._b] is not None

    def __getitem__(self, name):
        if self._live():
            st = self._store
            _, c1, _ = st._chunk_span(self._ui, name)
            if c1 > st._frontier[self._b]:
                st._gather_plain(self._ui, self._b, c1)
        return dict.__getitem__(self, name)

    def gemm(self, a, name):
        st = self._store
        if self._live() and name in st._FUSE_AT:
            _, c1, _ = st._chunk_span(self._ui, name)
            if c1 > st._frontier[self._b]:
                return st._gemm_gathering(self._ui, self._b, a, name)
        return ops.gemm(a, self[name])


class FSDPParamStore:
    def __init__(self, layout: ParamLayout, device, seed: int = 0, init_std: float = 0.02,
                 comm: str = "fused", group: Optional[dist.ProcessGroup] = None,
                 n_buffers: int = 3, gather: Optional[str] = None,
                 gather_chunk: int = 1 << 18):
        """``gather``: how the layer units reach the compute stream when ``comm`` is
        "fused".  "dma" (default) and "prefetch" bring unit i+1 in on a side stream while
        unit i computes, with the copy engines or with a pull kernel.  Measured on 4 GPUs
        (Llama-3-8B, seq 8192): dma 557.8 ms/step, prefetch 575.1, gemm 586.8 -- the pull
        kernel's CTAs and the fused kernel's copy CTAs both slow the tensor-core work they
        run beside.  "gemm" issues no separate gather for a layer: the layer's QKV GEMM
        launch also pulls the attention half of the unit and its gate/up GEMM launch the
        MLP half (``mb200_ag_gemm``: copy CTAs pull chunks over NVLink, the tensor-core
        CTAs of the same kernel start on a weight tile as soon as its chunks are flagged),
        so nothing is held ahead of use and no second stream competes for SMs."""
        self.layout = layout
        self.device = torch.device(device)
        self.group = group or dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.device.type != "cuda" and comm == "fused":
            comm = "nccl"
        self.comm = comm
        gather = gather or os.environ.get("MB200_FSDP_GATHER", "dma")
        if gather not in ("prefetch", "gemm", "dma"):
            raise ValueError(f"unknown gather mode {gather!r}")
        self.gather = gather if (comm == "fused" and self.device.type == "cuda") else "prefetch"
        W = self.world
        for u in layout.units:
            if u.size % (W * 8):
                raise ValueError(f"unit {u.name} of {u.size} elements is not divisible by "
                                 f"{W} ranks x 8")
        self.shard_sizes = [u.size // W for u in layout.units]
        self.shard_offsets = [0]
        for s in self.shard_sizes:
            self.shard_offsets.append(self.shard_offsets[-1] + s)
        shard_total = self.shard_offsets[-1]
        self.max_unit = max(u.size for u in layout.units)
        dev = self.device

        self.master = torch.empty(shard_total, dtype=torch.float32, device=dev)
        self.m = torch.zeros(shard_total, dtype=torch.float32, device=dev)
        self.v = torch.zeros(shard_total, dtype=torch.float32, device=dev)
        for ui, u in enumerate(layout.units):
            lo = u.offset + self.rank * self.shard_sizes[ui]
            init_params_(layout, self._shard(self.master, ui), seed, init_std, lo,
                         lo + self.shard_sizes[ui])

        if comm == "fused":
            from .symm import FlagArray, SymmBuffer
            self._shards_sym = SymmBuffer(shard_total, bf16, dev, self.group, zero=False)
            self.param_shards = self._shards_sym.tensor
            self._grads_sym = SymmBuffer(layout.total, bf16, dev, self.group)
            self.grads = self._grads_sym.tensor
            n_units = len(layout.units)
            self._flags = FlagArray(2 * n_units + 4, dev, self.group)
            self._comm_stream = torch.cuda.Stream(device=dev)
        else:
            self.param_shards = torch.empty(shard_total, dtype=bf16, device=dev)
            self.grads = torch.zeros(layout.total, dtype=bf16, device=dev)
            self._comm_stream = torch.cuda.Stream(device=dev) if dev.type == "cuda" else None
        self.param_shards.copy_(self.master)

        self._bufs = [torch.empty(self.max_unit, dtype=bf16, device=dev) for _ in range(n_buffers)]
        self._buf_unit: List[Optional[int]] = [None] * n_buffers
        self._buf_ready: List[Optional[torch.cuda.Event]] = [None] * n_buffers
        self._buf_free: List[Optional[torch.cuda.Event]] = [None] * n_buffers
        self._buf_refs = [0] * n_buffers
        self._buf_age = [0] * n_buffers
        self._clock = 0
        # Number of training steps begun.  Doubles as the epoch of the cross-rank flags:
        # the update of step k publishes epoch k, so gathers inside training step k wait
        # for epoch k-1 and gathers after it (evaluation, checkpointing) for epoch k.
        self.step_count = 0
        self._in_train_step = False
        self._adam_offset = 0
        self._phase = "fwd"
        self._hyper = dict(lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, grad_scale=1.0)
        self._pending_updates: List[int] = []
        # in-GEMM gather: per buffer, one ready flag per chunk and the gather frontier
        if gather_chunk <= 0 or gather_chunk % 8192:
            raise ValueError("gather_chunk must be a positive multiple of 8192 elements")
        self._chunk = gather_chunk
        self._n_chunks_max = (self.max_unit + self._chunk - 1) // self._chunk
        self._frontier: List[Optional[int]] = [None] * n_buffers   # None: gathered elsewhere
        self._peer_views: dict = {}
        self._chunk_epoch = [0] * n_buffers
        if self.gather == "gemm":
            self._cflags = [torch.zeros(self._n_chunks_max, dtype=torch.int32, device=dev)
                            for _ in range(n_buffers)]
        self.fused_gemm_launches = 0
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------------- helpers
    def _shard(self, t: torch.Tensor, ui: int) -> torch.Tensor:
        return t[self.shard_offsets[ui]: self.shard_offsets[ui + 1]]

    @property
    def _cuda(self) -> bool:
        return self.device.type == "cuda"

    def set_hyper(self, **kw) -> None:
        self._hyper.update(kw)

    # ----------------------------------------------------------------------- gathering
    def _find(self, ui: int) -> Optional[int]:
        for b, u in enumerate(self._buf_unit):
            if u == ui:
                return b
        return None

    def _free_buffer(self) -> Optional[int]:
        cands = [b for b in range(len(self._bufs)) if self._buf_refs[b] == 0]
        if not cands:
            return None
        empty = [b for b in cands if self._buf_unit[b] is None]
        return empty[0] if empty else min(cands, key=lambda b: self._buf_age[b])

    def _gather_into(self, ui: int, b: int) -> None:
        """Issue the all-gather of unit ``ui`` into buffer ``b`` on the comm stream."""
        u = self.layout.units[ui]
        s = self.shard_sizes[ui]
        dst = self._bufs[b][: u.size]
        self._frontier[b] = None
        if self._cuda:
            cs = self._comm_stream
            if self._buf_free[b] is not None:
                cs.wait_event(self._buf_free[b])
            # the previous optimizer update of this shard (queued on the comm stream) is
            # ordered before this gather by the stream itself
            with torch.cuda.stream(cs):
                self._issue_gather(ui, dst, s)
                ev = torch.cuda.Event()
                ev.record(cs)
            self._buf_ready[b] = ev
        else:
            self._issue_gather(ui, dst, s)
        self._buf_unit[b] = ui
        self._clock += 1
        self._buf_age[b] = self._clock

    def _issue_gather(self, ui: int, dst: torch.Tensor, s: int) -> None:
        if self.comm == "fused" and self.gather == "dma":
            # copy engines instead of SMs: one bounded wait for the peers' "shard updated"
            # flags, then one asynchronous copy per peer out of its mapped shard.  Nothing
            # of the gather runs on the SMs that the GEMMs of the other stream are using.
            n_units = len(self.layout.units)
            K.check(K.lib().mb200_wait_flags(self._flags.my_ptr, self.world, n_units + ui,
                                             self._wait_epoch(),
                                             K.status_word(self.device).data_ptr(),
                                             K.stream_ptr()), "wait_flags")
            srcs = self._peer_views.get(ui)
            if srcs is None:
                off = self.shard_offsets[ui] * 2           # bf16 shards
                srcs = self._peer_views[ui] = [p + off for p in self._shards_sym.ptrs]
            lib, base, st = K.lib(), dst.data_ptr(), K.stream_ptr()
            for k in range(self.world):
                p = (self.rank + k) % self.world          # every rank starts at a different peer
                K.check(lib.mb200_memcpy_d2d_async(base + p * s * 2, srcs[p], s * 2, st),
                        "memcpy_d2d", 0)          # a copy-engine transfer, not a kernel
            return
        if self.comm == "fused":
            n_units = len(self.layout.units)
            K.check(K.lib().mb200_allgather_pull(
                dst.data_ptr(), self._shards_sym.ptrs_at(self.shard_offsets[ui]), s, self.rank,
                self.world, self._flags.my_ptr, n_units + ui, self._wait_epoch(), None, 0, 0, 0,
                K.status_word(self.device).data_ptr(), K.stream_ptr()), "allgather_pull")
        else:
            src = self._shard(self.param_shards, ui)
            if dist.get_backend(self.group) == "nccl":
                dist.all_gather_into_tensor(dst, src, group=self.group)
            else:
                parts = [torch.empty_like(src) for _ in range(self.world)]
                dist.all_gather(parts, src, group=self.group)
                torch.cat(parts, out=dst)

    def _gathers_in_gemm(self, ui: int) -> bool:
        return self.gather == "gemm" and self.layout.units[ui].name.startswith("layer")

    def _acquire(self, ui: int) -> int:
        b = self._find(ui)
        if b is None:
            b = self._free_buffer()
            if b is None:
                raise RuntimeError("no free gather buffer (raise n_buffers)")
            if self._gathers_in_gemm(ui):
                # nothing is launched here: the unit's first GEMMs pull it (_DeferredUnit)
                if self._buf_free[b] is not None:
                    torch.cuda.current_stream().wait_event(self._buf_free[b])
                self._buf_unit[b] = ui
                self._buf_ready[b] = None
                self._frontier[b] = 0
                self._chunk_epoch[b] += 1
                self._clock += 1
                self._buf_age[b] = self._clock
            else:
                self._gather_into(ui, b)
        if self._cuda and self._buf_ready[b] is not None:
            torch.cuda.current_stream().wait_event(self._buf_ready[b])
        self._buf_refs[b] += 1
        return b

    def _prefetch(self, ui: int) -> None:
        if ui < 0 or ui >= len(self.layout.units) or self._find(ui) is not None:
            return
        if self._gathers_in_gemm(ui):
            return
        b = self._free_buffer()
        if b is not None:
            self._gather_into(ui, b)

    def _release(self, ui: int, invalidate: bool = False) -> None:
        b = self._find(ui)
        if b is None:
            return
        self._buf_refs[b] = max(0, self._buf_refs[b] - 1)
        if self._buf_refs[b] == 0:
            if self._cuda:
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream())
                self._buf_free[b] = ev
            if invalidate:
                self._buf_unit[b] = None

    # --------------------------------------------------------------------- store hooks
    def begin_step(self) -> None:
        self.step_count += 1
        self._in_train_step = True
        self._phase = "fwd"
        self._invalidate_gathered()

    def begin_eval(self) -> None:
        """Start of a forward-only pass: no optimizer step follows, so neither the flag
        epoch nor AdamW's step moves; gathered copies from before are dropped."""
        self._in_train_step = False
        self._phase = "fwd"
        self._invalidate_gathered()

    def _invalidate_gathered(self) -> None:
        for b in range(len(self._bufs)):  # gathered copies of the previous step are stale
            if self._buf_refs[b] == 0:
                self._buf_unit[b] = None

    def unit_params(self, ui: int) -> Dict[str, torch.Tensor]:
        b = self._find(ui)
        if b is None:
            raise RuntimeError(f"unit {ui} is not gathered; hooks out of order")
        u = self.layout.units[ui]
        views = self.layout.views(u, self._bufs[b][: u.size])
        if self._frontier[b] is not None:
            return _DeferredUnit(views, self, ui, b)
        return views

    # ---------------------------------------------------------------- in-GEMM gathering
    _FUSE_AT = ("wqkv", "w_gu")   # the GEMMs that carry a gather, in layout order

    def _chunk_span(self, ui: int, name: str):
        u = self.layout.units[ui]
        for p in u.params:
            if p.name == name:
                n = 1
                for d in p.shape:
                    n *= d
                return p.offset // self._chunk, (p.offset + n + self._chunk - 1) // self._chunk, p
        raise KeyError(name)

    def _n_chunks(self, ui: int) -> int:
        return (self.layout.units[ui].size + self._chunk - 1) // self._chunk

    def _wait_epoch(self) -> int:
        """The "shard updated" epoch a gather must see on every rank: the previous step's
        inside a training step (this step's updates come after its gathers), the last
        step's outside one.  0 (no wait) before the first update."""
        return max(0, self.step_count - 1 if self._in_train_step else self.step_count)

    def _gather_plain(self, ui: int, b: int, c_end: int) -> None:
        """Pull chunks [frontier, c_end) with the copy-only kernel on the compute stream
        (the chunk that holds a norm gain, read before the layer's first GEMM)."""
        c0 = self._frontier[b]
        if c0 is None or c_end <= c0:
            return
        n_units = len(self.layout.units)
        K.check(K.lib().mb200_gather_chunks(
            self._bufs[b].data_ptr(), self._shards_sym.ptrs_at(self.shard_offsets[ui]),
            self.shard_sizes[ui], self.rank, self.world, c0, c_end, self._chunk,
            self._cflags[b].data_ptr(), self._chunk_epoch[b], self._flags.my_ptr, n_units + ui,
            self._wait_epoch(), 0, K.status_word(self.device).data_ptr(), K.stream_ptr()),
            "gather_chunks")
        self._frontier[b] = c_end

    def _gemm_gathering(self, ui: int, b: int, a: torch.Tensor, name: str) -> torch.Tensor:
        """``a @ W[name]^T`` in the kernel that also pulls the unit's chunks from the
        frontier up to the next gather-carrying weight."""
        c0, c1, spec = self._chunk_span(ui, name)
        u = self.layout.units[ui]
        later = [q for q in u.params if q.name in self._FUSE_AT and q.offset > spec.offset]
        target = (later[0].offset + self._chunk - 1) // self._chunk if later else self._n_chunks(ui)
        target = max(target, c1)
        N, Kd = spec.shape
        a2 = a.reshape(-1, Kd)
        if not a2.is_contiguous():
            a2 = a2.contiguous()
        M = a2.shape[0]
        out = torch.empty(M, N, dtype=bf16, device=a.device)
        n_units = len(self.layout.units)
        K.check(K.lib().mb200_ag_gemm(
            a2.data_ptr(), Kd, 0, M, Kd, self._bufs[b].data_ptr(), spec.offset, N,
            out.data_ptr(), N, None, 0, self._shards_sym.ptrs_at(self.shard_offsets[ui]),
            self.shard_sizes[ui], self.rank, self.world, self._frontier[b], target, self._chunk,
            self._cflags[b].data_ptr(), self._chunk_epoch[b], self._flags.my_ptr, n_units + ui,
            self._wait_epoch(), 16, K.status_word(self.device).data_ptr(), K.stream_ptr()),
            "ag_gemm")
        self._frontier[b] = target
        self.fused_gemm_launches += 1
        return out.view(*a.shape[:-1], N)

    def unit_grads(self, ui: int) -> Dict[str, torch.Tensor]:
        u = self.layout.units[ui]
        return self.layout.views(u, self.grads[u.offset: u.offset + u.size])

    def pre_forward(self, ui: int) -> None:
        self._acquire(ui)
        self._prefetch(ui + 1)

    def post_forward(self, ui: int) -> None:
        self._release(ui)

    def pre_backward(self, ui: int) -> None:
        if ui == 0 and not self.layout.cfg.tie_embeddings:
            return  # the embedding backward only scatters into gradients
        self._acquire(ui)
        if ui >= 2:
            self._prefetch(ui - 1)

    def post_backward(self, ui: int) -> None:
        self._release(ui, invalidate=True)
        self._reduce_and_update(ui)

    # ---------------------------------------------------- reduce-scatter + optimizer step
    def _reduce_and_update(self, ui: int) -> None:
        u = self.layout.units[ui]
        s = self.shard_sizes[ui]
        h = self._hyper
        scale = h["grad_scale"] / self.world
        if self.comm == "fused":
            n_units = len(self.layout.units)
            cs = self._comm_stream
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            cs.wait_event(ev)
            with torch.cuda.stream(cs):
                K.check(K.lib().mb200_rs_adamw(
                    self._grads_sym.ptrs_at(u.offset), self._grads_sym.mc_at(u.offset),
                    self._flags.ptrs, self._shard(self.master, ui).data_ptr(), self._shard(self.m, ui).data_ptr(),
                    self._shard(self.v, ui).data_ptr(),
                    self._shard(self.param_shards, ui).data_ptr(), s, self.rank, self.world, ui,
                    n_units + ui, self.step_count, h["lr"], h["beta1"], h["beta2"], h["eps"],
                    h["wd"], self.step_count + self._adam_offset, scale,
                    self._flags.counter.data_ptr(), 0,
                    K.status_word(self.device).data_ptr(), K.stream_ptr()), "rs_adamw")
            return
        # library path
        g_unit = self.grads[u.offset: u.offset + u.size]
        g_shard = torch.empty(s, dtype=g_unit.dtype, device=self.device)
        if dist.get_backend(self.group) == "nccl":
            dist.reduce_scatter_tensor(g_shard, g_unit, group=self.group)
        else:
            tmp = g_unit.float()
            dist.all_reduce(tmp, group=self.group)
            g_shard.copy_(tmp[self.rank * s: (self.rank + 1) * s])
        ops.adamw_(self._shard(self.master, ui), self._shard(self.m, ui), self._shard(self.v, ui),
                   g_shard, self._shard(self.param_shards, ui), lr=h["lr"], beta1=h["beta1"],
                   beta2=h["beta2"], eps=h["eps"], wd=h["wd"],
                   step=self.step_count + self._adam_offset, grad_scale=scale)

    def optimizer_step(self, lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, grad_scale=1.0) -> None:
        """The per-unit updates were issued during backward with the hyper-parameters set
        by :meth:`set_hyper`; this joins the comm stream and records the values for the
        next step."""
        self.set_hyper(lr=lr, beta1=beta1, beta2=beta2, eps=eps, wd=wd, grad_scale=grad_scale)
        self._in_train_step = False
        if self._cuda and self._comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self._comm_stream)

    # ------------------------------------------------------------------ full parameters
    def full_params(self) -> torch.Tensor:
        """All-gather of every unit into one flat bf16 buffer (checkpointing)."""
        if self._cuda:
            torch.cuda.synchronize(self.device)
            K.check_status(self.device)   # shards behind a timed-out collective are not sound
        dist.barrier(group=self.group)
        full = torch.empty(self.layout.total, dtype=bf16, device=self.device)
        for ui, u in enumerate(self.layout.units):
            src = self._shard(self.param_shards, ui).clone()
            parts = [torch.empty_like(src) for _ in range(self.world)]
            dist.all_gather(parts, src, group=self.group)
            torch.cat(parts, out=full[u.offset: u.offset + u.size])
        return full

    def load_full_params(self, flat: torch.Tensor) -> None:
        for ui, u in enumerate(self.layout.units):
            s = self.shard_sizes[ui]
            lo = u.offset + self.rank * s
            self._shard(self.param_shards, ui).copy_(flat[lo: lo + s])
            self._shard(self.master, ui).copy_(flat[lo: lo + s])
        if self._cuda:
            torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def state_dict_shard(self) -> dict:
        """This rank's optimizer/parameter shard for resumable checkpoints."""
        return {"master": self.master, "m": self.m, "v": self.v,
                "step": self.step_count + self._adam_offset, "rank": self.rank,
                "world": self.world}

    def load_state_dict_shard(self, sd: dict) -> None:
        assert sd["world"] == self.world and sd["rank"] == self.rank
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        # step_count doubles as the epoch of the cross-rank flags of this process group and
        # must keep counting from where this process is; only the optimizer's step moves
        self._adam_offset = int(sd["step"]) - self.step_count
        self.param_shards.copy_(self.master)
        if self._cuda:
            torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
