"""Megatron-style tensor parallelism with sequence parallelism over one NVLink domain,
for one pipeline stage of a Llama-family model.

Between layers every rank holds T/tp rows of the residual stream ("sequence parallel").
A column-parallel GEMM (QKV, gate|up) first needs all rows of its normalised input; a
row-parallel GEMM (out, down) produces partial sums of all rows that must be summed and
scattered back to T/tp rows per rank.  With ``comm="fused"`` both are one kernel each:

* ``ag_gemm``  = ``mb200_ag_a_gemm``: the peers' rows arrive over NVLink while the tcgen05
  GEMM CTAs consume row blocks as they land (own rows first, then the peers in ring order);
  the rows are moved by the copy engines on a side stream, which raise the same per-chunk
  flags that the kernel's own copy CTAs raise in the ``MB200_TP_GATHER=kernel`` mode; the
  gathered input stays resident for the weight-gradient GEMM of the backward pass.
* ``gemm_rs``  = ``mb200_gemm_rs`` + ``mb200_rs_finish_sync``: the GEMM epilogue stores each
  bf16 partial tile straight into the owner rank's staging slot; the owner's next launch is
  the flag barrier and the fp32 sum of the slots together with the residual.

The cross-rank handshakes ride in launches that do work anyway (the copy of the local rows
publishes "rows in place", the GEMM's copy CTAs wait for it; the sum kernel signals and waits
for "tiles stored"): four launches per gather-GEMM / GEMM-scatter pair instead of six.

``comm="nccl"`` runs the same schedule with torch.distributed collectives and separate
GEMMs (the library baseline; under gloo it is the CPU test path).

The reference has no tensor parallelism (its mesh can be split into named dims such as
``tp``, python/monarch/_src/actor/shape.py:88-203, but no TP math exists); this module
is the net-new part that the ``{pp: 2, tp: 4}`` configuration needs.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..models.llama import LlamaConfig, LocalParamStore, ParamLayout
from ..ops import kernels as K

bf16 = torch.bfloat16


class TPComm:
    """Buffers, flags and the two fused primitives of one tensor-parallel group."""

    CHUNK = 1 << 16  # elements per readiness flag of a gathered activation
    SLOT_ROWS = 2    # flag slot: "my rows of the activation are in my symmetric buffer"
    SLOT_TILES = 3   # flag slot: "my GEMM has stored its partial tiles"

    def __init__(self, group, device, rows_local: int, d: int, comm: str = "fused"):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device(device)
        self.rows_local, self.d = rows_local, d
        self.rows = rows_local * self.world
        if self.device.type != "cuda" and comm == "fused":
            comm = "nccl"
        self.comm = comm
        self._n_ag = 0
        self._n_rs = 0
        self._epoch = 0
        self._rs_epoch = 0
        self._side = None
        # how the peers' rows reach the gather-GEMM: "dma" (copy engines on a side stream raise
        # the rows' chunk flags, the GEMM launch has no copy CTAs; Llama-2-13B tp=4 on 4 GPUs:
        # 2,125 ms/step) or "kernel" (copy CTAs inside the GEMM launch: 2,314 ms; the same
        # schedule over NCCL: 2,337 ms)
        self.gather = os.environ.get("MB200_TP_GATHER", "dma")
        if comm == "fused":
            from .symm import FlagArray, SymmBuffer
            n = rows_local * d
            # two shard buffers / two staging buffers used alternately: a buffer is written
            # again only after a flag handshake that every rank passes after its last read of
            # it (the handshake of the call in between)
            self._shard = [SymmBuffer(n, bf16, self.device, group, zero=False) for _ in range(2)]
            self._staging = [SymmBuffer(self.world * n, bf16, self.device, group)
                             for _ in range(2)]
            self._flags = FlagArray(4, self.device, group)
            n_chunks = (self.rows * d + self.CHUNK - 1) // self.CHUNK
            self._chunk_flags = torch.zeros(n_chunks, dtype=torch.int32, device=self.device)

    # ---------------------------------------------------------------- all-gather -> GEMM
    def ag_gemm(self, x_local: torch.Tensor, w: torch.Tensor, b_mn: bool = False):
        """x_local [rows_local, d] (this rank's rows) -> (AG(x) @ op(w), AG(x)).
        ``w`` is [N, d] (``b_mn=False``) or [d, N] (``b_mn=True``)."""
        T, d = self.rows, self.d
        N = w.shape[1] if b_mn else w.shape[0]
        x_full = torch.empty(T, d, dtype=x_local.dtype, device=x_local.device)
        if self.comm != "fused":
            dist.all_gather_into_tensor(x_full, x_local.contiguous(), group=self.group)
            return ops.gemm(x_full, w, b_mn=b_mn), x_full
        sb = self._shard[self._n_ag & 1]
        self._n_ag += 1
        self._epoch += 1
        xl = x_local.contiguous()
        if xl.data_ptr() % 16 == 0:
            # one launch copies this rank's rows into its symmetric buffer and publishes
            # "rows in place" on every rank; the copy CTAs of the GEMM launch wait for all
            # ranks' flags before they pull (no separate barrier launch)
            K.check(K.lib().mb200_coll_stage(
                sb.tensor.data_ptr(), xl.data_ptr(), xl.numel() * 2, self._flags.ptrs, self.rank,
                self.world, self.SLOT_ROWS, self._epoch, self._flags.counter.data_ptr(), 0,
                K.stream_ptr()), "coll_stage")
            wait_slot, wait_epoch = self.SLOT_ROWS, self._epoch
        else:
            sb.tensor.view(self.rows_local, d).copy_(xl)
            self._flags.barrier(0)  # every rank's rows are in place
            wait_slot, wait_epoch = 0, 0
        out = torch.empty(T, N, dtype=bf16, device=x_local.device)
        n_comm = 12
        shard = self.rows_local * d
        if self.gather == "dma" and wait_epoch and shard % self.CHUNK == 0:
            # the rows travel on the copy engines (a side stream: bounded flag wait, one copy
            # per rank in ring order starting with the own rows, the rows' chunk flags raised
            # behind each copy) while every SM of the GEMM launch multiplies
            self._dma_rows(sb, x_full, shard)
            n_comm, wait_slot, wait_epoch = -1, 0, 0
        K.check(K.lib().mb200_ag_a_gemm(
            x_full.data_ptr(), sb.ptrs_at(0), shard, self.rank, self.world, T, d,
            w.data_ptr(), w.stride(0), int(b_mn), N, out.data_ptr(), N, None, 0, self.CHUNK,
            self._chunk_flags.data_ptr(), self._epoch, self._flags.my_ptr, wait_slot, wait_epoch,
            n_comm, K.status_word(self.device).data_ptr(), K.stream_ptr()), "ag_a_gemm")
        if n_comm < 0:
            torch.cuda.current_stream().wait_stream(self._side)   # later readers of x_full
        return out, x_full

    def _dma_rows(self, sb, x_full: torch.Tensor, shard: int) -> None:
        main = torch.cuda.current_stream()
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        side = self._side
        side.wait_stream(main)                 # the staging copy and x_full's allocation
        x_full.record_stream(side)
        lib, per = K.lib(), shard // self.CHUNK
        with torch.cuda.stream(side):
            st = K.stream_ptr()
            K.check(lib.mb200_wait_flags(self._flags.my_ptr, self.world, self.SLOT_ROWS,
                                         self._epoch, K.status_word(self.device).data_ptr(), st),
                    "wait_flags")
            base, flags = x_full.data_ptr(), self._chunk_flags.data_ptr()
            for k in range(self.world):
                p = (self.rank + k) % self.world
                K.check(lib.mb200_memcpy_d2d_async(base + p * shard * 2, sb.ptrs[p], shard * 2, st),
                        "memcpy_d2d", 0)
                K.check(lib.mb200_memset_d32_async(flags + p * per * 4, self._epoch, per, st),
                        "memset_d32", 0)

    # ------------------------------------------------------------ GEMM -> reduce-scatter
    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, b_mn: bool = False,
                residual_local: Optional[torch.Tensor] = None) -> torch.Tensor:
        """sum over ranks of (a @ op(w)), rows scattered: returns this rank's
        [rows_local, N] (+ residual_local).  ``a`` is [rows, K_local]."""
        T = self.rows
        N = w.shape[1] if b_mn else w.shape[0]
        Kd = a.shape[1]
        if self.comm != "fused":
            part = ops.gemm(a, w, b_mn=b_mn).float()
            dist.all_reduce(part, group=self.group)
            out = part[self.rank * self.rows_local:(self.rank + 1) * self.rows_local]
            if residual_local is not None:
                out = out + residual_local.float()
            return out.to(a.dtype)
        assert N == self.d, "staging buffers are sized for d output columns"
        st = self._staging[self._n_rs & 1]
        self._n_rs += 1
        K.check(K.lib().mb200_gemm_rs(
            a.data_ptr(), w.data_ptr(), T, N, Kd, a.stride(0), w.stride(0), 0, int(b_mn),
            st.ptrs_at(0), self.world, self.rows_local, N, self.rank, K.gemm_impl(),
            K.status_word(self.device).data_ptr(), K.stream_ptr()), "gemm_rs")
        # the sum's launch is also the barrier that says every rank's partial tiles have landed
        self._rs_epoch += 1
        out = torch.empty(self.rows_local, N, dtype=bf16, device=a.device)
        K.check(K.lib().mb200_rs_finish_sync(
            st.tensor.data_ptr(), self.world, self.rows_local, N, N,
            0 if residual_local is None else residual_local.data_ptr(),
            0 if residual_local is None else residual_local.stride(0), out.data_ptr(), N,
            self._flags.ptrs, self.rank, self.SLOT_TILES, self._rs_epoch,
            K.status_word(self.device).data_ptr(), K.stream_ptr()), "rs_finish")
        return out

    def all_reduce_(self, t: torch.Tensor) -> None:
        """Sum a (small) tensor over the group in place: gradients of replicated params."""
        if t.dtype == bf16 and dist.get_backend(self.group) != "nccl":
            f = t.float()
            dist.all_reduce(f, group=self.group)
            t.copy_(f)
        else:
            dist.all_reduce(t, group=self.group)


class TPStageEngine:
    """Forward/backward of the layers [lo, hi) of a model on one tensor-parallel group,
    one micro-batch at a time (so a pipeline schedule can interleave them).

    ``forward(mb, x_in)`` takes this rank's rows of the stage input ([T/tp, d]; token ids
    [B, S] on the first stage) and returns this rank's rows of the stage output, or the
    local loss sum on the last stage (whose ``forward`` also runs the head's backward and
    keeps d(loss)/d(stage output rows)).  ``backward(mb, dy)`` returns d(loss)/d(stage
    input rows).  Only the stage input of each micro-batch is kept; layers are recomputed
    in ``backward`` (activation checkpointing).
    """

    def __init__(self, cfg: LlamaConfig, group, device, seq_len: int, micro_batch: int,
                 layers: tuple, has_embed: bool, has_head: bool, seed: int = 0,
                 comm: str = "fused", init_std: float = 0.02, n_microbatches: int = 1):
        self.cfg, self.group = cfg, group
        self.device = torch.device(device)
        self.tp = dist.get_world_size(group)
        self.tp_rank = dist.get_rank(group)
        self.S, self.B = seq_len, micro_batch
        self.T = seq_len * micro_batch
        if self.T % self.tp:
            raise ValueError("tokens per micro-batch must be divisible by tp")
        self.Tl = self.T // self.tp
        self.has_embed, self.has_head = has_embed, has_head
        self.n_mb = n_microbatches
        self.layout = ParamLayout(cfg, tp=self.tp, layers=layers, embed=has_embed, head=has_head)
        self.store = LocalParamStore(self.layout, self.device, seed=seed * 64 + 1 + self.tp_rank,
                                     init_std=init_std)
        self.comm = TPComm(group, self.device, self.Tl, cfg.d, comm)
        self._sync_replicated()
        self.cos, self.sin = ops.reference.rope_tables(seq_len, cfg.hd, cfg.theta,
                                                       device=self.device)
        self.Hq, self.Hkv = cfg.n_heads // self.tp, cfg.n_kv_heads // self.tp
        self._inputs: dict = {}
        self._dys: dict = {}
        self._grads_dirty = False

    # ---------------------------------------------------------------- replicated params
    def _replicated(self):
        """(unit index, name) of every parameter that all tp ranks hold in full."""
        for ui, u in enumerate(self.layout.units):
            for p in u.params:
                if len(p.shape) == 1 or p.name in ("embed", "lm_head"):
                    yield ui, p.name

    def _sync_replicated(self):
        src = dist.get_global_rank(self.group, 0)
        for ui, name in self._replicated():
            t = self.store.unit_params(ui)[name]
            if t.dtype == bf16 and dist.get_backend(self.group) != "nccl":
                f = t.float()
                dist.broadcast(f, src, group=self.group)
                t.copy_(f)
            else:
                dist.broadcast(t, src, group=self.group)
        self.store.master.copy_(self.store.params)

    # --------------------------------------------------------------------- one layer
    def _layer_fwd(self, w, x, keep):
        cfg, c = self.cfg, self.comm
        h1, rstd1 = ops.rmsnorm_fwd(x, w["attn_norm"], cfg.eps)
        qkv, h1f = c.ag_gemm(h1, w["wqkv"])
        ops.rope_(qkv, self.cos, self.sin, self.S, self.Hq + self.Hkv, cfg.hd)
        attn, actx = ops.attention_fwd(qkv, self.B, self.S, self.Hq, self.Hkv, cfg.hd,
                                       need_bwd=keep)
        x2 = c.gemm_rs(attn, w["wo"], residual_local=x)
        h2, rstd2 = ops.rmsnorm_fwd(x2, w["mlp_norm"], cfg.eps)
        gu, h2f = c.ag_gemm(h2, w["w_gu"])
        hmid = self._swiglu_fwd(gu)
        y = c.gemm_rs(hmid, w["w_down"], residual_local=x2)
        saved = (x, rstd1, h1f, actx, attn, x2, rstd2, h2f, gu, hmid) if keep else None
        return y, saved

    def _swiglu_fwd(self, gu):
        return ops.swiglu_fwd(gu)

    def _layer_bwd(self, w, g, saved, dy, acc, acc_w=None, defer=None):
        """Backward of one layer.  ``acc``: accumulate into the norm-gain gradients,
        ``acc_w`` (default ``acc``): into the matrix gradients.  With ``defer`` (a list) the
        weight-gradient GEMMs are not run: their operands are appended for
        :meth:`backward_weight` (zero-bubble schedules split B into BI and W)."""
        cfg, c = self.cfg, self.comm
        acc_w = acc if acc_w is None else acc_w

        def wgrad(d_out, inp, name):
            if defer is not None:
                defer.append((d_out, inp, g[name]))
            else:
                ops.gemm(d_out, inp, a_mn=True, b_mn=True, out=g[name], accumulate=acc_w)

        x, rstd1, h1f, actx, attn, x2, rstd2, h2f, gu, hmid = saved
        d_hmid, dyf = c.ag_gemm(dy, w["w_down"], b_mn=True)
        wgrad(dyf, hmid, "w_down")
        d_gu = ops.swiglu_bwd(gu, d_hmid)
        del d_hmid, dyf
        d_h2 = c.gemm_rs(d_gu, w["w_gu"], b_mn=True)
        wgrad(d_gu, h2f, "w_gu")
        del d_gu
        d_x2 = ops.rmsnorm_bwd(d_h2, x2, w["mlp_norm"], rstd2, g["mlp_norm"], accumulate=acc,
                               dres=dy)
        d_attn, dx2f = c.ag_gemm(d_x2, w["wo"], b_mn=True)
        wgrad(dx2f, attn, "wo")
        del dx2f
        d_qkv = ops.attention_bwd(actx, d_attn)
        ops.rope_(d_qkv, self.cos, self.sin, self.S, self.Hq + self.Hkv, cfg.hd, inverse=True)
        d_h1 = c.gemm_rs(d_qkv, w["wqkv"], b_mn=True)
        wgrad(d_qkv, h1f, "wqkv")
        return ops.rmsnorm_bwd(d_h1, x, w["attn_norm"], rstd1, g["attn_norm"], accumulate=acc,
                               dres=d_x2)

    def _layer_units(self):
        lo, hi = self.layout.layer_range
        base = 1 if self.has_embed else 0
        return [(base + k) for k in range(hi - lo)]

    # ------------------------------------------------------------------ micro-batch API
    def begin_step(self):
        self._inputs.clear()
        self._dys.clear()
        self._seen_bwd = 0
        self._seen_w = 0
        self._wstash = {}
        if self.has_embed:
            self.store.unit_grads(0)["embed"].zero_()

    def forward(self, mb: int, x_in: torch.Tensor, targets: Optional[torch.Tensor] = None):
        st, cfg = self.store, self.cfg
        r0, r1 = self.tp_rank * self.Tl, (self.tp_rank + 1) * self.Tl
        if self.has_embed:
            ids = x_in.reshape(-1)[r0:r1].contiguous()
            self._inputs[mb] = ids
            x = ops.embedding_fwd(st.unit_params(0)["embed"], ids)
        else:
            self._inputs[mb] = x_in
            x = x_in
        ckpt = []
        for ui in self._layer_units():
            ckpt.append(x)
            x, _ = self._layer_fwd(st.unit_params(ui), x, keep=False)
        self._inputs[mb] = (self._inputs[mb], ckpt)
        if not self.has_head:
            return x
        # ---- head on this rank's rows (sequence-parallel), loss and its backward
        hu = len(self.layout.units) - 1
        wh, gh = st.unit_params(hu), st.unit_grads(hu)
        acc = mb > 0
        if cfg.tie_embeddings:
            w_out, g_out = st.unit_params(0)["embed"], st.unit_grads(0)["embed"]
            acc = True  # zeroed in begin_step, shared with the embedding gradient
        else:
            w_out, g_out = wh["lm_head"], gh["lm_head"]
        hf, rstdf = ops.rmsnorm_fwd(x, wh["final_norm"], cfg.eps)
        logits = ops.gemm(hf, w_out)
        tg = targets.reshape(-1)[r0:r1].contiguous()
        loss_rows = ops.cross_entropy_(logits, tg, 1.0 / (self.T * self.n_mb))
        d_hf = ops.gemm(logits, w_out, b_mn=True)
        ops.gemm(logits, hf, a_mn=True, b_mn=True, out=g_out, accumulate=acc)
        del logits
        self._dys[mb] = ops.rmsnorm_bwd(d_hf, x, wh["final_norm"], rstdf, gh["final_norm"],
                                        accumulate=mb > 0)
        return loss_rows.sum()

    def backward(self, mb: int, dy: Optional[torch.Tensor] = None,
                 split: bool = False) -> Optional[torch.Tensor]:
        """Backward of micro-batch ``mb`` through this stage; returns the gradient for the
        previous stage (None on the first).  ``split=True`` is the BI action of a
        zero-bubble schedule: only input gradients (and the cheap norm-gain gradients) are
        computed now, the weight-gradient GEMMs wait for :meth:`backward_weight`."""
        st = self.store
        if self.has_head:
            dy = self._dys.pop(mb)
        first, ckpt = self._inputs.pop(mb)
        acc = self._seen_bwd > 0
        self._seen_bwd += 1
        defer = [] if split else None
        acc_w = self._seen_w > 0
        if not split:
            self._seen_w += 1
        units = self._layer_units()
        for k in reversed(range(len(units))):
            ui = units[k]
            w, g = st.unit_params(ui), st.unit_grads(ui)
            _, saved = self._layer_fwd(w, ckpt[k], keep=True)
            dy = self._layer_bwd(w, g, saved, dy, acc, acc_w, defer)
            ckpt[k] = None
        if split:
            self._wstash[mb] = defer
        if self.has_embed:
            ops.embedding_bwd_(dy, first, st.unit_grads(0)["embed"])
            return None
        return dy

    def backward_weight(self, mb: int) -> None:
        """The W action: weight gradients of micro-batch ``mb`` from the operands that its
        BI action kept."""
        acc_w = self._seen_w > 0
        self._seen_w += 1
        for d_out, inp, g_out in self._wstash.pop(mb):
            ops.gemm(d_out, inp, a_mn=True, b_mn=True, out=g_out, accumulate=acc_w)

    def optimizer_step(self, lr: float, **kw):
        # gradients of replicated parameters: every rank saw only its own rows
        for ui, name in self._replicated():
            self.comm.all_reduce_(self.store.unit_grads(ui)[name])
        self.store.optimizer_step(lr, **kw)

    # ------------------------------------------------------- state_dict interchange
    def _split(self, name: str, full: torch.Tensor) -> torch.Tensor:
        """This rank's shard of a full (Hugging Face shaped, fused) layer parameter."""
        cfg, W, r = self.cfg, self.tp, self.tp_rank
        hd = cfg.hd
        if name == "wqkv":
            q, k, v = full.split([cfg.n_heads * hd, cfg.n_kv_heads * hd, cfg.n_kv_heads * hd], 0)
            return torch.cat([t.chunk(W, 0)[r] for t in (q, k, v)], 0)
        if name == "w_gu":
            gate, up = full.split([cfg.ffn, cfg.ffn], 0)
            return torch.cat([gate.chunk(W, 0)[r], up.chunk(W, 0)[r]], 0)
        if name in ("wo", "w_down"):
            return full.chunk(W, 1)[r]
        return full

    def _merge(self, name: str, shards: list) -> torch.Tensor:
        cfg, W = self.cfg, self.tp
        hd = cfg.hd
        if name == "wqkv":
            nq, nk = cfg.n_heads * hd // W, cfg.n_kv_heads * hd // W
            parts = [s.split([nq, nk, nk], 0) for s in shards]
            return torch.cat([torch.cat([p[i] for p in parts], 0) for i in range(3)], 0)
        if name == "w_gu":
            parts = [s.split([cfg.ffn // W, cfg.ffn // W], 0) for s in shards]
            return torch.cat([torch.cat([p[i] for p in parts], 0) for i in range(2)], 0)
        if name in ("wo", "w_down"):
            return torch.cat(shards, 1)
        return shards[0]

    def load_full_units(self, full_layout: ParamLayout, full_flat: torch.Tensor) -> None:
        """Fill this rank's parameters from a full (tp=1, all layers) flat buffer."""
        for ui, u in enumerate(self.layout.units):
            fu = full_layout.units[full_layout.unit_index(u.name)]
            src = full_layout.views(fu, full_flat[fu.offset: fu.offset + fu.size])
            dst = self.store.unit_params(ui)
            for name, t in dst.items():
                t.copy_(self._split(name, src[name]).to(t.device))
        self.store.master.copy_(self.store.params)

    def gather_full_units(self) -> dict:
        """{unit name: {param name: full tensor (CPU)}} of this stage, on every rank."""
        out = {}
        for ui, u in enumerate(self.layout.units):
            views = self.store.unit_params(ui)
            d = {}
            for name, t in views.items():
                if len(t.shape) == 1 or name in ("embed", "lm_head"):
                    d[name] = t.detach().cpu().clone()
                    continue
                tt = t.contiguous()
                if tt.dtype == bf16 and dist.get_backend(self.group) != "nccl":
                    tt = tt.float()
                parts = [torch.empty_like(tt) for _ in range(self.tp)]
                dist.all_gather(parts, tt, group=self.group)
                d[name] = self._merge(name, parts).to(t.dtype).cpu()
            out[u.name] = d
        return out
