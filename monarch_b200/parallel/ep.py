"""Expert parallelism for Mixtral-style mixture-of-experts layers: one expert per rank of
the ``ep`` mesh dim, top-k routing, attention and router replicated (data parallel).

``comm="fused"`` (GPU): token dispatch and combine are fused with the expert GEMMs --
``mb200_moe_gather_gemm`` pulls the routed token rows from every rank over NVLink while
its tcgen05 CTAs multiply row blocks as they land, and the second GEMM's epilogue stores
each output row straight into the (token, k) slot of the token's home rank
(``mb200_gemm_bf16_ex`` with the scatter epilogue).  Row counts stay on the device: the
kernels read them from the ranks' routing tables, so the step has no host synchronisation.
The backward pass runs the same two kernels with gradients in place of activations.

``comm="nccl"``: ``all_to_all_single`` with explicit split sizes (one host sync per
dispatch) around separate GEMMs -- the library baseline and the CPU (gloo) test path.

Router weights multiply the expert's hidden activation (h = w * silu(g) * u), so the
combine is a plain sum and the backward dispatch needs no scaling.

The reference has no expert parallelism; its closest primitive is the all-to-all behind
``reduce("stack", scatter=True)`` (python/monarch/common/tensor.py:251-254).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops import kernels as K
from ..ops import reference as R

bf16 = torch.bfloat16


def _swiglu_scaled_fwd(gu: torch.Tensor, w_row: torch.Tensor) -> torch.Tensor:
    F = gu.shape[1] // 2
    g, u = gu[:, :F].float(), gu[:, F:].float()
    return (torch.nn.functional.silu(g) * u * w_row[:, None]).to(gu.dtype)


def _swiglu_scaled_bwd(gu, dh, w_row):
    F = gu.shape[1] // 2
    g, u, d = gu[:, :F].float(), gu[:, F:].float(), dh.float()
    sg = torch.sigmoid(g)
    silu = g * sg
    dw = (d * silu * u).sum(1)
    dhw = d * w_row[:, None]
    dg = dhw * u * (sg * (1 + g * (1 - sg)))
    du = dhw * silu
    return torch.cat([dg, du], 1).to(gu.dtype), dw


class _Saved:
    __slots__ = ("a", "gu", "h", "w_row", "order", "send_counts", "recv_counts", "row_rank",
                 "row_slot", "m_count", "cap")


class EPComm:
    """Dispatch -> expert FFN -> combine for one expert-parallel group."""

    def __init__(self, group, device, tokens: int, d: int, ffn: int, top_k: int = 2,
                 comm: str = "fused", capacity: Optional[int] = None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device(device)
        self.T, self.d, self.F, self.k = tokens, d, ffn, top_k
        if self.device.type != "cuda" and comm == "fused":
            comm = "nccl"
        self.comm = comm
        # rows one expert can receive; the default covers the worst case (every rank sends
        # every token), smaller values drop the overflow like a capacity factor does
        self.cap = capacity or self.world * tokens
        self._epoch = 0
        if comm == "fused":
            from .symm import FlagArray, SymmBuffer
            E = self.world
            mk = lambda n, dt: SymmBuffer(n, dt, self.device, group)
            self._counts = mk(max(E, 8), torch.int32)
            self._lists = mk(E * tokens, torch.int32)
            self._rows = mk(tokens * d, bf16)
            self._wts = mk(tokens * top_k, torch.float32)
            self._comb = mk(tokens * top_k * d, bf16)
            self._dw = mk(tokens * top_k, torch.float32)
            self._flags = FlagArray(4, self.device, group)
            self._row_flags = torch.zeros((self.cap + 15) // 16, dtype=torch.int32,
                                          device=self.device)

    # ------------------------------------------------------------------ fused helpers
    def _gather_gemm(self, w, b_mn, with_weights):
        cap, d = self.cap, self.d
        dev = self.device
        N = w.shape[1] if b_mn else w.shape[0]
        a = torch.empty(cap, d, dtype=bf16, device=dev)
        out = torch.empty(cap, N, dtype=bf16, device=dev)
        row_rank = torch.empty(cap, dtype=torch.int32, device=dev)
        row_slot = torch.empty(cap, dtype=torch.int32, device=dev)
        row_w = torch.empty(cap, dtype=torch.float32, device=dev)
        m_count = torch.empty(1, dtype=torch.int32, device=dev)
        self._epoch += 1
        K.check(K.lib().mb200_moe_gather_gemm(
            self._counts.ptrs_at(0), self._lists.ptrs_at(0), self._rows.ptrs_at(0),
            self._wts.ptrs_at(0) if with_weights else None, self.world, self.rank, self.T, self.k,
            d, cap, a.data_ptr(), row_rank.data_ptr(), row_slot.data_ptr(), row_w.data_ptr(),
            m_count.data_ptr(), self._row_flags.data_ptr(), self._epoch, w.data_ptr(),
            w.stride(0), int(b_mn), N, out.data_ptr(), N, 24,
            K.status_word(dev).data_ptr(), K.stream_ptr()), "moe_gather_gemm")
        return out, a, row_rank, row_slot, row_w, m_count

    def _gemm_ex(self, a, b, out, M, N, Kd, a_mn, b_mn, accumulate=False, dyn_m=None, dyn_k=None,
                 scatter=None):
        sc = scatter
        K.check(K.lib().mb200_gemm_bf16_ex(
            a.data_ptr(), b.data_ptr(), 0 if out is None else out.data_ptr(), M, N, Kd,
            a.stride(0), b.stride(0), 0 if out is None else out.stride(0), int(a_mn), int(b_mn),
            int(accumulate), 0 if dyn_m is None else dyn_m.data_ptr(),
            0 if dyn_k is None else dyn_k.data_ptr(),
            0 if sc is None else sc[0].data_ptr(), 0 if sc is None else sc[1].data_ptr(),
            None if sc is None else self._comb.ptrs_at(0), self.world, self.d, K.gemm_impl(),
            K.status_word(self.device).data_ptr(), K.stream_ptr()), "gemm_bf16_ex")

    def _combine(self, residual):
        out = torch.empty(self.T, self.d, dtype=bf16, device=self.device)
        K.check(K.lib().mb200_moe_combine(
            self._comb.tensor.data_ptr(), self.T, self.k, self.d,
            0 if residual is None else residual.data_ptr(),
            0 if residual is None else residual.stride(0), out.data_ptr(), self.d,
            K.stream_ptr()), "moe_combine")
        return out

    # ------------------------------------------------------------------------ forward
    def forward(self, x, top_idx, wts, w_gu, w_down, residual=None):
        """x [T, d]; top_idx [T, k] int32 expert ids; wts [T, k] fp32 router weights.
        Returns (y [T, d] = sum_k w_k * expert_k(x) + residual, saved-for-backward)."""
        sv = _Saved()
        if self.comm == "fused":
            if self.cap < self.world * self.T:
                self._comb.tensor.zero_()   # slots of tokens dropped by the capacity limit
            self._wts.tensor.copy_(wts.reshape(-1))
            self._rows.tensor.view(self.T, self.d).copy_(x)
            K.check(K.lib().mb200_moe_route(top_idx.data_ptr(), self.T, self.k, self.world,
                                            self._counts.tensor.data_ptr(),
                                            self._lists.tensor.data_ptr(), K.stream_ptr()),
                    "moe_route", 1)
            self._flags.barrier(0)
            gu, a, rr, rs, rw, mc = self._gather_gemm(w_gu, False, True)
            h = torch.empty(self.cap, self.F, dtype=bf16, device=self.device)
            K.check(K.lib().mb200_moe_swiglu_fwd(gu.data_ptr(), rw.data_ptr(), mc.data_ptr(),
                                                 h.data_ptr(), self.cap, self.F, K.stream_ptr()),
                    "moe_swiglu_fwd")
            self._gemm_ex(h, w_down, None, self.cap, self.d, self.F, False, False, dyn_m=mc,
                          scatter=(rr, rs))
            self._flags.barrier(1)
            y = self._combine(residual)
            sv.a, sv.gu, sv.h, sv.w_row, sv.row_rank, sv.row_slot, sv.m_count = a, gu, h, rw, rr, rs, mc
            return y, sv
        # ---- library path
        flat_e = top_idx.reshape(-1).long()
        order = torch.argsort(flat_e, stable=True)
        send_counts = torch.bincount(flat_e, minlength=self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        a = self._a2a(x[order // self.k], rc, sc)
        w_row = self._a2a(wts.reshape(-1)[order].contiguous(), rc, sc)
        gu = ops.gemm(a, w_gu)
        h = _swiglu_scaled_fwd(gu, w_row)
        back = self._a2a(ops.gemm(h, w_down), sc, rc)
        comb = torch.zeros(self.T * self.k, self.d, dtype=torch.float32, device=x.device)
        comb[order] = back.float()
        y = comb.view(self.T, self.k, self.d).sum(1)
        if residual is not None:
            y = y + residual.float()
        sv.a, sv.gu, sv.h, sv.w_row, sv.order, sv.send_counts, sv.recv_counts = \
            a, gu, h, w_row, order, sc, rc
        return y.to(x.dtype), sv

    def _a2a(self, send, recv_counts, send_counts):
        shape = (sum(recv_counts),) + tuple(send.shape[1:])
        if send.dtype == bf16 and dist.get_backend(self.group) != "nccl":
            out = torch.empty(shape, dtype=torch.float32, device=send.device)
            dist.all_to_all_single(out, send.float().contiguous(), recv_counts, send_counts,
                                   group=self.group)
            return out.to(bf16)
        out = torch.empty(shape, dtype=send.dtype, device=send.device)
        dist.all_to_all_single(out, send.contiguous(), recv_counts, send_counts, group=self.group)
        return out

    # ----------------------------------------------------------------------- backward
    def backward(self, dy, sv: _Saved, w_gu, w_down, g_gu, g_down, acc: bool):
        """dy [T, d] -> (d_x [T, d] through the experts, d_wts [T, k] fp32); accumulates
        (``acc``) or writes the expert weight gradients."""
        if self.comm == "fused":
            if self.cap < self.world * self.T:
                self._comb.tensor.zero_()
                self._dw.tensor.zero_()
            self._rows.tensor.view(self.T, self.d).copy_(dy)
            self._flags.barrier(0)
            d_h, dye, rr, rs, _, mc = self._gather_gemm(w_down, True, False)
            self._gemm_ex(dye, sv.h, g_down, self.d, self.F, self.cap, True, True, accumulate=acc,
                          dyn_k=mc)
            d_gu = torch.empty(self.cap, 2 * self.F, dtype=bf16, device=self.device)
            K.check(K.lib().mb200_moe_swiglu_bwd(
                sv.gu.data_ptr(), d_h.data_ptr(), sv.w_row.data_ptr(), mc.data_ptr(),
                rr.data_ptr(), rs.data_ptr(), d_gu.data_ptr(), self._dw.ptrs_at(0), self.world,
                self.cap, self.F, K.stream_ptr()), "moe_swiglu_bwd")
            self._gemm_ex(d_gu, sv.a, g_gu, 2 * self.F, self.d, self.cap, True, True,
                          accumulate=acc, dyn_k=mc)
            self._gemm_ex(d_gu, w_gu, None, self.cap, self.d, 2 * self.F, False, True, dyn_m=mc,
                          scatter=(rr, rs))
            self._flags.barrier(1)
            d_x = self._combine(None)
            return d_x, self._dw.tensor.view(self.T, self.k).clone()
        order, sc, rc = sv.order, sv.send_counts, sv.recv_counts
        dye = self._a2a(dy[order // self.k], rc, sc)
        d_h = ops.gemm(dye, w_down, b_mn=True)
        ops.gemm(dye, sv.h, a_mn=True, b_mn=True, out=g_down, accumulate=acc)
        d_gu, dw_row = _swiglu_scaled_bwd(sv.gu, d_h, sv.w_row)
        ops.gemm(d_gu, sv.a, a_mn=True, b_mn=True, out=g_gu, accumulate=acc)
        back = self._a2a(ops.gemm(d_gu, w_gu, b_mn=True), sc, rc)
        dw_back = self._a2a(dw_row.contiguous(), sc, rc)
        dcomb = torch.zeros(self.T * self.k, self.d, dtype=torch.float32, device=dy.device)
        dcomb[order] = back.float()
        d_wts = torch.zeros(self.T * self.k, dtype=torch.float32, device=dy.device)
        d_wts[order] = dw_back
        return dcomb.view(self.T, self.k, self.d).sum(1).to(dy.dtype), d_wts.view(self.T, self.k)


# ===================================================================== engine and store
from ..models.llama import LlamaEngine, ParamLayout  # noqa: E402
from .ddp import DDPParamStore  # noqa: E402


class EPParamStore(DDPParamStore):
    """Replicated attention/router/norm/embedding parameters (gradients all-reduced in
    buckets, overlapped with backward) plus this rank's expert, which is private: its
    gradient already holds the contributions of every rank's tokens.

    The engine scales the loss by 1/(tokens * world), so the all-reduce is a plain sum."""

    def __init__(self, layout: ParamLayout, device, seed: int = 0, init_std: float = 0.02,
                 comm: str = "fused", group=None, bucket_bytes: int = 25 * 1024 * 1024):
        super().__init__(layout, device, seed=seed, init_std=init_std, comm=comm, group=group,
                         bucket_bytes=bucket_bytes)
        self.reduce_scale = 1.0
        # experts differ per rank: redraw them with a rank-specific stream
        g = torch.Generator(device=self.device)
        for ui, u in enumerate(layout.units):
            for p in u.params:
                if p.name.startswith(("w_gu", "w_down")) and p.name not in ("w_gu", "w_down"):
                    n = 1
                    for x in p.shape:
                        n *= x
                    a = u.offset + p.offset
                    g.manual_seed((seed * 7907 + self.rank * 104729 + u.seed_id * 131 +
                                   hash(p.name) % 997) & 0x7FFFFFFF)
                    self.master[a: a + n].normal_(0.0, init_std, generator=g)
        self.params.copy_(self.master)

    def _reduced_extent(self, ui: int) -> int:
        u = self.layout.units[ui]
        for p in u.params:
            if p.name.startswith(("w_gu", "w_down")) and p.name not in ("w_gu", "w_down"):
                return p.offset // 8 * 8
        return u.size


class MoEEngine(LlamaEngine):
    """Llama engine whose MLP is a top-k mixture of experts, one expert per ``ep`` rank."""

    def __init__(self, cfg, store, seq_len: int, ep: EPComm, checkpoint: bool = True):
        super().__init__(cfg, store, seq_len, checkpoint=checkpoint)
        assert cfg.n_experts == ep.world, "one expert per rank of the ep group"
        self.ep = ep
        self.world = ep.world

    def _route(self, h2, wr, need_grad: bool):
        ctx = torch.enable_grad() if need_grad else torch.no_grad()
        with ctx:
            logits = h2.float() @ wr.float().t()
            probs = torch.softmax(logits, dim=-1)
            top_p, top_i = torch.topk(probs, self.cfg.top_k, dim=-1)
            wts = top_p / top_p.sum(-1, keepdim=True)
        return top_i, wts

    def _mlp_fwd(self, w, x2, keep):
        h2, rstd2 = ops.rmsnorm_fwd(x2, w["mlp_norm"], self.cfg.eps)
        top_i, wts = self._route(h2, w["router"], False)
        y, sv = self.ep.forward(h2, top_i.to(torch.int32).contiguous(), wts.contiguous(),
                                w["w_gu0"], w["w_down0"], residual=x2)
        return y, ((x2, rstd2, h2, top_i, sv) if keep else None)

    def _mlp_bwd(self, w, g, sm, dy):
        x2, rstd2, h2, top_i, sv = sm
        d_h2, d_wts = self.ep.backward(dy, sv, w["w_gu0"], w["w_down0"], g["w_gu0"], g["w_down0"],
                                       acc=False)
        # router: gradient of the renormalised top-k softmax weights (tiny [T, E] problem)
        h2f = h2.detach().float().requires_grad_(True)
        wr = w["router"].detach().float().requires_grad_(True)
        with torch.enable_grad():
            probs = torch.softmax(h2f @ wr.t(), dim=-1)
            top_p = probs.gather(1, top_i)
            wts = top_p / top_p.sum(-1, keepdim=True)
        gh, gwr = torch.autograd.grad(wts, (h2f, wr), d_wts.to(wts.dtype))
        g["router"].copy_(gwr.to(g["router"].dtype))
        d_h2 = (d_h2.float() + gh).to(dy.dtype)
        return ops.rmsnorm_bwd(d_h2, x2, w["mlp_norm"], rstd2, g["mlp_norm"], dres=dy)

    def forward_backward(self, tokens, targets, loss_scale=None):
        T = tokens.numel()
        loss = super().forward_backward(tokens, targets,
                                        loss_scale=loss_scale or 1.0 / (T * self.world))
        return loss


class MoETrainer:
    """Per-rank driver of a Mixtral-style model on an ``{ep: N}`` mesh (see Trainer)."""

    def __init__(self, model, seq_len: int, micro_batch: int = 1, device=None, comm: str = "fused",
                 lr: float = 3e-4, seed: int = 0, init_std: float = 0.02, capacity=None):
        from ..models.llama import PRESETS
        self.cfg = PRESETS[model] if isinstance(model, str) else model
        self.device = torch.device(device if device is not None else "cpu")
        self.world = dist.get_world_size()
        self.lr = lr
        self.parallelism = "ep"
        self.layout = ParamLayout(self.cfg, local_experts=1)
        self.store = EPParamStore(self.layout, self.device, seed=seed, init_std=init_std,
                                  comm=comm)
        self.ep = EPComm(dist.group.WORLD, self.device, seq_len * micro_batch, self.cfg.d,
                         self.cfg.ffn, self.cfg.top_k, comm=comm, capacity=capacity)
        self.engine = MoEEngine(self.cfg, self.store, seq_len, self.ep)
        shape = (micro_batch, seq_len)
        self._tok = torch.empty(shape, dtype=torch.int64, device=self.device)
        self._tgt = torch.empty(shape, dtype=torch.int64, device=self.device)

    def step_device(self, tokens, targets):
        loss = self.engine.forward_backward(tokens, targets)
        self.engine.optimizer_step(self.lr)
        return loss

    def step(self, tokens, targets) -> float:
        self._tok.copy_(tokens, non_blocking=True)
        self._tgt.copy_(targets, non_blocking=True)
        return float(self.step_device(self._tok, self._tgt).item())

    @property
    def h2d_bytes_per_step(self) -> int:
        return 2 * self._tok.numel() * 8

    @property
    def d2h_bytes_per_step(self) -> int:
        return 4
