"""Llama-family decoder with an explicit forward/backward engine.

The training step is written as explicit kernel launches (no autograd graph, no tracing
compiler): every GEMM is the tcgen05 kernel, every normalisation / activation /
loss / optimizer op is a hand-written sm_100a kernel, and the backward pass is spelled
out per layer so that activation checkpointing, parameter gathering and gradient
reduction can be placed exactly (see :mod:`monarch_b200.parallel`).

Parameters live in one flat bf16 buffer split into *units* (embedding, each decoder
layer, head); a unit is the granularity of FSDP gathering and gradient reduction.
Parameter names and shapes match the Hugging Face Llama ``state_dict`` so checkpoints
interchange with stock torch modules (:func:`to_hf_state_dict`,
:func:`load_hf_state_dict`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from .. import ops

bf16 = torch.bfloat16


@dataclass
class LlamaConfig:
    vocab: int = 128256
    d: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn: int = 14336
    eps: float = 1e-5
    theta: float = 500000.0
    tie_embeddings: bool = False
    name: str = "llama"
    n_experts: int = 0   # > 0: Mixtral-style mixture of SwiGLU experts in place of the MLP
    top_k: int = 2

    @property
    def hd(self) -> int:
        return self.d // self.n_heads

    @property
    def qkv_dim(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * self.hd

    def n_params(self) -> int:
        per_layer = (2 * self.d + self.qkv_dim * self.d + self.d * self.d +
                     2 * self.ffn * self.d + self.d * self.ffn)
        n = self.vocab * self.d + self.n_layers * per_layer + self.d
        if not self.tie_embeddings:
            n += self.vocab * self.d
        return n

    def flops_per_token(self, seq_len: int, recompute: bool = False) -> float:
        """FLOPs per token of one training step; with experts, the ``top_k`` active ones.

        ``recompute=False``: *model* FLOPs, the figure MFU is quoted on -- forward plus
        twice that for backward (3x the forward, attention included).
        ``recompute=True``: what the hardware executes with every layer checkpointed -- the
        GEMMs of the forward run once more (4x), while attention's forward is not repeated
        (its output and log-sum-exp are kept) but its backward recomputes the scores
        (2.5x its forward), 3.5x in all."""
        act = self.top_k if self.n_experts else 1
        mm = self.n_layers * (self.qkv_dim * self.d + self.d * self.d +
                              act * 3 * self.ffn * self.d + self.n_experts * self.d)
        mm += self.vocab * self.d
        attn = self.n_layers * 2 * seq_len * self.d / 2  # causal QK^T + PV, per token
        if not recompute:
            return 3 * (2 * mm + 2 * attn)
        head = self.vocab * self.d                       # the head is not checkpointed
        return 2 * (4 * (mm - head) + 3 * head) + 2 * attn * 3.5

PRESETS: dict[str, LlamaConfig] = {
    "llama3-8b": LlamaConfig(128256, 4096, 32, 32, 8, 14336, 1e-5, 500000.0, False, "llama3-8b"),
    "llama3.2-1b": LlamaConfig(128256, 2048, 16, 32, 8, 8192, 1e-5, 500000.0, True,
                               "llama3.2-1b"),
    "llama2-13b": LlamaConfig(32000, 5120, 40, 40, 40, 13824, 1e-5, 10000.0, False, "llama2-13b"),
    "mixtral-8x7b": LlamaConfig(32000, 4096, 32, 32, 8, 14336, 1e-5, 1e6, False, "mixtral-8x7b",
                                n_experts=8, top_k=2),
    "tiny-moe": LlamaConfig(512, 256, 2, 4, 2, 512, 1e-5, 500000.0, False, "tiny-moe",
                            n_experts=2, top_k=2),
    "tiny-moe4": LlamaConfig(512, 256, 2, 4, 2, 512, 1e-5, 500000.0, False, "tiny-moe4",
                             n_experts=4, top_k=2),
    "tiny": LlamaConfig(512, 256, 2, 4, 2, 512, 1e-5, 500000.0, False, "tiny"),
    "tiny-tied": LlamaConfig(512, 256, 2, 4, 2, 512, 1e-5, 500000.0, True, "tiny-tied"),
}


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    offset: int  # element offset inside its unit


@dataclass
class Unit:
    name: str
    offset: int  # element offset of the unit inside the flat buffer
    size: int    # padded size (multiple of ParamLayout.ALIGN)
    params: list = field(default_factory=list)
    seed_id: int = 0  # position in the full model (embed 0, layer i -> 1+i, head L+1)


class ParamLayout:
    """Flat layout: [embed | layer 0 | ... | layer L-1 | head]; units padded to ALIGN."""
    ALIGN = 8192  # elements: keeps every 1/8 shard 16-byte aligned with room to spare

    def __init__(self, cfg: LlamaConfig, tp: int = 1, layers: Optional[tuple] = None,
                 embed: bool = True, head: bool = True, local_experts: Optional[int] = None):
        """``tp`` > 1: the layout of ONE tensor-parallel rank (Megatron split: wqkv and w_gu
        by output rows -- whole heads / gate and up halves --, wo and w_down by input
        columns; embedding, head and norm gains replicated).  ``layers=(lo, hi)`` with
        ``embed``/``head``: the layout of one pipeline stage."""
        self.cfg = cfg
        self.tp = tp
        # experts held by this rank (expert parallel: n_experts / ep); all of them by default
        self.local_experts = cfg.n_experts if local_experts is None else local_experts
        self.units: list[Unit] = []
        off = 0
        lo, hi = layers if layers is not None else (0, cfg.n_layers)
        self.layer_range = (lo, hi)
        if tp > 1 and (cfg.n_heads % tp or cfg.n_kv_heads % tp or cfg.ffn % tp):
            raise ValueError(f"heads/ffn of {cfg.name} are not divisible by tp={tp}")

        def add_unit(name, specs, seed_id):
            nonlocal off
            u = Unit(name, off, 0, seed_id=seed_id)
            o = 0
            for n, shape in specs:
                u.params.append(ParamSpec(n, tuple(shape), o))
                numel = 1
                for s in shape:
                    numel *= s
                o += _round_up(numel, 8)
            u.size = _round_up(o, self.ALIGN)
            off += u.size
            self.units.append(u)

        d, F = cfg.d, cfg.ffn
        if embed:
            add_unit("embed", [("embed", (cfg.vocab, d))], 0)
        for i in range(lo, hi):
            specs = [("attn_norm", (d,)), ("wqkv", (cfg.qkv_dim // tp, d)),
                     ("wo", (d, cfg.n_heads * cfg.hd // tp)), ("mlp_norm", (d,))]
            if cfg.n_experts:
                # replicated (data-parallel) parameters first, this rank's experts last
                specs.append(("router", (cfg.n_experts, d)))
                for e in range(self.local_experts):
                    specs += [(f"w_gu{e}", (2 * F, d)), (f"w_down{e}", (d, F))]
            else:
                specs += [("w_gu", (2 * F // tp, d)), ("w_down", (d, F // tp))]
            add_unit(f"layer{i}", specs, 1 + i)
        if head:
            hp = [("final_norm", (d,))]
            if not cfg.tie_embeddings:
                hp.append(("lm_head", (cfg.vocab, d)))
            add_unit("head", hp, cfg.n_layers + 1)
        self.total = off

    def unit_index(self, name: str) -> int:
        for i, u in enumerate(self.units):
            if u.name == name:
                return i
        raise KeyError(name)

    def views(self, unit: Unit, flat_unit: torch.Tensor) -> dict:
        out = {}
        for p in unit.params:
            n = 1
            for s in p.shape:
                n *= s
            out[p.name] = flat_unit[p.offset: p.offset + n].view(p.shape)
        return out


class LocalParamStore:
    """All parameters, gradients and optimizer state resident on one device."""

    def __init__(self, layout: ParamLayout, device, seed: int = 0, init_std: float = 0.02):
        self.layout = layout
        self.device = torch.device(device)
        self.params = torch.empty(layout.total, dtype=bf16, device=device)
        self.grads = torch.zeros(layout.total, dtype=bf16, device=device)
        self.master = torch.empty(layout.total, dtype=torch.float32, device=device)
        self.m = torch.zeros(layout.total, dtype=torch.float32, device=device)
        self.v = torch.zeros(layout.total, dtype=torch.float32, device=device)
        init_params_(layout, self.master, seed, init_std)
        self.params.copy_(self.master)
        self.step_count = 0
        # AdamW inside backward (see set_hyper): hyper-parameters of the coming step, the
        # side stream the per-unit updates run on, how many units this step has updated
        self._hyper: Optional[dict] = None
        self._opt_stream = None
        self._updating = False
        self._updated_units = 0

    def set_hyper(self, **kw) -> None:
        """Hyper-parameters of the coming step.  Once they are known before the backward
        pass (``Trainer.step`` sets them), every unit's AdamW update is issued on a side
        stream as soon as that unit's gradients are final: the optimizer is bound by HBM
        bandwidth (28 bytes per parameter), the GEMMs of the remaining backward by the
        tensor cores, so the two overlap instead of the optimizer running alone at the end of
        the step.  The same element-wise kernel runs either way: results are bit-identical.
        ``optimizer_step`` then only joins the side stream."""
        if self._hyper is None:
            self._hyper = dict(lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, grad_scale=1.0)
        self._hyper.update(kw)

    # --- unit access -----------------------------------------------------------------
    def unit_params(self, ui: int) -> dict:
        u = self.layout.units[ui]
        return self.layout.views(u, self.params[u.offset: u.offset + u.size])

    def unit_grads(self, ui: int) -> dict:
        u = self.layout.units[ui]
        return self.layout.views(u, self.grads[u.offset: u.offset + u.size])

    # --- hooks (a resident store has nothing to gather) ------------------------------
    def begin_step(self):
        self._updating = self._hyper is not None and self.device.type == "cuda"
        self._updated_units = 0
        if self._updating and self._opt_stream is None:
            self._opt_stream = torch.cuda.Stream(device=self.device)

    def begin_eval(self):
        self._updating = False

    def pre_forward(self, ui: int):
        pass

    def post_forward(self, ui: int):
        pass

    def pre_backward(self, ui: int):
        pass

    def post_backward(self, ui: int):
        if not self._updating:
            return
        u = self.layout.units[ui]
        lo, hi = u.offset, u.offset + u.size
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self._opt_stream.wait_event(ev)          # the unit's gradients are final
        with torch.cuda.stream(self._opt_stream):
            ops.adamw_(self.master[lo:hi], self.m[lo:hi], self.v[lo:hi], self.grads[lo:hi],
                       self.params[lo:hi], step=self.step_count + 1, **self._hyper)
        self._updated_units += 1

    def optimizer_step(self, lr, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, grad_scale=1.0):
        self.step_count += 1
        if self._updating and self._updated_units == len(self.layout.units):
            # issued unit by unit during backward with the values given to set_hyper; these
            # are recorded for the next step (the contract of the sharded stores)
            self._updating = False
            torch.cuda.current_stream().wait_stream(self._opt_stream)
            self.set_hyper(lr=lr, beta1=beta1, beta2=beta2, eps=eps, wd=wd, grad_scale=grad_scale)
            return
        self._updating = False
        ops.adamw_(self.master, self.m, self.v, self.grads, self.params, lr=lr, beta1=beta1,
                   beta2=beta2, eps=eps, wd=wd, step=self.step_count, grad_scale=grad_scale)

    def full_params(self) -> torch.Tensor:
        return self.params

    def load_full_params(self, flat: torch.Tensor) -> None:
        self.params.copy_(flat)
        self.master.copy_(flat)

    def state_dict_shard(self) -> dict:
        """Everything a resumed run needs from this store (fp32 master weights and moments,
        optimizer step)."""
        return {"master": self.master, "m": self.m, "v": self.v, "step": self.step_count,
                "rank": 0, "world": 1}

    def load_state_dict_shard(self, sd: dict) -> None:
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.step_count = int(sd["step"])
        self.params.copy_(self.master)


def init_params_(layout: ParamLayout, master: torch.Tensor, seed: int, std: float,
                 lo: int = 0, hi: Optional[int] = None) -> None:
    """Deterministic init of the flat fp32 master buffer range [lo, hi): N(0, std) for
    matrices, ones for norm gains, zeros for padding.  Generated per parameter on the
    buffer's device so a shard-only store initialises just its slice consistently."""
    hi = layout.total if hi is None else hi
    for ui, u in enumerate(layout.units):
        if u.offset + u.size <= lo or u.offset >= hi:
            continue
        s, e = max(lo, u.offset), min(hi, u.offset + u.size)
        master[s - lo: e - lo].zero_()
        for pi, p in enumerate(u.params):
            n = 1
            for x in p.shape:
                n *= x
            a, b = u.offset + p.offset, u.offset + p.offset + n
            s, e = max(a, lo), min(b, hi)
            if s >= e:
                continue
            if len(p.shape) == 1:
                master[s - lo: e - lo].fill_(1.0)
                continue
            # Row-chunked generation keyed by (seed, unit, param, chunk): identical values
            # whichever slice of the parameter a rank owns.
            CH = 1 << 22
            c0 = (s - a) // CH
            c1 = (e - a + CH - 1) // CH
            for c in range(c0, c1):
                g = torch.Generator(device=master.device)
                g.manual_seed((seed * 1000003 + u.seed_id * 1009 + pi * 101 + c) & 0x7FFFFFFF)
                cn = min(CH, n - c * CH)
                vals = torch.empty(cn, dtype=torch.float32, device=master.device)
                vals.normal_(0.0, std, generator=g)
                ca, cb = a + c * CH, a + c * CH + cn
                ss, ee = max(ca, s), min(cb, e)
                master[ss - lo: ee - lo].copy_(vals[ss - ca: ee - ca])


def _unit_gemm(w, a: torch.Tensor, name: str) -> torch.Tensor:
    """``a @ w[name]^T``.  A parameter store may hand out a unit whose weights are still
    sharded across ranks and offer ``gemm(a, name)`` to fetch them inside the GEMM kernel
    (FSDP with in-GEMM gathering); a plain dict of views takes the ordinary kernel."""
    f = getattr(w, "gemm", None)
    return f(a, name) if f is not None else ops.gemm(a, w[name])


class LlamaEngine:
    """Explicit training engine: ``loss = engine.forward_backward(tokens, targets)``
    then ``engine.optimizer_step(lr)``.

    ``store`` provides parameters/gradients per unit and receives hooks around each
    unit's forward and backward so that FSDP / DDP / TP variants only swap the store.
    """

    def __init__(self, cfg: LlamaConfig, store, seq_len: int, checkpoint: bool = True,
                 recompute_layers: Optional[int] = None):
        """``checkpoint``: keep only each layer's input (and attention output) in the forward
        and recompute the rest in the backward.  ``recompute_layers`` (with ``checkpoint``):
        how many of the layers, counted from the first, are treated that way; the remaining
        last layers keep all their activations (about 17 bytes per token per model-dim
        element each), trading spare HBM for one skipped forward per kept layer.  Default:
        all layers are recomputed."""
        self.cfg = cfg
        self.store = store
        self.seq_len = seq_len
        self.checkpoint = checkpoint
        if recompute_layers is None:
            recompute_layers = cfg.n_layers if checkpoint else 0
        self.recompute_layers = max(0, min(cfg.n_layers, recompute_layers)) if checkpoint else 0
        dev = store.device
        self.cos, self.sin = ops.reference.rope_tables(seq_len, cfg.hd, cfg.theta, device=dev)
        self.n_units = cfg.n_layers + 2
        # with checkpointing, keep each layer's attention output and log-sum-exp so the
        # recompute pass skips the attention kernel (only with the hand-written kernels,
        # whose backward needs nothing else from the forward)
        self.keep_attention = checkpoint and ops.have_attention_kernel() and \
            torch.device(dev).type == "cuda"

    # ------------------------------------------------------------------ layer forward
    def _attn_fwd(self, w: dict, x: torch.Tensor, B: int, S: int, keep: bool, attn_saved=None):
        """x -> x + attention(norm(x)).  ``attn_saved`` = (o, lse) kept from the first
        forward: the recompute pass then rebuilds q/k/v but does not run the attention kernel
        again (selective checkpointing: 2 bytes per activation element per layer)."""
        cfg = self.cfg
        h1, rstd1 = ops.rmsnorm_fwd(x, w["attn_norm"], cfg.eps)
        qkv = _unit_gemm(w, h1, "wqkv")
        ops.rope_(qkv, self.cos, self.sin, S, cfg.n_heads + cfg.n_kv_heads, cfg.hd)
        if attn_saved is not None:
            attn, actx = ops.attention_ctx_from_saved(qkv, attn_saved, B, S, cfg.n_heads,
                                                      cfg.n_kv_heads, cfg.hd)
        else:
            attn, actx = ops.attention_fwd(qkv, B, S, cfg.n_heads, cfg.n_kv_heads, cfg.hd,
                                           need_bwd=keep or self.keep_attention)
        x2 = ops.gemm(attn, w["wo"], residual=x)
        return x2, (x, rstd1, h1, actx, attn)

    def _mlp_fwd(self, w: dict, x2: torch.Tensor, keep: bool):
        """x2 -> x2 + mlp(norm(x2))."""
        h2, rstd2 = ops.rmsnorm_fwd(x2, w["mlp_norm"], self.cfg.eps)
        gu = _unit_gemm(w, h2, "w_gu")
        hmid = ops.swiglu_fwd(gu)
        y = ops.gemm(hmid, w["w_down"], residual=x2)
        return y, ((x2, rstd2, h2, gu, hmid) if keep else None)

    def _layer_fwd(self, w: dict, x: torch.Tensor, B: int, S: int, keep: bool,
                   attn_saved=None):
        x2, sa = self._attn_fwd(w, x, B, S, keep, attn_saved)
        y, sm = self._mlp_fwd(w, x2, keep)
        if keep:
            return y, (sa, sm)
        actx = sa[3]
        if self.keep_attention and actx.lse is not None:
            return y, (actx.o, actx.lse)
        return y, None

    def _mlp_bwd(self, w: dict, g: dict, sm, dy: torch.Tensor):
        """Gradient w.r.t. x2 (residual path included)."""
        x2, rstd2, h2, gu, hmid = sm
        d_hmid = ops.gemm(dy, w["w_down"], b_mn=True)
        ops.gemm(dy, hmid, a_mn=True, b_mn=True, out=g["w_down"])
        d_gu = ops.swiglu_bwd(gu, d_hmid)
        del d_hmid
        d_h2 = ops.gemm(d_gu, w["w_gu"], b_mn=True)
        ops.gemm(d_gu, h2, a_mn=True, b_mn=True, out=g["w_gu"])
        del d_gu
        return ops.rmsnorm_bwd(d_h2, x2, w["mlp_norm"], rstd2, g["mlp_norm"], dres=dy)

    def _attn_bwd(self, w: dict, g: dict, sa, d_x2: torch.Tensor):
        cfg = self.cfg
        x, rstd1, h1, actx, attn = sa
        d_attn = ops.gemm(d_x2, w["wo"], b_mn=True)
        ops.gemm(d_x2, attn, a_mn=True, b_mn=True, out=g["wo"])
        d_qkv = ops.attention_bwd(actx, d_attn)
        ops.rope_(d_qkv, self.cos, self.sin, actx.S, cfg.n_heads + cfg.n_kv_heads, cfg.hd,
                  inverse=True)
        d_h1 = ops.gemm(d_qkv, w["wqkv"], b_mn=True)
        ops.gemm(d_qkv, h1, a_mn=True, b_mn=True, out=g["wqkv"])
        return ops.rmsnorm_bwd(d_h1, x, w["attn_norm"], rstd1, g["attn_norm"], dres=d_x2)

    def _layer_bwd(self, w: dict, g: dict, saved, dy: torch.Tensor):
        sa, sm = saved
        d_x2 = self._mlp_bwd(w, g, sm, dy)
        return self._attn_bwd(w, g, sa, d_x2)

    # ------------------------------------------------------------------------- step
    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor,
                         loss_scale: Optional[float] = None) -> torch.Tensor:
        """tokens/targets: [B, S] int64 on the engine's device.  Returns the mean
        token loss as a 0-d fp32 device tensor; gradients are left in the store."""
        cfg, st = self.cfg, self.store
        B, S = tokens.shape
        T = B * S
        L = cfg.n_layers
        ids = tokens.reshape(-1)
        tg = targets.reshape(-1)
        st.begin_step()

        # ---- forward
        st.pre_forward(0)
        x = ops.embedding_fwd(st.unit_params(0)["embed"], ids)
        st.post_forward(0)
        ckpt = []
        saved_all = []
        for i in range(L):
            st.pre_forward(1 + i)
            w = st.unit_params(1 + i)
            ckpt.append(x)
            x, saved = self._layer_fwd(w, x, B, S, keep=i >= self.recompute_layers)
            saved_all.append(saved)
            st.post_forward(1 + i)

        # ---- head: final norm, logits, loss, and its backward
        hu = L + 1
        st.pre_forward(hu)
        st.pre_backward(hu)
        wh = st.unit_params(hu)
        gh = st.unit_grads(hu)
        if cfg.tie_embeddings:
            st.pre_backward(0)
            w_out = st.unit_params(0)["embed"]
            g_out = st.unit_grads(0)["embed"]
        else:
            w_out, g_out = wh["lm_head"], gh["lm_head"]
        hf, rstdf = ops.rmsnorm_fwd(x, wh["final_norm"], cfg.eps)
        logits = ops.gemm(hf, w_out)
        scale = (1.0 / T) if loss_scale is None else loss_scale
        loss_rows = ops.cross_entropy_(logits, tg, scale)
        loss = loss_rows.mean()
        d_hf = ops.gemm(logits, w_out, b_mn=True)
        ops.gemm(logits, hf, a_mn=True, b_mn=True, out=g_out)
        del logits
        dx = ops.rmsnorm_bwd(d_hf, x, wh["final_norm"], rstdf, gh["final_norm"])
        del d_hf, hf
        st.post_forward(hu)
        st.post_backward(hu)

        # ---- layers backward (recompute from the checkpoint when enabled)
        for i in reversed(range(L)):
            st.pre_backward(1 + i)
            w = st.unit_params(1 + i)
            g = st.unit_grads(1 + i)
            if i < self.recompute_layers:
                _, saved = self._layer_fwd(w, ckpt[i], B, S, keep=True,
                                           attn_saved=saved_all[i])
                saved_all[i] = None
            else:
                saved = saved_all[i]
                saved_all[i] = None
            dx = self._layer_bwd(w, g, saved, dx)
            ckpt[i] = None
            del saved
            st.post_backward(1 + i)

        # ---- embedding backward
        if not cfg.tie_embeddings:
            st.pre_backward(0)
            st.unit_grads(0)["embed"].zero_()
        ops.embedding_bwd_(dx, ids, st.unit_grads(0)["embed"])
        st.post_backward(0)
        return loss

    def forward_loss(self, tokens, targets) -> torch.Tensor:
        """Forward only (evaluation): mean token loss."""
        cfg, st = self.cfg, self.store
        B, S = tokens.shape
        st.begin_eval()
        st.pre_forward(0)
        x = ops.embedding_fwd(st.unit_params(0)["embed"], tokens.reshape(-1))
        st.post_forward(0)
        for i in range(cfg.n_layers):
            st.pre_forward(1 + i)
            x, _ = self._layer_fwd(st.unit_params(1 + i), x, B, S, keep=False)
            st.post_forward(1 + i)
        hu = cfg.n_layers + 1
        st.pre_forward(hu)
        wh = st.unit_params(hu)
        if cfg.tie_embeddings:
            st.pre_forward(0)
            w_out = st.unit_params(0)["embed"]
        else:
            w_out = wh["lm_head"]
        hf, _ = ops.rmsnorm_fwd(x, wh["final_norm"], cfg.eps)
        logits = ops.gemm(hf, w_out)
        loss = ops.cross_entropy_(logits, targets.reshape(-1), 0.0).mean()
        if cfg.tie_embeddings:
            st.post_forward(0)
        st.post_forward(hu)
        return loss

    def optimizer_step(self, lr: float, **kw):
        self.store.optimizer_step(lr, **kw)


# ------------------------------------------------------------------ state_dict interchange
def to_hf_state_dict(cfg: LlamaConfig, layout: ParamLayout, flat: torch.Tensor) -> dict:
    """Full flat parameter buffer -> Hugging Face Llama ``state_dict`` (tensor views are
    cloned so the result is an ordinary, independently owned state_dict)."""
    sd = {}
    hd, Hq, Hkv, F = cfg.hd, cfg.n_heads, cfg.n_kv_heads, cfg.ffn
    for ui, u in enumerate(layout.units):
        v = layout.views(u, flat[u.offset: u.offset + u.size])
        if u.name == "embed":
            sd["model.embed_tokens.weight"] = v["embed"].clone()
        elif u.name == "head":
            sd["model.norm.weight"] = v["final_norm"].clone()
            sd["lm_head.weight"] = (v["lm_head"] if "lm_head" in v
                                    else sd["model.embed_tokens.weight"]).clone()
        else:
            i = ui - 1
            p = f"model.layers.{i}."
            sd[p + "input_layernorm.weight"] = v["attn_norm"].clone()
            sd[p + "post_attention_layernorm.weight"] = v["mlp_norm"].clone()
            q, k, vv = v["wqkv"].split([Hq * hd, Hkv * hd, Hkv * hd], dim=0)
            sd[p + "self_attn.q_proj.weight"] = q.clone()
            sd[p + "self_attn.k_proj.weight"] = k.clone()
            sd[p + "self_attn.v_proj.weight"] = vv.clone()
            sd[p + "self_attn.o_proj.weight"] = v["wo"].clone()
            gate, up = v["w_gu"].split([F, F], dim=0)
            sd[p + "mlp.gate_proj.weight"] = gate.clone()
            sd[p + "mlp.up_proj.weight"] = up.clone()
            sd[p + "mlp.down_proj.weight"] = v["w_down"].clone()
    return sd


def load_hf_state_dict(cfg: LlamaConfig, layout: ParamLayout, sd: dict,
                       flat: torch.Tensor) -> None:
    """Inverse of :func:`to_hf_state_dict`: fill a full flat buffer from HF names."""
    for ui, u in enumerate(layout.units):
        v = layout.views(u, flat[u.offset: u.offset + u.size])
        if u.name == "embed":
            v["embed"].copy_(sd["model.embed_tokens.weight"])
        elif u.name == "head":
            v["final_norm"].copy_(sd["model.norm.weight"])
            if "lm_head" in v:
                v["lm_head"].copy_(sd["lm_head.weight"])
        else:
            p = f"model.layers.{ui - 1}."
            v["attn_norm"].copy_(sd[p + "input_layernorm.weight"])
            v["mlp_norm"].copy_(sd[p + "post_attention_layernorm.weight"])
            v["wqkv"].copy_(torch.cat([sd[p + "self_attn.q_proj.weight"],
                                       sd[p + "self_attn.k_proj.weight"],
                                       sd[p + "self_attn.v_proj.weight"]], dim=0))
            v["wo"].copy_(sd[p + "self_attn.o_proj.weight"])
            v["w_gu"].copy_(torch.cat([sd[p + "mlp.gate_proj.weight"],
                                       sd[p + "mlp.up_proj.weight"]], dim=0))
            v["w_down"].copy_(sd[p + "mlp.down_proj.weight"])
