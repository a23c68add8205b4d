"""Pipeline runtime: executes one rank's action list of a schedule over a
:class:`~monarch_b200.parallel.tp.TPStageEngine`.

Mesh ``{pp: P, tp: W}`` with global rank ``pp * W + tp``.  Stage boundaries move this
rank's rows of the activation ([T/tp, d]) to the same tp rank of the neighbouring stage
with NCCL point-to-point (``send_tensor`` in the reference's terms).  Each direction of
each stage boundary has its own process group, hence its own NCCL communicator and
stream: receives are posted ahead of time without being queued behind sends of the other
direction, and the transfers overlap the compute stream.

Parity: python/monarch/parallel/pipelining/runtime.py:230-301 (stage construction),
:601-776 (schedule execution with a p2p stream and ``to_mesh``) in the reference.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ...models.llama import PRESETS, LlamaConfig
from ..tp import TPStageEngine
from . import schedule_ir as ir


def build_mesh_groups(pp: int, tp: int):
    """Create (collectively, on every rank) the tp group of each stage and one group per
    stage boundary and direction.  Returns (tp_group, fwd_groups, bwd_groups) where
    fwd_groups[s] links stage s -> s+1 for this rank's tp index (None if not a member)."""
    world = dist.get_world_size()
    rank = dist.get_rank()
    assert world == pp * tp, f"world {world} != pp {pp} x tp {tp}"
    my_pp, my_tp = divmod(rank, tp)
    tp_group = None
    for s in range(pp):
        g = dist.new_group([s * tp + t for t in range(tp)])
        if s == my_pp:
            tp_group = g
    fwd: List[Optional[dist.ProcessGroup]] = [None] * max(pp - 1, 0)
    bwd: List[Optional[dist.ProcessGroup]] = [None] * max(pp - 1, 0)
    for s in range(pp - 1):
        for t in range(tp):
            pair = [s * tp + t, (s + 1) * tp + t]
            gf = dist.new_group(pair)
            gb = dist.new_group(pair)
            if rank in pair:
                fwd[s], bwd[s] = gf, gb
    return tp_group, fwd, bwd


class PipelineTrainer:
    """One object per rank of a ``{pp, tp}`` mesh: owns the stage engine and runs a
    schedule (default 1F1B) over ``n_microbatches`` micro-batches per optimizer step."""

    def __init__(self, model: str | LlamaConfig, pp: int, tp: int, seq_len: int,
                 micro_batch: int = 1, n_microbatches: int = 8, device=None,
                 schedule: str = "1f1b", comm: str = "fused", lr: float = 3e-4, seed: int = 0,
                 init_std: float = 0.02):
        self.cfg = PRESETS[model] if isinstance(model, str) else model
        self.pp, self.tp = pp, tp
        self.rank = dist.get_rank()
        self.stage, self.tp_rank = divmod(self.rank, tp)
        self.device = torch.device(device if device is not None else "cpu")
        self.n_mb, self.lr = n_microbatches, lr
        self.seq_len, self.micro_batch = seq_len, micro_batch
        self.tp_group, self._fwd_groups, self._bwd_groups = build_mesh_groups(pp, tp)
        L = self.cfg.n_layers
        per = (L + pp - 1) // pp
        lo, hi = self.stage * per, min(L, (self.stage + 1) * per)
        self.engine = TPStageEngine(self.cfg, self.tp_group, self.device, seq_len, micro_batch,
                                    (lo, hi), has_embed=self.stage == 0,
                                    has_head=self.stage == pp - 1, seed=seed, comm=comm,
                                    init_std=init_std, n_microbatches=n_microbatches)
        self._warm_up_links()
        sched = ir.GENERATORS[schedule](pp, n_microbatches)
        ir.validate(sched, pp, n_microbatches)
        self.actions = ir.add_communication(sched, pp)[self.stage]
        self.parallelism = f"pp{pp}xtp{tp}"
        import os
        # receives are posted right before they are needed unless asked otherwise: a
        # receive posted far ahead is a kernel that sits on the GPU until its sender runs
        self.prepost = os.environ.get("MB200_PP_PREPOST", "0") == "1"
        self._debug = os.environ.get("MB200_PP_DEBUG", "0") == "1" and \
            self.device.type == "cuda"
        self.Tl = self.engine.Tl
        self._tok = torch.empty(n_microbatches, micro_batch, seq_len, dtype=torch.int64,
                                device=self.device)
        self._tgt = torch.empty_like(self._tok)

    # -------------------------------------------------------------------------------
    def _warm_up_links(self) -> None:
        """The first send/recv on a communicator sets up the connection and blocks the host
        until the peer has entered the matching call.  Do that here, one boundary and one
        direction at a time in an order every rank agrees on, so that the receives posted
        ahead of time in ``step_device`` never meet an unconnected link (two stages each
        blocked in the set-up of a different link would wait for each other forever)."""
        s = self.stage
        t = torch.zeros(8, dtype=torch.float32, device=self.device)
        for b in range(self.pp - 1):
            if s == b:
                dist.send(t, self._peer(b + 1), group=self._fwd_groups[b])
            elif s == b + 1:
                dist.recv(t, self._peer(b), group=self._fwd_groups[b])
        for b in range(self.pp - 1):
            if s == b + 1:
                dist.send(t, self._peer(b), group=self._bwd_groups[b])
            elif s == b:
                dist.recv(t, self._peer(b + 1), group=self._bwd_groups[b])
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def _peer(self, stage: int) -> int:
        return stage * self.tp + self.tp_rank

    def step_device(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """tokens/targets: [n_microbatches, micro_batch, seq_len] on the device.  Runs the
        schedule and the optimizer step; returns the mean token loss (valid on ranks of
        the last stage, zero elsewhere) as a device tensor."""
        eng, cfg = self.engine, self.cfg
        s = self.stage
        eng.begin_step()
        dt = eng.store.params.dtype
        recv_f: Dict[int, tuple] = {}
        recv_b: Dict[int, tuple] = {}

        def post(a):
            buf = torch.empty(self.Tl, cfg.d, dtype=dt, device=self.device)
            if a.kind == "RECV_F":
                recv_f[a.mb] = (buf, dist.irecv(buf, self._peer(s - 1),
                                                group=self._fwd_groups[s - 1]))
            else:
                recv_b[a.mb] = (buf, dist.irecv(buf, self._peer(s + 1),
                                                group=self._bwd_groups[s]))

        if self.prepost:
            # every receive of the step up front, in schedule order per direction
            for a in self.actions:
                if a.kind in ("RECV_F", "RECV_B"):
                    post(a)
        outs: Dict[int, torch.Tensor] = {}
        dxs: Dict[int, torch.Tensor] = {}
        sends = []
        loss_sum = torch.zeros((), dtype=torch.float32, device=self.device)
        for a in self.actions:
            if a.kind == "RECV_F":
                if not self.prepost:
                    post(a)
                recv_f[a.mb][1].wait()
            elif a.kind == "RECV_B":
                if not self.prepost:
                    post(a)
                recv_b[a.mb][1].wait()
            elif a.kind == "F":
                x_in = tokens[a.mb] if s == 0 else recv_f.pop(a.mb)[0]
                out = eng.forward(a.mb, x_in, targets[a.mb] if s == self.pp - 1 else None)
                if s == self.pp - 1:
                    loss_sum += out
                else:
                    outs[a.mb] = out
            elif a.kind == "SEND_F":
                t = outs.pop(a.mb)
                sends.append((t, dist.isend(t, self._peer(s + 1), group=self._fwd_groups[s])))
            elif a.kind in ("B", "BI"):
                dy = None if s == self.pp - 1 else recv_b.pop(a.mb)[0]
                dx = eng.backward(a.mb, dy, split=a.kind == "BI")
                if dx is not None:
                    dxs[a.mb] = dx
            elif a.kind == "W":
                eng.backward_weight(a.mb)
            elif a.kind == "SEND_B":
                t = dxs.pop(a.mb)
                sends.append((t, dist.isend(t, self._peer(s - 1),
                                            group=self._bwd_groups[s - 1])))
            else:
                raise NotImplementedError(f"action {a.kind} is not supported by this runtime")
            if self._debug:
                torch.cuda.synchronize(self.device)
                print(f"[pp rank {self.rank}] done {a}", flush=True)
        for _, w in sends:
            w.wait()
        eng.optimizer_step(self.lr)
        if s == self.pp - 1:
            dist.all_reduce(loss_sum, group=self.tp_group)
        return loss_sum / (self.n_mb * eng.T)

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> float:
        """Host inputs [n_microbatches, micro_batch, seq_len] -> loss as a float."""
        self._tok.copy_(tokens, non_blocking=True)
        self._tgt.copy_(targets, non_blocking=True)
        return float(self.step_device(self._tok, self._tgt).item())

    @property
    def h2d_bytes_per_step(self) -> int:
        return 2 * self._tok.numel() * 8

    @property
    def d2h_bytes_per_step(self) -> int:
        return 4

    # ---------------------------------------------------------------- checkpointing
    def state_dict(self) -> dict:
        """Hugging Face-named full ``state_dict`` (CPU tensors) on every rank: shards are
        gathered over tp, stages over pp."""
        from ...models.llama import ParamLayout, to_hf_state_dict
        mine = self.engine.gather_full_units()
        allu: List[Optional[dict]] = [None] * dist.get_world_size()
        dist.all_gather_object(allu, mine if self.tp_rank == 0 else {})
        full_layout = ParamLayout(self.cfg)
        flat = torch.zeros(full_layout.total, dtype=self.engine.store.params.dtype)
        for part in allu:
            for uname, params in (part or {}).items():
                u = full_layout.units[full_layout.unit_index(uname)]
                v = full_layout.views(u, flat[u.offset: u.offset + u.size])
                for name, t in params.items():
                    v[name].copy_(t)
        return to_hf_state_dict(self.cfg, full_layout, flat)

    def load_state_dict(self, sd: dict) -> None:
        from ...models.llama import ParamLayout, load_hf_state_dict
        full_layout = ParamLayout(self.cfg)
        flat = torch.zeros(full_layout.total, dtype=self.engine.store.params.dtype)
        load_hf_state_dict(self.cfg, full_layout, sd, flat)
        self.engine.load_full_units(full_layout, flat)
