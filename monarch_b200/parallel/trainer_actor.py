"""A training rank behind an actor: what a controller spawns on every proc of a mesh to
drive data-parallel / sharded / pipelined training with ``step`` messages.

    trainers = mesh.spawn("trainer", TrainerActor, {"model": "llama3-8b", "seq_len": 8192})
    for i in range(steps):
        losses = trainers.step.call(i).get()        # ValueMesh of per-rank losses

Each actor owns a :class:`~monarch_b200.parallel.trainer.Trainer` (or the pipeline / MoE /
stock-PyTorch variant), a few synthetic batches in pinned host memory, and runs on the GPU
named by ``LOCAL_RANK`` (or its rank in the mesh).  The control plane is the actor runtime;
the data plane (NVLink kernels or NCCL) never leaves the GPUs.  When the procs of the mesh
belong to an SPMD launch (:func:`monarch_b200.actor.attach_proc_mesh`) the actor uses the
process group the launcher's ranks created; otherwise it creates one from ``MASTER_ADDR`` /
``MASTER_PORT`` when the mesh has more than one rank.

The reference has no trainer; this is the shape of its SPMD examples (one actor per GPU,
``step`` endpoints: docs/source/examples/spmd_ddp.py) applied to this package's engine.
"""
from __future__ import annotations

import gc
import os
import re
from typing import Any, Dict, Optional

import torch

from ..actor import Actor, current_rank, current_size, endpoint


class TrainerActor(Actor):
    def __init__(self, spec: Dict[str, Any]):
        """``spec``: ``impl`` ("ours" | "aten"), ``model``, ``seq_len``, ``micro_batch``,
        ``parallelism`` ("auto", "single", "fsdp", "ddp", "ep", "ppPxtpT"), ``comm``,
        ``recompute_layers``, ``microbatches``, ``schedule``, ``n_batches``, ``cuda``."""
        self.spec = dict(spec)
        self.rank = current_rank().rank
        self.world = 1
        for v in current_size().values():
            self.world *= v
        self.cuda = bool(spec.get("cuda", torch.cuda.is_available()))
        self.local_rank = int(os.environ.get("LOCAL_RANK", self.rank))
        if self.cuda:
            self.device = torch.device("cuda", self.local_rank % torch.cuda.device_count())
            torch.cuda.set_device(self.device)       # this actor's thread launches the kernels
        else:
            self.device = torch.device("cpu")
        self._own_pg = False
        if self.world > 1:
            import torch.distributed as dist
            if not dist.is_initialized():
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                dist.init_process_group("nccl" if self.cuda else "gloo", rank=self.rank,
                                        world_size=self.world,
                                        **({"device_id": self.device} if self.cuda else {}))
                self._own_pg = True
        self.trainer = None
        self._build()

    # ------------------------------------------------------------------------- set-up
    def _build(self) -> None:
        s = self.spec
        impl = s.get("impl", "ours")
        model, seq, mb = s.get("model", "llama3-8b"), int(s.get("seq_len", 8192)), \
            int(s.get("micro_batch", 1))
        par = s.get("parallelism", "auto")
        comm = s.get("comm", "fused") if self.cuda else "nccl"
        self.n_mb = 1
        m_pp = re.fullmatch(r"pp(\d+)xtp(\d+)", par)
        if impl == "aten":
            from .aten_baseline import AtenTrainer
            self.trainer = AtenTrainer(model, seq, mb, device=self.device)
        elif m_pp:
            from .pipelining import PipelineTrainer
            self.n_mb = int(s.get("microbatches", 8))
            self.trainer = PipelineTrainer(model, int(m_pp.group(1)), int(m_pp.group(2)), seq, mb,
                                           self.n_mb, device=self.device, comm=comm,
                                           schedule=s.get("schedule", "1f1b"))
        elif par == "ep":
            from .ep import MoETrainer
            self.trainer = MoETrainer(model, seq, mb, device=self.device, comm=comm)
        else:
            from .trainer import Trainer
            self.trainer = Trainer(model, seq_len=seq, micro_batch=mb, parallelism=par,
                                   device=self.device, comm=comm,
                                   recompute_layers=s.get("recompute_layers"),
                                   lr=float(s.get("lr", 3e-4)))
        self._pipeline = bool(m_pp)
        cfg = self.trainer.cfg
        # a pipeline is one data-parallel replica: every stage sees the same batch
        gen = torch.Generator().manual_seed(int(s.get("seed", 1234)) +
                                            (0 if self._pipeline else self.rank))
        shape = (self.n_mb, mb, seq) if self._pipeline else (mb, seq)
        n_batches = int(s.get("n_batches", 4))
        pin = (lambda t: t.pin_memory()) if self.cuda else (lambda t: t)
        self.host_tok = [pin(torch.randint(0, cfg.vocab, shape, generator=gen))
                         for _ in range(n_batches)]
        self.host_tgt = [pin(torch.randint(0, cfg.vocab, shape, generator=gen))
                         for _ in range(n_batches)]
        self.dev_tok = [t.to(self.device) for t in self.host_tok]
        self.dev_tgt = [t.to(self.device) for t in self.host_tgt]
        self.tokens_per_step = self.n_mb * mb * seq if self._pipeline else mb * seq * self.world

    def _barrier(self) -> None:
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        if self.cuda:
            torch.cuda.synchronize(self.device)

    # ---------------------------------------------------------------------- endpoints
    @endpoint
    def step(self, i: int) -> float:
        """One optimizer step on batch ``i`` taken from pinned host memory; returns the loss
        (read back from the device, so the step is finished when the reply leaves)."""
        n = len(self.host_tok)
        return self.trainer.step(self.host_tok[i % n], self.host_tgt[i % n])

    @endpoint
    def sync(self) -> int:
        """Barrier across the ranks and device synchronisation; returns the rank."""
        self._barrier()
        return self.rank

    @endpoint
    def timed_steps(self, warmup: int, steps: int) -> Dict[str, Any]:
        """``warmup`` untimed steps, then exactly ``steps`` steps on device-resident batches
        between two CUDA events (barrier + synchronize on both sides); clocks are sampled
        during the timed region."""
        from ..ops import kernels as K
        from ..utils.clocks import ClockSampler
        n = len(self.dev_tok)
        loss = None
        for i in range(warmup):
            loss = self.trainer.step_device(self.dev_tok[i % n], self.dev_tgt[i % n])
        self._barrier()
        if self.cuda:
            K.check_status(self.device)
        sampler = ClockSampler(self.device.index if self.cuda else 0).start() if self.cuda else None
        l0 = K.launch_count
        if self.cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        import time
        t0 = time.perf_counter()
        for i in range(steps):
            loss = self.trainer.step_device(self.dev_tok[i % n], self.dev_tgt[i % n])
        if self.cuda:
            e1.record()
        self._barrier()
        wall = (time.perf_counter() - t0) * 1e3
        clocks = sampler.stop() if sampler is not None else None
        launches = K.launch_count - l0
        if self.cuda:
            K.check_status(self.device)
            ms = e0.elapsed_time(e1)
        else:
            ms = wall
        if self._pipeline and self.world > 1 and loss is not None:
            import torch.distributed as dist
            dist.all_reduce(loss, op=dist.ReduceOp.MAX)   # the last stage holds the loss
        return {"rank": self.rank, "ms": ms, "wall_ms": wall, "launches": launches,
                "clocks": clocks, "loss": float(loss.item()) if loss is not None else None,
                "max_mem_gb": torch.cuda.max_memory_allocated(self.device) / 1e9
                if self.cuda else 0.0}

    @endpoint
    def info(self) -> Dict[str, Any]:
        t = self.trainer
        return {"rank": self.rank, "world": self.world, "parallelism": t.parallelism,
                "tokens_per_step": self.tokens_per_step, "device": str(self.device),
                "pid": os.getpid(), "h2d_bytes_per_step": t.h2d_bytes_per_step,
                "d2h_bytes_per_step": t.d2h_bytes_per_step,
                "fsdp_gather": getattr(getattr(t, "store", None), "gather", None),
                "comm": getattr(getattr(t, "store", None), "comm", None)}

    @endpoint
    def release(self) -> None:
        """Drop the trainer and give its device memory back (another trainer may follow on
        the same GPU)."""
        self._barrier()
        self.trainer = None
        self.host_tok = self.host_tgt = self.dev_tok = self.dev_tgt = None
        gc.collect()
        if self.cuda:
            torch.cuda.empty_cache()
            torch.cuda.reset_peak_memory_stats(self.device)

    @endpoint
    def shutdown(self) -> None:
        self._barrier()
        if self._own_pg:
            import torch.distributed as dist
            dist.destroy_process_group()
