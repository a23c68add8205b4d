"""User-facing training driver: one object per rank that owns the model engine, the
parameter store for the chosen parallelism and the host<->device staging.

``Trainer.step(tokens, targets)`` is the call a user makes every iteration: it takes
*host* tensors (pinned or not), copies them to the device, runs forward + backward +
optimizer through the hand-written kernels and returns the loss as a Python float.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..models.llama import PRESETS, LlamaConfig, LlamaEngine, LocalParamStore, ParamLayout


def _dist_info():
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


class Trainer:
    def __init__(self, model: str | LlamaConfig = "llama3-8b", seq_len: int = 8192,
                 micro_batch: int = 1, parallelism: str = "auto", device=None,
                 checkpoint: bool = True, lr: float = 3e-4, seed: int = 0,
                 comm: str = "fused", recompute_layers: Optional[int] = None):
        self.cfg = PRESETS[model] if isinstance(model, str) else model
        self.seq_len = seq_len
        self.micro_batch = micro_batch
        self.lr = lr
        rank, world = _dist_info()
        self.rank, self.world = rank, world
        if device is None:
            if torch.cuda.is_available():
                device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
                torch.cuda.set_device(device)
            else:
                device = torch.device("cpu")
        self.device = torch.device(device)
        if parallelism == "auto":
            parallelism = "single" if world == 1 else "fsdp"
        self.parallelism = parallelism
        self.layout = ParamLayout(self.cfg)
        if parallelism == "single":
            self.store = LocalParamStore(self.layout, self.device, seed=seed)
        elif parallelism == "fsdp":
            from .fsdp import FSDPParamStore
            self.store = FSDPParamStore(self.layout, self.device, seed=seed, comm=comm)
        elif parallelism == "ddp":
            from .ddp import DDPParamStore
            self.store = DDPParamStore(self.layout, self.device, seed=seed, comm=comm)
        else:
            raise ValueError(f"unknown parallelism {parallelism!r}")
        self.engine = LlamaEngine(self.cfg, self.store, seq_len, checkpoint=checkpoint,
                                  recompute_layers=recompute_layers)
        shape = (micro_batch, seq_len)
        self._tok_dev = torch.empty(shape, dtype=torch.int64, device=self.device)
        self._tgt_dev = torch.empty(shape, dtype=torch.int64, device=self.device)
        # Device-side waits are bounded and report through a status word; a step whose
        # collective gave up must not pass for a step that trained.
        self._watch = None
        if self.device.type == "cuda":
            from ..ops.kernels import StatusWatch
            self._watch = StatusWatch(self.device)

    # -------------------------------------------------------------------------------
    def step_device(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One optimizer step on device-resident inputs; returns the device loss tensor.
        Never blocks on the device: a bounded wait that ran out inside a kernel of this
        step raises :class:`~monarch_b200.ops.kernels.KernelError` from the next call (or
        from :meth:`check`)."""
        if self._watch is not None:
            self._watch.poll()
        loss = self._step_device(tokens, targets)
        if self._watch is not None:
            self._watch.post()
        return loss

    def check(self) -> None:
        """Wait for the device and raise if any kernel since the last check recorded a
        failed wait.  Called before anything is written from the parameters."""
        if self._watch is not None:
            self._watch.poll(wait=True)
            from ..ops import kernels as K
            K.check_status(self.device)

    def _step_device(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        if hasattr(self.store, "set_hyper"):
            self.store.set_hyper(lr=self.lr)  # sharded stores update inside backward
        loss = self.engine.forward_backward(tokens, targets)
        self.engine.optimizer_step(self.lr)
        return loss

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> float:
        """One optimizer step on host inputs ([micro_batch, seq_len] int64).  Copies the
        batch to the device, runs the step and reads the loss back."""
        self._tok_dev.copy_(tokens, non_blocking=True)
        self._tgt_dev.copy_(targets, non_blocking=True)
        loss = self.step_device(self._tok_dev, self._tgt_dev)
        value = float(loss.item())       # synchronises: the status copy has landed too
        if self._watch is not None:
            self._watch.poll(wait=True)
        return value

    @property
    def h2d_bytes_per_step(self) -> int:
        return 2 * self._tok_dev.numel() * self._tok_dev.element_size()

    @property
    def d2h_bytes_per_step(self) -> int:
        return 4

    # ---------------------------------------------------------------- checkpointing
    def state_dict(self) -> dict:
        """Hugging Face-named model ``state_dict`` (full tensors, on every rank)."""
        from ..models.llama import to_hf_state_dict
        self.check()
        return to_hf_state_dict(self.cfg, self.layout, self.store.full_params())

    def save_checkpoint(self, path: str) -> None:
        """Resumable checkpoint: every rank writes ``<path>/shard_<rank>.pt`` (its fp32 master
        weights, AdamW moments, optimizer step, RNG states) and rank 0 writes
        ``<path>/manifest.json`` (model, parallelism, world size, step).  The model-only,
        Hugging Face-named view of the same weights is :meth:`state_dict`."""
        import json
        from ..random import get_rng_state_all
        self.check()      # never write shards that a timed-out collective left inconsistent
        os.makedirs(path, exist_ok=True)
        sd = {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v)
              for k, v in self.store.state_dict_shard().items()}
        sd["rng"] = get_rng_state_all()
        torch.save(sd, os.path.join(path, f"shard_{self.rank}.pt"))
        if self.rank == 0:
            with open(os.path.join(path, "manifest.json"), "w") as f:
                json.dump({"model": self.cfg.name, "parallelism": self.parallelism,
                           "world": self.world, "step": int(sd["step"]),
                           "seq_len": self.seq_len, "format": 1}, f)
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()

    def load_checkpoint(self, path: str) -> int:
        """Restore what :meth:`save_checkpoint` wrote (same parallelism and world size);
        returns the optimizer step to continue from."""
        import json
        from ..random import set_rng_state_all
        with open(os.path.join(path, "manifest.json")) as f:
            man = json.load(f)
        if man["world"] != self.world or man["parallelism"] != self.parallelism or \
                man["model"] != self.cfg.name:
            raise ValueError(f"checkpoint is for {man['model']} {man['parallelism']} x "
                             f"{man['world']}, this trainer is {self.cfg.name} "
                             f"{self.parallelism} x {self.world}; re-shard through state_dict()")
        sd = torch.load(os.path.join(path, f"shard_{self.rank}.pt"), map_location="cpu",
                        weights_only=False)
        self.store.load_state_dict_shard(sd)
        set_rng_state_all(sd["rng"])
        return int(sd["step"])

    def load_state_dict(self, sd: dict) -> None:
        from ..models.llama import load_hf_state_dict
        flat = torch.empty(self.layout.total, dtype=torch.bfloat16, device=self.device)
        flat.zero_()
        load_hf_state_dict(self.cfg, self.layout, sd, flat)
        self.store.load_full_params(flat)
