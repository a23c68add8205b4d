"""Library-path trainer: the same model and step as :class:`Trainer`, but every op is a
stock PyTorch call -- ``nn.Linear`` (cuBLAS), SDPA (cuDNN/flash), autograd with
activation checkpointing, ``torch.optim.AdamW(fused=True)`` on fp32 master weights under
bf16 autocast-free mixed precision, and ``torch.distributed.fsdp.fully_shard`` (NCCL
all-gather / reduce-scatter) when there is more than one rank.

This is what the reference's tensor worker executes for the same program (ATen ops via
``call_op``, monarch_tensor_worker/src/stream.rs:758-784; NCCL via
torch-sys-cuda/src/nccl.rs:464-835), so it stands in for the reference on the headline
benchmark when the reference itself cannot be built.  None of this package's kernels
run on this path.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.llama import PRESETS, LlamaConfig
from ..models.torch_llama import TorchLlama


class AtenTrainer:
    def __init__(self, model: str | LlamaConfig = "llama3-8b", seq_len: int = 8192,
                 micro_batch: int = 1, device=None, lr: float = 3e-4, seed: int = 0):
        self.cfg = PRESETS[model] if isinstance(model, str) else model
        self.seq_len, self.micro_batch, self.lr = seq_len, micro_batch, lr
        self.device = torch.device(device if device is not None else "cuda")
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.parallelism = "single" if self.world == 1 else "fsdp"
        torch.manual_seed(seed)
        fused = self.device.type == "cuda"
        with torch.device("meta"):
            net = TorchLlama(self.cfg, checkpoint=True)
        if self.world > 1:
            # fp32 master parameters, sharded; bf16 all-gathered compute copies
            from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
            # inputs are not cast at module boundaries: the activations are bf16 already (the
            # embedding's gathered weight is), and the fp32 rotary tables must stay fp32 in
            # the forward and in the checkpointed recomputation alike
            mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32,
                                      cast_forward_inputs=False)
            for blk in net.model.layers:
                fully_shard(blk, mp_policy=mp)
            fully_shard(net, mp_policy=mp)
            net.to_empty(device=self.device)
            self._init(net)
            self.net = net
            self._bf16_shadow = None
        else:
            # one GPU: bf16 module for compute + fp32 master copy stepped by fused AdamW
            net.to_empty(device=self.device)
            self._init(net)
            self.net = net.to(torch.bfloat16)
            self._bf16_shadow = [p for p in self.net.parameters()]
        self.net.train()
        if self._bf16_shadow is not None:
            # one optimizer per top-level block, so that only one block's fp32 gradient
            # copy exists at a time (all of them at once would not fit beside the state)
            groups = [list(self.net.model.embed_tokens.parameters())]
            groups += [list(b.parameters()) for b in self.net.model.layers]
            tail = list(self.net.model.norm.parameters())
            if not self.cfg.tie_embeddings:
                tail += list(self.net.lm_head.parameters())
            groups.append(tail)
            self.groups = []
            for g in groups:
                master = [p.detach().float().clone().requires_grad_(True) for p in g]
                opt = torch.optim.AdamW(master, lr=lr, betas=(0.9, 0.95), eps=1e-8,
                                        weight_decay=0.1, fused=fused)
                self.groups.append((g, master, opt))
        else:
            self.opt = torch.optim.AdamW(self.net.parameters(), lr=lr, betas=(0.9, 0.95),
                                         eps=1e-8, weight_decay=0.1, fused=fused)
        shape = (micro_batch, seq_len)
        self._tok_dev = torch.empty(shape, dtype=torch.int64, device=self.device)
        self._tgt_dev = torch.empty(shape, dtype=torch.int64, device=self.device)

    @staticmethod
    def _init(net):
        with torch.no_grad():
            for n, p in net.named_parameters():
                if p.dim() == 1:
                    p.fill_(1.0)
                else:
                    p.normal_(0.0, 0.02)

    def step_device(self, tokens, targets):
        loss = self.net(tokens, targets)
        loss.backward()
        if self._bf16_shadow is not None:
            for g, master, opt in self.groups:
                for m, p in zip(master, g):
                    m.grad = p.grad.float()
                    p.grad = None
                opt.step()
                with torch.no_grad():
                    torch._foreach_copy_(g, master)
                for m in master:
                    m.grad = None
        else:
            self.opt.step()
            self.opt.zero_grad(set_to_none=True)
        return loss.detach()

    def step(self, tokens, targets) -> float:
        self._tok_dev.copy_(tokens, non_blocking=True)
        self._tgt_dev.copy_(targets, non_blocking=True)
        return float(self.step_device(self._tok_dev, self._tgt_dev).item())

    @property
    def h2d_bytes_per_step(self) -> int:
        return 2 * self._tok_dev.numel() * 8

    @property
    def d2h_bytes_per_step(self) -> int:
        return 4
