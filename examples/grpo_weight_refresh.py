#!/usr/bin/env python
"""GRPO-style actor program: a learner publishes its weights as RDMABuffers, generators
pull them one-sidedly before producing rollouts, a scorer rates the rollouts and the
learner takes a policy-gradient step on them.  Tiny numbers, real data flow.

    python examples/grpo_weight_refresh.py

Parity: docs/source/examples/grpo_actor.py of the reference (learner / generator / scorer
actors, weights shared through RDMA buffer handles in ordinary messages)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from monarch_b200.actor import Actor, current_rank, endpoint, this_host  # noqa: E402
from monarch_b200.tensor_engine import RDMABuffer  # noqa: E402

D, ACTIONS = 8, 4


def _policy():
    torch.manual_seed(0)
    return torch.nn.Linear(D, ACTIONS)


class Learner(Actor):
    def __init__(self):
        self.model = _policy()
        self.opt = torch.optim.SGD(self.model.parameters(), lr=0.5)
        self.version = 0
        self._export()

    def _export(self):
        self.flat = torch.cat([p.detach().reshape(-1) for p in self.model.parameters()]).clone()
        self.buf = RDMABuffer(self.flat.view(torch.uint8))

    @endpoint
    def weights(self):
        return self.version, self.buf

    @endpoint
    def step(self, states, actions, rewards) -> float:
        logp = torch.log_softmax(self.model(states), -1).gather(1, actions[:, None])[:, 0]
        adv = rewards - rewards.mean()
        loss = -(logp * adv).mean()
        self.opt.zero_grad()
        loss.backward()
        self.opt.step()
        self.version += 1
        self._export()
        return float(loss.detach())


class Generator(Actor):
    def __init__(self):
        self.model = _policy()
        self.version = -1
        self.gen = torch.Generator().manual_seed(100 + current_rank().rank)

    @endpoint
    def refresh(self, version: int, buf: RDMABuffer) -> int:
        n = sum(p.numel() for p in self.model.parameters())
        flat = torch.empty(n, dtype=torch.float32)
        buf.read_into(flat.view(torch.uint8)).get(timeout=30)   # one-sided pull
        off = 0
        with torch.no_grad():
            for p in self.model.parameters():
                p.copy_(flat[off: off + p.numel()].view_as(p))
                off += p.numel()
        self.version = version
        return version

    @endpoint
    def rollout(self, n: int):
        s = torch.randn(n, D, generator=self.gen)
        with torch.no_grad():
            a = torch.multinomial(torch.softmax(self.model(s), -1), 1, generator=self.gen)[:, 0]
        return s, a


class Scorer(Actor):
    @endpoint
    def score(self, states, actions):
        # the "environment": action index should match the sign pattern of the first 2 dims
        target = (states[:, 0] > 0).long() * 2 + (states[:, 1] > 0).long()
        return (actions == target).float()


def run(iters: int = 30, generators: int = 2):
    lm = this_host().spawn_procs(per_host={"gpus": 1})
    gm = this_host().spawn_procs(per_host={"gpus": generators})
    sm = this_host().spawn_procs(per_host={"gpus": 1})
    try:
        learner = lm.spawn("learner", Learner)
        gens = gm.spawn("generators", Generator)
        scorer = sm.spawn("scorer", Scorer)
        acc = []
        for it in range(iters):
            version, buf = learner.weights.call_one().get(timeout=30)
            got = [v for _, v in gens.refresh.call(version, buf).get(timeout=30).items()]
            assert got == [version] * generators
            rolls = [v for _, v in gens.rollout.call(64).get(timeout=30).items()]
            states = torch.cat([r[0] for r in rolls])
            actions = torch.cat([r[1] for r in rolls])
            rewards = scorer.score.call_one(states, actions).get(timeout=30)
            learner.step.call_one(states, actions, rewards).get(timeout=30)
            acc.append(float(rewards.mean()))
        return {"reward_first": sum(acc[:5]) / 5, "reward_last": sum(acc[-5:]) / 5,
                "versions": version + 1}
    finally:
        for m in (lm, gm, sm):
            m.stop().get()


if __name__ == "__main__":
    print(run())
