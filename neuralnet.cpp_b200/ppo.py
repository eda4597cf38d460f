"""PPO step driver for a ternary GPT policy with a value head: the update loop a user of the reference
writes around PpoObjective (include/neuralnet.cpp/rl_policy.hpp:799-846) with GaeAdvantage
(rl_experience.hpp:273-380), an ExperienceBuffer and a UniformBatchSampler
(rl_pipeline.hpp:68-152; the integration pattern is src/rl_training_integration_test.cpp:86-206):

    record  = GptRolloutSource.rollout()          rollout, old values, rewards, GAE advantages / returns
    for epoch in range(epochs):
        order = UniformBatchSampler(no replacement).sample(n, n)       a fresh shuffle per epoch
        for each of the `minibatches` slices of `order`:
            micro-batched nnb_policy_train_step (clipped policy + entropy bonus + clipped value)
            all-reduce(sum) of the gradients, optimizer step

Trajectories are sharded over the ranks (GAE couples only the steps of one trajectory); every minibatch
is normalised by its global count of valid decisions.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .grpo import _DistMixin
from .pipeline import DeterministicRng, GptRolloutSource, RolloutSpec, TensorRecord, UniformBatchSampler, micro_batched
from .policy import Policy


@dataclass
class PpoConfig:
    prompt_len: int = 64
    max_new: int = 256
    temperature: float = 1.0
    top_k: int = 0
    gamma: float = 0.99
    lam: float = 0.95
    clip_eps: float = 0.2
    value_clip_eps: float = 0.2
    value_coef: float = 0.5
    entropy_coef: float = 0.01          # PpoConfig default of the reference (rl_policy.hpp:780)
    normalize_advantage: bool = False   # MaskedNormalizer over the rollout batch before the epochs
    epochs: int = 4
    minibatches: int = 4
    lr: float = 1e-4
    weight_decay: float = 0.01
    max_grad_norm: float = 0.0
    micro_batch: int = 16
    rollout_chunk: int = 256


class PpoTrainer(_DistMixin):
    def __init__(self, policy: Policy, cfg: PpoConfig, dist_group=None, seed: int = 0):
        if not policy.cfg.value_head:
            raise ValueError("PpoTrainer needs a policy with a value head")
        self.policy, self.cfg = policy, cfg
        self._init_dist(dist_group)
        spec = RolloutSpec(prompt_len=cfg.prompt_len, max_new=cfg.max_new, group_size=1, temperature=cfg.temperature,
                           top_k=cfg.top_k, rollout_chunk=cfg.rollout_chunk, advantage="gae", gamma=cfg.gamma, lam=cfg.lam,
                           normalize_advantage=cfg.normalize_advantage, eval_micro_batch=cfg.micro_batch)
        self.source = GptRolloutSource(policy, spec, None, None, None)
        self.sampler = UniformBatchSampler(replacement=False)
        self.rng = DeterministicRng(seed)  # the same seed on every rank: ranks shuffle alike

    def collect(self, prompts: torch.Tensor, reward_fn, seed: int, timers=None) -> TensorRecord:
        src = self.source
        src.reward_fn = reward_fn
        src.seq0 = self.rank * prompts.shape[0]
        src.on_phase = (lambda name: timers.mark(name)) if timers else None
        return src.rollout(None, prompts=prompts, seed=seed)

    def minibatch_update(self, mb_rec: TensorRecord):
        """Gradients of one minibatch (micro-batched), all-reduce, optimizer step.  Returns the report[10]."""
        c, pol = self.cfg, self.policy
        tokens, mask = mb_rec["tokens"], mb_rec["action_mask"]
        n = tokens.shape[0]
        units = mask.sum().reshape(1)
        units_global = float(self._allreduce(units).item())

        def run(mb):
            pol.zero_grad()
            report = torch.zeros(10, device=tokens.device)
            for a in range(0, n, mb):
                sl = slice(a, a + mb)
                report += pol.train_step(tokens[sl].contiguous(), c.prompt_len, mask[sl].contiguous(),
                                         old_logp=mb_rec["old_log_prob"][sl].contiguous(),
                                         advantage=mb_rec["advantage"][sl].contiguous(),
                                         returns=mb_rec["return"][sl].contiguous(),
                                         old_value=mb_rec["old_value"][sl].contiguous(), units=units_global,
                                         clip_eps=c.clip_eps, entropy_coef=c.entropy_coef, value_coef=c.value_coef,
                                         value_clip_eps=c.value_clip_eps)
            return report

        # a workspace that does not fit halves the micro-batch (kept for the following minibatches)
        report, self._micro_batch = micro_batched(n, getattr(self, "_micro_batch", c.micro_batch), 1, run)
        if self.world > 1:
            self._allreduce(pol.grads_view())
            self._allreduce(report)
        report[7] = units_global
        pol.optimizer_step(c.lr, weight_decay=c.weight_decay, max_grad_norm=c.max_grad_norm)
        return report

    def update(self, record: TensorRecord, timers=None):
        c = self.cfg
        n = record.rows()
        if n % c.minibatches != 0:
            raise ValueError(f"{n} trajectories do not split into {c.minibatches} minibatches")
        per = n // c.minibatches
        last = None
        for _ in range(c.epochs):
            order = self.sampler.sample(n, n, self.rng)
            for m in range(c.minibatches):
                idx = torch.tensor(order[m * per:(m + 1) * per], device=record["tokens"].device, dtype=torch.int64)
                last = self.minibatch_update(record.select(idx))
        if timers:
            timers.mark("train")
        return {"report": last}

    def step(self, prompts: torch.Tensor, reward_fn, seed: int, timers=None):
        """One PPO step on this rank's trajectories: rollout + GAE, then epochs x minibatches updates.
        reward_fn(tokens (n, S)) -> (n, G) per-decision rewards on the device."""
        record = self.collect(prompts, reward_fn, seed, timers)
        out = self.update(record, timers)
        out.update(reward_mean=record["reward"].mean(), tokens=record["tokens"], record=record)
        return out
