"""GRPO step driver: the consumer side of the reference's RLTrainingPipeline
(include/neuralnet.cpp/rl_pipeline.hpp:312-350) for GrpoObjective (rl_policy.hpp:866-953) on the ternary
GPT policy: GptRolloutSource produces a TensorRecord on the device (rollout, rewards, GroupAdvantage,
reference log-probs), update() runs the micro-batched objective / backward, the gradient all-reduce and
the optimizer step.

Sharding: whole prompt groups stay on one rank (GroupAdvantage needs no collective); the only
collectives are the all-reduce (sum) of the flat gradient buffer and of a few report scalars.
torch.distributed is plumbing only; every numeric step is a call into libnn-b200.so.

The KL term against a frozen reference policy (kl_coef, ref_log_prob) is this engine's addition: the
reference's GrpoObjective has the clipped policy term and the entropy bonus only, and its
SampledKlObjective penalises logp - old_log_prob.  kl_coef = 0 gives the reference preset.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .pipeline import GptRolloutSource, RolloutSpec, TensorRecord, micro_batched
from .policy import Policy

# names of the ten floats nnb_policy_train_step reports (PpoReport / GrpoReport fields of the reference,
# rl_policy.hpp:787-797,858-864, plus the pieces they are sums of)
REPORT_FIELDS = ("policy_loss", "ratio_mean", "approx_kl", "policy_clip_fraction", "kl_loss", "entropy_loss", "entropy",
                 "units", "value_loss", "value_clip_fraction")


def report_dict(report: torch.Tensor) -> dict:
    """The report vector as the reference's report structs name it: PpoReport.loss = policy + entropy + value
    terms (plus this engine's KL term), PpoReport.policy_loss = clipped term + entropy term."""
    v = [float(x) for x in report.detach().cpu().tolist()]
    d = dict(zip(REPORT_FIELDS, v))
    d["clipped_policy_loss"] = d["policy_loss"]
    d["policy_loss"] = d["clipped_policy_loss"] + d["entropy_loss"]
    d["loss"] = d["policy_loss"] + d["value_loss"] + d["kl_loss"]
    return d


@dataclass
class GrpoConfig:
    group_size: int = 16
    prompt_len: int = 128
    max_new: int = 512
    temperature: float = 0.8
    top_k: int = 50
    clip_eps: float = 0.2
    kl_coef: float = 0.04
    entropy_coef: float = 0.0
    lr: float = 1e-4
    weight_decay: float = 0.01
    max_grad_norm: float = 0.0
    micro_batch: int = 16        # sequences per training micro-batch
    rollout_chunk: int = 512     # sequences decoded together (bounds the KV cache)
    advantage_eps: float = 1e-8


def hash_reward(tokens_gen: torch.Tensor, seed: int, p: float = 0.3) -> torch.Tensor:
    """Seeded hash of the generated tokens mapped to {0,1} with probability p of 1 (synthetic reward)."""
    t = tokens_gen.to(torch.int64)
    pos = torch.arange(1, t.shape[1] + 1, device=t.device, dtype=torch.int64)
    h = ((t + 1) * (pos * 2654435761 % 2147483647)).sum(1) + seed * 97003
    h = (h * 1103515245 + 12345) % 2147483648
    h = (h ^ (h >> 13)) * 1274126177 % 2147483648
    return ((h % 1000003).to(torch.float32) / 1000003.0 < p).to(torch.float32)


class _DistMixin:
    def _init_dist(self, dist_group):
        self.dist = dist_group if dist_group is not None else (
            torch.distributed if torch.distributed.is_available() and torch.distributed.is_initialized() else None)
        self.rank = self.dist.get_rank() if self.dist else 0
        self.world = self.dist.get_world_size() if self.dist else 1

    def _allreduce(self, t):
        if self.dist and self.world > 1:
            self.dist.all_reduce(t)
        return t


class GrpoTrainer(_DistMixin):
    def __init__(self, policy: Policy, ref_policy: Policy | None, cfg: GrpoConfig, dist_group=None):
        self.policy, self.ref, self.cfg = policy, ref_policy, cfg
        self._init_dist(dist_group)
        spec = RolloutSpec(prompt_len=cfg.prompt_len, max_new=cfg.max_new, group_size=cfg.group_size,
                           temperature=cfg.temperature, top_k=cfg.top_k, rollout_chunk=cfg.rollout_chunk,
                           advantage="group", advantage_eps=cfg.advantage_eps, eval_micro_batch=cfg.micro_batch)
        self.source = GptRolloutSource(policy, spec, None, None, ref_policy if cfg.kl_coef != 0.0 else None)

    def collect(self, prompts: torch.Tensor, reward_fn, seed: int, timers=None) -> TensorRecord:
        """This rank's prompt groups -> TensorRecord (tokens, action_mask, advantage, old_log_prob, ref_log_prob)."""
        src = self.source
        src.reward_fn = reward_fn
        src.seq0 = self.rank * prompts.shape[0] * self.cfg.group_size
        src.on_phase = (lambda name: timers.mark(name)) if timers else None
        return src.rollout(None, prompts=prompts, seed=seed)

    def update(self, record: TensorRecord, timers=None):
        c, pol = self.cfg, self.policy
        ev = (lambda name: timers.mark(name)) if timers else (lambda name: None)
        tokens, mask = record["tokens"], record["action_mask"]
        N = tokens.shape[0]
        units = torch.tensor([float(N * c.max_new)], device=tokens.device)
        units_global = float(self._allreduce(units).item()) if self.world > 1 else float(N * c.max_new)
        ref_lp = record.get("ref_log_prob")

        def run(mb):
            # micro-batches made of whole groups let the engine compute a group's shared prompt once
            gs = c.group_size if mb % c.group_size == 0 else 1
            pol.zero_grad()
            report = torch.zeros(10, device=tokens.device)
            for a in range(0, N, mb):
                sl = slice(a, a + mb)
                report += pol.train_step(tokens[sl].contiguous(), c.prompt_len, mask[sl].contiguous(),
                                         old_logp=record["old_log_prob"][sl].contiguous(),
                                         advantage=record["advantage"][sl].contiguous(),
                                         ref_logp=None if ref_lp is None else ref_lp[sl].contiguous(),
                                         units=units_global, clip_eps=c.clip_eps, kl_coef=c.kl_coef,
                                         entropy_coef=c.entropy_coef, group_size=gs)
            return report

        # a workspace that does not fit halves the micro-batch (kept for the following steps)
        report, self._micro_batch = micro_batched(N, getattr(self, "_micro_batch", c.micro_batch), c.group_size, run)
        report[7] = units_global  # every micro-batch reports the global count: it is not a sum
        ev("train")
        if self.world > 1:
            self._allreduce(pol.grads_view())
            self._allreduce(report)
            report[7] = units_global
        ev("allreduce")
        norm = pol.optimizer_step(c.lr, weight_decay=c.weight_decay, max_grad_norm=c.max_grad_norm)
        ev("optimizer")
        return {"report": report, "grad_norm": norm}

    def step(self, prompts: torch.Tensor, reward_fn, seed: int, timers=None):
        """One GRPO step on this rank's prompt groups.  reward_fn(tokens (N,S)) -> (N,) f32 on the device."""
        record = self.collect(prompts, reward_fn, seed, timers)
        out = self.update(record, timers)
        out.update(reward_mean=record["reward"].mean(), tokens=record["tokens"], record=record)
        return out
