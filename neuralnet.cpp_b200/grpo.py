"""GRPO / PPO step drivers: the consumer-side loop the reference leaves to the user of
RLTrainingPipeline (include/neuralnet.cpp/rl_pipeline.hpp:312-350): rollout source -> rewards ->
advantages -> micro-batched objective/backward -> gradient all-reduce -> optimizer step.

Sharding: whole prompt groups stay on one rank (GroupAdvantage needs no collective); the only
collectives are the all-reduce (sum) of the flat gradient buffer and of a few report scalars.
torch.distributed is plumbing only; every numeric step is a call into libnn-b200.so.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ._lib import NnbError
from .policy import Policy


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


class GrpoTrainer:
    def __init__(self, policy: Policy, ref_policy: Policy | None, cfg: GrpoConfig, dist_group=None):
        self.policy, self.ref, self.cfg = policy, ref_policy, cfg
        self.dist = dist_group if dist_group is not None else (
            torch.distributed if torch.distributed.is_available() and torch.distributed.is_initialized() else None)
        self.rank = self.dist.get_rank() if self.dist else 0
        self.world = self.dist.get_world_size() if self.dist else 1
        self.timings = {}
        self._chunk = cfg.rollout_chunk  # shrinks if a KV cache of that many sequences does not fit

    def _allreduce(self, t):
        if self.dist and self.world > 1:
            self.dist.all_reduce(t)
        return t

    def rollout(self, prompts: torch.Tensor, seed: int, seq0: int):
        """prompts (n_groups_local, P) -> tokens (N, P+G), old_logp (N, G); groups are contiguous rows."""
        c = self.cfg
        rep = prompts.repeat_interleave(c.group_size, dim=0).contiguous()
        n = rep.shape[0]
        chunk = max(c.group_size, (min(self._chunk, n) // c.group_size) * c.group_size)
        while True:
            toks, lps = [], []
            try:
                for a in range(0, n, chunk):
                    t, lp, _ = self.policy.rollout(rep[a:a + chunk].contiguous(), c.max_new, temperature=c.temperature,
                                                   top_k=c.top_k, seed=seed, seq0=seq0 + a, group_size=c.group_size)
                    toks.append(t)
                    lps.append(lp)
                return torch.cat(toks), torch.cat(lps)
            except NnbError as ex:
                # the engine refuses a KV cache that does not fit (status -4) before allocating it: decode
                # fewer sequences together.  The samples do not depend on the chunking (Philox counters are
                # per sequence), so the retry reproduces the same rollout.
                if getattr(ex, "status", 0) != -4 or chunk <= c.group_size:
                    raise
                chunk = max(c.group_size, (chunk // 2 // c.group_size) * c.group_size)
                self._chunk = chunk

    def step(self, prompts: torch.Tensor, reward_fn, seed: int, timers=None):
        """One GRPO step on this rank's prompt groups.  reward_fn(tokens (N,S)) -> (N,) f32 on the device."""
        c, pol, eng = self.cfg, self.policy, self.policy.engine
        n_groups = prompts.shape[0]
        N = n_groups * c.group_size
        seq0 = self.rank * N
        ev = (lambda name: timers.mark(name)) if timers else (lambda name: None)
        ev("start")
        tokens, old_lp = self.rollout(prompts, seed, seq0)
        ev("rollout")
        rewards = reward_fn(tokens).contiguous()
        adv_seq = eng.group_advantage(rewards, [(g * c.group_size, c.group_size) for g in range(n_groups)],
                                      eps=c.advantage_eps)
        adv = adv_seq[:, None].expand(N, c.max_new).contiguous()
        mask = torch.ones((N, c.max_new), device=tokens.device, dtype=torch.float32)
        units = torch.tensor([float(N * c.max_new)], device=tokens.device)
        units_global = float(self._allreduce(units).item()) if self.world > 1 else float(N * c.max_new)
        ev("advantage")
        mb = c.micro_batch
        # micro-batches made of whole groups let the engine compute a group's shared prompt once
        gs = c.group_size if mb % c.group_size == 0 else 1
        ref_lp = None
        if self.ref is not None and c.kl_coef != 0.0:
            parts = [self.ref.logprobs(tokens[a:a + mb].contiguous(), c.prompt_len, group_size=gs)[0] for a in range(0, N, mb)]
            ref_lp = torch.cat(parts)
        ev("reference")
        pol.zero_grad()
        report = torch.zeros(10, device=tokens.device)
        for a in range(0, N, mb):
            sl = slice(a, a + mb)
            report += pol.train_step(tokens[sl].contiguous(), c.prompt_len, mask[sl].contiguous(),
                                     old_logp=old_lp[sl].contiguous(), advantage=adv[sl].contiguous(),
                                     ref_logp=None if ref_lp is None else ref_lp[sl].contiguous(),
                                     units=units_global, clip_eps=c.clip_eps, kl_coef=c.kl_coef,
                                     entropy_coef=c.entropy_coef, group_size=gs)
        report[7] = units_global  # every micro-batch reports the global count: it is not a sum
        ev("train")
        if self.world > 1:
            self._allreduce(pol.grads_view())
            self._allreduce(report)
            report[7] = units_global
        ev("allreduce")
        norm = pol.optimizer_step(c.lr, weight_decay=c.weight_decay, max_grad_norm=c.max_grad_norm)
        ev("optimizer")
        return {"report": report, "grad_norm": norm, "reward_mean": rewards.mean(), "tokens": tokens}
