"""Host-side mirror of the reference's replaceable RL pipeline (include/neuralnet.cpp/rl_pipeline.hpp:29-350,
rl_experience.hpp:32-68): DeterministicRng, RolloutSource, TensorRecord / ExperienceSchema, ExperienceBuffer,
UniformBatchSampler, MetricSink, RLTrainingPipeline.run.  Same names, same argument meaning, same error
behaviour (a violated precondition raises PipelineError with the condition that failed); the tensors in a
record are device tensors produced and consumed by libnn-b200.so, so a rollout never leaves the GPU between
the source and the update.

GptRolloutSource is the device-side producer for the ternary GPT policy: one call = one batched rollout
(nnb_rollout_grouped), rewards, advantages (GroupAdvantage or GaeAdvantage) and, when a frozen reference
policy is given, its log-probs — all on the device, returned as one TensorRecord.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


class PipelineError(RuntimeError):
    pass


class DeterministicRng:
    """Seeded generator with save / restore (rl_pipeline.hpp:29-66).  The reference draws from
    std::mt19937_64; this mirror draws from numpy's MT19937, so index sequences are reproducible per seed
    but are not the reference's sequences."""

    def __init__(self, seed: int = 0):
        self._seed = int(seed)
        self._g = np.random.Generator(np.random.MT19937(self._seed))

    def seed(self) -> int:
        return self._seed

    def next_u64(self) -> int:
        return int(self._g.integers(0, 2**64, dtype=np.uint64))

    def uniform_index(self, upper_exclusive: int) -> int:
        if upper_exclusive <= 0:
            raise PipelineError("DeterministicRng: uniform_index upper bound must be > 0")
        return int(self._g.integers(0, upper_exclusive))

    def save_state(self):
        return {"tag": "RNGS1", "seed": self._seed, "state": self._g.bit_generator.state}

    def restore_state(self, state):
        if not isinstance(state, dict) or state.get("tag") != "RNGS1":
            raise PipelineError("DeterministicRng.restore_state: bad state header")
        self._seed = state["seed"]
        self._g.bit_generator.state = state["state"]


class TensorRecord(dict):
    """Named tensors of one rollout (rl_experience.hpp:32-68).  Field names follow the reference's
    ExperienceSchema: action, action_mask, advantage, return, old_value, old_log_prob (+ value_mask);
    `tokens` (prompt + generated ids), `ref_log_prob` and `reward` are this engine's additions."""

    REQUIRED = ("action", "action_mask", "advantage", "old_log_prob")

    @classmethod
    def create(cls, fields: dict):
        missing = [k for k in cls.REQUIRED if k not in fields]
        if missing:
            raise PipelineError(f"TensorRecord: missing fields {missing}")
        n = fields["action"].shape[0]
        for k, v in fields.items():
            if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.shape[0] != n:
                raise PipelineError(f"TensorRecord: field '{k}' has {v.shape[0]} rows, expected {n}")
        return cls(fields)

    def require(self, name):
        if name not in self:
            raise PipelineError(f"TensorRecord: no field '{name}'")
        return self[name]

    def rows(self) -> int:
        return int(self["action"].shape[0])

    def select(self, index: torch.Tensor):
        """The record restricted to the given rows (a minibatch)."""
        return TensorRecord({k: (v.index_select(0, index).contiguous() if isinstance(v, torch.Tensor) and v.dim() >= 1 else v)
                             for k, v in self.items()})


class RolloutSource:
    def rollout(self, rng: DeterministicRng) -> TensorRecord:
        raise NotImplementedError


class ExperienceBuffer:
    def __init__(self, capacity: int = 0):
        self._records, self._capacity = [], capacity

    def add(self, record: TensorRecord):
        if self._capacity > 0 and len(self._records) >= self._capacity:
            self._records.pop(0)
        self._records.append(record)

    def size(self):
        return len(self._records)

    def empty(self):
        return not self._records

    def capacity(self):
        return self._capacity

    def clear(self):
        self._records.clear()

    def at(self, index: int) -> TensorRecord:
        if index < 0 or index >= len(self._records):
            raise PipelineError("ExperienceBuffer.at: index out of range")
        return self._records[index]


class UniformBatchSampler:
    def __init__(self, replacement: bool = False):
        self._replacement = replacement

    def sample(self, available: int, batch_size: int, rng: DeterministicRng):
        if batch_size == 0:
            raise PipelineError("UniformBatchSampler: batch_size must be > 0")
        if available == 0:
            raise PipelineError("UniformBatchSampler: buffer is empty")
        if not self._replacement and batch_size > available:
            raise PipelineError("UniformBatchSampler: batch_size > buffer size without replacement")
        if self._replacement:
            return [rng.uniform_index(available) for _ in range(batch_size)]
        pool = list(range(available))
        out = []
        for i in range(batch_size):  # partial Fisher-Yates, as the reference does it
            pick = i + rng.uniform_index(available - i)
            pool[i], pool[pick] = pool[pick], pool[i]
            out.append(pool[i])
        return out


class CollectingMetricSink:
    def __init__(self):
        self.records = []

    def emit(self, name: str, value: float):
        self.records.append((name, float(value)))


class NullMetricSink:
    def emit(self, name, value):
        pass



def micro_batched(n: int, micro_batch: int, group_size: int, run):
    """Calls run(micro_batch), which walks n sequences in slices of micro_batch, and returns (its result, the micro-batch
    used).  The engine sizes a forward/backward workspace at the first call of a shape and refuses one that does not fit
    (status -4) before touching the device: run is then restarted from scratch with half the micro-batch (whole prompt
    groups while that is possible).  Gradients accumulate over a minibatch either way, so the result is the same sum."""
    from ._lib import NnbError

    mb = max(1, min(micro_batch, n))
    while True:
        try:
            return run(mb), mb
        except NnbError as ex:
            if getattr(ex, "status", 0) != -4 or mb <= 1:
                raise
            half = mb // 2
            if group_size > 1 and half >= group_size:
                half = half // group_size * group_size
            mb = max(1, half)

@dataclass
class RLPipelineConfig:
    batch_size: int = 1
    collect_per_update: int = 1
    buffer_capacity: int = 0
    min_buffer_size: int = 1
    clear_buffer_after_update: bool = False


class RLTrainingPipeline:
    """rollout -> buffer -> sample -> update (RLTrainingPipeline::run, rl_pipeline.hpp:312-350)."""

    def __init__(self, cfg: RLPipelineConfig, source: RolloutSource, sampler, metrics=None, seed: int = 0):
        if source is None or sampler is None:
            raise PipelineError("RLTrainingPipeline: source and sampler are required")
        if cfg.batch_size == 0 or cfg.collect_per_update == 0 or cfg.min_buffer_size == 0:
            raise PipelineError("RLTrainingPipeline: batch / collect / min_buffer must be > 0")
        if cfg.min_buffer_size < cfg.batch_size:
            raise PipelineError("RLTrainingPipeline: min_buffer_size must not be smaller than batch_size")
        if cfg.buffer_capacity > 0 and cfg.min_buffer_size > cfg.buffer_capacity:
            raise PipelineError("RLTrainingPipeline: min_buffer_size must not exceed buffer_capacity")
        self.cfg, self.source, self.sampler = cfg, source, sampler
        self.metrics = metrics or NullMetricSink()
        self.buffer = ExperienceBuffer(cfg.buffer_capacity)
        self.rng = DeterministicRng(seed)
        self.update_count = 0
        self.rollout_cursor = 0

    def run(self, updates: int, update, before_update=None, after_update=None):
        for _ in range(updates):
            for _ in range(self.cfg.collect_per_update):
                self.buffer.add(self.source.rollout(self.rng))
                self.rollout_cursor += 1
            if self.buffer.size() < self.cfg.min_buffer_size:
                raise PipelineError("RLTrainingPipeline: buffer below min_buffer_size")
            indices = self.sampler.sample(self.buffer.size(), self.cfg.batch_size, self.rng)
            if len(indices) != self.cfg.batch_size:
                raise PipelineError("RLTrainingPipeline: sampler returned a wrong batch size")
            selected = [self.buffer.at(i) for i in indices]
            if before_update:
                before_update(selected)
            update(selected, self.rng, self.metrics)
            self.update_count += 1
            try:
                if after_update:
                    after_update(selected)
            finally:
                if self.cfg.clear_buffer_after_update:
                    self.buffer.clear()

    def save_checkpoint(self):
        return {"pipeline_version": 1, "update_count": self.update_count, "rollout_cursor": self.rollout_cursor,
                "rng_state": self.rng.save_state()}

    def restore_checkpoint(self, state):
        if state.get("pipeline_version") != 1:
            raise PipelineError("RLTrainingPipeline.restore_checkpoint: incompatible version")
        self.update_count, self.rollout_cursor = state["update_count"], state["rollout_cursor"]
        self.rng.restore_state(state["rng_state"])


@dataclass
class RolloutSpec:
    prompt_len: int
    max_new: int
    group_size: int = 1
    temperature: float = 1.0
    top_k: int = 0
    rollout_chunk: int = 1024     # sequences decoded together (bounds the KV cache)
    advantage: str = "group"      # "group" (GroupAdvantage over the sequences of a prompt) or "gae"
    advantage_eps: float = 1e-8
    gamma: float = 0.99
    lam: float = 0.95
    normalize_advantage: bool = False  # MaskedNormalizer over the whole record (gae only)
    eval_micro_batch: int = 16         # sequences per teacher-forced evaluation pass (values, reference log-probs)


class GptRolloutSource(RolloutSource):
    """Device-side producer: prompts -> batched rollout -> rewards -> advantages -> TensorRecord.

    prompts_fn(cursor) -> (n_prompts, P) int32 device tensor; reward_fn(tokens (N, P+G)) -> (N,) sequence rewards
    for advantage="group", or (N, G) per-decision rewards for advantage="gae".  seq0 is the global index of
    this source's first sequence (the Philox counter), so sharding a batch over sources does not change samples."""

    def __init__(self, policy, spec: RolloutSpec, prompts_fn, reward_fn, ref_policy=None, seq0: int = 0):
        self.policy, self.spec, self.prompts_fn, self.reward_fn = policy, spec, prompts_fn, reward_fn
        self.ref, self.seq0 = ref_policy, seq0
        self.cursor = 0
        self._chunk = spec.rollout_chunk
        self.on_phase = None  # optional callback(name) at phase boundaries, for timing

    def _mark(self, name):
        if self.on_phase:
            self.on_phase(name)

    def _decode(self, rep, seed):
        from ._lib import NnbError

        c, n = self.spec, rep.shape[0]
        chunk = max(c.group_size, (min(self._chunk, n) // c.group_size) * c.group_size)
        while True:
            toks, lps = [], []
            try:
                for a in range(0, n, chunk):
                    t, lp, _ = self.policy.rollout(rep[a:a + chunk].contiguous(), c.max_new, temperature=c.temperature,
                                                   top_k=c.top_k, seed=seed, seq0=self.seq0 + a, group_size=c.group_size)
                    toks.append(t)
                    lps.append(lp)
                return torch.cat(toks), torch.cat(lps)
            except NnbError as ex:
                # the engine refuses a KV cache that does not fit (status -4) before allocating it: decode fewer
                # sequences together.  Samples do not depend on the chunking (Philox counters are per sequence).
                if getattr(ex, "status", 0) != -4 or chunk <= c.group_size:
                    raise
                chunk = max(c.group_size, (chunk // 2 // c.group_size) * c.group_size)
                self._chunk = chunk

    def rollout(self, rng: DeterministicRng = None, prompts=None, seed=None) -> TensorRecord:
        """RolloutSource::rollout.  `prompts` / `seed` override what prompts_fn and the generator would give (used
        by the step drivers, which are handed their prompts)."""
        c, pol, eng = self.spec, self.policy, self.policy.engine
        if prompts is None:
            prompts = self.prompts_fn(self.cursor)
        self.cursor += 1
        if seed is None:
            seed = rng.next_u64() if rng is not None else self.cursor
        self._mark("start")
        rep = prompts.repeat_interleave(c.group_size, dim=0).contiguous() if c.group_size > 1 else prompts.contiguous()
        tokens, old_lp = self._decode(rep, seed)
        self._mark("rollout")
        N, G, P = tokens.shape[0], c.max_new, c.prompt_len
        mask = torch.ones((N, G), device=tokens.device, dtype=torch.float32)
        fields = {"tokens": tokens, "action": tokens[:, P:].contiguous(), "action_mask": mask, "value_mask": mask,
                  "old_log_prob": old_lp}
        reward = self.reward_fn(tokens).contiguous()
        fields["reward"] = reward
        def evaluate(policy, pick, **kw):
            """teacher-forced pass over all N sequences in micro-batches; halves them if the workspace does not fit"""
            def run(mb):
                gs = c.group_size if mb % c.group_size == 0 else 1
                return torch.cat([policy.logprobs(tokens[a:a + mb].contiguous(), P, group_size=gs, **kw)[pick]
                                  for a in range(0, N, mb)])
            out, self._eval_mb = micro_batched(N, getattr(self, "_eval_mb", c.eval_micro_batch), c.group_size, run)
            return out

        if c.advantage == "group":
            adv_seq = eng.group_advantage(reward, [(g * c.group_size, c.group_size) for g in range(N // c.group_size)],
                                          eps=c.advantage_eps)
            fields["advantage"] = adv_seq[:, None].expand(N, G).contiguous()
            self._mark("advantage")
        else:
            if not pol.cfg.value_head:
                raise PipelineError("GptRolloutSource: advantage='gae' needs a policy with a value head")
            old_value = evaluate(pol, 2, want_value=True)
            # GaeAdvantage works on (steps, batch) with row = time
            adv_t, ret_t = eng.gae(reward.t().contiguous(), old_value.t().contiguous(), mask=mask.t().contiguous(),
                                   gamma=c.gamma, lam=c.lam)
            adv = adv_t.t().contiguous()
            if c.normalize_advantage:
                adv = eng.masked_normalize(adv.view(-1), mask.view(-1), eps=c.advantage_eps).view(N, G)
            fields.update(advantage=adv, old_value=old_value)
            fields["return"] = ret_t.t().contiguous()
            self._mark("advantage")
        if self.ref is not None:
            fields["ref_log_prob"] = evaluate(self.ref, 0)
        self._mark("reference")
        return TensorRecord.create(fields)
