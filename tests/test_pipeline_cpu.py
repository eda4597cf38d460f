"""Host logic of the RL pipeline mirror (neuralnet.cpp_b200/pipeline.py, ppo.py) without a GPU: buffer capacity,
sampling without replacement, the run loop's order of calls and its precondition errors
(include/neuralnet.cpp/rl_pipeline.hpp:68-152,312-350; pattern of src/rl_pipeline_test.cpp), and a world-size-2
gloo run of the PPO epochs x minibatches loop on a stub policy (trajectories sharded, one all-reduce per minibatch)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rec(pkg, n=4, tag=0.0):
    return pkg.TensorRecord.create({"action": torch.zeros(n, 2), "action_mask": torch.ones(n, 2),
                                    "advantage": torch.full((n, 2), tag), "old_log_prob": torch.zeros(n, 2)})


def test_buffer_sampler_and_record(pkg):
    buf = pkg.ExperienceBuffer(capacity=2)
    for t in range(3):
        buf.add(_rec(pkg, tag=float(t)))
    assert buf.size() == 2 and float(buf.at(0)["advantage"][0, 0]) == 1.0  # the oldest record was dropped
    with pytest.raises(pkg.PipelineError):
        buf.at(2)
    rng = pkg.DeterministicRng(5)
    s = pkg.UniformBatchSampler(False).sample(10, 10, rng)
    assert sorted(s) == list(range(10))  # without replacement: a permutation
    with pytest.raises(pkg.PipelineError):
        pkg.UniformBatchSampler(False).sample(3, 4, rng)
    assert len(pkg.UniformBatchSampler(True).sample(3, 8, rng)) == 8
    state = rng.save_state()
    a = [rng.uniform_index(100) for _ in range(5)]
    rng.restore_state(state)
    assert a == [rng.uniform_index(100) for _ in range(5)]
    with pytest.raises(pkg.PipelineError):
        pkg.TensorRecord.create({"action": torch.zeros(2, 2)})
    sub = _rec(pkg, 6).select(torch.tensor([4, 1]))
    assert sub.rows() == 2


def test_pipeline_run_order_and_preconditions(pkg):
    class Source(pkg.RolloutSource):
        def __init__(self):
            self.n = 0

        def rollout(self, rng):
            self.n += 1
            return _rec(pkg, tag=float(self.n))

    calls = []
    cfg = pkg.RLPipelineConfig(batch_size=2, collect_per_update=2, min_buffer_size=2, clear_buffer_after_update=True)
    sink = pkg.CollectingMetricSink()
    pipe = pkg.RLTrainingPipeline(cfg, Source(), pkg.UniformBatchSampler(False), sink, seed=3)

    def update(selected, rng, metrics):
        calls.append(("update", sorted(float(r["advantage"][0, 0]) for r in selected)))
        metrics.emit("loss", 1.0)

    pipe.run(2, update, before_update=lambda sel: calls.append(("before", len(sel))),
             after_update=lambda sel: calls.append(("after", len(sel))))
    assert calls == [("before", 2), ("update", [1.0, 2.0]), ("after", 2), ("before", 2), ("update", [3.0, 4.0]), ("after", 2)]
    assert pipe.update_count == 2 and pipe.rollout_cursor == 4 and pipe.buffer.empty() and len(sink.records) == 2
    st = pipe.save_checkpoint()
    pipe.update_count = 0
    pipe.restore_checkpoint(st)
    assert pipe.update_count == 2
    with pytest.raises(pkg.PipelineError):
        pkg.RLTrainingPipeline(pkg.RLPipelineConfig(batch_size=4, min_buffer_size=2), Source(), pkg.UniformBatchSampler())
    with pytest.raises(pkg.PipelineError):
        pkg.RLTrainingPipeline(pkg.RLPipelineConfig(), None, pkg.UniformBatchSampler())


class _StubEngine:
    device = torch.device("cpu")

    def gae(self, rewards, values, mask=None, gamma=0.99, lam=0.95):
        return rewards - values, rewards.clone()

    def group_advantage(self, rewards, spans, eps=1e-6):
        out = torch.zeros_like(rewards)
        for f, c in spans:
            out[f:f + c] = rewards[f:f + c] - rewards[f:f + c].mean()
        return out


class _StubCfg:
    value_head = True


class _StubPolicy:
    def __init__(self, rank):
        self.engine, self.cfg, self.rank = _StubEngine(), _StubCfg(), rank
        self.g = torch.zeros(4)
        self.calls, self.stepped = [], 0

    def rollout(self, prompts, max_new, temperature, top_k, seed, seq0, group_size=1):
        self.calls.append(("rollout", prompts.shape[0], seq0))
        n = prompts.shape[0]
        gen = (torch.arange(n)[:, None] + seq0 + torch.arange(max_new)[None, :]).to(torch.int32)
        return torch.cat([prompts, gen], 1), torch.full((n, max_new), -1.0), None

    def logprobs(self, tokens, prompt_len, want_value=False, group_size=1):
        n, g = tokens.shape[0], tokens.shape[1] - prompt_len
        return torch.full((n, g), -1.0), None, torch.zeros(n, g)

    def zero_grad(self):
        self.g.zero_()

    def train_step(self, tokens, prompt_len, mask, units=0.0, **kw):
        self.calls.append(("train", tokens.shape[0], units, sorted(int(t) for t in tokens[:, prompt_len])))
        self.g += tokens.shape[0]
        rep = torch.zeros(10)
        rep[7] = mask.sum()
        return rep

    def grads_view(self):
        return self.g

    def optimizer_step(self, lr, **kw):
        self.calls.append(("opt", float(self.g[0])))
        self.stepped += 1
        return torch.zeros(1)


def _ppo_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package

    pkg = load_package()
    cfg = pkg.PpoConfig(prompt_len=2, max_new=3, epochs=2, minibatches=2, micro_batch=2, rollout_chunk=8)
    pol = _StubPolicy(rank)
    tr = pkg.PpoTrainer(pol, cfg, seed=9)
    prompts = torch.zeros((4, 2), dtype=torch.int32)  # 4 trajectories on this rank
    out = tr.step(prompts, lambda t: torch.ones(t.shape[0], 3), seed=1)
    q.put((rank, pol.calls, pol.stepped, float(out["report"][7])))
    dist.destroy_process_group()


def test_two_rank_ppo_epochs_and_minibatches():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_ppo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in procs], key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, c0, s0, u0), (_, c1, s1, u1) = res
    assert c0[0] == ("rollout", 4, 0) and c1[0] == ("rollout", 4, 4)  # sequence offsets continue over the ranks
    # 2 epochs x 2 minibatches = 4 optimizer steps per rank, each after ONE micro-batch of 2 trajectories here,
    # normalised by the global decision count of the minibatch (2 ranks x 2 trajectories x 3 decisions)
    assert s0 == 4 and s1 == 4 and u0 == 12.0 and u1 == 12.0
    trains0 = [c for c in c0 if c[0] == "train"]
    assert len(trains0) == 4 and all(c[1] == 2 and c[2] == 12.0 for c in trains0)
    # every epoch visits each local trajectory exactly once
    for ep in range(2):
        seen = sorted(t for c in trains0[2 * ep:2 * ep + 2] for t in c[3])
        assert seen == [0, 1, 2, 3]
    # gradients are summed over the ranks before each optimizer step: 2 + 2
    assert all(c[1] == 4.0 for c in c0 + c1 if c[0] == "opt")


def test_micro_batch_halves_when_the_workspace_does_not_fit(pkg):
    """The engine refuses a training workspace that does not fit (status -4) before it touches the device; the trainers
    then restart the accumulation with half the micro-batch (whole prompt groups while possible) and keep the smaller
    size.  Other errors pass through."""
    from neuralnet_cpp_b200._lib import NnbError
    from neuralnet_cpp_b200.pipeline import micro_batched

    class Tight(_StubPolicy):
        limit = 4

        def train_step(self, tokens, prompt_len, mask, units=0.0, **kw):
            if tokens.shape[0] > self.limit:
                err = NnbError("nnb_status -4: training workspace does not fit")
                err.status = -4
                raise err
            self.groups = kw.get("group_size")
            return super().train_step(tokens, prompt_len, mask, units=units, **kw)

        def logprobs(self, tokens, prompt_len, want_value=False, group_size=1):
            if tokens.shape[0] > 8:
                err = NnbError("nnb_status -4: workspace does not fit")
                err.status = -4
                raise err
            self.calls.append(("eval", tokens.shape[0], group_size))
            return super().logprobs(tokens, prompt_len, want_value=want_value, group_size=group_size)

    pol, ref = Tight(0), Tight(0)
    cfg = pkg.GrpoConfig(group_size=2, prompt_len=2, max_new=3, micro_batch=16, rollout_chunk=64, kl_coef=0.04)
    tr = pkg.GrpoTrainer(pol, ref, cfg)
    prompts = torch.zeros((6, 2), dtype=torch.int32)  # 6 groups of 2
    out = tr.step(prompts, lambda t: torch.arange(t.shape[0]).float(), seed=1)
    trains = [c for c in pol.calls if c[0] == "train"]
    # 12 sequences: 16 -> 12 (all) refused, 6 refused, 2 (6 // 2 = 3, rounded down to whole groups) accepted
    assert [c[1] for c in trains] == [2] * 6 and pol.groups == 2
    assert float(pol.g[0]) == 12.0 and pol.stepped == 1 and float(out["report"][7]) == 36.0
    # the frozen policy's log-probs: 12 at once refused, 6 accepted (whole groups)
    assert [c for c in ref.calls if c[0] == "eval"] == [("eval", 6, 2), ("eval", 6, 2)]
    # the smaller size is kept: the next step does not try 12 again
    pol.calls.clear()
    tr.step(prompts, lambda t: torch.arange(t.shape[0]).float(), seed=2)
    assert [c[1] for c in pol.calls if c[0] == "train"] == [2] * 6

    # other errors, and a refusal at one sequence, are the caller's
    def boom(mb):
        err = NnbError("nnb_status -2: bad argument")
        err.status = -2
        raise err

    with pytest.raises(NnbError):
        micro_batched(8, 4, 1, boom)

    def never_fits(mb):
        err = NnbError("nnb_status -4")
        err.status = -4
        raise err

    with pytest.raises(NnbError):
        micro_batched(8, 4, 1, never_fits)
    assert micro_batched(8, 4, 1, lambda mb: mb * 10) == (40, 4)
