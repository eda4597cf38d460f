"""World-size-2 gloo test of the multi-rank host logic of the GRPO step (no GPU): whole prompt
groups per rank, distinct Philox sequence offsets, the global unit count, and the all-reduce (sum)
of the flat gradient buffer and of the report.  The engine is replaced by a CPU stub so only the
orchestration in neuralnet.cpp_b200/grpo.py is under test."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class StubEngine:
    device = torch.device("cpu")

    def group_advantage(self, rewards, spans, eps=1e-8):
        out = torch.zeros_like(rewards)
        for f, c in spans:
            r = rewards[f:f + c]
            var = r.var(unbiased=False)
            out[f:f + c] = 0 if var <= eps * eps else (r - r.mean()) / var.sqrt()
        return out


class StubPolicy:
    def __init__(self, rank):
        self.engine = StubEngine()
        self.rank = rank
        self.g = torch.zeros(8)
        self.calls = []
        self.stepped = 0

    def rollout(self, prompts, max_new, temperature, top_k, seed, seq0, group_size=1):
        self.calls.append(("rollout", prompts.shape[0], seq0))
        n, p = prompts.shape
        gen = (torch.arange(n)[:, None] + seq0 + torch.arange(max_new)[None, :]).to(torch.int32) % 7
        return torch.cat([prompts, gen], 1), torch.full((n, max_new), -1.0), None

    def logprobs(self, tokens, prompt_len, group_size=1):
        return torch.full((tokens.shape[0], tokens.shape[1] - prompt_len), -1.1), None, None

    def zero_grad(self):
        self.g.zero_()

    def train_step(self, tokens, prompt_len, mask, units=0.0, **kw):
        self.calls.append(("train", tokens.shape[0], units))
        self.g += (self.rank + 1) * tokens.shape[0]
        rep = torch.zeros(10)
        rep[7] = mask.sum()
        return rep

    def grads_view(self):
        return self.g

    def optimizer_step(self, lr, **kw):
        self.stepped += 1
        return torch.tensor([float(self.g.norm())])


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package

    pkg = load_package()
    cfg = pkg.GrpoConfig(group_size=4, prompt_len=3, max_new=5, micro_batch=4, rollout_chunk=8, kl_coef=0.04)
    pol, ref = StubPolicy(rank), StubPolicy(rank)
    tr = pkg.GrpoTrainer(pol, ref, cfg)
    prompts = torch.arange(3 * 3).reshape(3, 3).to(torch.int32) + 100 * rank  # 3 groups on this rank
    out = tr.step(prompts, lambda t: (t[:, 3:].sum(1) % 2).float(), seed=1)
    q.put((rank, pol.g.clone(), pol.calls, out["report"].clone(), pol.stepped, out["tokens"].shape))
    dist.destroy_process_group()


def test_two_rank_grpo_step_host_logic():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in procs], key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (r0, g0, c0, rep0, s0, shape0), (r1, g1, c1, rep1, s1, shape1) = res
    # 3 groups x 4 sequences per rank; rollout in chunks of 8 (whole groups), offsets continue per rank
    assert shape0 == (12, 8) and shape1 == (12, 8)
    assert [c for c in c0 if c[0] == "rollout"] == [("rollout", 8, 0), ("rollout", 4, 8)]
    assert [c for c in c1 if c[0] == "rollout"] == [("rollout", 8, 12), ("rollout", 4, 20)]
    # every micro-batch is normalised by the GLOBAL unit count (2 ranks x 12 sequences x 5 decisions)
    assert all(c[2] == 120.0 for c in c0 + c1 if c[0] == "train")
    # gradient buffers hold the sum over ranks and are identical: (1 + 2) * 12
    assert torch.equal(g0, g1) and torch.all(g0 == 36)
    assert rep0[7] == 120 and rep1[7] == 120
    assert s0 == 1 and s1 == 1


class TightStubPolicy(StubPolicy):
    """refuses a training micro-batch of more than `limit` sequences the way the engine refuses a workspace that does
    not fit: status -4, nothing accumulated"""
    limit = 4

    def train_step(self, tokens, prompt_len, mask, units=0.0, **kw):
        if tokens.shape[0] > self.limit:
            from neuralnet_cpp_b200._lib import NnbError

            err = NnbError("nnb_status -4: training workspace does not fit")
            err.status = -4
            raise err
        return super().train_step(tokens, prompt_len, mask, units=units, **kw)


def _uneven_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package

    pkg = load_package()
    cfg = pkg.GrpoConfig(group_size=4, prompt_len=3, max_new=5, micro_batch=12, rollout_chunk=16)
    # only rank 1 runs short of memory: it falls back to 4-sequence micro-batches, rank 0 keeps 12
    pol = TightStubPolicy(rank) if rank == 1 else StubPolicy(rank)
    tr = pkg.GrpoTrainer(pol, None, cfg)
    prompts = torch.arange(3 * 3).reshape(3, 3).to(torch.int32) + 100 * rank
    out = tr.step(prompts, lambda t: (t[:, 3:].sum(1) % 2).float(), seed=1)
    q.put((rank, pol.g.clone(), [c for c in pol.calls if c[0] == "train"], float(out["report"][7]), pol.stepped))
    dist.destroy_process_group()


def test_ranks_may_fall_back_to_different_micro_batches():
    """the collectives of a step come after the micro-batch loop, so a rank that halves its micro-batch still meets the
    others at the same all-reduces and the summed gradient is the same"""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 33500 + os.getpid() % 2000
    procs = [ctx.Process(target=_uneven_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in procs], key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, g0, t0, u0, s0), (_, g1, t1, u1, s1) = res
    assert [c[1] for c in t0] == [12] and [c[1] for c in t1] == [4, 4, 4]
    assert torch.equal(g0, g1) and torch.all(g0 == 36) and u0 == 120 and u1 == 120 and s0 == 1 and s1 == 1
