"""Pins the decode-path oracle (oracle/oracle_model.c): sampler rules from src/sampling_test.cpp,
the bit-reproducible exp, Philox known answers, and self-consistency of the GPT step path."""
import math

import numpy as np
import pytest


def test_expf_close_to_libm(orc):
    xs = np.concatenate([np.linspace(-85, 85, 20001), np.random.default_rng(0).normal(0, 3, 20000)]).astype(np.float32)
    worst = 0.0
    for x in xs[::7]:
        got = orc.expf(float(x))
        ref = math.exp(float(x))
        worst = max(worst, abs(got - ref) / ref)
    assert worst < 2.5e-7  # ~2 ulp
    assert orc.expf(0.0) == 1.0
    assert orc.expf(-100.0) == 0.0


def test_philox_known_answer(orc):
    # Philox4x32-10 known-answer vectors of the Random123 distribution (kat_vectors):
    # counter 0,0,0,0 key 0,0 -> 6627e8d5 e169c58d bc57ac4c 9b00dbd8
    u = orc.philox_uniform(0, 0, 0)
    assert u == (0x6627E8D5 >> 8) / 16777216.0
    # counter ffffffff x4, key ffffffff x2 -> 408f276d ...
    # (our counter is (sequence, step, 0, 0) so only the all-zero vector applies directly)
    us = [orc.philox_uniform(1234, s, t) for s in range(4) for t in range(4)]
    assert len(set(us)) == 16 and all(0.0 <= v < 1.0 for v in us)


# ---- src/sampling_test.cpp:114-151 (top-k), :290-301 (greedy), ties -> smallest index ------------
def test_sampler_top_k_support(orc):
    logits = [1.0, 4.0, 2.0, 3.0]
    rs = np.random.default_rng(1).uniform(0, 1, 500)
    assert all(orc.sample_token(logits, 1.0, 2, float(r)) in (1, 3) for r in rs)
    assert all(orc.sample_token(logits, 1.0, 1, float(r)) == 1 for r in rs[:50])  # top_k=1 == argmax
    tie = [2.0, 2.0, 2.0]
    assert all(orc.sample_token(tie, 1.0, 2, float(r)) <= 1 for r in rs[:50])  # ties keep the smaller index


def test_sampler_greedy_rules(orc):
    assert orc.sample_token([1.0, 5.0, 2.0, 3.0], 0.0, 3, 0.123) == 1
    assert orc.sample_token([5.0, 5.0, 1.0], 0.0, 0, 0.9) == 0  # ties -> smallest index
    assert orc.sample_token([5.0, 5.0, 1.0], -1.0, 0, 0.9) == 0


def test_sampler_inverse_cdf(orc):
    logits = np.log(np.array([0.1, 0.2, 0.3, 0.4], np.float32))
    assert orc.sample_token(logits, 1.0, 0, 0.05) == 0
    assert orc.sample_token(logits, 1.0, 0, 0.25) == 1
    assert orc.sample_token(logits, 1.0, 0, 0.55) == 2
    assert orc.sample_token(logits, 1.0, 0, 0.95) == 3
    assert orc.sample_token(logits, 1.0, 0, 0.99999994) == 3  # fallback = last candidate
    # temperature sharpens: at T=0.1 nearly all mass sits on index 3
    assert orc.sample_token(logits, 0.1, 0, 0.2) == 3
    # frequencies follow softmax
    rs = np.random.default_rng(2).uniform(0, 1, 4000)
    counts = np.bincount([orc.sample_token(logits, 1.0, 0, float(r)) for r in rs], minlength=4) / 4000
    assert np.abs(counts - [0.1, 0.2, 0.3, 0.4]).max() < 0.03


def test_rmsnorm_formula(orc):
    rng = np.random.default_rng(3)
    x = rng.normal(0, 2, 256).astype(np.float32)
    g = rng.normal(1, 0.1, 256).astype(np.float32)
    got = orc.rmsnorm(x, g)
    ref = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-5) * g
    assert np.abs(got - ref).max() < 1e-5


def _tiny(pkgmod, act, pos, seed=1):
    cfg = pkgmod.GptConfig(n_layer=2, d_model=64, n_head=2, d_ff=128, vocab=97, ctx=24, act=act, pos=pos)
    return cfg, cfg.init_params(seed, bias_std=0.01)


@pytest.mark.parametrize("act,pos", [(0, 0), (1, 1)])
def test_layout_and_quantisation_agree(pkg, orc, act, pos):
    from oracle_binding import OracleGpt

    cfg, flat = _tiny(pkg, act, pos)
    layout, n = cfg.param_layout()
    m = OracleGpt(cfg, flat)
    assert m.param_count() == n
    lay = {name: (off, shape) for name, off, shape in layout}
    off, shape = lay["blocks.1.ffn.fc1.weight"]
    W = flat[off:off + shape[0] * shape[1]].reshape(shape)
    tau, trit = m.linear(1, 4, shape[0], shape[1])
    assert np.array_equal(tau, orc.absmean_tau(W))
    assert np.array_equal(trit, orc.trit_unpack(orc.trit_pack(W, tau), shape[1]))


@pytest.mark.parametrize("act,pos", [(0, 0), (1, 1)])
def test_rollout_is_consistent_with_teacher_forced_step_logits(pkg, act, pos):
    from oracle_binding import OracleGpt

    cfg, flat = _tiny(pkg, act, pos)
    m = OracleGpt(cfg, flat)
    prompts = np.random.default_rng(5).integers(0, cfg.vocab, (3, 5)).astype(np.int32)
    tokens, logp, logits = m.rollout(prompts, 6, 0.0, 0, seed=7, want_logits=True)
    assert np.array_equal(tokens[:, :5], prompts)
    for b in range(3):
        full = m.step_logits(tokens[b])
        # logits that produced generated token t sit at position P-1+t of the teacher-forced pass
        assert np.array_equal(full[4:10], logits[b])
        assert np.array_equal(tokens[b, 5:], full[4:10].argmax(1))
        lse = np.log(np.exp(full[4:10].astype(np.float64) - full[4:10].max(1, keepdims=True)).sum(1)) + full[4:10].max(1)
        ref_lp = full[4:10][np.arange(6), tokens[b, 5:]] - lse
        assert np.abs(logp[b] - ref_lp).max() < 1e-5
    # sampled rollouts are reproducible and depend on the seed
    t1, _, _ = m.rollout(prompts, 6, 1.0, 10, seed=7)
    t2, _, _ = m.rollout(prompts, 6, 1.0, 10, seed=7)
    t3, _, _ = m.rollout(prompts, 6, 1.0, 10, seed=8)
    assert np.array_equal(t1, t2) and not np.array_equal(t1, t3)


# src/sampling_test.cpp:153-176: nucleus sampling
def test_sampler_top_p(orc):
    rs = np.random.default_rng(1).uniform(size=300).astype(np.float32)
    assert {orc.sample_token_cfg([10.0, 0.0, 0.0, 0.0], top_p=0.5, r=float(r)) for r in rs} == {0}  # near one-hot: the peak only
    assert 0 in {orc.sample_token_cfg([10.0, 0.0, 0.0, 0.0], top_p=1e-9, r=float(r)) for r in rs[:50]}  # never an empty set
    flat = {orc.sample_token_cfg([1.0, 1.0, 1.0, 1.0], top_p=0.5, r=float(r)) for r in rs}
    assert len(flat) <= 2 and flat <= {0, 1}  # four equal entries, p = 0.5: two kept, ties to the smaller indices


# src/sampling_test.cpp:178-222: repeat penalty, window, and the multiplicative branch for negative logits
def test_sampler_repeat_penalty(orc):
    assert orc.sample_token_cfg([5.0, 4.0], temperature=0.0, history=[0]) == 0
    assert orc.sample_token_cfg([5.0, 4.0], temperature=0.0, repeat_penalty=10.0, history=[0]) == 1
    assert orc.sample_token_cfg([5.0, 4.0], temperature=0.0, repeat_penalty=10.0, repeat_window=1, history=[1, 0]) == 1
    assert orc.sample_token_cfg([5.0, 4.0], temperature=0.0, repeat_penalty=10.0, repeat_window=0, history=[1, 0]) == 0
    assert orc.sample_token_cfg([-1.0, -5.0], temperature=0.0, repeat_penalty=10.0, history=[1]) == 0
    # a token that occurs twice in the window is penalised once
    assert orc.sample_token_cfg([5.0, 0.6], temperature=0.0, repeat_penalty=3.0, history=[0, 0]) == 0  # 5/3 > 0.6, 5/9 < 0.6


# logits_transform (src/sampling_test.cpp, the hook runs before every other rule): a bias of -inf forbids a token
def test_sampler_bias_comes_first(orc):
    bias = np.array([-np.inf, 0.0, 0.0], np.float32)
    assert orc.sample_token_cfg([9.0, 1.0, 2.0], temperature=0.0, bias=bias) == 2
    rs = np.random.default_rng(2).uniform(size=100).astype(np.float32)
    assert {orc.sample_token_cfg([9.0, 1.0, 2.0], bias=bias, r=float(r)) for r in rs} <= {1, 2}


def test_sampler_cfg_defaults_equal_the_plain_sampler(orc):
    rng = np.random.default_rng(3)
    for _ in range(50):
        lg = rng.normal(0, 2, 40).astype(np.float32)
        r = float(rng.uniform())
        assert orc.sample_token_cfg(lg, temperature=0.7, top_k=5, r=r) == orc.sample_token(lg, 0.7, 5, r)
