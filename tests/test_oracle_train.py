"""Self-consistency of the numpy training oracle (oracle/oracle_train.py): its forward agrees with
the C restatement of the step path, and its smooth sub-blocks pass finite-difference checks."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle_train as ot  # noqa: E402


@pytest.mark.parametrize("act,pos", [(0, 0), (1, 1)])
def test_forward_matches_step_path(pkg, orc, act, pos):
    from oracle_binding import OracleGpt

    cfg = pkg.GptConfig(n_layer=2, d_model=64, n_head=2, d_ff=128, vocab=97, ctx=24, act=act, pos=pos)
    flat = cfg.init_params(1, bias_std=0.01)
    tr = ot.OracleTrainer(cfg, flat)
    m = OracleGpt(cfg, flat)
    tokens = np.random.default_rng(0).integers(0, 97, (3, 12)).astype(np.int32)
    logp, ent, _ = tr.forward(tokens, 4)
    # quantisation of weights and activations is bit-identical to the C oracle
    tau, trit = m.linear(1, 4, tr.lin["blocks.1.ffn.fc1"].trit.shape[0], 64)
    assert np.array_equal(tau, tr.lin["blocks.1.ffn.fc1"].tau) and np.array_equal(trit, tr.lin["blocks.1.ffn.fc1"].trit)
    for b in range(3):
        full = m.step_logits(tokens[b])[3:11]
        ref_lp = [orc.logprob_entropy(full[g], int(tokens[b, 4 + g])) for g in range(8)]
        assert np.abs(logp[b] - [r[0] for r in ref_lp]).max() < 2e-4
        assert np.abs(ent[b] - [r[1] for r in ref_lp]).max() < 2e-4
    q, s = ot.act_quant(np.random.default_rng(1).normal(0, 1, (5, 64)).astype(np.float32))
    q2, s2 = orc.act_quant_tm(np.random.default_rng(1).normal(0, 1, (5, 64)).astype(np.float32))
    assert np.array_equal(q, q2) and np.array_equal(s, s2)


def test_rmsnorm_backward_finite_differences():
    rng = np.random.default_rng(2)
    x = rng.normal(0, 1, (3, 16)).astype(np.float32)
    g = rng.normal(1, 0.1, 16)
    dy = rng.normal(0, 1, (3, 16))
    _, cache = ot.rmsnorm_fwd(x, g)
    dx, dg = ot.rmsnorm_bwd(dy, g, cache)

    def f(xx, gg):
        x64 = xx.astype(np.float64)
        return ((x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + 1e-5) * gg) * dy).sum()

    eps = 1e-4
    for i in range(3):
        for j in range(0, 16, 5):
            a, b = x.astype(np.float64).copy(), x.astype(np.float64).copy()
            a[i, j] += eps
            b[i, j] -= eps
            assert abs((f(a, g) - f(b, g)) / (2 * eps) - dx[i, j]) < 1e-5
    for j in range(0, 16, 3):
        a, b = g.copy(), g.copy()
        a[j] += eps
        b[j] -= eps
        assert abs((f(x, a) - f(x, b)) / (2 * eps) - dg[j]) < 1e-5


def test_objective_matches_c_oracle():
    from oracle_binding import OracleRL

    rl = OracleRL()
    rng = np.random.default_rng(3)
    n = 200
    logp = rng.normal(-3, 1, n)
    old = logp + rng.normal(0, 0.3, n)
    ref = logp + rng.normal(0, 0.1, n)
    adv = rng.normal(0, 1, n)
    ent = rng.uniform(0, 4, n)
    mask = (rng.uniform(size=n) < 0.8).astype(np.float64)
    rep, up_lp, up_ent, _ = ot.OracleTrainer.objective(logp, ent, mask, old, adv, ref, clip_eps=0.2, kl_coef=0.04, entropy_coef=0.01)
    up_p, m = rl.clipped_policy(logp, old, adv, mask, 0.2)
    kl, up_k = rl.sampled_kl(logp, ref, mask, 0.04)
    el, up_e = rl.entropy_bonus(ent, mask, 0.01)
    assert np.abs(up_lp - (up_p + up_k)).max() < 1e-6 and np.abs(up_ent - up_e).max() < 1e-7
    assert abs(rep["policy_loss"] - m["loss"]) < 1e-5 and abs(rep["kl_loss"] - kl) < 1e-6 and abs(rep["entropy_loss"] - el) < 1e-6
    assert abs(rep["clip_fraction"] - m["clip_fraction"]) < 1e-6 and abs(rep["approx_kl"] - m["approx_kl"]) < 1e-6


def test_grpo_preset_equals_its_parts_on_the_reference_case():
    """src/rl_grpo_test.cpp:85-151: two groups of three samples, three classes, returns {1,2,3 | 10,10,10}, old log-probs
    0, the preset's defaults (clip 0.2, entropy coefficient 0.01, no KL term: include/neuralnet.cpp/rl_policy.hpp:848-856).
    Group advantages {-1/s, 0, 1/s, 0, 0, 0} with s = sqrt(2/3); the preset's loss and logit gradient equal
    ClippedPolicyObjective + EntropyBonusObjective on those advantages."""
    from oracle_binding import OracleRL

    rl = OracleRL()
    # the reference stores logits as (classes, samples); row-major list from the test
    lg = np.array([1, 0, 0, 0, 0, 0, 0, 1, 0, 0, 0, 0, -1, 0, 1, 0, 0, 0], np.float32).reshape(3, 6).T.copy()
    actions = np.array([0, 1, 2, 0, 1, 2], np.int32)
    mask = np.ones(6)
    s = np.sqrt(2.0 / 3.0)
    adv = rl.group_advantage([1, 2, 3, 10, 10, 10], [(0, 3), (3, 3)], eps=1e-8)
    assert np.abs(adv - np.array([-1 / s, 0, 1 / s, 0, 0, 0])).max() < 2e-5
    logp, ent = rl.categorical_logp_entropy(lg, actions)
    old = np.zeros(6)
    rep, up_lp, up_ent, _ = ot.OracleTrainer.objective(logp, ent, mask, old, adv, None, clip_eps=0.2, kl_coef=0.0,
                                                       entropy_coef=0.01)
    up_p, m = rl.clipped_policy(logp, old, adv, mask, 0.2)
    el, up_e = rl.entropy_bonus(ent, mask, 0.01)
    total = rep["policy_loss"] + rep["kl_loss"] + rep["entropy_loss"] + rep["value_loss"]
    assert abs(total - (m["loss"] + el)) < 1e-5 and rep["kl_loss"] == 0 and rep["value_loss"] == 0
    grad = rl.categorical_backward(lg, actions, np.asarray(up_lp, np.float32), np.asarray(up_ent, np.float32))
    want = rl.categorical_backward(lg, actions, up_p, None) + rl.categorical_backward(lg, actions, None, up_e)
    assert np.abs(grad - want).max() < 1e-6
    # the second group has zero variance: its advantages, and with them its policy gradient, vanish
    assert np.abs(rl.categorical_backward(lg, actions, up_p, None)[3:]).max() == 0
