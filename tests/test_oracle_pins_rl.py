"""Pins oracle/oracle_rl.c to the known answers of the reference's RL tests
(src/rl_experience_test.cpp, src/rl_policy_test.cpp, src/rl_ppo_test.cpp, src/rl_grpo_test.cpp)."""
import numpy as np
import pytest

from oracle_binding import OracleRL


@pytest.fixture(scope="module")
def rl():
    return OracleRL()


def near(a, b, tol=1e-5):
    return np.allclose(np.asarray(a, np.float64), np.asarray(b, np.float64), atol=tol, rtol=0)


# src/rl_experience_test.cpp:107-123
def test_gae_hand_calculation(rl):
    adv, ret = rl.gae([[1], [2], [3]], [[0.5], [0.5], [0.5]], done=[[0], [0], [1]], bootstrap=[0.7], gamma=0.5, lam=0.8)
    assert near(adv.ravel(), [1.85, 2.75, 2.5])
    assert near(ret.ravel(), [2.35, 3.25, 3.0])


# src/rl_experience_test.cpp:125-158
def test_gae_done_mask_bootstrap(rl):
    adv, _ = rl.gae([[1], [2], [3]], [[0], [0], [0]], done=[[0], [1], [0]], mask=[[1], [0], [1]], gamma=1.0, lam=1.0)
    assert near(adv.ravel(), [1.0, 0.0, 3.0])
    adv, _ = rl.gae([[1], [1]], [[0], [0]], bootstrap=[2.0], gamma=0.5, lam=1.0)
    assert near(adv.ravel(), [2.0, 2.0])
    adv, _ = rl.gae([[1], [2], [3]], [[0], [10], [0]], mask=[[1], [0], [1]], gamma=0.5, lam=1.0)
    assert near(adv.ravel(), [1.0, 0.0, 3.0])


# src/rl_experience_test.cpp:160-190
def test_masked_normalizer(rl):
    s = np.sqrt(2.0 / 3.0)
    assert near(rl.masked_normalize([1, 2, 3], [1, 1, 1]), [-1 / s, 0, 1 / s])
    assert near(rl.masked_normalize([2, 2, 2], [1, 1, 1]), [0, 0, 0])  # zero variance -> 0, not NaN
    assert near(rl.masked_normalize([1, 2, 3], [0, 0, 0]), [0, 0, 0])


# src/rl_experience_test.cpp:192-212
def test_group_advantage(rl):
    s = np.sqrt(2.0 / 3.0)
    out = rl.group_advantage([1, 2, 3, 10, 10, 10], [(0, 3), (3, 3)])
    assert near(out, [-1 / s, 0, 1 / s, 0, 0, 0])
    assert rl.group_advantage([1, 2, 3, 10, 10, 10], [(0, 2), (3, 1)]) is None  # non-contiguous spans rejected


# src/rl_policy_test.cpp:160-205: logits (3,2) column per decision = {1,0,-1} and {0,2,0}
LOGITS_TM = np.array([[1, 0, -1], [0, 2, 0]], np.float32)
ACTIONS = np.array([0, 1], np.int32)


def _softmax(x):
    e = np.exp(x - x.max())
    return e / e.sum()


def test_categorical_hand_reference(rl):
    p0, p1 = _softmax(LOGITS_TM[0].astype(np.float64)), _softmax(LOGITS_TM[1].astype(np.float64))
    logp, ent = rl.categorical_logp_entropy(LOGITS_TM, ACTIONS)
    assert near(logp, [np.log(p0[0]), np.log(p1[1])])
    assert near(ent, [-(p0 * np.log(p0)).sum(), -(p1 * np.log(p1)).sum()])
    g = rl.categorical_backward(LOGITS_TM, ACTIONS, up_lp=[1, 1])
    want0, want1 = -p0, -p1
    want0[0] += 1
    want1[1] += 1
    assert near(g, [want0, want1])  # onehot - softmax


def test_entropy_gradient_matches_finite_differences(rl):
    rng = np.random.default_rng(0)
    lg = rng.normal(0, 1, (3, 7)).astype(np.float32)
    act = np.array([1, 2, 3], np.int32)
    g = rl.categorical_backward(lg, act, up_ent=[1, 1, 1])
    eps = 1e-3
    for t in range(3):
        for j in range(7):
            a, b = lg.copy(), lg.copy()
            a[t, j] += eps
            b[t, j] -= eps
            num = (rl.categorical_logp_entropy(a, act)[1][t] - rl.categorical_logp_entropy(b, act)[1][t]) / (2 * eps)
            assert abs(num - g[t, j]) < 3e-3


# src/rl_ppo_test.cpp:119-195: ratios {0.5, 1.5}, A = +1 -> loss -0.85; A = -1 -> 1.15
def test_ppo_clip_branches(rl):
    logp, _ = rl.categorical_logp_entropy(LOGITS_TM, ACTIONS)
    old = logp - np.log(np.array([0.5, 1.5], np.float32))
    up, m = rl.clipped_policy(logp, old, [1, 1], [1, 1], 0.2)
    assert abs(m["loss"] - (-0.85)) < 1e-5
    assert abs(m["ratio_mean"] - 1.0) < 1e-5
    assert abs(m["clip_fraction"] - 1.0) < 1e-5
    _, m = rl.clipped_policy(logp, old, [-1, -1], [1, 1], 0.2)
    assert abs(m["loss"] - 1.15) < 1e-5
    # finite differences of the loss w.r.t. logits (3e-3, as the reference test)
    up, _ = rl.clipped_policy(logp, old, [1, 1], [1, 1], 0.2)
    g = rl.categorical_backward(LOGITS_TM, ACTIONS, up_lp=up)
    eps = 1e-3
    for t in range(2):
        for j in range(3):
            a, b = LOGITS_TM.copy(), LOGITS_TM.copy()
            a[t, j] += eps
            b[t, j] -= eps
            la = rl.clipped_policy(rl.categorical_logp_entropy(a, ACTIONS)[0], old, [1, 1], [1, 1], 0.2)[1]["loss"]
            lb = rl.clipped_policy(rl.categorical_logp_entropy(b, ACTIONS)[0], old, [1, 1], [1, 1], 0.2)[1]["loss"]
            assert abs((la - lb) / (2 * eps) - g[t, j]) < 3e-3


# src/rl_ppo_test.cpp:262-281
def test_value_clip(rl):
    loss, grad, cf = rl.clipped_value([1, 1.8], [0, 1], [0, 1], [1, 1], 0.2, 1.0)
    assert abs(loss - 0.82) < 1e-5
    assert near(grad, [1, 0.8])
    assert abs(cf - 1.0) < 1e-5


def test_kl_and_entropy_terms(rl):
    loss, up = rl.sampled_kl([-1.0, -2.0, -3.0], [-1.5, -2.0, -2.0], [1, 1, 0], 0.04)
    assert abs(loss - 0.04 * (0.5 + 0.0) / 2) < 1e-7
    assert near(up, [0.02, 0.02, 0.0])
    loss, up = rl.entropy_bonus([1.0, 2.0, 5.0], [1, 1, 0], 0.01)
    assert abs(loss - (-0.01 * 3.0 / 2)) < 1e-7
    assert near(up, [-0.005, -0.005, 0.0])
    # units == 0 -> zero loss and zero gradient (rl_policy.hpp:579-584)
    up, m = rl.clipped_policy([-1.0], [-1.0], [1.0], [0.0])
    assert m["loss"] == 0 and up[0] == 0


def test_adamw_single_step_hand_reference(rl):
    p, g = np.array([1.0, -2.0], np.float32), np.array([0.5, -0.25], np.float32)
    p2, m2, v2 = rl.adamw(p, g, np.zeros(2), np.zeros(2), lr=0.1, t=1, wd=0.01)
    # t=1: m_hat = g, v_hat = g^2 -> step = lr * g/(|g| + eps) = lr*sign(g); decay first
    want = p * (1 - 0.1 * 0.01) - 0.1 * np.sign(g)
    assert near(p2, want, 1e-6)
    assert np.allclose(m2, 0.1 * g, rtol=1e-4) and np.allclose(v2, 0.001 * g * g, rtol=1e-4)


# src/optimizer_test.cpp:167-235: one AdamW step on a 3 x 4 tensor (p = 0.5 + 0.03 i, g = -0.2 + 0.02 i, lr 0.05,
# betas 0.9 / 0.999, eps 1e-8, weight decay 0.1) against the decay-first formula, relative 1e-5; with the two writes
# swapped the result must differ by more than 1e-6 (the order is part of the contract)
def test_adamw_decay_first_order_case(rl):
    f = np.float32
    i = np.arange(12, dtype=np.float32)
    p0, g0 = (f(0.5) + i * f(0.03)).astype(np.float32), (f(-0.2) + i * f(0.02)).astype(np.float32)
    lr, b1, b2, eps, wd = f(0.05), f(0.9), f(0.999), f(1e-8), f(0.1)

    def reference(decay_first):
        bc1, bc2 = f(1) - b1, f(1) - b2  # t = 1
        m = (f(1) - b1) * g0
        v = (f(1) - b2) * g0 * g0
        p = p0.copy()
        if decay_first:
            p = p * (f(1) - lr * wd)
        p = p - lr * (m / bc1) / (np.sqrt(v / bc2) + eps)
        if not decay_first:
            p = p * (f(1) - lr * wd)
        return p.astype(np.float32)

    got, _, _ = rl.adamw(p0, g0, np.zeros(12), np.zeros(12), lr=0.05, t=1, wd=0.1, beta1=0.9, beta2=0.999, eps=1e-8)
    ref = reference(True)
    rel = np.abs(got - ref) / np.maximum(np.abs(ref), 1e-6)
    assert rel.max() < 1e-5
    assert np.abs(ref - reference(False)).max() > 1e-6
    assert np.abs(got - reference(False)).max() > 1e-6


def test_clip_grad_norm(rl):
    g, norm = rl.clip_grad_norm([3.0, 4.0], 1.0)
    assert abs(norm - 5.0) < 1e-6 and near(g, [0.6, 0.8], 1e-6)
    g, norm = rl.clip_grad_norm([0.3, 0.4], 1.0)
    assert np.array_equal(g, np.array([0.3, 0.4], np.float32))  # below the limit: untouched


# src/rl_experience_test.cpp:160-169: rewards {1,2,3}, gamma 0.5 -> {2.75, 3.5, 3.0}
def test_monte_carlo_return_known_answer(rl):
    assert near(rl.mc_return([[1], [2], [3]], gamma=0.5).ravel(), [2.75, 3.5, 3.0])
    # done stops the carry, the mask zeroes the row and what is carried
    assert near(rl.mc_return([[1], [2], [3]], done=[[0], [1], [0]], gamma=1.0).ravel(), [3.0, 2.0, 3.0])
    assert near(rl.mc_return([[1], [2], [3]], mask=[[1], [0], [1]], gamma=1.0).ravel(), [1.0, 0.0, 3.0])


# src/rl_policy_test.cpp:301-307: value {0.5, 1}, returns {1, 2}, coefficient 2 -> loss 1.25, gradient {-1, -2}
def test_value_regression_known_answer(rl):
    loss, grad = rl.value_regression([0.5, 1.0], [1.0, 2.0], [1.0, 1.0], coef=2.0)
    assert abs(loss - 1.25) < 1e-6 and near(grad, [-1.0, -2.0])
    loss, grad = rl.value_regression([0.5, 1.0], [1.0, 2.0], [0.0, 0.0], coef=2.0)
    assert loss == 0.0 and near(grad, [0.0, 0.0])
