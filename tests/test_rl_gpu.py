"""Parity of the CUDA RL kernels with the CPU restatement (advantages bit-exact where the
arithmetic is elementwise, 1e-3 relative otherwise), through the C-ABI."""
import numpy as np
import pytest
import torch

from oracle_binding import OracleRL

pytestmark = pytest.mark.gpu
REL = 1e-3  # tolerance for f32 log-probs, advantages, losses and gradients


@pytest.fixture(scope="module")
def rl():
    return OracleRL()


def dev(a, eng, dt=np.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dt)).to(eng.device)


def close(got, ref, rel=REL):
    got = got.cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got)
    ref = np.asarray(ref)
    scale = max(np.abs(ref).max(), 1e-6)
    return np.abs(got - ref).max() <= rel * scale


def test_gae_hand_cases(eng, rl):
    adv, ret = eng.gae(dev([[1], [2], [3]], eng), dev([[0.5], [0.5], [0.5]], eng), done=dev([[0], [0], [1]], eng),
                       bootstrap=dev([0.7], eng), gamma=0.5, lam=0.8)
    assert np.allclose(adv.cpu().numpy().ravel(), [1.85, 2.75, 2.5], atol=1e-6)
    assert np.allclose(ret.cpu().numpy().ravel(), [2.35, 3.25, 3.0], atol=1e-6)


@pytest.mark.parametrize("steps,batch,use_done,use_mask,use_boot", [
    (256, 256, True, True, True), (256, 256, False, False, False), (17, 3, True, False, True), (1, 1, False, True, False)])
def test_gae_bit_exact(eng, rl, steps, batch, use_done, use_mask, use_boot):
    rng = np.random.default_rng(steps * 7 + batch)
    r = rng.normal(0, 0.1, (steps, batch)).astype(np.float32)
    r[-1] += rng.normal(0, 1, batch).astype(np.float32)
    v = rng.normal(0, 1, (steps, batch)).astype(np.float32)
    done = (rng.uniform(size=(steps, batch)) < 0.05).astype(np.float32) if use_done else None
    mask = (rng.uniform(size=(steps, batch)) < 0.9).astype(np.float32) if use_mask else None
    boot = rng.normal(0, 1, batch).astype(np.float32) if use_boot else None
    a_ref, r_ref = rl.gae(r, v, done, mask, boot, 0.99, 0.95)
    a, rt = eng.gae(dev(r, eng), dev(v, eng), None if done is None else dev(done, eng),
                    None if mask is None else dev(mask, eng), None if boot is None else dev(boot, eng), 0.99, 0.95)
    assert np.array_equal(a.cpu().numpy().view(np.uint32), a_ref.view(np.uint32))
    assert np.array_equal(rt.cpu().numpy().view(np.uint32), r_ref.view(np.uint32))


def test_group_advantage(eng, rl):
    s = np.sqrt(2.0 / 3.0)
    out = eng.group_advantage(dev([1, 2, 3, 10, 10, 10], eng), [(0, 3), (3, 3)])
    assert np.allclose(out.cpu().numpy(), [-1 / s, 0, 1 / s, 0, 0, 0], atol=1e-6)
    # 64 groups x 16 with binary rewards (p = 0.3), ragged groups, and a group larger than a warp
    rng = np.random.default_rng(1)
    for sizes in ([16] * 64, [8] * 8, [1, 2, 3, 70, 5], [1]):
        n = sum(sizes)
        ret = (rng.uniform(size=n) < 0.3).astype(np.float32)
        spans, c = [], 0
        for k in sizes:
            spans.append((c, k))
            c += k
        ref = rl.group_advantage(ret, spans)
        got = eng.group_advantage(dev(ret, eng), spans).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_group_advantage_rejects_bad_spans(eng, pkg):
    with pytest.raises(pkg.NnbError):
        eng.group_advantage(dev([1, 2, 3, 10, 10, 10], eng), [(0, 2), (3, 1)])
    with pytest.raises(pkg.NnbError):
        eng.group_advantage(dev([1, 2, 3], eng), [(0, 2)])


def test_masked_normalize(eng, rl):
    rng = np.random.default_rng(2)
    x = rng.normal(1, 2, 5000).astype(np.float32)
    m = (rng.uniform(size=5000) < 0.7).astype(np.float32)
    assert close(eng.masked_normalize(dev(x, eng), dev(m, eng)), rl.masked_normalize(x, m), 1e-5)
    assert close(eng.masked_normalize(dev(x, eng)), rl.masked_normalize(x), 1e-5)
    z = eng.masked_normalize(dev(np.full(10, 2.0), eng), dev(np.ones(10), eng)).cpu().numpy()
    assert np.all(z == 0)
    z = eng.masked_normalize(dev(x, eng), dev(np.zeros(5000), eng)).cpu().numpy()
    assert np.all(z == 0)


@pytest.mark.parametrize("t,v", [(2, 3), (33, 1000), (7, 10000), (5, 32002)])
def test_categorical_forward_backward(eng, rl, t, v):
    rng = np.random.default_rng(v)
    lg = rng.normal(0, 2, (t, v)).astype(np.float32)
    act = rng.integers(0, v, t).astype(np.int32)
    lp_ref, h_ref = rl.categorical_logp_entropy(lg, act)
    lp, h = eng.categorical_logp_entropy(dev(lg, eng), dev(act, eng, np.int32))
    assert close(lp, lp_ref) and close(h, h_ref)
    ul = rng.normal(0, 1, t).astype(np.float32)
    ue = rng.normal(0, 1, t).astype(np.float32)
    g_ref = rl.categorical_backward(lg, act, ul, ue)
    g = eng.categorical_backward(dev(lg, eng), dev(act, eng, np.int32), dev(ul, eng), dev(ue, eng))
    assert close(g, g_ref)
    g1 = eng.categorical_backward(dev(lg, eng), dev(act, eng, np.int32), dev(ul, eng), None)
    assert close(g1, rl.categorical_backward(lg, act, ul, None))


def test_ppo_known_answers(eng, rl):
    lg = np.array([[1, 0, -1], [0, 2, 0]], np.float32)
    act = np.array([0, 1], np.int32)
    lp, _ = eng.categorical_logp_entropy(dev(lg, eng), dev(act, eng, np.int32))
    old = lp.cpu().numpy() - np.log(np.array([0.5, 1.5], np.float32))
    one = dev([1, 1], eng)
    _, _, rep = eng.token_objective(lp, one, old_logp=dev(old, eng), advantage=one, clip_eps=0.2)
    rep = rep.cpu().numpy()
    assert abs(rep[0] - (-0.85)) < 1e-5 and abs(rep[1] - 1.0) < 1e-5 and abs(rep[3] - 1.0) < 1e-5
    _, _, rep = eng.token_objective(lp, one, old_logp=dev(old, eng), advantage=dev([-1, -1], eng), clip_eps=0.2)
    assert abs(rep.cpu().numpy()[0] - 1.15) < 1e-5
    grad, rep = eng.clipped_value(dev([1, 1.8], eng), dev([0, 1], eng), dev([0, 1], eng), one, clip_eps=0.2, coef=1.0)
    assert np.allclose(grad.cpu().numpy(), [1, 0.8], atol=1e-6)
    assert abs(rep.cpu().numpy()[0] - 0.82) < 1e-5 and abs(rep.cpu().numpy()[1] - 1.0) < 1e-5


@pytest.mark.parametrize("n", [1, 1000, 65536])
def test_token_objective_matches_components(eng, rl, n):
    rng = np.random.default_rng(n)
    logp = rng.normal(-3, 1, n).astype(np.float32)
    old = (logp + rng.normal(0, 0.3, n)).astype(np.float32)
    ref = (logp + rng.normal(0, 0.1, n)).astype(np.float32)
    adv = rng.normal(0, 1, n).astype(np.float32)
    ent = rng.uniform(0, 5, n).astype(np.float32)
    mask = (rng.uniform(size=n) < 0.8).astype(np.float32)
    up_p, m = rl.clipped_policy(logp, old, adv, mask, 0.2)
    kl_loss, up_k = rl.sampled_kl(logp, ref, mask, 0.04)
    e_loss, up_e = rl.entropy_bonus(ent, mask, 0.01)
    up_lp, up_ent, rep = eng.token_objective(dev(logp, eng), dev(mask, eng), old_logp=dev(old, eng), advantage=dev(adv, eng),
                                             ref_logp=dev(ref, eng), entropy=dev(ent, eng), clip_eps=0.2, kl_coef=0.04,
                                             entropy_coef=0.01)
    rep = rep.cpu().numpy()
    assert close(up_lp, up_p + up_k) and close(up_ent, up_e)
    want = [m["loss"], m["ratio_mean"], m["approx_kl"], m["clip_fraction"], kl_loss, e_loss]
    for got, ref_v in zip(rep[:6], want):
        assert abs(got - ref_v) <= REL * max(abs(ref_v), 1e-3)
    assert rep[7] == mask.sum()
    # sharded batch: passing the global unit count scales the gradient accordingly
    up2, _, _ = eng.token_objective(dev(logp, eng), dev(mask, eng), old_logp=dev(old, eng), advantage=dev(adv, eng),
                                    units=float(2 * mask.sum() + 2), clip_eps=0.2)
    if mask.sum() > 0:
        assert close(up2 * (2 * mask.sum() + 2) / mask.sum(), up_p)


def test_zero_units_gives_zero_loss_and_gradient(eng):
    up, _, rep = eng.token_objective(dev([-1.0, -2.0], eng), dev([0, 0], eng), old_logp=dev([-1.0, -2.0], eng),
                                     advantage=dev([1, 1], eng))
    assert torch.all(up == 0) and rep.cpu().numpy()[0] == 0


def test_clipped_value_random(eng, rl):
    rng = np.random.default_rng(5)
    n = 5000
    v, r, ov = (rng.normal(0, 1, n).astype(np.float32) for _ in range(3))
    m = (rng.uniform(size=n) < 0.9).astype(np.float32)
    loss, grad, cf = rl.clipped_value(v, r, ov, m, 0.2, 0.5)
    g, rep = eng.clipped_value(dev(v, eng), dev(r, eng), dev(ov, eng), dev(m, eng), clip_eps=0.2, coef=0.5)
    assert close(g, grad)
    assert abs(rep.cpu().numpy()[0] - loss) <= REL * abs(loss) and abs(rep.cpu().numpy()[1] - cf) <= 1e-5


def test_monte_carlo_return_and_value_regression(eng, rl):
    # src/rl_experience_test.cpp:160-169 and src/rl_policy_test.cpp:301-307 on the GPU, then random cases bit for bit
    out = eng.monte_carlo_return(dev([[1], [2], [3]], eng), gamma=0.5)
    assert np.allclose(out.cpu().numpy().ravel(), [2.75, 3.5, 3.0], atol=1e-6)
    g, rep = eng.value_regression(dev([0.5, 1.0], eng), dev([1.0, 2.0], eng), dev([1.0, 1.0], eng), coef=2.0)
    assert np.allclose(g.cpu().numpy(), [-1.0, -2.0], atol=1e-6) and abs(rep.cpu().numpy()[0] - 1.25) < 1e-6
    rng = np.random.default_rng(11)
    steps, batch = 256, 256
    r = rng.normal(0, 1, (steps, batch)).astype(np.float32)
    done = (rng.uniform(size=(steps, batch)) < 0.02).astype(np.float32)
    mask = (rng.uniform(size=(steps, batch)) < 0.9).astype(np.float32)
    for d, m in ((None, None), (done, None), (done, mask)):
        want = rl.mc_return(r, d, m, gamma=0.99)
        got = eng.monte_carlo_return(dev(r, eng), None if d is None else dev(d, eng), None if m is None else dev(m, eng), gamma=0.99)
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    n = 5000
    v, ret = (rng.normal(0, 1, n).astype(np.float32) for _ in range(2))
    m = (rng.uniform(size=n) < 0.9).astype(np.float32)
    loss, grad = rl.value_regression(v, ret, m, coef=0.5)
    g, rep = eng.value_regression(dev(v, eng), dev(ret, eng), dev(m, eng), coef=0.5)
    assert close(g, grad) and abs(rep.cpu().numpy()[0] - loss) <= REL * abs(loss)


def test_adamw_and_clip(eng, rl):
    rng = np.random.default_rng(6)
    n = 100003
    p = rng.normal(0, 0.02, n).astype(np.float32)
    m, v = np.zeros(n, np.float32), np.zeros(n, np.float32)
    dp, dm, dv = dev(p, eng), dev(m, eng), dev(v, eng)
    for t in range(1, 4):
        g = rng.normal(0, 1e-3, n).astype(np.float32)
        g_ref, norm_ref = rl.clip_grad_norm(g, 0.1)
        dg = dev(g, eng)
        norm = eng.clip_grad_norm(dg, 0.1)
        assert abs(norm.item() - norm_ref) <= 1e-5 * norm_ref
        assert close(dg, g_ref, 1e-6)
        p, m, v = rl.adamw(p, g_ref, m, v, lr=1e-4, t=t, wd=0.01)
        eng.adamw_step(dp, dev(g_ref, eng), dm, dv, lr=1e-4, t=t, weight_decay=0.01)
        assert np.array_equal(dp.cpu().numpy().view(np.uint32), p.view(np.uint32))  # elementwise: bit-exact
        assert np.array_equal(dm.cpu().numpy().view(np.uint32), m.view(np.uint32))
        assert np.array_equal(dv.cpu().numpy().view(np.uint32), v.view(np.uint32))


def test_plain_c_client_runs(pkg, tmp_path):
    """The C99 client of tests/cabi/ against the GPU: engine description and the reference's group-advantage
    known answer ({1,2,3} -> {-1/s, 0, 1/s}, s = sqrt(2/3); a constant group -> zeros)."""
    import subprocess

    from test_abi_symbols import _compile_client

    r = subprocess.run([_compile_client(tmp_path, pkg)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()
    assert "nn-b200 engine" in lines[0]
    got = [float(x) for x in lines[1].split()]
    s = (2.0 / 3.0) ** 0.5
    assert np.allclose(got, [-1 / s, 0, 1 / s, 0, 0, 0], atol=1e-5)


def test_cpp_engine_shim_runs(pkg, tmp_path):
    """tests/cabi/shim_test.cpp on the GPU: BitLinear forward (Y bitwise) / backward through the reference's call
    sequence, the write-epoch cache, the data-movement verbs, and RLTrainingPipeline::run over a device-side rollout
    source with a GRPO-style update."""
    import subprocess

    from test_abi_symbols import _compile_shim_test

    r = subprocess.run([_compile_shim_test(tmp_path, pkg)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr + r.stdout
    assert "shim ok" in r.stdout
