"""PPO on a ternary GPT policy with a value head: one minibatch at the GPT-2-small shape of the PPO
configuration (12 layers, d 768, 12 heads, MLP 3072, vocab 32000, prompt 64 + 256 generated) against the numpy
restatement of PpoObjective / GaeAdvantage within 1e-3 (exact mode), and the step driver (rollout source,
GAE record, epochs x minibatches) end to end on a small policy."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle_train as ot  # noqa: E402
from oracle_binding import OracleRL  # noqa: E402

pytestmark = pytest.mark.gpu
REL = 1e-3


def dev(a, eng, dt=np.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dt)).to(eng.device)


def rel_err(got, ref):
    ref, got = np.asarray(ref, np.float64), np.asarray(got, np.float64)
    return np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-12)


def test_ppo_minibatch_at_gpt2_small_shape(pkg, eng):
    cfg = pkg.GptConfig(n_layer=12, d_model=768, n_head=12, d_ff=3072, vocab=32000, ctx=512, act=0, pos=0, value_head=True)
    flat = cfg.init_params(1)
    layout = {nm: (off, shape) for nm, off, shape in cfg.param_layout()[0]}
    off, _ = layout["value_head.weight"]
    flat[off:off + 768] = np.random.default_rng(9).normal(0, 0.05, 768)
    pol = pkg.Policy(eng, cfg)
    pol.upload_params(flat)
    tr = ot.OracleTrainer(cfg, flat)
    rng = np.random.default_rng(3)
    n, P, G = 2, 64, 256
    tokens = rng.integers(0, 32000, (n, P + G)).astype(np.int32)
    lp_ref, ent_ref, val_ref = tr.forward(tokens, P)
    lp, ent, val = pol.logprobs(dev(tokens, eng, np.int32), P, want_entropy=True, want_value=True)
    assert rel_err(lp.cpu().numpy(), lp_ref) <= REL and rel_err(ent.cpu().numpy(), ent_ref) <= REL
    assert rel_err(val.cpu().numpy(), val_ref) <= REL
    # rewards of the configuration: per-token N(0, 0.1) plus a terminal N(0, 1); GAE gamma 0.99, lambda 0.95
    reward = rng.normal(0, 0.1, (n, G)).astype(np.float32)
    reward[:, -1] += rng.normal(0, 1, n).astype(np.float32)
    old_value = (val_ref + rng.normal(0, 0.2, (n, G))).astype(np.float32)
    adv_ref, ret_ref = OracleRL().gae(reward.T, old_value.T, gamma=0.99, lam=0.95)
    adv_t, ret_t = eng.gae(dev(reward.T, eng), dev(old_value.T, eng), gamma=0.99, lam=0.95)
    assert np.array_equal(adv_t.cpu().numpy().view(np.uint32), adv_ref.view(np.uint32))
    adv, ret = adv_ref.T.copy(), ret_ref.T.copy()
    old = (lp_ref + rng.normal(0, 0.2, (n, G))).astype(np.float32)
    mask = np.ones((n, G), np.float32)
    kw = dict(clip_eps=0.2, entropy_coef=0.01, value_coef=0.5, value_clip_eps=0.2)
    rep_ref, up_lp, up_ent, dv = tr.objective(lp_ref, ent_ref, mask, old, adv, None, val_ref, ret, old_value, **kw)
    g_ref = tr.backward(up_lp, up_ent, dv)
    pol.zero_grad()
    rep = pol.train_step(dev(tokens, eng, np.int32), P, dev(mask, eng), old_logp=dev(old, eng), advantage=dev(adv, eng),
                         returns=dev(ret, eng), old_value=dev(old_value, eng), **kw).cpu().numpy()
    for i, nm in ((0, "policy_loss"), (2, "approx_kl"), (3, "clip_fraction"), (5, "entropy_loss"), (8, "value_loss"),
                  (9, "value_clip_fraction")):
        assert abs(rep[i] - rep_ref[nm]) <= REL * max(abs(rep_ref[nm]), 1e-2), nm
    named = pkg.report_dict(torch.from_numpy(rep))
    assert abs(named["loss"] - (rep_ref["policy_loss"] + rep_ref["entropy_loss"] + rep_ref["value_loss"])) <= 1e-3
    g = pol.grads_view().cpu().numpy().astype(np.float64)
    for name, (off, shape) in layout.items():
        size = int(np.prod(shape))
        a, b = g[off:off + size], g_ref[off:off + size]
        scale = np.abs(b).max()
        if scale < 1e-12:
            continue
        assert np.abs(a - b).max() <= REL * scale, f"{name}: {np.abs(a - b).max() / scale:.2e}"
    pol.release_workspaces()


@pytest.mark.parametrize("exact", [True, False])
def test_ppo_step_driver(pkg, eng, exact):
    cfg = pkg.GptConfig(n_layer=2, d_model=128, n_head=2, d_ff=256, vocab=300, ctx=96, act=0, pos=0, value_head=True, exact=exact)
    pol = pkg.Policy(eng, cfg)
    flat = cfg.init_params(2, bias_std=0.01)
    pol.upload_params(flat)
    pcfg = pkg.PpoConfig(prompt_len=64, max_new=32, epochs=2, minibatches=2, micro_batch=4, rollout_chunk=8, lr=1e-3)
    tr = pkg.PpoTrainer(pol, pcfg, seed=3)
    prompts = dev(np.random.default_rng(4).integers(0, 300, (8, 64)), eng, np.int32)
    gen = torch.Generator(device=eng.device)
    gen.manual_seed(5)

    def reward_fn(tokens):
        r = torch.randn((tokens.shape[0], 32), device=eng.device, generator=gen) * 0.1
        r[:, -1] += torch.randn(tokens.shape[0], device=eng.device, generator=gen)
        return r

    p0 = pol.params_view().clone()
    out = tr.step(prompts, reward_fn, seed=7)
    eng.check_device_errors()
    rec = out["record"]
    # the record's advantages and returns are GaeAdvantage of its rewards and old values, bit for bit
    adv_ref, ret_ref = OracleRL().gae(rec["reward"].cpu().numpy().T, rec["old_value"].cpu().numpy().T, mask=np.ones((32, 8), np.float32),
                                      gamma=0.99, lam=0.95)
    assert np.array_equal(rec["advantage"].cpu().numpy().view(np.uint32), adv_ref.T.copy().view(np.uint32))
    assert np.array_equal(rec["return"].cpu().numpy().view(np.uint32), ret_ref.T.copy().view(np.uint32))
    # the old values are the value head's output at the decisions; the old log-probs those of the sampled tokens
    rep = pkg.report_dict(out["report"])
    assert all(np.isfinite(v) for v in rep.values()) and rep["units"] == 4 * 32
    assert rep["value_loss"] > 0 and rep["entropy"] > 0
    assert (pol.params_view() - p0).abs().max().item() > 0  # four optimizer steps moved the weights
    assert pol.engine.launch_count() > 0
