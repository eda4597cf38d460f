"""Finite-difference checks of the training oracle's backward pass, in the manner of the reference's own
gradient checks: loss L = <outputs, random upstream>, every checked parameter entry perturbed by +-eps, central
difference against the analytic gradient (src/attn_gradcheck.cpp, src/swiglu_gradcheck.cpp,
src/rmsnorm_gradcheck.cpp, src/gpt_gradcheck.cpp: eps 1e-3, tolerance 5e-2 in f32).  The checks run on the
oracle's differentiable twin (dense float64 linears, no f32 roundings, everything else the same code), so the
tolerance here is 1e-6: attention (with and without RoPE), QuickGELU / SwiGLU, RMSNorm, residuals, embeddings,
head, categorical log-prob / entropy and the value port are pinned by something other than the oracle's own
algebra.  The quantised linear's forward / backward rules are pinned separately by the reference's known answers
(tests/test_oracle_pins.py).  Also restated: the reference's bound on KV-cache decode against the full causal
forward, max |logit difference| <= 5e-2 (src/attn_consistency_test.cpp:262-264)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle_train as ot  # noqa: E402


def _loss(cfg, flat, tokens, P, up_lp, up_ent, dv):
    tr = ot.OracleTrainer(cfg, flat, smooth=True)
    lp, ent, val = tr.forward(tokens, P)
    total = (lp.reshape(-1) * up_lp).sum() + (ent.reshape(-1) * up_ent).sum()
    if val is not None:
        total += (val.reshape(-1) * dv).sum()
    return total


# the last cases switch on, one at a time and then together, the structure of BitNet b1.58 2B4T: SubLN, grouped-query
# attention, tied embeddings (the reference exercises them in src/bitnet_struct_test.cpp: gradients reach the sub-norm
# gains, GQA equals MHA with block-replicated KV weights, the tied head's two gradient paths sum in one tensor)
@pytest.mark.parametrize("act,pos,value_head,extra", [
    (0, 0, False, {}), (1, 1, True, {}), (0, 1, True, {}), (1, 0, False, {}), (2, 1, False, {}),
    (1, 1, False, dict(sub_ln=True)), (1, 1, False, dict(n_head=4, n_head_kv=2)), (0, 0, True, dict(tie_embeddings=True)),
    (2, 1, True, dict(sub_ln=True, n_head=4, n_head_kv=1, tie_embeddings=True))])
def test_whole_model_backward_by_finite_differences(pkg, act, pos, value_head, extra):
    kw = dict(n_layer=2, d_model=16, n_head=2, d_ff=24, vocab=13, ctx=8, act=act, pos=pos, value_head=value_head)
    kw.update(extra)
    cfg = pkg.GptConfig(**kw)
    rng = np.random.default_rng(10 + act + 2 * pos)
    layout, n_params = cfg.param_layout()
    flat = rng.normal(0, 0.3, n_params)
    for name, off, shape in layout:
        if name.endswith("gamma"):
            size = int(np.prod(shape))
            flat[off:off + size] = 1.0 + rng.normal(0, 0.1, size)
    n, S, P = 2, 7, 3
    tokens = rng.integers(0, cfg.vocab, (n, S)).astype(np.int32)
    T = n * (S - P)
    up_lp, up_ent = rng.normal(0, 1, T), rng.normal(0, 1, T)
    dv = rng.normal(0, 1, T) if value_head else None
    tr = ot.OracleTrainer(cfg, flat, smooth=True)
    tr.forward(tokens, P)
    g = tr.backward(up_lp, up_ent, dv)
    eps = 1e-5
    worst = 0.0
    for name, off, shape in layout:
        size = int(np.prod(shape))
        scale = max(np.abs(g[off:off + size]).max(), 1e-8)
        picks = rng.choice(size, size=min(4, size), replace=False)
        if name == "tok_emb":  # rows of tokens that occur, so that the entries are live
            picks = [int(tokens[0, 0]) * cfg.d_model + 1, int(tokens[1, 2]) * cfg.d_model + 5]
        for j in picks:
            a, b = flat.copy(), flat.copy()
            a[off + j] += eps
            b[off + j] -= eps
            num = (_loss(cfg, a, tokens, P, up_lp, up_ent, dv) - _loss(cfg, b, tokens, P, up_lp, up_ent, dv)) / (2 * eps)
            # the key bias has an exactly zero gradient without RoPE (softmax is shift-invariant): absolute floor
            err = abs(num - g[off + j]) / (scale + 1e-3)
            worst = max(worst, err)
            assert err <= 1e-6, f"{name}[{j}]: numeric {num:.8e} vs analytic {g[off + j]:.8e}"
    assert worst <= 1e-6


def test_quantised_model_reduces_to_its_twin_where_nothing_is_quantised(pkg):
    """The quantised oracle and its differentiable twin share every line except the linears: with weights that are
    exactly ternary times a scale and activations that are exactly representable, their outputs agree, so the
    finite-difference checks above speak for the quantised model's attention / norm / activation code too."""
    cfg = pkg.GptConfig(n_layer=1, d_model=16, n_head=2, d_ff=16, vocab=11, ctx=6, act=1, pos=1)
    rng = np.random.default_rng(3)
    flat = cfg.init_params(1, bias_std=0.01)
    tokens = rng.integers(0, 11, (2, 6)).astype(np.int32)
    a = ot.OracleTrainer(cfg, flat)
    b = ot.OracleTrainer(cfg, flat, smooth=True)
    # replace the twin's dense weights by the dequantised ternary ones: the only remaining difference is the
    # int8 rounding of activations, at most half a step of 1/127 of the row maximum per feature
    for name, lin in b.lin.items():
        lin.w = (a.lin[name].trit.astype(np.float64) * a.lin[name].tau.astype(np.float64)[:, None])
    lp_a, _, _ = a.forward(tokens, 2)
    lp_b, _, _ = b.forward(tokens, 2)
    assert np.abs(lp_a - lp_b).max() < 5e-2


@pytest.mark.parametrize("act,pos,extra", [(0, 0, {}), (1, 1, {}),
                                           (2, 1, dict(sub_ln=True, n_head=4, n_head_kv=2, tie_embeddings=True))])
def test_decode_step_logits_within_the_reference_bound_of_the_full_forward(pkg, act, pos, extra):
    """src/attn_consistency_test.cpp:262-264: KV-cache decode and the full causal forward may differ by at most
    5e-2 on any logit.  The C restatement of the step path against the numpy restatement of the full forward."""
    from oracle_binding import OracleGpt

    kw = dict(n_layer=2, d_model=64, n_head=2, d_ff=128, vocab=97, ctx=24, act=act, pos=pos)
    kw.update(extra)
    cfg = pkg.GptConfig(**kw)
    flat = cfg.init_params(1, bias_std=0.01)
    tr = ot.OracleTrainer(cfg, flat)
    m = OracleGpt(cfg, flat)
    tokens = np.random.default_rng(0).integers(0, 97, (2, 16)).astype(np.int32)
    tr.forward(tokens, 1)  # decisions at every position but the last
    full = tr.logits.reshape(2, 15, 97)
    for b in range(2):
        step = m.step_logits(tokens[b])[:15]
        assert np.abs(step.astype(np.float64) - full[b]).max() <= 5e-2
