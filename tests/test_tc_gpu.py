"""The tcgen05 / TMEM / TMA GEMMs against the CPU oracle and the mma.sync path: the int8 forward
is bit-exact; the bf16 backward GEMMs are within bf16 rounding of the f64 reference."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev(a, eng):
    return torch.from_numpy(np.ascontiguousarray(a)).to(eng.device)


def _case(orc, t, k, out, seed):
    rng = np.random.default_rng(seed)
    W = rng.normal(0, 0.02, (out, k)).astype(np.float32)
    tau = orc.absmean_tau(W)
    X = rng.normal(0, 1, (t, k)).astype(np.float32)
    bias = rng.normal(0, 0.05, out).astype(np.float32)
    return W, tau, X, bias


def test_expand_weights(eng, orc):
    W, tau, _, _ = _case(orc, 1, 256, 70, 1)
    packed = orc.trit_pack(W, tau)
    trit = orc.trit_unpack(packed, 256)
    w8, wb = eng.expand_weights(_dev(packed.view(np.int32), eng), 256)
    assert np.array_equal(eng.actq_to_plain(w8).cpu().numpy(), trit)  # same K permutation as the activations
    assert np.array_equal(wb.float().cpu().numpy(), trit.astype(np.float32))


@pytest.mark.parametrize("t,k,out", [(128, 128, 256), (64, 64, 40), (130, 192, 300), (300, 2048, 384), (1000, 320, 1000),
                                     (2048, 2048, 5632)])
def test_forward_tc_bit_exact(eng, orc, t, k, out):
    W, tau, X, bias = _case(orc, t, k, out, t + k + out)
    packed = orc.trit_pack(W, tau)
    q_ref, s_ref = orc.act_quant_tm(X)
    y_ref = orc.bitlinear_i8_tm(packed, tau, bias, q_ref, s_ref, want_acc=False)
    q, s, qsum = eng.act_quant_tm(_dev(X, eng))
    w8, _ = eng.expand_weights(_dev(packed.view(np.int32), eng), k, want_bf16=False)
    y = eng.bitlinear_fwd_tc(w8, _dev(tau, eng), _dev(bias, eng), q, s)
    eng.check_device_errors()
    assert np.array_equal(y.cpu().numpy().view(np.uint32), y_ref.view(np.uint32))
    res = torch.randn((t, out), device=eng.device)
    y2 = eng.bitlinear_fwd_tc(w8, _dev(tau, eng), _dev(bias, eng), q, s, residual=res)
    y_mma = eng.bitlinear_fwd_tm(_dev(packed.view(np.int32), eng), _dev(tau, eng), _dev(bias, eng), q, s, qsum)
    assert torch.equal(y2, res + y_mma)


@pytest.mark.parametrize("bn", [64, 128, 192, 256])
@pytest.mark.parametrize("t,k,out", [(130, 192, 300), (512, 2048, 2048), (300, 5632, 1000)])
def test_forward_tc_every_tile_width(eng, orc, bn, t, k, out):
    """The result of the forward does not depend on the width of its output tile."""
    W, tau, X, bias = _case(orc, t, k, out, t + k + out + bn)
    packed = orc.trit_pack(W, tau)
    q_ref, s_ref = orc.act_quant_tm(X)
    y_ref = orc.bitlinear_i8_tm(packed, tau, bias, q_ref, s_ref, want_acc=False)
    q, s, _ = eng.act_quant_tm(_dev(X, eng))
    w8, _ = eng.expand_weights(_dev(packed.view(np.int32), eng), k, want_bf16=False)
    eng.set_tc_forward_tile(bn)
    try:
        y = eng.bitlinear_fwd_tc(w8, _dev(tau, eng), _dev(bias, eng), q, s)
        eng.check_device_errors()
    finally:
        eng.set_tc_forward_tile(0)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), y_ref.view(np.uint32))


def test_forward_tile_width_rejected(eng):
    with pytest.raises(Exception):
        eng.set_tc_forward_tile(100)


@pytest.mark.parametrize("t,k,out", [(128, 256, 256), (64, 64, 64), (130, 192, 328), (300, 2048, 384), (1000, 320, 1000),
                                     (2100, 192, 328), (4096, 768, 768), (3000, 704, 1000), (256, 2048, 2048)])
def test_backward_tc(eng, orc, t, k, out):
    """from 2048 tokens up the weight-gradient GEMM of a small matrix splits the token axis (2100 tokens: two slices, the
    second ragged; 4096 x 768 x 768: four slices of 18 tiles; 3000 x 704 x 1000: two slices with ragged tiles)"""
    W, tau, X, _ = _case(orc, t, k, out, t + 3 * k + out)
    packed = orc.trit_pack(W, tau)
    trit = orc.trit_unpack(packed, k).astype(np.float64)
    q_ref, s_ref = orc.act_quant_tm(X)
    dY = np.random.default_rng(2).normal(0, 1, (t, out)).astype(np.float32)
    dx_ref = (dY.astype(np.float64) * tau[None, :]) @ trit
    dw_ref = ((dY.astype(np.float64) * s_ref[:, None]).T @ q_ref.astype(np.float64)) * tau[:, None]
    q, s, _ = eng.act_quant_tm(_dev(X, eng))
    _, wb = eng.expand_weights(_dev(packed.view(np.int32), eng), k)
    dw = torch.zeros((out, k), device=eng.device)
    dx, dw = eng.bitlinear_bwd_tc(_dev(dY, eng), _dev(tau, eng), wb, q, s, k, dw=dw)
    eng.check_device_errors()
    assert np.abs(dx.cpu().numpy() - dx_ref).max() <= 2e-2 * np.abs(dx_ref).max()
    assert np.abs(dw.cpu().numpy() - dw_ref).max() <= 2e-2 * np.abs(dw_ref).max()
    # accumulation
    dx2, dw2 = eng.bitlinear_bwd_tc(_dev(dY, eng), _dev(tau, eng), wb, q, s, k, dw=dw, dx=dx, accumulate_dx=True)
    assert np.abs(dx2.cpu().numpy() - 2 * dx_ref).max() <= 2e-2 * 2 * np.abs(dx_ref).max()
    assert np.abs(dw2.cpu().numpy() - 2 * dw_ref).max() <= 2e-2 * 2 * np.abs(dw_ref).max()


@pytest.mark.parametrize("t,k,v", [(128, 128, 256), (200, 192, 536), (1024, 2048, 32000), (70, 256, 10000)])
def test_lmhead_fused_logprob_entropy_forward_and_backward(eng, orc, t, k, v):
    """The LM head fused with CategoricalDistribution::log_prob / entropy and their gradients: logits are never stored.
    Against the same quantities computed in f64 from the materialised logits of the bit-exact forward: log-prob, entropy
    and log-sum-exp within 1e-5 of the logits' range, the bf16 backward operand within bf16 rounding, the bias gradient
    within 1e-3 (ragged last tiles: 536 = 2 x 256 + 24, 10000 = 39 x 256 + 16)."""
    W, tau, X, bias = _case(orc, t, k, v, t + k + v)
    packed = orc.trit_pack(W, tau)
    q, s, _ = eng.act_quant_tm(_dev(X, eng))
    w8, _ = eng.expand_weights(_dev(packed.view(np.int32), eng), k, want_bf16=False)
    d_tau, d_bias = _dev(tau, eng), _dev(bias, eng)
    rng = np.random.default_rng(7)
    actions = rng.integers(0, v, t).astype(np.int32)
    actions[:4] = [0, v - 1, 255 % v, 256 % v]  # tile borders
    d_act = _dev(actions, eng)
    logits = eng.bitlinear_fwd_tc(w8, d_tau, d_bias, q, s).double()
    lse_ref = torch.logsumexp(logits, 1)
    lp_all = logits - lse_ref[:, None]
    p = lp_all.exp()
    ent_ref = -(p * lp_all).sum(1)
    idx = torch.arange(t, device=eng.device)
    logp_ref = lp_all[idx, d_act.long()]
    logp, ent, lse = eng.lmhead_logprob_entropy(w8, d_tau, d_bias, q, s, d_act)
    eng.check_device_errors()
    scale = float(logits.abs().max())
    assert (lse.double() - lse_ref).abs().max().item() <= 1e-5 * max(scale, 1.0)
    assert (logp.double() - logp_ref).abs().max().item() <= 2e-5 * max(scale, 1.0)
    assert (ent.double() - ent_ref).abs().max().item() <= 1e-4 * max(float(ent_ref.abs().max()), 1.0)
    up_lp = _dev(rng.normal(0, 1, t).astype(np.float32), eng)
    up_ent = _dev(rng.normal(0, 0.1, t).astype(np.float32), eng)
    for ue in (None, up_ent):
        onehot = torch.zeros_like(p)
        onehot[idx, d_act.long()] = 1.0
        dl = (onehot - p) * up_lp.double()[:, None]
        if ue is not None:
            dl = dl - p * (lp_all + ent_ref[:, None]) * ue.double()[:, None]
        dyb_ref = dl * d_tau.double()[None, :]
        db0 = _dev(rng.normal(0, 1, v).astype(np.float32), eng)
        dyb, db = eng.lmhead_logprob_entropy_backward(w8, d_tau, d_bias, q, s, d_act, lse, ent, up_lp, ue, dbias=db0.clone())
        eng.check_device_errors()
        err = (dyb.double() - dyb_ref).abs().max().item()
        assert err <= 2.0 ** -7 * float(dyb_ref.abs().max()), err  # bf16 rounding of the operand
        db_ref = dl.sum(0) + db0.double()
        assert (db.double() - db_ref).abs().max().item() <= 1e-3 * float(db_ref.abs().max())
