"""The structure switches of BitNet b1.58 2B4T in the CPU restatements, checked the way the reference checks them
(src/bitnet_struct_test.cpp): SubLN adds layers x (d_model + d_ff) gains [1] and changes the forward [3]; grouped-query
attention with as many KV heads as heads is multi-head attention [7] and otherwise equals multi-head attention with
block-replicated KV weights, the head map being h // (H / Hkv) [8]; a tied head removes vocab x d_model + vocab
parameters [10] and equals an untied dense head holding the embedding (here: the numpy restatement's smooth twin)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import oracle_train as ot  # noqa: E402
from oracle_binding import OracleGpt  # noqa: E402


def _cfg(pkg, **kw):
    base = dict(n_layer=2, d_model=64, n_head=4, d_ff=128, vocab=53, ctx=20, act=1, pos=1)
    base.update(kw)
    return pkg.GptConfig(**base)


def test_parameter_counts(pkg):
    a = _cfg(pkg)
    n = a.param_layout()[1]
    assert _cfg(pkg, sub_ln=True).param_layout()[1] == n + a.n_layer * (a.d_model + a.d_ff)
    assert n - _cfg(pkg, tie_embeddings=True).param_layout()[1] == a.vocab * a.d_model + a.vocab
    assert _cfg(pkg, n_head_kv=4).param_layout()[1] == n
    dk = a.d_model // a.n_head
    assert n - _cfg(pkg, n_head_kv=2).param_layout()[1] == a.n_layer * 2 * (2 * dk) * (a.d_model + 1)


def test_subln_changes_the_forward_and_gqa_with_all_heads_does_not(pkg):
    a, g = _cfg(pkg), _cfg(pkg, n_head_kv=4)
    flat = a.init_params(3, bias_std=0.01)
    tokens = np.random.default_rng(0).integers(0, a.vocab, (1, 12)).astype(np.int32)
    la = OracleGpt(a, flat).step_logits(tokens[0])
    assert np.array_equal(la, OracleGpt(g, flat).step_logits(tokens[0]))
    s = _cfg(pkg, sub_ln=True)
    fs = s.init_params(3, bias_std=0.01)
    # same weights, gains at 1: only the extra normalisations differ
    lay_a = {nm: (off, shape) for nm, off, shape in a.param_layout()[0]}
    for nm, off, shape in s.param_layout()[0]:
        if nm in lay_a:
            o = lay_a[nm][0]
            fs[off:off + int(np.prod(shape))] = flat[o:o + int(np.prod(shape))]
    ls = OracleGpt(s, fs).step_logits(tokens[0])
    assert np.abs(ls - la).max() > 1e-3


@pytest.mark.parametrize("hkv", [1, 2])
def test_gqa_is_multi_head_attention_with_block_replicated_kv_weights(pkg, hkv):
    H = 4
    g, m = _cfg(pkg, n_head_kv=hkv), _cfg(pkg)
    dk, rep = g.d_model // H, H // hkv
    fg = g.init_params(5, bias_std=0.01)
    lay_g = {nm: (off, shape) for nm, off, shape in g.param_layout()[0]}
    fm = np.zeros(m.param_layout()[1], np.float32)
    for nm, off, shape in m.param_layout()[0]:
        o, s = lay_g[nm]
        src = fg[o:o + int(np.prod(s))].reshape(s)
        if ".attn.k." in nm or ".attn.v." in nm:
            src = np.repeat(src.reshape(hkv, dk, -1), rep, axis=0)
        fm[off:off + int(np.prod(shape))] = src.reshape(-1)
    tokens = np.random.default_rng(1).integers(0, g.vocab, (2, 14)).astype(np.int32)
    # the C restatement of the step path: bit for bit (a row's ternarisation depends on that row only)
    for b in range(2):
        assert np.array_equal(OracleGpt(g, fg).step_logits(tokens[b]), OracleGpt(m, fm).step_logits(tokens[b]))
    # the numpy restatement of the teacher-forced pass: forward equal, K/V gradients are the sums over each group
    tg, tm = ot.OracleTrainer(g, fg), ot.OracleTrainer(m, fm)
    lg, eg, _ = tg.forward(tokens, 4)
    lm, em, _ = tm.forward(tokens, 4)
    assert np.array_equal(lg, lm)
    up = np.random.default_rng(2).normal(0, 1, lg.size)
    gg, gm = tg.backward(up), tm.backward(up)
    scale = np.abs(gm).max()
    for nm, off, shape in m.param_layout()[0]:
        o, s = lay_g[nm]
        a = gm[off:off + int(np.prod(shape))].reshape(shape[0], -1)
        b = gg[o:o + int(np.prod(s))].reshape(s[0], -1)
        if ".attn.k." in nm or ".attn.v." in nm:
            a = a.reshape(hkv, rep, dk, -1).sum(1).reshape(hkv * dk, -1)
        assert np.abs(a - b).max() <= 1e-9 * scale, nm


def test_tied_head_is_the_embedding_used_as_a_dense_head(pkg):
    """smooth twin (dense float64 linears): an untied model whose head weight is the embedding and whose head bias is
    zero gives the tied model's outputs, and the tied embedding gradient is the sum of the two paths"""
    t, u = _cfg(pkg, tie_embeddings=True, pos=0), _cfg(pkg, pos=0)
    rng = np.random.default_rng(7)
    ft = rng.normal(0, 0.3, t.param_layout()[1])
    lay_t = {nm: (off, shape) for nm, off, shape in t.param_layout()[0]}
    fu = np.zeros(u.param_layout()[1])
    for nm, off, shape in u.param_layout()[0]:
        n = int(np.prod(shape))
        if nm == "lm_head.weight":
            fu[off:off + n] = ft[:n]  # tok_emb sits first
        elif nm == "lm_head.bias":
            fu[off:off + n] = 0.0
        else:
            o = lay_t[nm][0]
            fu[off:off + n] = ft[o:o + n]
    tokens = rng.integers(0, t.vocab, (2, 10)).astype(np.int32)
    a, b = ot.OracleTrainer(t, ft, smooth=True), ot.OracleTrainer(u, fu, smooth=True)
    la, ea, _ = a.forward(tokens, 3)
    lb, eb, _ = b.forward(tokens, 3)
    assert np.abs(la - lb).max() <= 1e-12 and np.abs(ea - eb).max() <= 1e-12
    up = rng.normal(0, 1, la.size)
    ga, gb = a.backward(up), b.backward(up)
    n_emb = t.vocab * t.d_model
    lay_u = {nm: off for nm, off, _ in u.param_layout()[0]}
    both = gb[:n_emb] + gb[lay_u["lm_head.weight"]:lay_u["lm_head.weight"] + n_emb]
    assert np.abs(ga[:n_emb] - both).max() <= 1e-10 * np.abs(both).max()
