"""Model files of the ternary GPT policy in both roles (model_serialization.hpp:40-89; src/model_roles_test.cpp's checks):
a model-role file restores packed weights and tau bit for bit, so logits are bit-identical, and comes back trainable at the
quantiser's fixed point; a checkpoint-role file restores the latent bit for bit; the model file is much smaller;
a corrupted or truncated file is refused before anything is loaded."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _policy(pkg, eng, seed):
    cfg = pkg.GptConfig(n_layer=2, d_model=64, n_head=2, d_ff=128, vocab=211, ctx=24, act=1, pos=1, value_head=True)
    pol = pkg.Policy(eng, cfg)
    pol.upload_params(cfg.init_params(seed, bias_std=0.01))
    return cfg, pol


def test_model_and_checkpoint_roles_round_trip(pkg, eng, tmp_path):
    cfg, a = _policy(pkg, eng, 1)
    _, b = _policy(pkg, eng, 2)
    prompts = torch.from_numpy(np.random.default_rng(0).integers(0, 211, (3, 5)).astype(np.int32)).to(eng.device)
    tok_a, lp_a, lg_a = a.rollout(prompts, 8, temperature=0.0, want_logits=True)
    model_file, ckpt_file = str(tmp_path / "p.nnmodel"), str(tmp_path / "p.nnckpt")
    a.save(model_file, "model")
    a.save(ckpt_file, "checkpoint")
    assert os.path.getsize(model_file) < 0.6 * os.path.getsize(ckpt_file)  # base-3 packing, no latent
    b.load(model_file)
    for layer, which in ((0, 0), (1, 4), (1, 5), (-1, 0)):
        pa, ta = a.linear(layer, which)
        pb, tb = b.linear(layer, which)
        assert torch.equal(pa, pb) and torch.equal(ta, tb)
    tok_b, lp_b, lg_b = b.rollout(prompts, 8, temperature=0.0, want_logits=True)
    assert torch.equal(lg_a, lg_b) and torch.equal(tok_a, tok_b)
    # trainable again, at the fixed point: re-quantising the loaded latent gives the same trits and tau within an ulp
    packed_before, tau_before = (t.clone() for t in b.linear(0, 4))
    b.requantize()
    packed_after, tau_after = b.linear(0, 4)
    assert torch.equal(packed_before, packed_after)
    assert (tau_after - tau_before).abs().max().item() <= 2e-6 * tau_before.abs().max().item()
    # the non-ternary parameters came back bit for bit
    layout = {nm: (off, shape) for nm, off, shape in cfg.param_layout()[0]}
    for name in ("tok_emb", "blocks.0.ln1.gamma", "lm_head.bias", "value_head.weight"):
        off, shape = layout[name]
        n = int(np.prod(shape))
        assert torch.equal(a.params_view()[off:off + n], b.params_view()[off:off + n])
    # checkpoint role: the whole latent, bit for bit
    _, c = _policy(pkg, eng, 3)
    c.load(ckpt_file)
    assert torch.equal(c.params_view(), a.params_view())
    tok_c, _, lg_c = c.rollout(prompts, 8, temperature=0.0, want_logits=True)
    assert torch.equal(lg_a, lg_c)


def test_damaged_files_are_refused(pkg, eng, tmp_path):
    cfg, a = _policy(pkg, eng, 1)
    path = str(tmp_path / "p.nnmodel")
    a.save(path, "model")
    raw = bytearray(open(path, "rb").read())
    before = a.params_view().clone()
    bad = bytearray(raw)
    bad[len(bad) // 2] ^= 0x40
    open(path, "wb").write(bad)
    with pytest.raises(pkg.NnbError, match="checksum"):
        a.load(path)
    open(path, "wb").write(raw[:-100])
    with pytest.raises(pkg.NnbError):
        a.load(path)
    assert torch.equal(a.params_view(), before)  # nothing was loaded
    other = pkg.Policy(eng, pkg.GptConfig(n_layer=1, d_model=64, n_head=2, d_ff=128, vocab=211, ctx=24, act=1, pos=1, value_head=True))
    open(path, "wb").write(raw)
    with pytest.raises(pkg.NnbError, match="different model"):
        other.load(path)
