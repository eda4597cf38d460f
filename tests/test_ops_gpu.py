"""Standalone RMSNorm and rotary-embedding operators of the C-ABI (nnb_rmsnorm_fwd/bwd, nnb_rope_tables/apply/step)
against float64 restatements of RMSNorm::forward / backward (compute_layer_mlp.hpp:686-746) and
RotaryEmbedding::apply / apply_step (compute_position_encoding.hpp:64-80,126-168); tolerance 1e-5 relative."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _p(t):
    return C.c_void_p(t.data_ptr())


def test_rmsnorm_forward_backward(pkg, eng):
    lib = pkg.lib()
    rng = np.random.default_rng(0)
    t, f = 37, 192
    x = torch.from_numpy(rng.normal(0, 1, (t, f)).astype(np.float32)).to(eng.device)
    g = torch.from_numpy(rng.normal(1, 0.1, f).astype(np.float32)).to(eng.device)
    dy = torch.from_numpy(rng.normal(0, 1, (t, f)).astype(np.float32)).to(eng.device)
    y = torch.empty_like(x)
    assert lib.nnb_rmsnorm_fwd(eng.handle, _p(x), _p(g), t, f, _p(y)) == 0, lib.nnb_last_error()
    x64 = x.double().requires_grad_(True)
    g64 = g.double().requires_grad_(True)
    y64 = x64 * torch.rsqrt((x64 * x64).mean(-1, keepdim=True) + 1e-5) * g64
    assert (y.double() - y64).abs().max().item() <= 1e-5 * float(y64.abs().max())
    (y64 * dy.double()).sum().backward()
    dx = torch.empty_like(x)
    dg = torch.full((f,), 0.5, device=eng.device)
    assert lib.nnb_rmsnorm_bwd(eng.handle, _p(x), _p(g), _p(dy), t, f, _p(dx), _p(dg)) == 0, lib.nnb_last_error()
    assert (dx.double() - x64.grad).abs().max().item() <= 1e-5 * float(x64.grad.abs().max())
    assert (dg.double() - 0.5 - g64.grad).abs().max().item() <= 1e-4 * float(g64.grad.abs().max())  # added to what was there


def test_rope_tables_apply_and_step(pkg, eng):
    lib = pkg.lib()
    rng = np.random.default_rng(1)
    n_seq, S, H, dk = 3, 10, 2, 20
    half = dk // 2
    cos = torch.empty((S, half), device=eng.device)
    sin = torch.empty((S, half), device=eng.device)
    assert lib.nnb_rope_tables(eng.handle, dk, S, _p(cos), _p(sin)) == 0
    pos = np.arange(S)[:, None].astype(np.float32)
    theta = pos / np.power(np.float32(10000.0), (2 * np.arange(half)).astype(np.float32) / np.float32(dk))
    assert np.abs(cos.cpu().numpy() - np.cos(theta)).max() <= 1e-6 and np.abs(sin.cpu().numpy() - np.sin(theta)).max() <= 1e-6
    x0 = rng.normal(0, 1, (n_seq * S, H * dk)).astype(np.float32)
    x = torch.from_numpy(x0).to(eng.device)
    assert lib.nnb_rope_apply(eng.handle, _p(x), _p(cos), _p(sin), n_seq * S, S, H, dk, 0) == 0
    v = x0.reshape(n_seq, S, H, dk).astype(np.float64)
    a, b = v[..., :half], v[..., half:]
    c, s = np.cos(theta)[None, :, None, :], np.sin(theta)[None, :, None, :]
    want = np.concatenate([a * c - b * s, b * c + a * s], -1).reshape(n_seq * S, H * dk)
    assert np.abs(x.cpu().numpy() - want).max() <= 1e-5
    # the inverse rotation (the gradient) undoes it
    assert lib.nnb_rope_apply(eng.handle, _p(x), _p(cos), _p(sin), n_seq * S, S, H, dk, 1) == 0
    assert np.abs(x.cpu().numpy() - x0).max() <= 1e-5
    # one new token per sequence at position 7
    xs = torch.from_numpy(x0[:n_seq].copy()).to(eng.device)
    assert lib.nnb_rope_step(eng.handle, _p(xs), _p(cos), _p(sin), n_seq, 7, H, dk) == 0
    v = x0[:n_seq].reshape(n_seq, H, dk).astype(np.float64)
    a, b = v[..., :half], v[..., half:]
    c, s = np.cos(theta[7])[None, None, :], np.sin(theta[7])[None, None, :]
    want = np.concatenate([a * c - b * s, b * c + a * s], -1).reshape(n_seq, H * dk)
    assert np.abs(xs.cpu().numpy() - want).max() <= 1e-5
