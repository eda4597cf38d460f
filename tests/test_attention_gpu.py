"""Causal attention forward/backward: the CUDA-core path against a float64 reference of the reference's
formulas (compute_layer_attention.hpp:752-828, 873-960), and the bf16 tensor-core path against it within
bf16 rounding."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(q, k, v, dout, n, S, H):
    d = q.shape[1]
    dk = d // H
    scale = 1.0 / np.sqrt(dk)
    q4, k4, v4, g4 = (a.astype(np.float64).reshape(n, S, H, dk) for a in (q, k, v, dout))
    qs = q4 * scale
    sc = np.einsum("bihd,bjhd->bhij", qs, k4)
    sc = np.where(np.tril(np.ones((S, S), bool))[None, None], sc, -np.inf)
    mx = sc.max(-1, keepdims=True)
    w = np.exp(sc - mx)
    l = w.sum(-1, keepdims=True)
    w = w / l
    out = np.einsum("bhij,bjhd->bihd", w, v4)
    lse = (mx + np.log(l))[..., 0]
    dv = np.einsum("bhij,bihd->bjhd", w, g4)
    dp = np.einsum("bihd,bjhd->bhij", g4, v4)
    r = (w * dp).sum(-1, keepdims=True)
    x = w * (dp - r)
    dq = np.einsum("bhij,bjhd->bihd", x, k4) * scale
    dkk = np.einsum("bhij,bihd->bjhd", x, qs)
    return out.reshape(n * S, d), lse, dq.reshape(n * S, d), dkk.reshape(n * S, d), dv.reshape(n * S, d)


def _err(a, b):
    return np.abs(a.cpu().numpy() - b).max() / np.abs(b).max()


@pytest.mark.parametrize("n,S,H,dk", [(2, 33, 2, 64), (3, 150, 2, 128), (1, 64, 1, 64), (2, 97, 3, 64), (1, 200, 2, 128),
                                      (2, 40, 2, 100), (2, 17, 4, 32)])
def test_attention_paths(eng, n, S, H, dk):
    rng = np.random.default_rng(S * dk)
    d = H * dk
    q, k, v, g = (rng.normal(0, 1, (n * S, d)).astype(np.float32) for _ in range(4))
    out_ref, lse_ref, dq_ref, dk_ref, dv_ref = _ref(q, k, v, g, n, S, H)
    tq, tk, tv, tg = (torch.from_numpy(a).to(eng.device) for a in (q, k, v, g))
    for exact, tol in ((True, 1e-4), (False, 2e-2)):
        out, lse = eng.attention_fwd(tq, tk, tv, n, S, H, exact=exact)
        assert _err(out, out_ref) <= tol
        assert np.abs(lse.cpu().numpy() - lse_ref).max() <= tol * max(1.0, np.abs(lse_ref).max())
        dq, dkk, dv = eng.attention_bwd(tq, tk, tv, out, tg, lse, n, S, H, exact=exact)
        assert _err(dq, dq_ref) <= tol and _err(dkk, dk_ref) <= tol and _err(dv, dv_ref) <= tol


def _rope(x, n, S, H, cos, sin, sign=1.0):
    """Rotate pairs (j, j + dk/2) of every head by the row's position; sign=-1 is the inverse."""
    d = x.shape[1]
    dk = d // H
    half = dk // 2
    x4 = x.astype(np.float64).reshape(n, S, H, dk)
    a, b = x4[..., :half], x4[..., half:]
    c, s = cos[None, :, None, :], sign * sin[None, :, None, :]
    return np.concatenate([a * c - b * s, b * c + a * s], -1).reshape(n * S, d)


@pytest.mark.parametrize("n,S,H,dk", [(2, 33, 2, 64), (2, 150, 2, 128), (1, 257, 3, 128), (2, 40, 2, 100)])
def test_attention_with_rope_inside(eng, n, S, H, dk):
    """q and k un-rotated, gradients with respect to the un-rotated q and k, both numeric modes."""
    rng = np.random.default_rng(S + dk)
    d = H * dk
    half = dk // 2
    q, k, v, g = (rng.normal(0, 1, (n * S, d)).astype(np.float32) for _ in range(4))
    ang = np.arange(S)[:, None] * (10000.0 ** (-np.arange(half) / half))[None, :]
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    qr, kr = _rope(q, n, S, H, cos, sin), _rope(k, n, S, H, cos, sin)
    out_ref, lse_ref, dqr, dkr, dv_ref = _ref(qr, kr, v, g, n, S, H)
    dq_ref, dk_ref = _rope(dqr, n, S, H, cos, sin, -1.0), _rope(dkr, n, S, H, cos, sin, -1.0)
    tq, tk, tv, tg, tc, ts = (torch.from_numpy(a).to(eng.device) for a in (q, k, v, g, cos, sin))
    for exact, tol in ((True, 1e-4), (False, 2e-2)):
        out, lse = eng.attention_rope_fwd(tq, tk, tv, tc, ts, n, S, H, exact=exact)
        assert _err(out, out_ref) <= tol
        assert np.abs(lse.cpu().numpy() - lse_ref).max() <= tol * max(1.0, np.abs(lse_ref).max())
        dq, dkk, dv = eng.attention_rope_bwd(tq, tk, tv, tc, ts, out, tg, lse, n, S, H, exact=exact)
        assert _err(dq, dq_ref) <= tol and _err(dkk, dk_ref) <= tol and _err(dv, dv_ref) <= tol


def _bf16_round(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).float().numpy()


@pytest.mark.parametrize("n,H,dk,pos,pre_len,group", [(4, 4, 64, 17, 0, 1), (3, 16, 128, 40, 0, 1), (4, 2, 128, 21, 8, 2),
                                                      (6, 3, 64, 9, 9, 3), (2, 2, 32, 5, 0, 1), (2, 32, 100, 30, 0, 1)])
def test_attention_decode_step(eng, n, H, dk, pos, pre_len, group):
    """One new token against the cache: rotation, append, attention over prefix + own positions; the exact path
    against float64, the bf16 paths (per-head kernel and all-heads kernel with the fused int8 output) within
    bf16 rounding, and the fused quantisation against the quantisation of its own f32 output."""
    rng = np.random.default_rng(n * 1000 + pos)
    d, half, ctx_alloc, pre_alloc = H * dk, dk // 2, 48, max(pre_len, 1) + 3
    qkv = rng.normal(0, 1, (3, n, d)).astype(np.float32)
    kown = rng.normal(0, 1, (n, H, ctx_alloc, dk)).astype(np.float32)
    vown = rng.normal(0, 1, (n, H, ctx_alloc, dk)).astype(np.float32)
    kpre = rng.normal(0, 1, (n // group, H, pre_alloc, dk)).astype(np.float32)
    vpre = rng.normal(0, 1, (n // group, H, pre_alloc, dk)).astype(np.float32)
    ang = np.arange(64)[:, None] * (10000.0 ** (-np.arange(half) / half))[None, :]
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)

    def reference(rnd):
        q4, k4, v4 = (qkv[i].astype(np.float64).reshape(n, H, dk) for i in range(3))
        c, s = cos[pos].astype(np.float64), sin[pos].astype(np.float64)
        rot = lambda x: np.concatenate([x[..., :half] * c - x[..., half:] * s, x[..., half:] * c + x[..., :half] * s], -1)
        qr, kr = rot(q4), rnd(rot(k4))
        out = np.zeros((n, H, dk))
        for b in range(n):
            keys = np.concatenate([rnd(kpre[b // group][:, :pre_len]), rnd(kown[b][:, :pos - pre_len]), kr[b][:, None]], 1)
            vals = np.concatenate([rnd(vpre[b // group][:, :pre_len]), rnd(vown[b][:, :pos - pre_len]), rnd(v4[b])[:, None]], 1)
            sc = np.einsum("hd,hjd->hj", qr[b], keys.astype(np.float64)) / np.sqrt(dk)
            w = np.exp(sc - sc.max(-1, keepdims=True))
            w /= w.sum(-1, keepdims=True)
            out[b] = np.einsum("hj,hjd->hd", w, vals.astype(np.float64))
        return out.reshape(n, d), kr

    dev = eng.device
    tq = torch.from_numpy(qkv).to(dev)
    tpos = torch.tensor([pos], device=dev, dtype=torch.int32)
    rope = (torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev))
    for exact in (True, False):
        dt = torch.float32 if exact else torch.bfloat16
        rnd = (lambda a: a) if exact else _bf16_round
        ref, kr = reference(rnd)
        for fused in ((False,) if exact else (False, True)):
            if fused and dk not in (64, 128):
                continue
            kc, vc = torch.from_numpy(kown).to(dev).to(dt), torch.from_numpy(vown).to(dev).to(dt)
            prefix = (torch.from_numpy(kpre).to(dev).to(dt), torch.from_numpy(vpre).to(dev).to(dt), pre_len) if pre_len else None
            out, q8, s, qsum = eng.attention_decode(tq, kc, vc, tpos, H, rope=rope, prefix=prefix, group=group, exact=exact,
                                                    want_q8=fused)
            tol = 1e-5 if exact else 2e-2
            assert _err(out, ref) <= tol
            # the new key and value were appended at row pos - pre_len
            assert np.abs(kc[:, :, pos - pre_len].float().cpu().numpy() - kr).max() <= (1e-5 if exact else 2e-2)
            assert np.abs(vc[:, :, pos - pre_len].float().cpu().numpy() - qkv[2].reshape(n, H, dk)).max() <= (1e-6 if exact else 2e-2)
            if fused:
                q_ref, s_ref, qs_ref = eng.act_quant_tm(out)
                assert torch.allclose(s, s_ref, rtol=1e-6, atol=0)
                dq = (q8.int() - q_ref.int()).abs()
                assert int(dq.max()) <= 1 and float((dq > 0).float().mean()) < 1e-3  # x/s against x*(1/s) at a rounding tie
                assert torch.equal(qsum, eng.actq_to_plain(q8).int().sum(1).int())
