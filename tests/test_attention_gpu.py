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
