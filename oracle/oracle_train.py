"""oracle_train.py — numpy restatement of the reference's teacher-forced forward, objectives and
backward pass for the ternary GPT policy.

TEST INFRASTRUCTURE ONLY: imported by tests (and the CPU-baseline leg of the benchmark), never by
the product.  Follows, formula by formula (paths under include/neuralnet.cpp/ of the reference):
  GPTModel::forward / backward          compute_layer_gpt.hpp:460-636
  prenorm residual blocks               compute_layer_base.hpp:598-605, compute_layer_gpt.hpp:173-182
  BitLinear::forward / backward (int8)  compute_layer_bitlinear.hpp:417-472, 475-544
  RMSNorm forward / backward            compute_layer_mlp.hpp:686-746
  GeLU (QuickGELU), SwiGLU fwd / bwd    compute_layer_mlp.hpp:243-270, 317-369
  RotaryEmbedding apply (fwd / bwd)     compute_position_encoding.hpp:126-145
  AttentionBase forward / backward      compute_layer_attention.hpp:698-988
  CategoricalDistribution, objectives   rl_policy.hpp:92-187, 460-773, 799-953
Quantisation decisions (int8 activations, ternary weights) are taken in f32 exactly as the engine
takes them; everything downstream of them is evaluated in float64, so this file is the
high-precision side of the 1e-3 relative gates.  Float accumulation order of the reference is
engine-defined: parity unpinned bitwise, tolerance-gated.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

F32 = np.float32
_LIB = None


def _lib():
    """liboracle.so supplies the bit-reproducible exp and the RoPE tables of the step path."""
    global _LIB
    if _LIB is None:
        L = C.CDLL(os.path.join(os.path.dirname(os.path.abspath(__file__)), "liboracle.so"))
        fp = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
        L.orc_expf_array.argtypes = [fp, C.c_size_t, fp]
        L.orc_rope_tables.argtypes = [C.c_int, C.c_int, fp, fp]
        _LIB = L
    return _LIB


def expf32(x):
    x = np.ascontiguousarray(x, F32)
    out = np.empty_like(x)
    _lib().orc_expf_array(x.reshape(-1), x.size, out.reshape(-1))
    return out


def unflatten(cfg, flat):
    layout, n = cfg.param_layout()
    assert flat.size == n
    return {name: flat[off:off + int(np.prod(shape))].reshape(shape) for name, off, shape in layout}


def absmean_tau(w):
    k = w.shape[1]
    inv = F32(1.0) / F32(k)
    return (np.abs(w).astype(F32) * inv).astype(np.float64).sum(1).astype(F32)


def ternarise(w, tau):
    hi = (tau * F32(0.5))[:, None]
    lo = (tau * F32(-0.5))[:, None]
    return np.where(w > hi, 1, np.where(w < lo, -1, 0)).astype(np.int8)


def act_quant(x):
    """x (T,K) f32 -> q (T,K) int8, s (T) f32: s = absmax*(1/127), q = round_half_away(clamp(x/s))."""
    x = x.astype(F32)
    mx = np.abs(x).max(1)
    s = (mx * (F32(1.0) / F32(127.0))).astype(F32)
    with np.errstate(divide="ignore", invalid="ignore"):
        v = (x / s[:, None]).astype(F32)
    v = np.where(np.isnan(v), 0, v)
    v = np.clip(v, -127, 127)
    q = np.where(s[:, None] == 0, 0, np.sign(v) * np.floor(np.abs(v).astype(np.float64) + 0.5)).astype(np.int8)
    return q, s


class Linear:
    """BitLinear with int8 activations.  smooth=True replaces it by the dense float64 linear y = x W^T + b with its
    exact derivative: the model around it then has no quantiser, so that finite differences apply to it (the
    reference's gradient checks run on dense layers for the same reason, src/gpt_gradcheck.cpp:1-20)."""

    def __init__(self, w, b, smooth=False):
        self.w, self.b, self.smooth = w, b, smooth
        self.tau = absmean_tau(w)
        self.trit = ternarise(w, self.tau)

    def forward(self, x):
        """x (T,K) f32 -> y (T,out) f32 evaluated like the engine: (tau*s)*float(acc) + b in f32."""
        if self.smooth:
            self.x64 = np.asarray(x, np.float64)
            return self.x64 @ self.w.astype(np.float64).T + self.b.astype(np.float64)[None, :]
        q, s = act_quant(x)
        acc = q.astype(np.float64) @ self.trit.astype(np.float64).T  # exact integers
        y = (self.tau[None, :] * s[:, None]).astype(F32) * acc.astype(F32)
        y = (y + self.b[None, :]).astype(F32)
        self.q, self.s = q, s
        return y

    def backward(self, dy):
        """dy (T,out) f64 -> dx (T,K); accumulates dw, db (STE, int8 path)."""
        if self.smooth:
            self.dw = dy.T @ self.x64
            self.db = dy.sum(0)
            return dy @ self.w.astype(np.float64)
        t = self.tau.astype(np.float64)
        dx = (dy * t[None, :]) @ self.trit.astype(np.float64)
        self.dw = ((dy * self.s.astype(np.float64)[:, None]).T @ self.q.astype(np.float64)) * t[:, None]
        self.db = dy.sum(0)
        return dx


def rmsnorm_fwd(x, g, smooth=False):
    """Output in the engine's f32 rounding order (it feeds a quantiser); cache in float64.
    smooth=True: everything in float64, no f32 rounding."""
    if smooth:
        x64 = np.asarray(x, np.float64)
        sinv = 1.0 / np.sqrt((x64 * x64).mean(-1, keepdims=True) + 1e-5)
        return x64 * sinv * np.asarray(g, np.float64), (x64 * sinv, sinv)
    x = x.astype(F32)
    f = x.shape[-1]
    ss = (x * x).astype(np.float64).sum(-1, keepdims=True).astype(F32)
    v = (ss * (F32(1.0) / F32(f)) + F32(1e-5)).astype(F32)
    sinv32 = (F32(1.0) / np.sqrt(v).astype(F32)).astype(F32)
    out = ((x * sinv32).astype(F32) * g.astype(F32)).astype(F32)
    x64 = x.astype(np.float64)
    sinv = 1.0 / np.sqrt((x64 * x64).mean(-1, keepdims=True) + 1e-5)
    return out, (x64 * sinv, sinv)


def rmsnorm_bwd(dy, g, cache):
    normed, sinv = cache
    gy = dy * g
    m = (gy * normed).mean(-1, keepdims=True)
    dx = (gy - m * normed) * sinv
    dg = (dy * normed).reshape(-1, normed.shape[-1]).sum(0)
    return dx, dg


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def rope_tables(cfg, S):
    dk = cfg.d_model // cfg.n_head
    half = dk // 2
    cos, sin = np.empty((S, half), F32), np.empty((S, half), F32)
    _lib().orc_rope_tables(dk, S, cos, sin)
    return cos, sin


def rope_apply(x, cos, sin, sign=1.0):
    """x (n,S,H,dk); out = x*cos + rotate_half(x)*sin (sign=-1: the inverse rotation).
    f32 inputs are rotated with the engine's f32 roundings, float64 inputs in float64."""
    half = x.shape[-1] // 2
    a, b = x[..., :half], x[..., half:]
    dt = x.dtype
    c, s = cos[None, :, None, :].astype(dt), (sign * sin[None, :, None, :]).astype(dt)
    return np.concatenate([(a * c).astype(dt) + ((-b) * s).astype(dt), (b * c).astype(dt) + (a * s).astype(dt)], -1).astype(dt)


class OracleTrainer:
    """Holds the parameters (dict of f32 arrays in the engine's flat layout) and runs forward/backward."""

    def __init__(self, cfg, flat, smooth=False):
        """smooth=True: dense float64 linears and no f32 roundings anywhere (flat may then be float64) — the
        differentiable twin of the model, on which the backward pass is checked by finite differences."""
        self.cfg = cfg
        self.smooth = smooth
        self.flat = np.ascontiguousarray(flat, np.float64 if smooth else F32)
        self.p = unflatten(cfg, self.flat)
        self.lin = {}
        for name in list(self.p):
            if name.endswith(".weight") and not name.startswith("value_head"):
                base = name[:-7]
                self.lin[base] = Linear(self.p[name], self.p[base + ".bias"], smooth)

    # ------------------------------------------------------------------ forward
    def forward(self, tokens, prompt_len):
        cfg, p = self.cfg, self.p
        n, S = tokens.shape
        d, H = cfg.d_model, cfg.n_head
        dk = d // H
        F = cfg.d_ff
        # grouped-query attention (compute_layer_attention.hpp:444-454): Hkv key/value heads, query head h reads
        # KV head h // (H / Hkv); the reference expands K and V to H heads (gather_rows) and runs plain MHA
        Hkv = getattr(cfg, "n_head_kv", 0) or H
        rep = H // Hkv
        sub_ln = bool(getattr(cfg, "sub_ln", False))
        tie = bool(getattr(cfg, "tie_embeddings", False))
        self.tokens, self.P = tokens, prompt_len
        sm = self.smooth
        R = (lambda a: np.asarray(a, np.float64)) if sm else (lambda a: np.asarray(a).astype(F32))  # the engine's f32 rounding
        ex = np.exp if sm else expf32
        x = p["tok_emb"][tokens]  # (n,S,d) f32
        if cfg.pos == 0:
            x = R(x + p["pos_emb"][None, :S])
        self.cache = []
        cos = sin = None
        if cfg.pos == 1:
            cos, sin = rope_tables(cfg, S)
        scale = 1.0 / np.sqrt(np.float64(dk))
        causal = np.tril(np.ones((S, S), bool))
        for l in range(cfg.n_layer):
            pre = f"blocks.{l}."
            c = {}
            c["x_in"] = x
            n1, c["n1"] = rmsnorm_fwd(x, p[pre + "ln1.gamma"], sm)
            flat1 = n1.reshape(n * S, d)
            q = self.lin[pre + "attn.q"].forward(flat1).reshape(n, S, H, dk)
            k = self.lin[pre + "attn.k"].forward(flat1).reshape(n, S, Hkv, dk)
            v = self.lin[pre + "attn.v"].forward(flat1).astype(np.float64).reshape(n, S, Hkv, dk)
            if cfg.pos == 1:
                q, k = rope_apply(q, cos, sin), rope_apply(k, cos, sin)
            if rep > 1:
                k, v = np.repeat(k, rep, axis=2), np.repeat(v, rep, axis=2)
            # the reference folds the scale into Q after RoPE (one f32 multiply)
            qs = R(q * (1.0 / np.sqrt(np.float64(dk)) if sm else F32(1.0 / np.sqrt(F32(dk))))).astype(np.float64)
            k = k.astype(np.float64)
            sc = np.einsum("bihd,bjhd->bhij", qs, k)
            sc = np.where(causal[None, None], sc, -np.inf)
            sc = sc - sc.max(-1, keepdims=True)
            w = np.exp(sc)
            w = w / w.sum(-1, keepdims=True)
            att = np.einsum("bhij,bjhd->bihd", w, v)
            c.update(qs=qs, k=k, v=v, w=w)
            a = R(att.reshape(n * S, d))
            if sub_ln:  # SubLN (compute_layer_attention.hpp:482-489,820-826): heads' output -> norm -> o projection
                a, c["sn_a"] = rmsnorm_fwd(a, p[pre + "attn.sub_norm.gamma"], sm)
            o = self.lin[pre + "attn.o"].forward(a)
            x_mid = R(x + o.reshape(n, S, d))
            c["x_mid"] = x_mid
            n2, c["n2"] = rmsnorm_fwd(x_mid, p[pre + "ln2.gamma"], sm)
            h1 = self.lin[pre + "ffn.fc1"].forward(n2.reshape(n * S, d))
            c["h1"] = h1
            one = 1.0 if sm else F32(1.0)
            if cfg.act == 0:
                act = R(h1 / R(one + ex(-R(h1 * (1.702 if sm else F32(1.702))))))
            elif cfg.act == 2:  # ReLU2GLU (compute_layer_mlp.hpp:384-440): relu(gate)^2 * up
                g, u = h1[:, :F], h1[:, F:]
                r = np.maximum(g, 0)
                act = R(R(r * r) * u)
            else:
                g, u = h1[:, :F], h1[:, F:]
                sg = R(one / R(one + ex(-g)))
                act = R(R(g * sg) * u)
            act = R(act)
            if sub_ln:  # SubLN (compute_layer_feedforward.hpp:37-47,201-206): activated hidden -> norm -> fc2
                act, c["sn_f"] = rmsnorm_fwd(act, p[pre + "ffn.sub_norm.gamma"], sm)
            f2 = self.lin[pre + "ffn.fc2"].forward(act)
            x = R(x_mid + f2.reshape(n, S, d))
            self.cache.append(c)
        self.x_final = x
        G = S - prompt_len
        xd = x[:, prompt_len - 1:S - 1].reshape(n * G, d)
        hn, self.cf = rmsnorm_fwd(xd, p["ln_f.gamma"], sm)
        self.hn = hn
        if tie:
            # tied embeddings (compute_layer_gpt.hpp:286-297): logits = tok_emb . hn, a dense product, no bias
            logits = hn.astype(np.float64) @ p["tok_emb"].astype(np.float64).T
            if not sm:
                logits = logits.astype(F32).astype(np.float64)
        else:
            logits = self.lin["lm_head"].forward(hn).astype(np.float64)
        self.logits = logits
        actions = tokens[:, prompt_len:].reshape(-1)
        self.actions = actions
        mx = logits.max(1, keepdims=True)
        lse = mx[:, 0] + np.log(np.exp(logits - mx).sum(1))
        self.logp_all = logits - lse[:, None]
        logp = self.logp_all[np.arange(len(actions)), actions]
        prob = np.exp(self.logp_all)
        ent = -(prob * self.logp_all).sum(1)
        value = None
        if cfg.value_head:
            value = hn.astype(np.float64) @ p["value_head.weight"].astype(np.float64).reshape(-1) + float(p["value_head.bias"][0])
        self.value = value
        return logp.reshape(n, G), ent.reshape(n, G), None if value is None else value.reshape(n, G)

    # ---------------------------------------------------------------- objective
    @staticmethod
    def objective(logp, ent, mask, old_logp=None, adv=None, ref_logp=None, value=None, returns=None, old_value=None,
                  units=0.0, clip_eps=0.2, kl_coef=0.0, entropy_coef=0.0, value_coef=0.0, value_clip_eps=0.2):
        """Returns (report dict, d loss/d logp, d loss/d entropy, d loss/d value), all flattened."""
        logp, ent, mask = (np.asarray(a, np.float64).reshape(-1) for a in (logp, ent, mask))
        units = float(mask.sum()) if units <= 0 else float(units)
        rep = dict(policy_loss=0.0, ratio_mean=0.0, approx_kl=0.0, clip_fraction=0.0, kl_loss=0.0, entropy_loss=0.0,
                   value_loss=0.0, value_clip_fraction=0.0, units=units)
        up_lp, up_ent = np.zeros_like(logp), np.zeros_like(logp)
        dv = None
        if units <= 0:
            return rep, up_lp, up_ent, dv
        if old_logp is not None:
            old, a = np.asarray(old_logp, np.float64).reshape(-1), np.asarray(adv, np.float64).reshape(-1)
            diff = logp - old
            ratio = np.exp(diff)
            lo, hi = 1 - clip_eps, 1 + clip_eps
            surr = np.minimum(ratio * a, np.clip(ratio, lo, hi) * a)
            rep["policy_loss"] = -(surr * mask).sum() / units
            pos = np.where(ratio > hi, 0.0, ratio * a)
            neg = np.where(ratio < lo, 0.0, ratio * a)
            up_lp += np.where(a > 0, pos, neg) * mask * (-1.0 / units)
            rep["ratio_mean"] = (ratio * mask).sum() / units
            rep["approx_kl"] = 0.5 * (diff * diff * mask).sum() / units
            rep["clip_fraction"] = (((ratio < lo) | (ratio > hi)) * mask).sum() / units
        if ref_logp is not None and kl_coef != 0:
            ref = np.asarray(ref_logp, np.float64).reshape(-1)
            rep["kl_loss"] = kl_coef * ((logp - ref) * mask).sum() / units
            up_lp += mask * (kl_coef / units)
        if entropy_coef != 0:
            rep["entropy_loss"] = -entropy_coef * (ent * mask).sum() / units
            up_ent += mask * (-entropy_coef / units)
        if value_coef != 0:
            v, r, ov = (np.asarray(x, np.float64).reshape(-1) for x in (value, returns, old_value))
            lo, hi = ov - value_clip_eps, ov + value_clip_eps
            cl = np.clip(v, lo, hi)
            dsq, csq = (v - r) ** 2, (cl - r) ** 2
            rep["value_loss"] = value_coef * (np.maximum(dsq, csq) * mask).sum() / units
            outside = (v < lo) | (v > hi)
            ug = 2 * (v - r)
            cg = np.where(outside, 0.0, ug)
            dv = np.where(csq > dsq, cg, ug) * mask * (value_coef / units)
            rep["value_clip_fraction"] = (outside * mask).sum() / units
        return rep, up_lp, up_ent, dv

    # ----------------------------------------------------------------- backward
    def backward(self, up_lp, up_ent=None, dvalue=None):
        """Gradients of sum(up_lp*logp) + sum(up_ent*H) + sum(dvalue*value) w.r.t. every parameter.
        Returns a flat float64 vector in the parameter layout."""
        cfg, p = self.cfg, self.p
        n, S = self.tokens.shape
        d, H, F = cfg.d_model, cfg.n_head, cfg.d_ff
        dk = d // H
        P = self.P
        G = S - P
        grads = {name: np.zeros(v.shape, np.float64) for name, v in p.items()}
        prob = np.exp(self.logp_all)
        onehot = np.zeros_like(prob)
        onehot[np.arange(len(self.actions)), self.actions] = 1.0
        dlogits = (onehot - prob) * up_lp[:, None]
        if up_ent is not None:
            ent = -(prob * self.logp_all).sum(1)
            dlogits += -prob * (self.logp_all + ent[:, None]) * up_ent[:, None]
        Hkv = getattr(cfg, "n_head_kv", 0) or H
        rep = H // Hkv
        sub_ln = bool(getattr(cfg, "sub_ln", False))
        if getattr(cfg, "tie_embeddings", False):
            # dX = g . E ; dE += g^T . hn, into the same gradient as the embedding lookup (compute_layer_gpt.hpp:556-575)
            dhn = dlogits @ p["tok_emb"].astype(np.float64)
            grads["tok_emb"] += dlogits.T @ np.asarray(self.hn, np.float64)
        else:
            head = self.lin["lm_head"]
            dhn = head.backward(dlogits)
            grads["lm_head.weight"] += head.dw
            grads["lm_head.bias"] += head.db
        if cfg.value_head and dvalue is not None:
            w = p["value_head.weight"].astype(np.float64).reshape(-1)
            dhn = dhn + dvalue[:, None] * w[None, :]
            grads["value_head.weight"] += (dvalue[:, None] * self.hn.astype(np.float64)).sum(0).reshape(1, -1)
            grads["value_head.bias"] += dvalue.sum()
        dxd, dg = rmsnorm_bwd(dhn, p["ln_f.gamma"].astype(np.float64), self.cf)
        grads["ln_f.gamma"] += dg
        g = np.zeros((n, S, d))
        g[:, P - 1:S - 1] = dxd.reshape(n, G, d)
        cos = sin = None
        if cfg.pos == 1:
            cos, sin = rope_tables(cfg, S)
        scale = 1.0 / np.sqrt(np.float64(dk))
        for l in range(cfg.n_layer - 1, -1, -1):
            pre = f"blocks.{l}."
            c = self.cache[l]
            fc2, fc1 = self.lin[pre + "ffn.fc2"], self.lin[pre + "ffn.fc1"]
            da = fc2.backward(g.reshape(n * S, d))
            grads[pre + "ffn.fc2.weight"] += fc2.dw
            grads[pre + "ffn.fc2.bias"] += fc2.db
            if sub_ln:
                da, dg = rmsnorm_bwd(da, p[pre + "ffn.sub_norm.gamma"].astype(np.float64), c["sn_f"])
                grads[pre + "ffn.sub_norm.gamma"] += dg
            h = c["h1"].astype(np.float64)
            if cfg.act == 0:
                bx = h * 1.702
                s = sigmoid(bx)
                dh = da * (s * (1 + bx * (1 - s)))
            elif cfg.act == 2:
                gt, up = h[:, :F], h[:, F:]
                r = np.maximum(gt, 0)
                dh = np.concatenate([da * up * (2 * r), da * r * r], 1)
            else:
                gt, up = h[:, :F], h[:, F:]
                s = sigmoid(gt)
                dh = np.concatenate([da * up * (s * (1 + gt * (1 - s))), da * gt * s], 1)
            dn2 = fc1.backward(dh)
            grads[pre + "ffn.fc1.weight"] += fc1.dw
            grads[pre + "ffn.fc1.bias"] += fc1.db
            dx, dg = rmsnorm_bwd(dn2.reshape(n, S, d), p[pre + "ln2.gamma"].astype(np.float64), c["n2"])
            grads[pre + "ln2.gamma"] += dg
            g2 = g + dx
            lo = self.lin[pre + "attn.o"]
            datt = lo.backward(g2.reshape(n * S, d))
            grads[pre + "attn.o.weight"] += lo.dw
            grads[pre + "attn.o.bias"] += lo.db
            if sub_ln:
                datt, dg = rmsnorm_bwd(datt, p[pre + "attn.sub_norm.gamma"].astype(np.float64), c["sn_a"])
                grads[pre + "attn.sub_norm.gamma"] += dg
            datt = datt.reshape(n, S, H, dk)
            w, qs, k, v = c["w"], c["qs"], c["k"], c["v"]
            dv = np.einsum("bhij,bihd->bjhd", w, datt)
            dp = np.einsum("bihd,bjhd->bhij", datt, v)
            r = (w * dp).sum(-1, keepdims=True)
            xs = w * (dp - r)
            dq = np.einsum("bhij,bjhd->bihd", xs, k) * scale
            dk_ = np.einsum("bhij,bihd->bjhd", xs, qs)
            if rep > 1:  # the replicas of a KV head sum (scatter_add_rows of the reference)
                dk_ = dk_.reshape(n, S, Hkv, rep, dk).sum(3)
                dv = dv.reshape(n, S, Hkv, rep, dk).sum(3)
            if cfg.pos == 1:
                dq, dk_ = rope_apply(dq, cos, sin, -1.0), rope_apply(dk_, cos, sin, -1.0)
            dn1 = 0
            for nm, dd in (("attn.q", dq), ("attn.k", dk_), ("attn.v", dv)):
                li = self.lin[pre + nm]
                dn1 = dn1 + li.backward(dd.reshape(n * S, -1))
                grads[pre + nm + ".weight"] += li.dw
                grads[pre + nm + ".bias"] += li.db
            dx, dg = rmsnorm_bwd(dn1.reshape(n, S, d), p[pre + "ln1.gamma"].astype(np.float64), c["n1"])
            grads[pre + "ln1.gamma"] += dg
            g = g2 + dx
        np.add.at(grads["tok_emb"], self.tokens.reshape(-1), g.reshape(n * S, d))
        if cfg.pos == 0:
            grads["pos_emb"][:S] += g.sum(0)
        layout, total = cfg.param_layout()
        flat = np.zeros(total, np.float64)
        for name, off, shape in layout:
            flat[off:off + int(np.prod(shape))] = grads[name].reshape(-1)
        return flat
