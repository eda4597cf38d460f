"""ctypes binding of oracle/liboracle.so — the CPU checker.  Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_SO = os.path.join(ROOT, "oracle", "liboracle.so")

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_SZ = C.c_size_t


def _ensure_built():
    srcs = [os.path.join(ROOT, "oracle", f) for f in ("oracle.c", "oracle_model.c", "oracle_rl.c")]
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < max(os.path.getmtime(f) for f in srcs):
        subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle")], check=True)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


class Oracle:
    def __init__(self):
        _ensure_built()
        L = C.CDLL(_SO)
        self.L = L
        L.orc_trit_code_of.restype = C.c_uint32
        L.orc_trit_code_of.argtypes = [C.c_float, C.c_float]
        L.orc_trit_value_of.restype = C.c_float
        L.orc_trit_value_of.argtypes = [C.c_uint32]
        L.orc_trit_words_per_row.restype = _SZ
        L.orc_trit_words_per_row.argtypes = [_SZ]
        L.orc_trit_bytes_per_row.restype = _SZ
        L.orc_trit_bytes_per_row.argtypes = [_SZ]
        L.orc_trit_pack_row.argtypes = [_f32p, _SZ, C.c_float, _u32p]
        L.orc_trit_at.restype = C.c_float
        L.orc_trit_at.argtypes = [_u32p, _SZ]
        L.orc_absmean_tau.argtypes = [_f32p, _SZ, _SZ, _f32p]
        L.orc_trit_pack.argtypes = [_f32p, _f32p, _SZ, _SZ, _u32p]
        L.orc_i8_quantize.restype = C.c_int8
        L.orc_i8_quantize.argtypes = [C.c_float, C.c_float]
        L.orc_i8_words_per_row.restype = _SZ
        L.orc_i8_words_per_row.argtypes = [_SZ]
        L.orc_i8_at.restype = C.c_int8
        L.orc_i8_at.argtypes = [_u32p, _SZ]
        L.orc_quantize_i8.argtypes = [_f32p, _SZ, _SZ, _f32p, C.c_int, _u32p]
        L.orc_unpack_i8.argtypes = [_u32p, _SZ, _SZ, _f32p]
        L.orc_col_absmax_scale.argtypes = [_f32p, _SZ, _SZ, _f32p]
        L.orc_matmul_q.argtypes = [_u32p, _f32p, _f32p, _SZ, _SZ, _SZ, _f32p]
        L.orc_matmul_q_t.argtypes = [_u32p, _f32p, _f32p, _SZ, _SZ, _SZ, _f32p]
        L.orc_matmul_q_i8.argtypes = [_u32p, _f32p, _u32p, _f32p, _SZ, _SZ, _SZ, C.c_void_p, C.c_void_p]
        L.orc_bitlinear_i8_tm.argtypes = [_u32p, _f32p, C.c_void_p, _i8p, _f32p, _SZ, _SZ, _SZ,
                                          C.c_void_p, C.c_void_p]
        L.orc_act_quant_tm.argtypes = [_f32p, _SZ, _SZ, _i8p, _f32p]

    # ---- codecs
    def trit_code_of(self, w, tau):
        return int(self.L.orc_trit_code_of(w, tau))

    def trit_value_of(self, code):
        return float(self.L.orc_trit_value_of(code))

    def trit_words_per_row(self, k):
        return int(self.L.orc_trit_words_per_row(k))

    def trit_bytes_per_row(self, k):
        return int(self.L.orc_trit_bytes_per_row(k))

    def trit_pack_row(self, w, tau):
        w = _c(w, np.float32)
        out = np.zeros(self.trit_words_per_row(len(w)), np.uint32)
        self.L.orc_trit_pack_row(w, len(w), tau, out)
        return out

    def trit_at(self, words, i):
        return float(self.L.orc_trit_at(_c(words, np.uint32), i))

    def absmean_tau(self, latent):
        latent = _c(latent, np.float32)
        tau = np.empty(latent.shape[0], np.float32)
        self.L.orc_absmean_tau(latent, latent.shape[0], latent.shape[1], tau)
        return tau

    def trit_pack(self, latent, tau):
        latent = _c(latent, np.float32)
        rows, k = latent.shape
        out = np.empty((rows, self.trit_words_per_row(k)), np.uint32)
        self.L.orc_trit_pack(latent, _c(tau, np.float32), rows, k, out)
        return out

    def trit_unpack(self, packed, k):
        """decode to int8 trits (rows, k) with numpy"""
        packed = _c(packed, np.uint32)
        idx = np.arange(k)
        codes = (packed[:, idx // 16] >> (2 * (idx % 16)).astype(np.uint32)) & 3
        return codes.astype(np.int8) - 2

    def i8_quantize(self, x, s):
        return int(self.L.orc_i8_quantize(x, s))

    def i8_at(self, words, i):
        return int(self.L.orc_i8_at(_c(words, np.uint32), i))

    def quantize_i8(self, x, scale, col_scale=True):
        x = _c(x, np.float32)
        m, n = x.shape
        out = np.empty((m, (n + 3) // 4), np.uint32)
        self.L.orc_quantize_i8(x, m, n, _c(scale, np.float32), int(col_scale), out)
        return out

    def unpack_i8(self, packed, n):
        packed = _c(packed, np.uint32)
        out = np.empty((packed.shape[0], n), np.float32)
        self.L.orc_unpack_i8(packed, packed.shape[0], n, out)
        return out

    def col_absmax_scale(self, x):
        x = _c(x, np.float32)
        s = np.empty(x.shape[1], np.float32)
        self.L.orc_col_absmax_scale(x, x.shape[0], x.shape[1], s)
        return s

    # ---- matmuls (reference layout)
    def matmul_q(self, packed, tau, x, k):
        packed = _c(packed, np.uint32)
        x = _c(x, np.float32)
        rows, n = packed.shape[0], x.shape[1]
        c = np.empty((rows, n), np.float32)
        self.L.orc_matmul_q(packed, _c(tau, np.float32), x, rows, k, n, c)
        return c

    def matmul_q_t(self, packed, tau, b, mcols):
        packed = _c(packed, np.uint32)
        b = _c(b, np.float32)
        rows, n = packed.shape[0], b.shape[1]
        c = np.empty((mcols, n), np.float32)
        self.L.orc_matmul_q_t(packed, _c(tau, np.float32), b, rows, mcols, n, c)
        return c

    def matmul_q_i8(self, packed, tau, xq, s, k, n):
        packed = _c(packed, np.uint32)
        xq = _c(xq, np.uint32)
        rows = packed.shape[0]
        y = np.empty((rows, n), np.float32)
        acc = np.empty((rows, n), np.int32)
        self.L.orc_matmul_q_i8(packed, _c(tau, np.float32), xq, _c(s, np.float32), rows, k, n,
                               y.ctypes.data, acc.ctypes.data)
        return y, acc

    # ---- token-major
    def act_quant_tm(self, x):
        x = _c(x, np.float32)
        t, k = x.shape
        q = np.empty((t, k), np.int8)
        s = np.empty(t, np.float32)
        self.L.orc_act_quant_tm(x, t, k, q, s)
        return q, s

    def bitlinear_i8_tm(self, packed, tau, bias, q, s, want_acc=True):
        packed = _c(packed, np.uint32)
        q = _c(q, np.int8)
        t, k = q.shape
        out = packed.shape[0]
        y = np.empty((t, out), np.float32)
        acc = np.empty((t, out), np.int32) if want_acc else None
        b = _c(bias, np.float32) if bias is not None else None
        self.L.orc_bitlinear_i8_tm(packed, _c(tau, np.float32), b.ctypes.data if b is not None else None,
                                   q, _c(s, np.float32), t, k, out, y.ctypes.data,
                                   acc.ctypes.data if acc is not None else None)
        return (y, acc) if want_acc else y


# ------------------------------------------------------------------ GPT model (oracle_model.c)
class _OrcCfg(C.Structure):
    _fields_ = [(n, C.c_int) for n in
                ("n_layer", "d_model", "n_head", "d_ff", "vocab", "ctx", "act", "pos", "value_head",
                 "sub_ln", "n_head_kv", "tie")]


class OracleGpt:
    """CPU restatement of the GPT decode path on a flat parameter buffer (same order as the engine's)."""

    def __init__(self, cfg, flat_params: np.ndarray):
        _ensure_built()
        L = C.CDLL(_SO)
        self.L = L
        self.cfg = cfg
        self._c = _OrcCfg(cfg.n_layer, cfg.d_model, cfg.n_head, cfg.d_ff, cfg.vocab, cfg.ctx, cfg.act, cfg.pos,
                          int(cfg.value_head), int(getattr(cfg, "sub_ln", False)),
                          int(getattr(cfg, "n_head_kv", 0)), int(getattr(cfg, "tie_embeddings", False)))
        L.orc_gpt_param_count.restype = _SZ
        L.orc_gpt_param_count.argtypes = [C.POINTER(_OrcCfg)]
        L.orc_gpt_create.restype = C.c_void_p
        L.orc_gpt_create.argtypes = [C.POINTER(_OrcCfg), _f32p]
        L.orc_gpt_destroy.argtypes = [C.c_void_p]
        L.orc_gpt_get_linear.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.orc_gpt_rollout.restype = C.c_int
        L.orc_gpt_rollout.argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int,
                                      C.c_uint64, C.c_uint32, _i32p, C.c_void_p, C.c_void_p]
        L.orc_gpt_step_logits.restype = C.c_int
        L.orc_gpt_step_logits.argtypes = [C.c_void_p, _i32p, C.c_int, _f32p]
        self.params = np.ascontiguousarray(flat_params, np.float32)  # keep alive: the model points into it
        assert self.params.size == L.orc_gpt_param_count(C.byref(self._c))
        self.h = L.orc_gpt_create(C.byref(self._c), self.params)

    def __del__(self):
        try:
            if self.h:
                self.L.orc_gpt_destroy(self.h)
                self.h = None
        except Exception:
            pass

    def param_count(self):
        return int(self.L.orc_gpt_param_count(C.byref(self._c)))

    def linear(self, layer, which, rows, cols):
        tau = np.empty(rows, np.float32)
        trit = np.empty((rows, cols), np.int8)
        self.L.orc_gpt_get_linear(self.h, layer, which, tau.ctypes.data, trit.ctypes.data)
        return tau, trit

    def rollout(self, prompts, max_new, temperature, top_k, seed, seq0=0, want_logits=False):
        prompts = np.ascontiguousarray(prompts, np.int32)
        B, P = prompts.shape
        tokens = np.empty((B, P + max_new), np.int32)
        logp = np.empty((B, max_new), np.float32)
        logits = np.empty((B, max_new, self.cfg.vocab), np.float32) if want_logits else None
        rc = self.L.orc_gpt_rollout(self.h, prompts, B, P, max_new, temperature, top_k, seed, seq0, tokens,
                                    logp.ctypes.data, logits.ctypes.data if logits is not None else None)
        assert rc == 0
        return tokens, logp, logits

    def rollout_cfg(self, prompts, max_new, temperature=1.0, top_k=0, top_p=1.0, repeat_penalty=1.0, repeat_window=0,
                    bias=None, eos=-1, min_new=0, seed=0, seq0=0):
        prompts = np.ascontiguousarray(prompts, np.int32)
        B, P = prompts.shape
        L = self.L
        L.orc_gpt_rollout_cfg.restype = C.c_int
        L.orc_gpt_rollout_cfg.argtypes = [C.c_void_p, _i32p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float,
                                          C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_uint64, C.c_uint32, _i32p, _f32p, _i32p]
        tokens = np.empty((B, P + max_new), np.int32)
        logp = np.empty((B, max_new), np.float32)
        glen = np.empty(B, np.int32)
        b = np.ascontiguousarray(bias, np.float32) if bias is not None else None
        rc = L.orc_gpt_rollout_cfg(self.h, prompts, B, P, max_new, temperature, top_k, top_p, repeat_penalty, repeat_window,
                                   b.ctypes.data if b is not None else None, eos, min_new, seed, seq0, tokens, logp, glen)
        assert rc == 0
        return tokens, logp, glen

    def step_logits(self, tokens):
        tokens = np.ascontiguousarray(tokens, np.int32)
        out = np.empty((len(tokens), self.cfg.vocab), np.float32)
        assert self.L.orc_gpt_step_logits(self.h, tokens, len(tokens), out) == 0
        return out


def _bind_extra(L):
    L.orc_expf.restype = C.c_float
    L.orc_expf.argtypes = [C.c_float]
    L.orc_philox_uniform.restype = C.c_float
    L.orc_philox_uniform.argtypes = [C.c_uint64, C.c_uint32, C.c_uint32]
    L.orc_sample_token.restype = C.c_int
    L.orc_sample_token.argtypes = [_f32p, C.c_int, C.c_float, C.c_int, C.c_float]
    L.orc_rmsnorm.argtypes = [_f32p, _f32p, C.c_int, C.c_float, _f32p]
    L.orc_logprob_entropy.argtypes = [_f32p, C.c_int, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float)]


def _oracle_extra(self):
    _bind_extra(self.L)


def _expf(self, x):
    return float(self.L.orc_expf(x))


def _philox(self, seed, seq, step):
    return float(self.L.orc_philox_uniform(seed, seq, step))


def _sample(self, logits, temperature, top_k, r):
    work = np.ascontiguousarray(logits, np.float32).copy()
    return int(self.L.orc_sample_token(work, len(work), temperature, top_k, r))


def _rmsnorm(self, x, gamma, eps=1e-5):
    x = _c(x, np.float32)
    out = np.empty_like(x)
    self.L.orc_rmsnorm(x, _c(gamma, np.float32), len(x), eps, out)
    return out


def _logprob_entropy(self, logits, token):
    lp, h = C.c_float(), C.c_float()
    self.L.orc_logprob_entropy(_c(logits, np.float32), len(logits), token, C.byref(lp), C.byref(h))
    return lp.value, h.value


_orig_init = Oracle.__init__


def _init(self):
    _orig_init(self)
    _bind_extra(self.L)


Oracle.__init__ = _init
Oracle.expf = _expf
Oracle.philox_uniform = _philox
def _sample_cfg(self, logits, temperature=1.0, top_k=0, top_p=1.0, repeat_penalty=1.0, repeat_window=0, bias=None,
                history=(), r=0.5):
    work = np.ascontiguousarray(logits, np.float32).copy()
    hist = np.ascontiguousarray(history, np.int32)
    self.L.orc_sample_token_cfg.restype = C.c_int
    self.L.orc_sample_token_cfg.argtypes = [_f32p, C.c_int, C.c_float, C.c_int, C.c_float, C.c_float, C.c_int, C.c_void_p,
                                            _i32p, C.c_int, C.c_float]
    b = np.ascontiguousarray(bias, np.float32) if bias is not None else None
    return int(self.L.orc_sample_token_cfg(work, len(work), temperature, top_k, top_p, repeat_penalty, repeat_window,
                                           b.ctypes.data if b is not None else None, hist, len(hist), r))


Oracle.sample_token = _sample
Oracle.sample_token_cfg = _sample_cfg
Oracle.rmsnorm = _rmsnorm
Oracle.logprob_entropy = _logprob_entropy


# ------------------------------------------------------------------ RL (oracle_rl.c)
class _PolicyMetrics(C.Structure):
    _fields_ = [("loss", C.c_float), ("ratio_mean", C.c_float), ("approx_kl", C.c_float),
                ("clip_fraction", C.c_float)]


def _opt(a):
    return None if a is None else _c(a, np.float32).ctypes.data_as(C.c_void_p)


class OracleRL:
    def __init__(self):
        _ensure_built()
        L = C.CDLL(_SO)
        self.L = L
        vp = C.c_void_p
        L.orc_gae.argtypes = [_f32p, _f32p, vp, vp, vp, _SZ, _SZ, C.c_float, C.c_float, _f32p, _f32p]
        L.orc_masked_normalize.argtypes = [_f32p, vp, _SZ, C.c_float, _f32p]
        L.orc_group_advantage.restype = C.c_int
        L.orc_group_advantage.argtypes = [_f32p, _SZ, _i32p, _i32p, _SZ, C.c_float, _f32p]
        L.orc_categorical_logp_entropy.argtypes = [_f32p, _i32p, _SZ, _SZ, _f32p, _f32p]
        L.orc_categorical_backward.argtypes = [_f32p, _i32p, vp, vp, _SZ, _SZ, _f32p]
        L.orc_clipped_policy.argtypes = [_f32p, _f32p, _f32p, _f32p, _SZ, C.c_float, _f32p, C.POINTER(_PolicyMetrics)]
        L.orc_entropy_bonus.restype = C.c_float
        L.orc_entropy_bonus.argtypes = [_f32p, _f32p, _SZ, C.c_float, _f32p]
        L.orc_sampled_kl.restype = C.c_float
        L.orc_sampled_kl.argtypes = [_f32p, _f32p, _f32p, _SZ, C.c_float, _f32p]
        L.orc_mc_return.argtypes = [_f32p, vp, vp, _SZ, _SZ, C.c_float, _f32p]
        L.orc_value_regression.restype = C.c_float
        L.orc_value_regression.argtypes = [_f32p, _f32p, _f32p, _SZ, C.c_float, _f32p]
        L.orc_clipped_value.restype = C.c_float
        L.orc_clipped_value.argtypes = [_f32p, _f32p, _f32p, _f32p, _SZ, C.c_float, C.c_float, _f32p,
                                        C.POINTER(C.c_float)]
        L.orc_clip_grad_norm.restype = C.c_float
        L.orc_clip_grad_norm.argtypes = [_f32p, _SZ, C.c_float]
        L.orc_adamw.argtypes = [_f32p, _f32p, _f32p, _f32p, _SZ, C.c_float, C.c_float, C.c_float, C.c_float,
                                C.c_float, C.c_int]

    def gae(self, rewards, values, done=None, mask=None, bootstrap=None, gamma=0.99, lam=0.95):
        r = _c(rewards, np.float32)
        steps, batch = r.shape
        adv, ret = np.empty_like(r), np.empty_like(r)
        keep = [_c(x, np.float32) if x is not None else None for x in (done, mask, bootstrap)]
        ptr = [k.ctypes.data_as(C.c_void_p) if k is not None else None for k in keep]
        self.L.orc_gae(r, _c(values, np.float32), ptr[0], ptr[1], ptr[2], steps, batch, gamma, lam, adv, ret)
        return adv, ret

    def masked_normalize(self, values, mask=None, eps=1e-8):
        v = _c(values, np.float32)
        out = np.empty_like(v)
        m = _c(mask, np.float32) if mask is not None else None
        self.L.orc_masked_normalize(v.ravel(), m.ctypes.data_as(C.c_void_p) if m is not None else None, v.size, eps,
                                    out.ravel())
        return out

    def group_advantage(self, returns, spans, eps=1e-8):
        r = _c(returns, np.float32)
        out = np.empty_like(r)
        first = np.ascontiguousarray([s[0] for s in spans], np.int32)
        count = np.ascontiguousarray([s[1] for s in spans], np.int32)
        rc = self.L.orc_group_advantage(r, r.size, first, count, len(spans), eps, out)
        return out if rc == 0 else None

    def categorical_logp_entropy(self, logits, actions):
        lg = _c(logits, np.float32)
        t, v = lg.shape
        logp, ent = np.empty(t, np.float32), np.empty(t, np.float32)
        self.L.orc_categorical_logp_entropy(lg, _c(actions, np.int32), t, v, logp, ent)
        return logp, ent

    def categorical_backward(self, logits, actions, up_lp=None, up_ent=None):
        lg = _c(logits, np.float32)
        t, v = lg.shape
        out = np.empty_like(lg)
        a = _c(up_lp, np.float32) if up_lp is not None else None
        b = _c(up_ent, np.float32) if up_ent is not None else None
        self.L.orc_categorical_backward(lg, _c(actions, np.int32), a.ctypes.data_as(C.c_void_p) if a is not None else None,
                                        b.ctypes.data_as(C.c_void_p) if b is not None else None, t, v, out)
        return out

    def clipped_policy(self, logp, old_logp, adv, mask, clip_eps=0.2):
        n = len(logp)
        up = np.empty(n, np.float32)
        m = _PolicyMetrics()
        self.L.orc_clipped_policy(_c(logp, np.float32), _c(old_logp, np.float32), _c(adv, np.float32),
                                  _c(mask, np.float32), n, clip_eps, up, C.byref(m))
        return up, dict(loss=m.loss, ratio_mean=m.ratio_mean, approx_kl=m.approx_kl, clip_fraction=m.clip_fraction)

    def entropy_bonus(self, entropy, mask, coef):
        n = len(entropy)
        up = np.empty(n, np.float32)
        loss = self.L.orc_entropy_bonus(_c(entropy, np.float32), _c(mask, np.float32), n, coef, up)
        return float(loss), up

    def sampled_kl(self, logp, ref, mask, coef):
        n = len(logp)
        up = np.empty(n, np.float32)
        loss = self.L.orc_sampled_kl(_c(logp, np.float32), _c(ref, np.float32), _c(mask, np.float32), n, coef, up)
        return float(loss), up

    def clipped_value(self, value, returns, old_value, mask, clip_eps=0.2, coef=1.0):
        n = len(value)
        grad = np.empty(n, np.float32)
        cf = C.c_float()
        loss = self.L.orc_clipped_value(_c(value, np.float32), _c(returns, np.float32), _c(old_value, np.float32),
                                        _c(mask, np.float32), n, clip_eps, coef, grad, C.byref(cf))
        return float(loss), grad, cf.value

    def value_regression(self, value, returns, mask, coef=1.0):
        n = len(value)
        grad = np.empty(n, np.float32)
        loss = self.L.orc_value_regression(_c(value, np.float32), _c(returns, np.float32), _c(mask, np.float32), n, coef, grad)
        return float(loss), grad

    def mc_return(self, rewards, done=None, mask=None, gamma=0.99):
        r = _c(rewards, np.float32)
        steps, batch = r.shape
        out = np.empty_like(r)
        keep = [_c(x, np.float32) if x is not None else None for x in (done, mask)]
        ptr = [k.ctypes.data_as(C.c_void_p) if k is not None else None for k in keep]
        self.L.orc_mc_return(r, ptr[0], ptr[1], steps, batch, gamma, out)
        return out

    def clip_grad_norm(self, g, max_norm):
        g = np.ascontiguousarray(g, np.float32).copy()
        norm = self.L.orc_clip_grad_norm(g, g.size, max_norm)
        return g, float(norm)

    def adamw(self, p, g, m, v, lr, t, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.01):
        p, m, v = (np.ascontiguousarray(x, np.float32).copy() for x in (p, m, v))
        self.L.orc_adamw(p, _c(g, np.float32), m, v, p.size, lr, beta1, beta2, eps, wd, t)
        return p, m, v
