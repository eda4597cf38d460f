"""Engine: the reference's ComputeEngine operator names over the C-ABI, on torch device tensors.

torch is plumbing only (device memory, streams); every operator below is one call into
libnn-b200.so.  Names, argument meaning and layouts follow the reference's call sites in
include/neuralnet.cpp/compute_layer_bitlinear.hpp (trit_pack :650, quantize_i8 :447,
matmul_q_i8 :454, matmul_q :464, matmul_q_t :494, unpack_i8 :516).
"""
from __future__ import annotations

import ctypes as C

import torch

from ._lib import NnbError, check, lib

F32, BF16 = 0, 1


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise NnbError(f"unsupported activation dtype {t.dtype}")


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda or not t.is_contiguous():
        raise NnbError("operands must be contiguous CUDA tensors")
    return C.c_void_p(t.data_ptr())


class Engine:
    """One engine per device and per thread (the reference's threading contract,
    docs/usage/07-thread-safety.md:11-17)."""

    def __init__(self, device: int = 0, use_torch_stream: bool = True):
        self._lib = lib()
        if not torch.cuda.is_available():
            raise NnbError("no CUDA device: the nn-b200 engine needs a B200 and has no CPU fallback")
        h = C.c_void_p()
        check(self._lib.nnb_engine_create(device, C.byref(h)))
        self._h = h
        self.device = torch.device("cuda", device)
        if use_torch_stream:
            # launch on torch's current stream so torch allocations, copies and events order with us
            s = torch.cuda.current_stream(self.device)
            check(self._lib.nnb_engine_set_stream(self._h, C.c_void_p(s.cuda_stream)))

    def close(self):
        if getattr(self, "_h", None):
            self._lib.nnb_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def describe(self) -> str:
        buf = C.create_string_buffer(512)
        check(self._lib.nnb_engine_describe(self._h, buf, 512))
        return buf.value.decode()

    def sync(self):
        check(self._lib.nnb_engine_sync(self._h))

    def set_stream(self, stream: "torch.cuda.Stream | None"):
        ptr = C.c_void_p(stream.cuda_stream) if stream is not None else C.c_void_p(-1)  # -1: the engine's own
        check(self._lib.nnb_engine_set_stream(self._h, ptr))

    def launch_count(self) -> int:
        return int(self._lib.nnb_engine_launch_count(self._h))

    # ------------------------------------------------------------ reference layout
    def absmean_tau(self, latent: torch.Tensor) -> torch.Tensor:
        rows, k = latent.shape
        tau = torch.empty(rows, device=self.device, dtype=torch.float32)
        check(self._lib.nnb_absmean_tau(self._h, _ptr(latent), rows, k, _ptr(tau)))
        return tau

    def trit_pack(self, latent: torch.Tensor, tau: torch.Tensor) -> torch.Tensor:
        """(rows,K) f32 + (rows) -> (rows, ceil(K/16)) int32 words (bit pattern of the uint32 codes)."""
        rows, k = latent.shape
        packed = torch.empty((rows, (k + 15) // 16), device=self.device, dtype=torch.int32)
        check(self._lib.nnb_trit_pack(self._h, _ptr(latent), _ptr(tau), rows, k, _ptr(packed)))
        return packed

    def col_absmax_scale(self, x: torch.Tensor) -> torch.Tensor:
        k, n = x.shape
        s = torch.empty(n, device=self.device, dtype=torch.float32)
        check(self._lib.nnb_col_absmax_scale(self._h, _ptr(x), k, n, _ptr(s)))
        return s

    def quantize_i8(self, x: torch.Tensor, scale: torch.Tensor, col_scale: bool = True) -> torch.Tensor:
        m, n = x.shape
        out = torch.empty((m, (n + 3) // 4), device=self.device, dtype=torch.int32)
        check(self._lib.nnb_quantize_i8(self._h, _ptr(x), m, n, _ptr(scale), int(col_scale), _ptr(out)))
        return out

    def unpack_i8(self, packed: torch.Tensor, cols: int) -> torch.Tensor:
        m = packed.shape[0]
        out = torch.empty((m, cols), device=self.device, dtype=torch.float32)
        check(self._lib.nnb_unpack_i8(self._h, _ptr(packed), m, cols, _ptr(out)))
        return out

    def matmul_q_i8(self, wq, tau, xq, s, k: int, n: int, want_acc: bool = False):
        rows = wq.shape[0]
        y = torch.empty((rows, n), device=self.device, dtype=torch.float32)
        acc = torch.empty((rows, n), device=self.device, dtype=torch.int32) if want_acc else None
        check(self._lib.nnb_matmul_q_i8(self._h, _ptr(wq), _ptr(tau), _ptr(xq), _ptr(s), rows, k, n,
                                        _ptr(y), _ptr(acc)))
        return (y, acc) if want_acc else y

    def matmul_q(self, wq, tau, x, k: int) -> torch.Tensor:
        rows = wq.shape[0]
        n = x.shape[1]
        c = torch.empty((rows, n), device=self.device, dtype=torch.float32)
        check(self._lib.nnb_matmul_q(self._h, _ptr(wq), _ptr(tau), _ptr(x), rows, k, n, _ptr(c)))
        return c

    def matmul_q_t(self, wq, tau, b, mcols: int) -> torch.Tensor:
        rows = wq.shape[0]
        n = b.shape[1]
        c = torch.empty((mcols, n), device=self.device, dtype=torch.float32)
        check(self._lib.nnb_matmul_q_t(self._h, _ptr(wq), _ptr(tau), _ptr(b), rows, mcols, n, _ptr(c)))
        return c

    # ------------------------------------------------------------------ token-major
    def act_quant_tm(self, x: torch.Tensor):
        """x (T,K) f32/bf16 -> (q private layout (T,K) int8, s (T) f32, qsum (T) int32)."""
        t, k = x.shape
        q = torch.empty((t, k), device=self.device, dtype=torch.int8)
        s = torch.empty(t, device=self.device, dtype=torch.float32)
        qsum = torch.empty(t, device=self.device, dtype=torch.int32)
        check(self._lib.nnb_act_quant_tm(self._h, _ptr(x), _dt(x), t, k, _ptr(q), _ptr(s), _ptr(qsum)))
        return q, s, qsum

    def actq_to_plain(self, q: torch.Tensor) -> torch.Tensor:
        t, k = q.shape
        out = torch.empty_like(q)
        check(self._lib.nnb_actq_to_plain(self._h, _ptr(q), t, k, _ptr(out)))
        return out

    def bitlinear_fwd_tm(self, wq, tau, bias, q, s, qsum, out_dtype=torch.float32, want_acc=False,
                         y=None):
        t, k = q.shape
        out = wq.shape[0]
        if y is None:
            y = torch.empty((t, out), device=self.device, dtype=out_dtype)
        acc = torch.empty((t, out), device=self.device, dtype=torch.int32) if want_acc else None
        check(self._lib.nnb_bitlinear_fwd_tm(self._h, _ptr(wq), _ptr(tau), _ptr(bias), _ptr(q), _ptr(s),
                                             _ptr(qsum), t, k, out, _ptr(y), _dt(y), _ptr(acc)))
        return (y, acc) if want_acc else y

    def bitlinear_fwd_tm_stack(self, wq, tau, bias, q, s, qsum, y):
        """wq (n_mats, out, K/16), tau/bias (n_mats, out), y (n_mats, T, out)."""
        n_mats, out, words = wq.shape
        t, k = q.shape
        check(self._lib.nnb_bitlinear_fwd_tm_stack(self._h, _ptr(wq), out * words, _ptr(tau), _ptr(bias),
                                                   _ptr(q), _ptr(s), _ptr(qsum), n_mats, t, k, out,
                                                   _ptr(y), t * out, _dt(y)))
        return y

    def bitlinear_fwd_host(self, wq, tau, bias, h_x: torch.Tensor, h_y: torch.Tensor):
        """h_x (T,K) f32 and h_y (T,out) f32 are HOST tensors (pinned for async copies)."""
        t, k = h_x.shape
        out = wq.shape[0]
        check(self._lib.nnb_bitlinear_fwd_host(self._h, _ptr(wq), _ptr(tau), _ptr(bias),
                                               C.c_void_p(h_x.data_ptr()), t, k, out,
                                               C.c_void_p(h_y.data_ptr())))
        return h_y


# ------------------------------------------------------------------ RL operators
def _f32(self, *shape):
    return torch.empty(shape, device=self.device, dtype=torch.float32)


def gae(self, rewards, values, done=None, mask=None, bootstrap=None, gamma=0.99, lam=0.95):
    """GaeAdvantage::apply — (steps, batch) tensors, row = time.  Returns (advantage, returns)."""
    steps, batch = rewards.shape
    adv, ret = _f32(self, steps, batch), _f32(self, steps, batch)
    check(self._lib.nnb_gae(self._h, _ptr(rewards), _ptr(values), _ptr(done), _ptr(mask), _ptr(bootstrap),
                            steps, batch, gamma, lam, _ptr(adv), _ptr(ret)))
    return adv, ret


def group_advantage(self, returns, spans, eps=1e-8):
    """GroupAdvantage::apply — returns (N,), spans = [(first_row, row_count), ...]."""
    import numpy as np

    first = np.ascontiguousarray([s[0] for s in spans], np.int32)
    count = np.ascontiguousarray([s[1] for s in spans], np.int32)
    out = _f32(self, returns.numel())
    check(self._lib.nnb_group_advantage(self._h, _ptr(returns), returns.numel(), first.ctypes.data_as(C.c_void_p),
                                        count.ctypes.data_as(C.c_void_p), len(spans), eps, _ptr(out)))
    return out


def masked_normalize(self, values, mask=None, eps=1e-8):
    out = torch.empty_like(values)
    check(self._lib.nnb_masked_normalize(self._h, _ptr(values), _ptr(mask), values.numel(), eps, _ptr(out)))
    return out


def categorical_logp_entropy(self, logits, actions):
    t, v = logits.shape
    logp, ent = _f32(self, t), _f32(self, t)
    check(self._lib.nnb_categorical_logp_entropy(self._h, _ptr(logits), _ptr(actions), t, v, _ptr(logp), _ptr(ent)))
    return logp, ent


def categorical_backward(self, logits, actions, up_logp=None, up_entropy=None):
    t, v = logits.shape
    out = torch.empty_like(logits)
    check(self._lib.nnb_categorical_backward(self._h, _ptr(logits), _ptr(actions), _ptr(up_logp), _ptr(up_entropy),
                                             t, v, _ptr(out)))
    return out


def token_objective(self, logp, mask, old_logp=None, advantage=None, ref_logp=None, entropy=None, units=0.0,
                    clip_eps=0.2, kl_coef=0.0, entropy_coef=0.0):
    """Clipped policy + sampled KL + entropy bonus.  Returns (up_logp, up_entropy, report[8])."""
    n = logp.numel()
    up_lp, up_ent, report = _f32(self, n), _f32(self, n), _f32(self, 8)
    check(self._lib.nnb_token_objective(self._h, _ptr(logp), _ptr(entropy), _ptr(old_logp), _ptr(ref_logp),
                                        _ptr(advantage), _ptr(mask), n, units, clip_eps, kl_coef, entropy_coef,
                                        _ptr(up_lp), _ptr(up_ent), _ptr(report)))
    return up_lp, up_ent, report


def clipped_value(self, value, returns, old_value, mask, units=0.0, clip_eps=0.2, coef=1.0):
    n = value.numel()
    grad, report = _f32(self, n), _f32(self, 2)
    check(self._lib.nnb_clipped_value(self._h, _ptr(value), _ptr(returns), _ptr(old_value), _ptr(mask), n, units,
                                      clip_eps, coef, _ptr(grad), _ptr(report)))
    return grad, report


def value_regression(self, value, returns, mask, units=0.0, coef=1.0):
    """ValueRegressionObjective — returns (grad, report[2] = loss, units)."""
    n = value.numel()
    grad, report = _f32(self, n), _f32(self, 2)
    check(self._lib.nnb_value_regression(self._h, _ptr(value), _ptr(returns), _ptr(mask), n, units, coef, _ptr(grad),
                                         _ptr(report)))
    return grad, report


def monte_carlo_return(self, rewards, done=None, mask=None, gamma=0.99):
    """MonteCarloReturn::apply — (steps, batch) tensors, row = time."""
    steps, batch = rewards.shape
    out = _f32(self, steps, batch)
    check(self._lib.nnb_monte_carlo_return(self._h, _ptr(rewards), _ptr(done), _ptr(mask), steps, batch, gamma, _ptr(out)))
    return out


def clip_grad_norm(self, grads, max_norm):
    norm = _f32(self, 1)
    check(self._lib.nnb_clip_grad_norm(self._h, _ptr(grads), grads.numel(), max_norm, _ptr(norm)))
    return norm


def scale_inplace(self, x, scale):
    check(self._lib.nnb_scale_inplace(self._h, _ptr(x), x.numel(), scale))
    return x


def adamw_step(self, params, grads, m, v, lr, t, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
    check(self._lib.nnb_adamw_step(self._h, _ptr(params), _ptr(grads), _ptr(m), _ptr(v), params.numel(), lr, beta1,
                                   beta2, eps, weight_decay, t))


for _f in (gae, group_advantage, masked_normalize, categorical_logp_entropy, categorical_backward,
           token_objective, clipped_value, value_regression, monte_carlo_return, clip_grad_norm, scale_inplace,
           adamw_step):
    setattr(Engine, _f.__name__, _f)


def bitlinear_dx_tm(self, dy, wq, tau, k, dx=None, accumulate=False, exact=True):
    """dX (t,k) (+)= (dY (t,out) * tau) . trit (out,k) — matmul_q_t, token-major."""
    t, out = dy.shape
    if dx is None:
        dx = torch.empty((t, k), device=self.device, dtype=torch.float32)
    check(self._lib.nnb_bitlinear_dx_tm(self._h, _ptr(dy), _ptr(wq), _ptr(tau), t, k, out, _ptr(dx), int(accumulate),
                                        int(exact)))
    return dx


def bitlinear_dw_tm(self, dy, q, s, tau, dw, exact=True):
    """dW (out,k) += tau * ((dY * s)^T . q) — the STE weight gradient of the int8-activation path."""
    t, out = dy.shape
    k = q.shape[1]
    check(self._lib.nnb_bitlinear_dw_tm(self._h, _ptr(dy), _ptr(q), _ptr(s), _ptr(tau), t, k, out, _ptr(dw), int(exact)))
    return dw


Engine.bitlinear_dx_tm = bitlinear_dx_tm
Engine.bitlinear_dw_tm = bitlinear_dw_tm


def expand_weights(self, wq, k, want_bf16=True):
    """2-bit container (rows, k/16) -> (int8 trits in the engine's K permutation, bf16 trits)."""
    rows = wq.shape[0]
    w8 = torch.empty((rows, k), device=self.device, dtype=torch.int8)
    wb = torch.empty((rows, k), device=self.device, dtype=torch.bfloat16) if want_bf16 else None
    check(self._lib.nnb_expand_weights(self._h, _ptr(wq), rows, k, _ptr(w8), _ptr(wb)))
    return w8, wb


def bitlinear_fwd_tc(self, w8, tau, bias, q, s, residual=None, y=None):
    t, k = q.shape
    out = w8.shape[0]
    if y is None:
        y = torch.empty((t, out), device=self.device, dtype=torch.float32)
    check(self._lib.nnb_bitlinear_fwd_tc(self._h, _ptr(w8), _ptr(tau), _ptr(bias), _ptr(residual), _ptr(q), _ptr(s), t, k,
                                         out, _ptr(y)))
    return y


def lmhead_logprob_entropy(self, w8, tau, bias, q, s, actions, want_entropy=True):
    """LM head fused with log-prob / entropy: returns (logp, entropy, lse), each (t,)."""
    t, k = q.shape
    v = w8.shape[0]
    logp, lse = _f32(self, t), _f32(self, t)
    ent = _f32(self, t) if want_entropy else None
    check(self._lib.nnb_lmhead_logprob_entropy_fwd(self._h, _ptr(w8), _ptr(tau), _ptr(bias), _ptr(q), _ptr(s), _ptr(actions), t, k, v,
                                                   _ptr(logp), _ptr(ent), _ptr(lse)))
    return logp, ent, lse


def lmhead_logprob_entropy_backward(self, w8, tau, bias, q, s, actions, lse, ent, up_logp, up_entropy=None, dbias=None):
    """Returns (dyb (t, v) bf16 = d logits * tau, dbias (v) incremented by the column sums of d logits)."""
    t, k = q.shape
    v = w8.shape[0]
    dyb = torch.empty((t, v), device=self.device, dtype=torch.bfloat16)
    if dbias is None:
        dbias = torch.zeros(v, device=self.device, dtype=torch.float32)
    check(self._lib.nnb_lmhead_logprob_entropy_bwd(self._h, _ptr(w8), _ptr(tau), _ptr(bias), _ptr(q), _ptr(s), _ptr(actions), _ptr(lse),
                                                   _ptr(ent), _ptr(up_logp), _ptr(up_entropy), t, k, v, _ptr(dyb), _ptr(dbias)))
    return dyb, dbias


def set_tc_forward_tile(self, bn: int = 0):
    """Process-wide width of the tensor-core forward's output tile (64/128/192/256; 0 = automatic)."""
    check(self._lib.nnb_tc_set_forward_tile(int(bn)))


def bitlinear_bwd_tc(self, dy, tau, wb, q, s, k, want_dx=True, dw=None, dx=None, accumulate_dx=False, scratch=None,
                     prepared=False):
    """scratch = (dyb, xs) bf16 buffers to reuse; prepared=True runs only the GEMMs on scratch filled by an earlier call."""
    t, out = dy.shape
    if scratch is not None:
        dyb, xs = scratch
    else:
        dyb = torch.empty((t, out), device=self.device, dtype=torch.bfloat16)
        xs = torch.empty((t, k), device=self.device, dtype=torch.bfloat16) if dw is not None else None
    if prepared:
        dy = None
    if want_dx and dx is None:
        dx = torch.empty((t, k), device=self.device, dtype=torch.float32)
    check(self._lib.nnb_bitlinear_bwd_tc(self._h, _ptr(dy), _ptr(tau), _ptr(wb), _ptr(q), _ptr(s), t, k, out, _ptr(dyb),
                                         _ptr(xs), _ptr(dx) if want_dx else None, int(accumulate_dx), _ptr(dw)))
    return dx, dw


def check_device_errors(self):
    check(self._lib.nnb_engine_check(self._h))


Engine.expand_weights = expand_weights
Engine.set_tc_forward_tile = set_tc_forward_tile
Engine.bitlinear_fwd_tc = bitlinear_fwd_tc
Engine.bitlinear_bwd_tc = bitlinear_bwd_tc
Engine.check_device_errors = check_device_errors


def attention_fwd(self, q, k, v, n_seq, seq_len, n_head, exact=True):
    d = q.shape[1]
    out = torch.empty_like(q)
    lse = torch.empty((n_seq, n_head, seq_len), device=self.device, dtype=torch.float32)
    check(self._lib.nnb_attention_fwd(self._h, _ptr(q), _ptr(k), _ptr(v), n_seq, seq_len, n_head, d // n_head,
                                      int(exact), _ptr(out), _ptr(lse)))
    return out, lse


def attention_bwd(self, q, k, v, out, dout, lse, n_seq, seq_len, n_head, exact=True):
    d = q.shape[1]
    delta = torch.empty_like(lse)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    check(self._lib.nnb_attention_bwd(self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(dout), _ptr(lse), n_seq, seq_len,
                                      n_head, d // n_head, int(exact), _ptr(delta), _ptr(dq), _ptr(dk), _ptr(dv)))
    return dq, dk, dv


def attention_rope_fwd(self, q, k, v, rope_cos, rope_sin, n_seq, seq_len, n_head, exact=True):
    """Attention with RoPE inside: q, k un-rotated, tables (seq_len, dk/2)."""
    d = q.shape[1]
    out = torch.empty_like(q)
    lse = torch.empty((n_seq, n_head, seq_len), device=self.device, dtype=torch.float32)
    check(self._lib.nnb_attention_rope_fwd(self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(rope_cos), _ptr(rope_sin), n_seq, seq_len,
                                           n_head, d // n_head, int(exact), _ptr(out), _ptr(lse)))
    return out, lse


def attention_rope_bwd(self, q, k, v, rope_cos, rope_sin, out, dout, lse, n_seq, seq_len, n_head, exact=True):
    d = q.shape[1]
    delta = torch.empty_like(lse)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    check(self._lib.nnb_attention_rope_bwd(self._h, _ptr(q), _ptr(k), _ptr(v), _ptr(rope_cos), _ptr(rope_sin), _ptr(out),
                                           _ptr(dout), _ptr(lse), n_seq, seq_len, n_head, d // n_head, int(exact), _ptr(delta),
                                           _ptr(dq), _ptr(dk), _ptr(dv)))
    return dq, dk, dv


def attention_decode(self, qkv, kcache, vcache, pos, n_head, rope=None, prefix=None, group=1, exact=True, want_out=True,
                     want_q8=False):
    """One new token per sequence against the KV cache.  qkv (3, n_seq, d); caches (n_seq, H, ctx_alloc, dk) f32 (exact)
    or bf16; pos: int32 device tensor of one element; rope = (cos, sin); prefix = (kpre, vpre, pre_len)."""
    _, n_seq, d = qkv.shape
    dk = d // n_head
    ctx_alloc = kcache.shape[2]
    kpre, vpre, pre_len = prefix if prefix is not None else (None, None, 0)
    pre_alloc = kpre.shape[2] if kpre is not None else 0
    cos, sin = rope if rope is not None else (None, None)
    out = torch.empty((n_seq, d), device=self.device, dtype=torch.float32) if want_out else None
    q8 = torch.empty((n_seq, d), device=self.device, dtype=torch.int8) if want_q8 else None
    s = torch.empty((n_seq,), device=self.device, dtype=torch.float32) if want_q8 else None
    qsum = torch.empty((n_seq,), device=self.device, dtype=torch.int32) if want_q8 else None
    check(self._lib.nnb_attention_decode(self._h, _ptr(qkv), _ptr(kcache), _ptr(vcache), ctx_alloc, _ptr(kpre), _ptr(vpre),
                                         pre_len, pre_alloc, group, _ptr(cos), _ptr(sin), _ptr(pos), n_seq, n_head, dk,
                                         int(exact), _ptr(out), _ptr(q8), _ptr(s), _ptr(qsum)))
    return out, q8, s, qsum


Engine.attention_decode = attention_decode
Engine.attention_fwd = attention_fwd
Engine.attention_bwd = attention_bwd
Engine.attention_rope_fwd = attention_rope_fwd
Engine.attention_rope_bwd = attention_rope_bwd


for _f in (lmhead_logprob_entropy, lmhead_logprob_entropy_backward):
    setattr(Engine, _f.__name__, _f)
