"""Policy: host-side handle of the ternary GPT policy inside libnn-b200.so.

Mirrors what a consumer of the reference does with build_gpt_model(engine, GptConfig)
(include/neuralnet.cpp/domain_gpt.hpp:33-77) plus GPTModel::generate
(include/neuralnet.cpp/compute_layer_gpt.hpp:740-852), batched over sequences.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from ._lib import NnbError, check, lib
from .engine import Engine, _ptr

GELU, SWIGLU, RELU2 = 0, 1, 2
LEARNED, ROPE = 0, 1


class _CConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("n_layer", "d_model", "n_head", "d_ff", "vocab", "ctx", "act", "pos", "value_head", "exact",
                 "sub_ln", "n_head_kv", "tie_embeddings")]


@dataclass
class GptConfig:
    n_layer: int
    d_model: int
    n_head: int
    d_ff: int
    vocab: int
    ctx: int
    act: int = GELU
    pos: int = LEARNED
    value_head: bool = False
    exact: bool = True
    sub_ln: bool = False          # RMSNorm between the heads' output and the o projection, and before fc2
    n_head_kv: int = 0            # grouped-query attention: KV heads (0 = n_head); query head h reads h // (H / Hkv)
    tie_embeddings: bool = False  # logits = tok_emb . ln_f(x): a dense head without bias, no lm_head tensors

    @property
    def kv_heads(self) -> int:
        return self.n_head_kv if self.n_head_kv > 0 else self.n_head

    def to_c(self) -> _CConfig:
        return _CConfig(self.n_layer, self.d_model, self.n_head, self.d_ff, self.vocab, self.ctx,
                        self.act, self.pos, int(self.value_head), int(self.exact),
                        int(self.sub_ln), int(self.n_head_kv), int(self.tie_embeddings))

    def param_layout(self):
        """(name, offset, shape) of every tensor in the flat parameter buffer, in order."""
        d, F, V = self.d_model, self.d_ff, self.vocab
        F1 = 2 * F if self.act in (SWIGLU, RELU2) else F
        dkv = self.kv_heads * (d // self.n_head)
        out, o = [], 0

        def add(name, *shape):
            nonlocal o
            out.append((name, o, shape))
            o += int(np.prod(shape))

        add("tok_emb", V, d)
        if self.pos == LEARNED:
            add("pos_emb", self.ctx, d)
        for l in range(self.n_layer):
            p = f"blocks.{l}."
            add(p + "ln1.gamma", d)
            add(p + "attn.q.weight", d, d); add(p + "attn.k.weight", dkv, d); add(p + "attn.v.weight", dkv, d)
            add(p + "attn.q.bias", d); add(p + "attn.k.bias", dkv); add(p + "attn.v.bias", dkv)
            if self.sub_ln:
                add(p + "attn.sub_norm.gamma", d)
            add(p + "attn.o.weight", d, d); add(p + "attn.o.bias", d)
            add(p + "ln2.gamma", d)
            add(p + "ffn.fc1.weight", F1, d); add(p + "ffn.fc1.bias", F1)
            if self.sub_ln:
                add(p + "ffn.sub_norm.gamma", F)
            add(p + "ffn.fc2.weight", d, F); add(p + "ffn.fc2.bias", d)
        add("ln_f.gamma", d)
        if not self.tie_embeddings:
            add("lm_head.weight", V, d); add("lm_head.bias", V)
        if self.value_head:
            add("value_head.weight", 1, d); add("value_head.bias", 1)
        return out, o

    def init_params(self, seed: int, linear_std: float = 0.02, bias_std: float = 0.0) -> np.ndarray:
        """Seeded synthetic initialisation: linears N(0, linear_std) (absmean-quantised by the engine),
        embeddings N(0, 0.02), norm gains 1, biases N(0, bias_std) (0 = zeros, the reference default)."""
        layout, n = self.param_layout()
        rng = np.random.default_rng(seed)
        flat = np.zeros(n, np.float32)
        for name, off, shape in layout:
            size = int(np.prod(shape))
            if name.endswith("gamma"):
                v = np.ones(size, np.float32)
            elif name.endswith(".bias"):
                v = rng.normal(0, bias_std, size).astype(np.float32) if bias_std > 0 else np.zeros(size, np.float32)
            elif name in ("tok_emb", "pos_emb"):
                v = rng.normal(0, 0.02, size).astype(np.float32)
            else:
                v = rng.normal(0, linear_std, size).astype(np.float32)
            flat[off:off + size] = v
        return flat


class Policy:
    def __init__(self, engine: Engine, cfg: GptConfig):
        self._lib = lib()
        self.engine = engine
        self.cfg = cfg
        h = C.c_void_p()
        cc = cfg.to_c()
        check(self._lib.nnb_policy_create(engine.handle, C.byref(cc), C.byref(h)))
        self._h = h
        self.n_params = int(self._lib.nnb_policy_param_count(self._h))

    def close(self):
        if getattr(self, "_h", None):
            self._lib.nnb_policy_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def handle(self):
        return self._h

    def tensors(self):
        out = []
        n = int(self._lib.nnb_policy_tensor_count(self._h))
        for i in range(n):
            name = C.create_string_buffer(128)
            off, rows, cols = C.c_size_t(), C.c_size_t(), C.c_size_t()
            check(self._lib.nnb_policy_tensor_info(self._h, i, name, 128, C.byref(off), C.byref(rows), C.byref(cols)))
            out.append((name.value.decode(), off.value, rows.value, cols.value))
        return out

    def params_view(self) -> torch.Tensor:
        """The flat f32 master parameters as a torch tensor aliasing the engine's buffer."""
        ptr = self._lib.nnb_policy_params(self._h)
        return _alias(ptr, self.n_params, torch.float32, self.engine.device)

    def upload_params(self, flat: np.ndarray):
        flat = np.ascontiguousarray(flat, np.float32)
        if flat.size != self.n_params:
            raise NnbError(f"expected {self.n_params} parameters, got {flat.size}")
        check(self._lib.nnb_policy_upload_params(self._h, flat.ctypes.data_as(C.c_void_p)))

    def requantize(self):
        check(self._lib.nnb_policy_requantize(self._h))

    def linear(self, layer: int, which: int):
        pk, tau = C.c_void_p(), C.c_void_p()
        i, o = C.c_size_t(), C.c_size_t()
        check(self._lib.nnb_policy_linear(self._h, layer, which, C.byref(pk), C.byref(tau), C.byref(i), C.byref(o)))
        packed = _alias(pk.value, o.value * (i.value // 16), torch.int32, self.engine.device).view(o.value, i.value // 16)
        return packed, _alias(tau.value, o.value, torch.float32, self.engine.device)

    def rollout(self, prompts: torch.Tensor, max_new: int, temperature: float = 1.0, top_k: int = 0,
                seed: int = 0, seq0: int = 0, want_logp: bool = True, want_logits: bool = False,
                group_size: int = 1):
        """prompts (B, P) int32 on the device -> tokens (B, P+max_new) int32, logp (B, max_new), [logits].
        group_size > 1: every group_size consecutive rows of `prompts` are the same prompt; the shared
        prefix is decoded once per group."""
        B, P = prompts.shape
        dev = self.engine.device
        tokens = torch.empty((B, P + max_new), device=dev, dtype=torch.int32)
        logp = torch.empty((B, max_new), device=dev, dtype=torch.float32) if want_logp else None
        logits = torch.empty((B, max_new, self.cfg.vocab), device=dev, dtype=torch.float32) if want_logits else None
        check(self._lib.nnb_rollout_grouped(self._h, _ptr(prompts), B, P, max_new, int(group_size), float(temperature),
                                            int(top_k), C.c_uint64(seed), C.c_uint32(seq0), _ptr(tokens), _ptr(logp),
                                            _ptr(logits)))
        return tokens, logp, logits

    def rollout_host(self, h_prompts: torch.Tensor, max_new: int, temperature: float, top_k: int, seed: int,
                     seq0: int, h_tokens: torch.Tensor, h_logp: torch.Tensor | None):
        B, P = h_prompts.shape
        check(self._lib.nnb_rollout_host(self._h, C.c_void_p(h_prompts.data_ptr()), B, P, max_new,
                                         float(temperature), int(top_k), C.c_uint64(seed), C.c_uint32(seq0),
                                         C.c_void_p(h_tokens.data_ptr()),
                                         C.c_void_p(h_logp.data_ptr()) if h_logp is not None else None))
        return h_tokens, h_logp


def _alias(ptr: int, numel: int, dtype, device) -> torch.Tensor:
    """A torch tensor over engine-owned device memory (no copy, no ownership)."""
    itemsize = torch.empty((), dtype=dtype).element_size()

    class _Iface:
        pass

    holder = _Iface()
    typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.int8: "|i1"}[dtype]
    holder.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (int(ptr), False),
                                       "version": 2, "strides": (itemsize,)}
    return torch.as_tensor(holder, device=device)


class _CSampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("repeat_penalty", C.c_float),
                ("repeat_window", C.c_int32), ("seed", C.c_uint64), ("d_logit_bias", C.c_void_p), ("eos_token", C.c_int32),
                ("min_new_tokens", C.c_int32)]


@dataclass
class SamplingConfig:
    """SamplingConfig of the reference (compute_layer_base.hpp:1002-1022); logit_bias (vocab,) f32 on the device stands
    for its host hook logits_transform; eos_token / min_new_tokens are GPTModel::generate's arguments."""
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repeat_penalty: float = 1.0
    repeat_window: int = 0
    seed: int = 0
    logit_bias: torch.Tensor | None = None
    eos_token: int = -1
    min_new_tokens: int = 0


def rollout_sampled(self, prompts: torch.Tensor, max_new: int, cfg: SamplingConfig, seq0: int = 0, group_size: int = 1,
                    want_logits: bool = False):
    """Batched generate with the full sampling configuration -> tokens (B, P+max_new), logp (B, max_new),
    gen_len (B,) tokens generated before the end-of-sequence token, [logits]."""
    B, P = prompts.shape
    dev = self.engine.device
    tokens = torch.empty((B, P + max_new), device=dev, dtype=torch.int32)
    logp = torch.empty((B, max_new), device=dev, dtype=torch.float32)
    glen = torch.empty((B,), device=dev, dtype=torch.int32)
    logits = torch.empty((B, max_new, self.cfg.vocab), device=dev, dtype=torch.float32) if want_logits else None
    cc = _CSampling(cfg.temperature, cfg.top_k, cfg.top_p, cfg.repeat_penalty, cfg.repeat_window, cfg.seed,
                    None if cfg.logit_bias is None else cfg.logit_bias.data_ptr(), cfg.eos_token, cfg.min_new_tokens)
    check(self._lib.nnb_rollout_sampled(self._h, _ptr(prompts), B, P, max_new, int(group_size), C.byref(cc), C.c_uint32(seq0),
                                        _ptr(tokens), _ptr(logp), _ptr(logits), _ptr(glen)))
    return tokens, logp, glen, logits


class _CObjective(C.Structure):
    _fields_ = [("d_mask", C.c_void_p), ("d_old_logp", C.c_void_p), ("d_advantage", C.c_void_p),
                ("d_ref_logp", C.c_void_p), ("d_returns", C.c_void_p), ("d_old_value", C.c_void_p),
                ("units", C.c_float), ("clip_eps", C.c_float), ("kl_coef", C.c_float), ("entropy_coef", C.c_float),
                ("value_coef", C.c_float), ("value_clip_eps", C.c_float)]


def _dp(t):
    return None if t is None else t.data_ptr()


def logprobs(self, tokens: torch.Tensor, prompt_len: int, want_entropy=False, want_value=False, group_size=1):
    """Teacher-forced log-probs (and entropy / values) of the decisions of tokens (n, S) int32.  group_size > 1:
    every group_size consecutive sequences share their prompt, which is then computed once per group."""
    n, S = tokens.shape
    G = S - prompt_len
    dev = self.engine.device
    logp = torch.empty((n, G), device=dev, dtype=torch.float32)
    ent = torch.empty((n, G), device=dev, dtype=torch.float32) if want_entropy else None
    val = torch.empty((n, G), device=dev, dtype=torch.float32) if want_value else None
    check(self._lib.nnb_policy_logprobs_grouped(self._h, _ptr(tokens), n, S, prompt_len, group_size, _ptr(logp), _ptr(ent),
                                                _ptr(val)))
    return logp, ent, val


def grads_view(self) -> torch.Tensor:
    ptr = self._lib.nnb_policy_grads(self._h)
    if not ptr:
        raise NnbError("out of device memory for the gradient buffer")
    return _alias(ptr, self.n_params, torch.float32, self.engine.device)


def zero_grad(self):
    check(self._lib.nnb_policy_zero_grad(self._h))


def train_step(self, tokens: torch.Tensor, prompt_len: int, mask, old_logp=None, advantage=None, ref_logp=None,
               returns=None, old_value=None, units=0.0, clip_eps=0.2, kl_coef=0.0, entropy_coef=0.0,
               value_coef=0.0, value_clip_eps=0.2, group_size=1):
    """One micro-batch: forward, objective, backward; gradients accumulate.  Returns report[10] (device).
    group_size > 1: every group_size consecutive sequences share their prompt (computed once per group)."""
    n, S = tokens.shape
    obj = _CObjective(_dp(mask), _dp(old_logp), _dp(advantage), _dp(ref_logp), _dp(returns), _dp(old_value),
                      units, clip_eps, kl_coef, entropy_coef, value_coef, value_clip_eps)
    report = torch.empty(10, device=self.engine.device, dtype=torch.float32)
    check(self._lib.nnb_policy_train_step_grouped(self._h, _ptr(tokens), n, S, prompt_len, group_size, C.byref(obj),
                                                  _ptr(report)))
    return report


def sft_step(self, tokens: torch.Tensor, prompt_len: int, mask, units=0.0, group_size=1):
    """Sparse cross-entropy of the next token on one micro-batch; gradients accumulate.  Returns report[10]
    (loss in [0], units in [7])."""
    n, S = tokens.shape
    report = torch.empty(10, device=self.engine.device, dtype=torch.float32)
    check(self._lib.nnb_policy_sft_step(self._h, _ptr(tokens), n, S, prompt_len, group_size, _ptr(mask), units, _ptr(report)))
    return report


def cached_activation(self, layer: int, which: int):
    """(q int8 (rows, cols) in the engine's K-permuted layout, s f32 (rows)) kept by the last training micro-batch for
    layer `layer`: which 0 = input of q|k|v, 1 = input of o, 2 = input of fc1, 3 = input of fc2."""
    rows, cols = C.c_size_t(), C.c_size_t()
    check(self._lib.nnb_policy_cached_activation(self._h, layer, which, None, None, C.byref(rows), C.byref(cols)))
    q = torch.empty((rows.value, cols.value), device=self.engine.device, dtype=torch.int8)
    s = torch.empty(rows.value, device=self.engine.device, dtype=torch.float32)
    check(self._lib.nnb_policy_cached_activation(self._h, layer, which, _ptr(q), _ptr(s), None, None))
    return q, s


def optimizer_step(self, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, max_grad_norm=0.0):
    norm = torch.empty(1, device=self.engine.device, dtype=torch.float32)
    check(self._lib.nnb_policy_optimizer_step(self._h, lr, beta1, beta2, eps, weight_decay, max_grad_norm, _ptr(norm)))
    return norm


def set_step_timing(self, stride: int):
    """Record a CUDA event every `stride` decode steps of the following rollouts (0 = off)."""
    check(self._lib.nnb_rollout_set_step_timing(self._h, int(stride)))


def step_times(self):
    """(ms, pos) arrays of the last rollout's timed segments: device time of each run of `stride` decode steps and
    the position its first step consumed."""
    n = C.c_size_t()
    check(self._lib.nnb_rollout_step_times(self._h, None, None, 0, C.byref(n)))
    ms = np.zeros(n.value, np.float32)
    pos = np.zeros(n.value, np.int32)
    if n.value:
        check(self._lib.nnb_rollout_step_times(self._h, ms.ctypes.data_as(C.c_void_p), pos.ctypes.data_as(C.c_void_p), n.value,
                                               C.byref(n)))
    return ms, pos


def save(self, path: str, role: str = "model"):
    """Write the policy as a model file: role "model" (ternary weights packed base-3 + tau) or "checkpoint" (f32 latent)."""
    check(self._lib.nnb_policy_save(self._h, str(path).encode(), {"model": 0, "checkpoint": 1}[role]))


def load(self, path: str):
    """Read a model file of either role into this policy (same architecture); a model-role file comes back trainable
    with bit-identical packed weights."""
    check(self._lib.nnb_policy_load(self._h, str(path).encode()))


def release_workspaces(self):
    check(self._lib.nnb_policy_release_workspaces(self._h))


for _f in (save, load, rollout_sampled, logprobs, grads_view, zero_grad, train_step, sft_step, optimizer_step, release_workspaces, set_step_timing,
           step_times, cached_activation):
    setattr(Policy, _f.__name__, _f)
