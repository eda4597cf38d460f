"""Runs one kernel (or one phase) of the RL-step path a few times on its benchmark shape.

    python kernel_cases.py <case> [args]

Used for Nsight Compute captures and quick timing; every case prints its CUDA-event time.  Cases:
  fwd          int8 ternary forward GEMM (tcgen05), T=10240 K=2048 O=11264
  dx | dw      bf16 backward GEMMs (tcgen05) of the same linear
  gemv [M [K N]]  2-bit packed weight stream, M (16) tokens, stack of 64 matrices (K 2048 x N 11264)
  attn_decode  decode attention of 512 sequences x 16 heads x 128 at position 400, fused int8 output
  train [n]    reference log-probs + one training micro-batch of n (16) sequences x 640 on the 1B policy
  trainppo [n] one PPO micro-batch (clipped policy + value loss + entropy bonus) of n (64) sequences x 320 on the
               GPT-2-small-shaped policy with a value head (12 layers, d 768, 12 heads, MLP 3072, vocab 32000)
  rollout [B P new]   batched rollout on the 1B policy (default 512 16 24)
  rollout3b [B P new [layers]] batched rollout on the 3B-shaped decode policy (26 layers, d 3200, 32 heads of 100;
               default 128 16 48); `layers` cuts the depth (same kernels, less memory: for profiler captures)
  rollout2b4t [B P new [layers]] the same on the BitNet-b1.58-2B4T structure (30 layers, d 2560, 20 heads on 5 KV heads of
               128, SubLN, ReLU2GLU, tied embeddings, vocab 128256)
  lmhead [T]   LM head fused with log-prob / entropy, forward and backward, T (8192) decisions x d 2048 x vocab 32000
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from __graft_entry__ import load_package  # noqa: E402

MODEL_1B = dict(n_layer=24, d_model=2048, n_head=16, d_ff=5632, vocab=32000, ctx=640, act=1, pos=1)
MODEL_GPT2S = dict(n_layer=12, d_model=768, n_head=12, d_ff=3072, vocab=32000, ctx=512, act=0, pos=0, value_head=True)
MODEL_3B = dict(n_layer=26, d_model=3200, n_head=32, d_ff=8640, vocab=32002, ctx=2048, act=1, pos=1)
MODEL_2B4T = dict(n_layer=30, d_model=2560, n_head=20, n_head_kv=5, d_ff=6912, vocab=128256, ctx=2048, act=2, pos=1,
                  sub_ln=True, tie_embeddings=True)


def _rand_packed(dev, *shape):
    """Random 2-bit containers without the unused code 0 (trit + 2 in {1, 2, 3})."""
    w = torch.randint(-2**31, 2**31 - 1, shape, device=dev, dtype=torch.int64) & 0xFFFFFFFF
    lo, hi = w & 0x55555555, (w >> 1) & 0x55555555
    w = w | (((~(lo | hi)) & 0x55555555) << 1)
    return torch.where(w >= 2**31, w - 2**32, w).to(torch.int32).contiguous()


def _timed(name, fn, reps=4):
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    print(f"{name}: {a.elapsed_time(b) / reps * 1e3:.1f} us per call")


def _policy(pkg, eng, model=MODEL_1B):
    cfg = pkg.GptConfig(exact=False, **model)
    pol = pkg.Policy(eng, cfg)
    g = torch.Generator(device=eng.device)
    g.manual_seed(1)
    pv = pol.params_view()
    pv.normal_(0, 0.02, generator=g)
    for name, off, shape in cfg.param_layout()[0]:
        size = int(np.prod(shape))
        if name.endswith("gamma"):
            pv[off:off + size] = 1.0
        elif name.endswith(".bias"):
            pv[off:off + size] = 0.0
    pol.requantize()
    return cfg, pol, g


def main(argv):
    case = argv[1] if len(argv) > 1 else "fwd"
    pkg = load_package()
    eng = pkg.Engine(0)
    dev = eng.device
    if case in ("fwd", "dx", "dw"):
        T, k, out = 10240, 2048, 11264
        w8, wb = eng.expand_weights(_rand_packed(dev, out, k // 16), k)
        tau = torch.rand(out, device=dev) * 0.05 + 0.01
        q, s, _ = eng.act_quant_tm(torch.randn(T, k, device=dev))
        if case == "fwd":
            y = torch.empty(T, out, device=dev)
            _timed("int8 forward GEMM", lambda: eng.bitlinear_fwd_tc(w8, tau, None, q, s, y=y))
        else:
            dy = torch.randn(T, out, device=dev)
            dx = torch.empty(T, k, device=dev)
            dw = torch.zeros(out, k, device=dev)
            scratch = (torch.empty(T, out, device=dev, dtype=torch.bfloat16), torch.empty(T, k, device=dev, dtype=torch.bfloat16))
            eng.bitlinear_bwd_tc(dy, tau, wb, q, s, k, dx=dx, dw=dw, scratch=scratch)  # fills the bf16 operands
            if case == "dx":
                _timed("bf16 dX GEMM", lambda: eng.bitlinear_bwd_tc(dy, tau, wb, q, s, k, dx=dx, scratch=scratch, prepared=True))
            else:
                _timed("bf16 dW GEMM", lambda: eng.bitlinear_bwd_tc(dy, tau, wb, q, s, k, want_dx=False, dw=dw, scratch=scratch,
                                                                    prepared=True))
    elif case == "gemv":
        k, out, n = (int(argv[3]), int(argv[4]), 64) if len(argv) > 4 else (2048, 11264, 64)
        wst = _rand_packed(dev, n, out, k // 16)
        taus = torch.rand(n, out, device=dev) * 0.05 + 0.01
        m = int(argv[2]) if len(argv) > 2 else 16
        q, s, qs = eng.act_quant_tm(torch.randn(m, k, device=dev))
        ys = torch.empty(n, m, out, device=dev)
        _timed(f"packed GEMV stack, {m} token(s), K {k}, N {out}, {n * (k * out // 4 + 4 * out * (1 + m)) / 1e6:.0f} MB",
               lambda: eng.bitlinear_fwd_tm_stack(wst, taus, None, q, s, qs, ys), reps=10)
    elif case == "attn_decode":
        B, H, dk, ctx, pos = 512, 16, 128, 512, 400
        kc = torch.randn(B, H, ctx, dk, device=dev).to(torch.bfloat16)
        vc = torch.randn(B, H, ctx, dk, device=dev).to(torch.bfloat16)
        qkv = torch.randn(3, B, H * dk, device=dev)
        tpos = torch.tensor([pos], device=dev, dtype=torch.int32)
        half = dk // 2
        ang = torch.arange(ctx, device=dev)[:, None] * (10000.0 ** (-torch.arange(half, device=dev) / half))[None, :]
        rope = (torch.cos(ang).contiguous(), torch.sin(ang).contiguous())
        _timed("decode attention (fused int8 output)",
               lambda: eng.attention_decode(qkv, kc, vc, tpos, H, rope=rope, exact=False, want_out=False, want_q8=True))
    elif case == "train":
        n = int(argv[2]) if len(argv) > 2 else 16
        cfg, pol, g = _policy(pkg, eng)
        tokens = torch.randint(0, cfg.vocab, (n, 640), device=dev, dtype=torch.int32, generator=g)
        mask = torch.ones((n, 512), device=dev)
        adv = torch.randn((n, 512), device=dev, generator=g)
        lp, _, _ = pol.logprobs(tokens, 128)
        pol.zero_grad()
        pol.train_step(tokens, 128, mask, old_logp=lp, advantage=adv, ref_logp=lp, kl_coef=0.04)
        _timed("reference log-probs", lambda: pol.logprobs(tokens, 128), reps=2)
        _timed("training micro-batch", lambda: pol.train_step(tokens, 128, mask, old_logp=lp, advantage=adv, ref_logp=lp,
                                                              kl_coef=0.04), reps=2)
    elif case == "trainppo":
        n = int(argv[2]) if len(argv) > 2 else 64
        cfg, pol, g = _policy(pkg, eng, MODEL_GPT2S)
        tokens = torch.randint(0, cfg.vocab, (n, 320), device=dev, dtype=torch.int32, generator=g)
        mask = torch.ones((n, 256), device=dev)
        adv = torch.randn((n, 256), device=dev, generator=g)
        ret = torch.randn((n, 256), device=dev, generator=g)
        lp, _, val = pol.logprobs(tokens, 64, want_value=True)
        pol.zero_grad()
        step = lambda: pol.train_step(tokens, 64, mask, old_logp=lp, advantage=adv, returns=ret, old_value=val,  # noqa: E731
                                      entropy_coef=0.01, value_coef=0.5)
        step()
        _timed("PPO training micro-batch", step, reps=2)
    elif case == "rollout":
        B, P, new = (int(a) for a in argv[2:5]) if len(argv) > 4 else (512, 16, 24)
        cfg, pol, g = _policy(pkg, eng)
        prompts = torch.randint(0, cfg.vocab, (B, P), device=dev, dtype=torch.int32, generator=g)
        pol.set_step_timing(32)
        _timed(f"rollout {B} x ({P}+{new})", lambda: pol.rollout(prompts, new, temperature=0.8, top_k=50, seed=1), reps=1)
        ms, pos = pol.step_times()
        print("ms per step by position:", " ".join(f"{p}:{m / 32:.3f}" for m, p in zip(ms, pos)))
    elif case in ("rollout3b", "rollout2b4t"):
        B, P, new = (int(a) for a in argv[2:5]) if len(argv) > 4 else (128, 16, 48)
        base = MODEL_3B if case == "rollout3b" else MODEL_2B4T
        model = dict(base, n_layer=int(argv[5])) if len(argv) > 5 else base
        cfg, pol, g = _policy(pkg, eng, model)
        prompts = torch.randint(0, cfg.vocab, (B, P), device=dev, dtype=torch.int32, generator=g)
        pol.set_step_timing(8)
        _timed(f"{case[7:]}-shaped rollout {B} x ({P}+{new})", lambda: pol.rollout(prompts, new, temperature=0.8, top_k=50, seed=1), reps=1)
        ms, pos = pol.step_times()
        print("ms per step by position:", " ".join(f"{p}:{m / 8:.3f}" for m, p in zip(ms, pos)))
    elif case == "lmhead":
        T, k, V = int(argv[2]) if len(argv) > 2 else 8192, 2048, 32000
        w8, _ = eng.expand_weights(_rand_packed(dev, V, k // 16), k)
        tau = torch.rand(V, device=dev) * 0.05 + 0.01
        bias = torch.randn(V, device=dev) * 0.01
        q, s, _ = eng.act_quant_tm(torch.randn(T, k, device=dev))
        actions = torch.randint(0, V, (T,), device=dev, dtype=torch.int32)
        up_lp, up_ent = torch.randn(T, device=dev), torch.randn(T, device=dev) * 0.01
        logp, ent, lse = eng.lmhead_logprob_entropy(w8, tau, bias, q, s, actions)
        dbias = torch.zeros(V, device=dev)
        _timed("fused LM head forward (log-prob, entropy)", lambda: eng.lmhead_logprob_entropy(w8, tau, bias, q, s, actions))
        _timed("fused LM head backward (bf16 d logits * tau, bias gradient)",
               lambda: eng.lmhead_logprob_entropy_backward(w8, tau, bias, q, s, actions, lse, ent, up_lp, up_ent, dbias=dbias))
    else:
        raise SystemExit(__doc__)
    eng.check_device_errors()


if __name__ == "__main__":
    main(sys.argv)
