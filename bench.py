"""bench.py — hot-path benchmark of the nn-b200 engine.

python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workloads (synthetic data, random-init weights; the default is the configuration the metric is quoted on):
  grpo1b     GRPO step on a 24-layer, d 2048, 16-head, RoPE, SwiGLU 5632, vocab 32000 ternary policy; 64 prompt
             groups x 16 samples, prompt 128 uniform-random ids, 512 generated tokens, top-k 50, temperature 0.8;
             reward = seeded hash of the generated tokens -> {0,1} with p 0.3; clip 0.2, KL 0.04 against a frozen
             copy of the initial weights; AdamW.  Prompt groups are sharded over the ranks (whole groups per rank,
             strong scaling); the policy gradient is all-reduced with NCCL.
             step = rollout + rewards/advantages + reference log-probs + forward/backward + optimizer.
  tiny       the CPU-runnable GRPO configuration (4 layers, d 256, 4 heads, GELU 1024, vocab 10000; 8 x 8 rollouts,
             prompt 32 + 64 generated, temperature 1.0, clip 0.2, KL 0).
  ppo_gpt2s  PPO with GAE on a GPT-2-small-shaped ternary policy with a value head (12 layers, d 768, 12 heads,
             MLP 3072, vocab 32000, ctx 512); 256 sequences, prompt 64 + 256 generated; terminal reward N(0,1) plus
             per-token N(0,0.1); gamma 0.99, lambda 0.95, clip 0.2, value coef 0.5, 4 epochs x 4 minibatches.
             Trajectories are sharded over the ranks.  step = rollout + values + GAE + 16 minibatch updates.
  decode3b   rollout-only decode on a BitNet-b1.58-3B-shaped policy (26 layers, d 3200, 32 heads of 100, SwiGLU
             8640, vocab 32002): 512 sequences, prompt 256, 1792 generated, bf16 KV cache to ctx 2048, sharded by
             sequence over the ranks and decoded in chunks of at most 128 sequences per GPU (the cache of one
             sequence is 0.71 GB).  step = all 512 sequences.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "grpo1b": dict(kind="grpo", model=dict(n_layer=24, d_model=2048, n_head=16, d_ff=5632, vocab=32000, ctx=640, act=1, pos=1),
                   groups=64, group_size=16, prompt_len=128, max_new=512, temperature=0.8, top_k=50, kl_coef=0.04,
                   micro_batch=32, rollout_chunk=1024,
                   text="GRPO step, ~1B ternary Llama-style policy (24 layers, d 2048, 16 heads, RoPE, SwiGLU 5632, vocab 32000), "
                        "64 prompts x group 16, prompt 128, 512 generated, top-k 50, T 0.8, clip 0.2, KL 0.04 vs frozen initial policy"),
    "tiny": dict(kind="grpo", model=dict(n_layer=4, d_model=256, n_head=4, d_ff=1024, vocab=10000, ctx=256, act=0, pos=0),
                 groups=8, group_size=8, prompt_len=32, max_new=64, temperature=1.0, top_k=0, kl_coef=0.0,
                 micro_batch=64, rollout_chunk=64,
                 text="GRPO step, tiny ternary GPT (4 layers, d 256, 4 heads, GELU 1024, vocab 10000), 8 prompts x group 8, "
                      "prompt 32, 64 generated, T 1.0, clip 0.2, KL 0"),
    "ppo_gpt2s": dict(kind="ppo", model=dict(n_layer=12, d_model=768, n_head=12, d_ff=3072, vocab=32000, ctx=512, act=0, pos=0,
                                             value_head=True),
                      n_seq=256, prompt_len=64, max_new=256, temperature=1.0, top_k=0, micro_batch=64, rollout_chunk=256,
                      epochs=4, minibatches=4,
                      text="PPO step with GAE, GPT-2-small-shaped ternary policy with a value head (12 layers, d 768, 12 heads, MLP 3072, "
                           "vocab 32000), 256 sequences, prompt 64, 256 generated, gamma 0.99, lambda 0.95, clip 0.2, value coef 0.5, "
                           "entropy coef 0.01, 4 epochs x 4 minibatches"),
    "decode3b": dict(kind="decode", model=dict(n_layer=26, d_model=3200, n_head=32, d_ff=8640, vocab=32002, ctx=2048, act=1, pos=1),
                     n_seq=512, prompt_len=256, max_new=1792, temperature=0.8, top_k=50, chunk=128,
                     text="rollout-only decode, BitNet-b1.58-3B-shaped ternary policy (26 layers, d 3200, 32 heads, SwiGLU 8640, "
                          "vocab 32002), 512 sequences, prompt 256, 1792 generated, bf16 KV cache to ctx 2048, top-k 50, T 0.8, "
                          "decoded in chunks of <= 128 sequences per GPU"),
    # the structure of BitNet b1.58 2B4T: SubLN, grouped-query attention (20 heads on 5 KV heads), tied embeddings, ReLU2GLU
    "grpo2b4t": dict(kind="grpo", model=dict(n_layer=30, d_model=2560, n_head=20, n_head_kv=5, d_ff=6912, vocab=128256, ctx=640,
                                             act=2, pos=1, sub_ln=True, tie_embeddings=True),
                     groups=64, group_size=16, prompt_len=128, max_new=512, temperature=0.8, top_k=50, kl_coef=0.04,
                     micro_batch=16, rollout_chunk=1024,
                     text="GRPO step, BitNet-b1.58-2B4T-structured ternary policy (30 layers, d 2560, 20 heads on 5 KV heads, RoPE, "
                          "SubLN, ReLU2GLU 6912, tied embeddings, vocab 128256), 64 prompts x group 16, prompt 128, 512 generated, "
                          "top-k 50, T 0.8, clip 0.2, KL 0.04 vs frozen initial policy"),
    "decode2b4t": dict(kind="decode", model=dict(n_layer=30, d_model=2560, n_head=20, n_head_kv=5, d_ff=6912, vocab=128256, ctx=2048,
                                                 act=2, pos=1, sub_ln=True, tie_embeddings=True),
                       n_seq=512, prompt_len=256, max_new=1792, temperature=0.8, top_k=50, chunk=128,
                       text="rollout-only decode, BitNet-b1.58-2B4T-structured ternary policy (30 layers, d 2560, 20 heads on 5 KV "
                            "heads, SubLN, ReLU2GLU 6912, tied embeddings, vocab 128256), 512 sequences, prompt 256, 1792 generated, "
                            "bf16 KV cache to ctx 2048, top-k 50, T 0.8, decoded in chunks of <= 128 sequences per GPU"),
}


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "src": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return

        def pump():
            for line in self.proc.stdout:
                self.rows.append((time.time(), line.strip()))

        threading.Thread(target=pump, daemon=True).start()

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons, power = [], None, set(), []
        for ts, line in self.rows:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not (t0 <= ts <= t1 + 0.2):
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None}


def _dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def _init_policy_device(pkg, eng, cfg, seed):
    """Random-init weights on the device: linears and embeddings N(0, 0.02), gains 1, biases 0."""
    import torch

    pol = pkg.Policy(eng, cfg)
    g = torch.Generator(device=eng.device)
    g.manual_seed(seed)
    pv = pol.params_view()
    pv.normal_(0, 0.02, generator=g)
    layout, _ = cfg.param_layout()
    for name, off, shape in layout:
        size = int(np.prod(shape))
        if name.endswith("gamma"):
            pv[off:off + size] = 1.0
        elif name.endswith(".bias"):
            pv[off:off + size] = 0.0
    pol.requantize()
    return pol


def _time_loop(torch, fn, reps, warm=3):
    for _ in range(warm):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


def _kernel_rooflines(torch, pkg, eng, pol, wl, peaks):
    """Times the dominant kernels ALONE (CUDA events on the launching stream, operands larger than L2, ten launches
    back to back after three warm-ups), so the tensor-core fractions are taken against the measured BURST rates."""
    m = wl["model"]
    d = m["d_model"]
    dev = eng.device
    out = {}
    # builder-measured int8 tensor peak: a plain cuBLASLt int8 GEMM (torch._int_mm), 8192^3, int32 accumulation
    int8_peak = None
    try:
        a8 = torch.randint(-127, 127, (8192, 8192), device=dev, dtype=torch.int8)
        b8 = torch.randint(-1, 2, (8192, 8192), device=dev, dtype=torch.int8).t()
        ms8 = _time_loop(torch, lambda: torch._int_mm(a8, b8), 10)
        int8_peak = 2.0 * 8192 ** 3 / (ms8 * 1e-3) / 1e12
        del a8, b8
    except Exception as ex:  # the library GEMM is only a yardstick
        out["int8_peak_error"] = str(ex)[:120]
    # (1) backward dX GEMM of fc1 at one micro-batch (tcgen05, bf16 operands, f32 accumulation in TMEM): the
    # backward GEMMs are the largest single share of the training phase.  Operands are prepared once; the timed
    # loop launches the GEMM kernel only.
    T = wl["micro_batch"] * (wl["prompt_len"] + wl["max_new"])
    packed, tau = pol.linear(0, 4)  # fc1
    O = packed.shape[0]
    w8, wb = eng.expand_weights(packed, d)
    dy = torch.randn((T, O), device=dev)
    dx = torch.empty((T, d), device=dev)
    x = torch.randn((T, d), device=dev)
    q, s, qsum = eng.act_quant_tm(x)
    dyb = torch.empty((T, O), device=dev, dtype=torch.bfloat16)
    eng.bitlinear_bwd_tc(dy, tau, wb, q, s, d, dx=dx, scratch=(dyb, None))
    ms = _time_loop(torch, lambda: eng.bitlinear_bwd_tc(dy, tau, wb, q, s, d, dx=dx, scratch=(dyb, None), prepared=True), 10)
    ach = 2.0 * T * d * O / (ms * 1e-3) / 1e12
    out["roofline"] = {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                       "frac": ach / peaks["bf16_tflops"], "traffic": None,
                       "traffic_note": "not measured in this run (DRAM bytes need a profiler capture; see profiles/)",
                       "peak_source": peaks["src"] + " cuBLAS bf16 burst (the kernel is timed alone)",
                       "frac_of_sustained": ach / peaks["bf16_tflops_sustained"],
                       "kernel": "gemm_tc_kernel<bf16 dX>", "kernel_ms": ms, "shape": f"T={T} K={O} N={d}",
                       "algorithmic_bytes": int(T * O * 2 + O * d * 2 + T * d * 4)}
    # (2) ternary forward GEMM at one micro-batch (tcgen05 kind::i8, int32 accumulation in TMEM)
    y = torch.empty((T, O), device=dev)
    ms = _time_loop(torch, lambda: eng.bitlinear_fwd_tc(w8, tau, None, q, s, y=y), 10)
    ach8 = 2.0 * T * d * O / (ms * 1e-3) / 1e12
    out["roofline_int8_gemm"] = {"bound": "tensor", "achieved": ach8, "unit": "TOP/s (int8)", "peak": int8_peak,
                                 "frac": (ach8 / int8_peak) if int8_peak else None,
                                 "peak_source": "torch._int_mm 8192^3 timed in this run (cuBLASLt int8, burst)",
                                 "kernel": "gemm_tc_kernel<int8 forward>", "kernel_ms": ms, "shape": f"T={T} K={d} O={O}"}
    eng.check_device_errors()
    del w8, wb, dy, dx, dyb, y
    # (3) decode attention of one step at a mid-rollout context: the HBM-bound kernel of the rollout
    H = m["n_head"]
    dk = d // H
    if dk in (64, 128):
        Bd, ctx, pos = 512, 512, 400
        kc = torch.randn((Bd, H, ctx, dk), device=dev).to(torch.bfloat16)
        vc = torch.randn((Bd, H, ctx, dk), device=dev).to(torch.bfloat16)
        qkv = torch.randn((3, Bd, d), device=dev)
        tpos = torch.tensor([pos], device=dev, dtype=torch.int32)
        ms = _time_loop(torch, lambda: eng.attention_decode(qkv, kc, vc, tpos, H, exact=False, want_out=False, want_q8=True), 10)
        alg = Bd * H * (pos + 1) * dk * 2 * 2 + 3 * Bd * d * 4 + Bd * d
        out["roofline_attn_decode"] = {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                       "frac": alg / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "kernel": "attn_decode_fused_kernel",
                                       "kernel_ms": ms, "shape": f"B={Bd} H={H} dk={dk} pos={pos}"}
        del kc, vc, qkv
    # (4) decode-sized ternary GEMV: packed-weight stream of a stack of fc1-shaped matrices (> L2)
    n_mats = 64
    wst = torch.randint(-2**31, 2**31 - 1, (n_mats, O, d // 16), device=dev, dtype=torch.int64)
    lo, hi = wst & 0x55555555, (wst >> 1) & 0x55555555
    wst = wst | ((~(lo | hi)) & 0x55555555) << 1
    wst = (wst & 0xFFFFFFFF)
    wst = torch.where(wst >= 2**31, wst - 2**32, wst).to(torch.int32).contiguous()
    taus = torch.rand((n_mats, O), device=dev) * 0.09 + 0.01
    for mtok in (1, 4, 16):
        xq = torch.randn((mtok, d), device=dev)
        q1, s1, qs1 = eng.act_quant_tm(xq)
        ys = torch.empty((n_mats, mtok, O), device=dev)
        ms = _time_loop(torch, lambda: eng.bitlinear_fwd_tm_stack(wst, taus, None, q1, s1, qs1, ys), 20)
        alg = n_mats * (d * O / 4 + 4 * O + mtok * d + 4 * mtok + 4 * mtok * O)
        ach = alg / (ms * 1e-3) / 1e9
        out[f"roofline_gemv_m{mtok}"] = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                          "frac": ach / peaks["hbm_gbs"],
                                          "kernel": "bitlinear_gemv_kernel (dp4a)" if mtok == 1 else "bitlinear_skinny_kernel",
                                          "kernel_ms": ms, "shape": f"M={mtok} K={d} N={O} x{n_mats}"}
    return out


class Phases:
    def __init__(self, torch):
        self.torch, self.ev = torch, []

    def mark(self, name):
        e = self.torch.cuda.Event(enable_timing=True)
        e.record()
        self.ev.append((name, e))

    def per_step(self, steps):
        ph = {}
        for i in range(1, len(self.ev)):
            nm = self.ev[i][0]
            if nm != "start":
                ph[nm] = ph.get(nm, 0.0) + self.ev[i - 1][1].elapsed_time(self.ev[i][1]) / steps
        return ph


# ----------------------------------------------------------------------------- jobs
class GrpoJob:
    metric, unit = "grpo_steps_per_s", "GRPO steps/s"
    dtype = "int8 x 2-bit -> int32 forward, bf16 backward, f32 master weights"

    def __init__(self, torch, pkg, eng, wl, rank, world):
        self.torch, self.pkg, self.eng, self.wl, self.rank, self.world = torch, pkg, eng, wl, rank, world
        cfg = pkg.GptConfig(exact=False, **wl["model"])
        assert wl["groups"] % world == 0, "prompt groups must divide over the ranks"
        self.groups_local = wl["groups"] // world
        self.pol = _init_policy_device(pkg, eng, cfg, seed=1)
        self.ref = _init_policy_device(pkg, eng, cfg, seed=1) if wl["kl_coef"] != 0.0 else None  # frozen initial weights
        gcfg = pkg.GrpoConfig(group_size=wl["group_size"], prompt_len=wl["prompt_len"], max_new=wl["max_new"],
                              temperature=wl["temperature"], top_k=wl["top_k"], clip_eps=0.2, kl_coef=wl["kl_coef"], lr=1e-4,
                              micro_batch=wl["micro_batch"], rollout_chunk=wl["rollout_chunk"])
        self.trainer = pkg.GrpoTrainer(self.pol, self.ref, gcfg)
        self.P, self.G = gcfg.prompt_len, gcfg.max_new
        rng = np.random.default_rng(2)
        allp = rng.integers(0, cfg.vocab, (wl["groups"], self.P)).astype(np.int32)
        self.h_prompts = torch.from_numpy(allp[rank * self.groups_local:(rank + 1) * self.groups_local].copy()).pin_memory()
        self.d_prompts = self.h_prompts.to(eng.device)
        self.step_no = 0
        self.last = None
        self.n_local = self.groups_local * wl["group_size"]
        self.gen_tokens = wl["groups"] * wl["group_size"] * self.G
        self.global_batch, self.seq_len = wl["groups"] * wl["group_size"], self.P + self.G
        self.parallelism = f"dp{world} by prompt group"
        self.scaling = "strong"

    def reward_dev(self, tokens):
        if self.wl["kl_coef"] == 0.0:  # the tiny configuration's reward: fraction of generated ids < 5000
            return (tokens[:, self.P:] < 5000).float().mean(1)
        return self.pkg.hash_reward(tokens[:, self.P:], 7)

    def reward_host(self, tokens):
        torch = self.torch
        tk = tokens[:, self.P:].cpu().numpy().astype(np.int64)
        if self.wl["kl_coef"] == 0.0:
            r = (tk < 5000).mean(1).astype(np.float32)
        else:
            pos = (np.arange(1, self.G + 1, dtype=np.int64) * 2654435761) % 2147483647
            h = ((tk + 1) * pos).sum(1) + 7 * 97003
            h = (h * 1103515245 + 12345) % 2147483648
            h = ((h ^ (h >> 13)) * 1274126177) % 2147483648
            r = ((h % 1000003).astype(np.float32) / np.float32(1000003.0) < 0.3).astype(np.float32)
        return torch.from_numpy(r).pin_memory().to(self.eng.device, non_blocking=True)

    def step(self, phases=None):
        self.step_no += 1
        self.last = self.trainer.step(self.d_prompts, self.reward_dev, seed=self.step_no, timers=phases)

    def e2e_step(self):
        """prompts start in pinned host memory, generated tokens go back to the host where the reward is computed,
        rewards come back up, and the step's report is read on the host"""
        self.step_no += 1
        out = self.trainer.step(self.h_prompts.to(self.eng.device, non_blocking=True), self.reward_host, seed=self.step_no)
        return out["report"].cpu()

    def e2e_bytes(self):
        return self.groups_local * self.P * 4 + self.n_local * 4, self.n_local * self.G * 4 + 10 * 4

    def extras(self, ph):
        out = {"rollout_tok_per_s": self.gen_tokens / (ph["rollout"] * 1e-3)} if ph.get("rollout") else {}
        out["last_report"] = self.pkg.report_dict(self.last["report"])
        return out

    def release(self):
        self.pol.release_workspaces()
        if self.ref is not None:
            self.ref.release_workspaces()


class PpoJob(GrpoJob):
    metric, unit = "ppo_steps_per_s", "PPO steps/s"

    def __init__(self, torch, pkg, eng, wl, rank, world):
        self.torch, self.pkg, self.eng, self.wl, self.rank, self.world = torch, pkg, eng, wl, rank, world
        cfg = pkg.GptConfig(exact=False, **wl["model"])
        assert wl["n_seq"] % (world * wl["minibatches"]) == 0, "trajectories must divide over ranks and minibatches"
        self.n_local = wl["n_seq"] // world
        self.pol = _init_policy_device(pkg, eng, cfg, seed=1)
        self.ref = None
        # a value head that is not identically zero, so that the value loss has something to fit
        pv = self.pol.params_view()
        for name, off, shape in cfg.param_layout()[0]:
            if name == "value_head.weight":
                g = torch.Generator(device=eng.device)
                g.manual_seed(5)
                pv[off:off + shape[1]].normal_(0, 0.05, generator=g)
        pcfg = pkg.PpoConfig(prompt_len=wl["prompt_len"], max_new=wl["max_new"], temperature=wl["temperature"], top_k=wl["top_k"],
                             epochs=wl["epochs"], minibatches=wl["minibatches"], micro_batch=min(wl["micro_batch"], self.n_local // wl["minibatches"]),
                             rollout_chunk=wl["rollout_chunk"])
        self.trainer = pkg.PpoTrainer(self.pol, pcfg, seed=11)
        self.P, self.G = pcfg.prompt_len, pcfg.max_new
        rng = np.random.default_rng(2)
        allp = rng.integers(0, cfg.vocab, (wl["n_seq"], self.P)).astype(np.int32)
        self.h_prompts = torch.from_numpy(allp[rank * self.n_local:(rank + 1) * self.n_local].copy()).pin_memory()
        self.d_prompts = self.h_prompts.to(eng.device)
        self.gen = torch.Generator(device=eng.device)
        self.gen.manual_seed(100 + rank)
        self.step_no, self.last = 0, None
        self.gen_tokens = wl["n_seq"] * self.G
        self.global_batch, self.seq_len = wl["n_seq"], self.P + self.G
        self.parallelism = f"dp{world} by trajectory"
        self.scaling = "strong"

    def reward_dev(self, tokens):
        torch = self.torch
        r = torch.randn((tokens.shape[0], self.G), device=self.eng.device, generator=self.gen) * 0.1
        r[:, -1] += torch.randn(tokens.shape[0], device=self.eng.device, generator=self.gen)
        return r

    def reward_host(self, tokens):
        tk = tokens[:, self.P:].cpu().numpy()  # the environment sees the generated tokens on the host
        rs = np.random.default_rng(int(tk[:, 0].sum()) & 0xFFFF)
        r = rs.normal(0, 0.1, tk.shape).astype(np.float32)
        r[:, -1] += rs.normal(0, 1, tk.shape[0]).astype(np.float32)
        return self.torch.from_numpy(r).pin_memory().to(self.eng.device, non_blocking=True)

    def e2e_bytes(self):
        return self.n_local * self.P * 4 + self.n_local * self.G * 4, self.n_local * self.G * 4 + 10 * 4


class DecodeJob:
    metric, unit = "rollout_tok_per_s", "generated tokens/s"
    dtype = "int8 x 2-bit -> int32 linears, bf16 KV cache, f32 accumulation"

    def __init__(self, torch, pkg, eng, wl, rank, world):
        self.torch, self.pkg, self.eng, self.wl, self.rank, self.world = torch, pkg, eng, wl, rank, world
        self.cfg = pkg.GptConfig(exact=False, **wl["model"])
        assert wl["n_seq"] % world == 0
        self.n_local = wl["n_seq"] // world
        self.chunk = min(wl["chunk"], self.n_local)
        assert self.n_local % self.chunk == 0
        self.pol = _init_policy_device(pkg, eng, self.cfg, seed=1)
        self.P, self.G = wl["prompt_len"], wl["max_new"]
        rng = np.random.default_rng(2)
        allp = rng.integers(0, self.cfg.vocab, (wl["n_seq"], self.P)).astype(np.int32)
        self.h_prompts = torch.from_numpy(allp[rank * self.n_local:(rank + 1) * self.n_local].copy()).pin_memory()
        self.d_prompts = self.h_prompts.to(eng.device)
        self.h_tokens = torch.empty((self.chunk, self.P + self.G), dtype=torch.int32).pin_memory()
        self.step_no, self.last = 0, None
        self.gen_tokens = wl["n_seq"] * self.G
        self.global_batch, self.seq_len = wl["n_seq"], self.P + self.G
        self.parallelism = f"dp{world} by sequence, {self.n_local // self.chunk} chunk(s) of {self.chunk} per GPU"
        self.scaling = "strong"
        self.fit = None

    def step(self, phases=None):
        self.step_no += 1
        if phases:
            phases.mark("start")
        for a in range(0, self.n_local, self.chunk):
            self.last = self.pol.rollout(self.d_prompts[a:a + self.chunk].contiguous(), self.G, temperature=self.wl["temperature"],
                                         top_k=self.wl["top_k"], seed=self.step_no, seq0=self.rank * self.n_local + a, want_logp=False)
        if phases:
            phases.mark("rollout")

    def e2e_step(self):
        self.step_no += 1
        for a in range(0, self.n_local, self.chunk):
            self.pol.rollout_host(self.h_prompts[a:a + self.chunk], self.G, self.wl["temperature"], self.wl["top_k"], self.step_no,
                                  self.rank * self.n_local + a, self.h_tokens, None)
        return self.h_tokens

    def e2e_bytes(self):
        return self.n_local * self.P * 4, self.n_local * (self.P + self.G) * 4

    def measure_fit(self, peaks):
        """One more chunk with an event every 64 decode steps: time per step = a + b * context.  b is the attention
        kernel's cost per cached position (KV bytes per position / b = its HBM rate); a is everything that does not
        grow with the context: the packed-weight stream of the 26 x 7 linears and the head, the quantisers, the sampler."""
        m = self.wl["model"]
        self.pol.set_step_timing(64)
        self.pol.rollout(self.d_prompts[:self.chunk].contiguous(), self.G, temperature=self.wl["temperature"], top_k=self.wl["top_k"],
                         seed=1, seq0=0, want_logp=False)
        ms, pos = self.pol.step_times()
        self.pol.set_step_timing(0)
        if len(ms) < 4:
            return {}
        n_steps = np.diff(np.append(pos, self.P + self.G - 1)).astype(np.float64)
        per_step = ms.astype(np.float64) / n_steps
        mid = pos.astype(np.float64) + n_steps / 2.0 + 1.0  # mean number of cached positions attended to
        gen = pos >= self.P  # steps that also run the head and the sampler
        b, a = np.polyfit(mid[gen], per_step[gen], 1)
        L, d, H = m["n_layer"], m["d_model"], m["n_head"]
        F = m["d_ff"]
        dk = d // H
        dkv = (m.get("n_head_kv") or H) * dk
        kv_per_pos = self.chunk * L * 2 * dkv * 2  # algorithmic bytes per cached position per step (bf16 K and V heads)
        # packed bytes of the linears: q and o (d x d), k and v (dkv x d), fc1 (gate | up) and fc2, the head unless tied
        packed = (L * (2 * d * d + 2 * dkv * d + 3 * d * F) + (0 if m.get("tie_embeddings") else m["vocab"] * d)) / 4
        if dk == 100:
            kernel, pad = "attn_decode_mma_kernel<100,104,112>", " (the cache rows are padded from 100 to 104 features: 4 % more is actually read)"
        else:
            kernel, pad = f"attn_decode_bf16_kernel<{dk},{dk}>", ""
        if m.get("n_head_kv") and m["n_head_kv"] != H:
            if dk in (64, 128):
                kernel = f"attn_decode_mma_kernel<{dk}>"
            pad += (f"; grouped-query attention: the cache holds {m['n_head_kv']} KV heads, each row loaded once for the "
                    f"{H // m['n_head_kv']} query heads of its group")
        attn = kv_per_pos / (b * 1e-3) / 1e9
        wstream = packed / (a * 1e-3) / 1e9
        return {"roofline": {"bound": "hbm", "achieved": attn, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": attn / peaks["hbm_gbs"],
                             "traffic": None, "kernel": kernel,
                             "how": "slope of the per-step time over the context, measured with CUDA events every 64 steps inside a "
                                    f"rollout of {self.chunk} sequences; algorithmic bytes = 2 x ctx x (KV heads x dk) x 2 B per sequence and layer"
                                    + pad,
                             "ms_per_step_per_position": float(b), "peak_source": peaks["src"] + " copy bandwidth"},
                "roofline_weight_stream": {"bound": "hbm", "achieved": wstream, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                           "frac": wstream / peaks["hbm_gbs"], "packed_bytes": int(packed),
                                           "ms_per_step_context_free": float(a),
                                           "how": "2-bit container bytes of all linears / the context-independent part of a decode "
                                                  "step (intercept of the same fit): a lower bound on the linears' own rate, since "
                                                  "the intercept also holds the quantisers, the sampler and launch gaps"}}

    def extras(self, ph):
        return {"rollout_tok_per_s": self.gen_tokens / (ph["rollout"] * 1e-3)} if ph.get("rollout") else {}

    def release(self):
        pass


JOBS = {"grpo": GrpoJob, "ppo": PpoJob, "decode": DecodeJob}


def run_ours(args):
    import torch
    from __graft_entry__ import load_package

    rank, world, local = _dist_env()
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = load_package()
    eng = pkg.Engine(local)
    dev = eng.device
    peaks = _peaks()
    wl = WORKLOADS[args.workload]
    if args.groups and wl["kind"] == "grpo":
        wl = dict(wl, groups=args.groups, text=wl["text"] + f" [prompt groups overridden: {args.groups}]")
    if args.micro_batch and "micro_batch" in wl:
        # the sequences one forward/backward takes; gradients accumulate over a minibatch either way
        wl = dict(wl, micro_batch=args.micro_batch, text=wl["text"] + f" [micro-batch overridden: {args.micro_batch}]")
    job = JOBS[wl["kind"]](torch, pkg, eng, wl, rank, world)

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    W = max(args.warmup, 3)
    for _ in range(W):
        job.step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.4)
    l0 = eng.launch_count()
    phases = Phases(torch)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.time()
    ev0.record()
    for _ in range(args.steps):
        job.step(phases)
    ev1.record()
    barrier()
    t1 = time.time()
    launches = eng.launch_count() - l0
    total_ms = ev0.elapsed_time(ev1)
    ph = phases.per_step(args.steps)
    if world > 1:
        tt = torch.tensor([total_ms, ph.get("rollout", 0.0)], device=dev)
        torch.distributed.all_reduce(tt, op=torch.distributed.ReduceOp.MAX)
        total_ms, ph["rollout"] = float(tt[0]), float(tt[1])
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    ms_per_step = total_ms / args.steps
    steps_per_s = 1000.0 / ms_per_step
    value = steps_per_s * job.gen_tokens if wl["kind"] == "decode" else steps_per_s

    n_e2e = max(1, args.steps // 2)
    barrier()
    te0 = time.perf_counter()
    for _ in range(n_e2e):
        host_result = job.e2e_step()
    barrier()
    te = time.perf_counter() - te0
    if world > 1:
        tt = torch.tensor([te], device=dev)
        torch.distributed.all_reduce(tt, op=torch.distributed.ReduceOp.MAX)
        te = float(tt[0])
    e2e_value = n_e2e / te * (job.gen_tokens if wl["kind"] == "decode" else 1.0)
    h2d, d2h = job.e2e_bytes()
    del host_result

    res = {
        "metric": job.metric, "value": value, "unit": job.unit, "n_gpus": world, "steps": args.steps,
        "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": job.scaling, "vs_baseline": None,
        "dtype": job.dtype, "data": "synthetic",
        "config": {"workload": wl["text"], "name": args.workload, "global_batch": job.global_batch, "seq_len": job.seq_len,
                   "parallelism": job.parallelism,
                   "l2": "working set per step (weights, KV cache, activations) far larger than L2"},
        "phase_ms": {k: round(v, 2) for k, v in ph.items()},
        "e2e": {"value": e2e_value, "unit": job.unit, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "steps": n_e2e},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    res.update(job.extras(ph))
    if rank == 0 and world == 1:
        if wl["kind"] == "decode":
            res.update(job.measure_fit(peaks))
        else:
            job.release()
            res.update(_kernel_rooflines(torch, pkg, eng, job.pol, wl, peaks))
            if not args.no_parity:
                from neuralnet_cpp_b200.parity import fast_vs_exact
                res["parity_fast"] = fast_vs_exact(pkg, eng)[0]
        if not args.no_cpu_baseline:
            res["cpu_baseline"] = cpu_baseline(args.workload, gpu=(torch, pkg, eng))
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        torch.distributed.destroy_process_group()


# ----------------------------------------------------------------------------- CPU arm
def _cpu_threads():
    """All host cores, set explicitly: launchers such as torch.distributed.run export OMP_NUM_THREADS=1, which would
    otherwise make this arm single-threaded at N > 1 and threaded at N = 1."""
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except Exception:
        pass
    os.environ["OMP_NUM_THREADS"] = str(cores)
    try:
        import ctypes
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(cores)
    except Exception:
        pass
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(cores)
    except Exception:
        pass
    return cores


def _cpu_imports():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from __graft_entry__ import load_package
    import oracle_binding as ob
    import oracle_train as ot

    return load_package(), ob, ot


def _cpu_flat(cfg, seed=1):
    layout, n = cfg.param_layout()
    rng = np.random.default_rng(seed)
    flat = rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)
    for name, off, shape in layout:
        size = int(np.prod(shape))
        if name.endswith("gamma"):
            flat[off:off + size] = 1.0
        elif name.endswith(".bias"):
            flat[off:off + size] = 0.0
    return flat


def cpu_config1_step(pkg, ob, ot):
    """A complete GRPO step of the tiny configuration on the CPU restatement, MEASURED end to end: 8 x 8 rollouts of
    32 + 64 tokens through the C step path (OpenMP over sequences), group advantages, teacher-forced forward, clipped
    surrogate, backward (numpy, threaded BLAS), AdamW."""
    wl = WORKLOADS["tiny"]
    cfg = pkg.GptConfig(exact=True, **wl["model"])
    flat = _cpu_flat(cfg)
    rng = np.random.default_rng(2)
    prompts = np.repeat(rng.integers(0, cfg.vocab, (wl["groups"], wl["prompt_len"])), wl["group_size"], axis=0).astype(np.int32)
    rl = ob.OracleRL()
    t0 = time.perf_counter()
    m = ob.OracleGpt(cfg, flat)
    tokens, old_lp, _ = m.rollout(prompts, wl["max_new"], wl["temperature"], wl["top_k"], seed=1)
    t_roll = time.perf_counter() - t0
    reward = (tokens[:, wl["prompt_len"]:] < 5000).mean(1).astype(np.float32)
    adv = rl.group_advantage(reward, [(wl["group_size"] * g, wl["group_size"]) for g in range(wl["groups"])])
    tr = ot.OracleTrainer(cfg, flat)
    lp, ent, _ = tr.forward(tokens, wl["prompt_len"])
    _, up_lp, _, _ = tr.objective(lp, ent, np.ones_like(lp), old_lp, np.repeat(adv[:, None], wl["max_new"], 1), clip_eps=0.2)
    g = tr.backward(up_lp)
    rl.adamw(flat, g.astype(np.float32), np.zeros_like(flat), np.zeros_like(flat), lr=1e-4, t=1)
    t_all = time.perf_counter() - t0
    return {"step_s": t_all, "rollout_s": t_roll, "rollout_tok_per_s": tokens.shape[0] * wl["max_new"] / t_roll}


def cpu_config2_sweep(ob, budget_s=12.0):
    """Threaded row-block matmul_q_i8 (decode 64 weight rows to a tile, dense kernel over it) on the operator sweep:
    M in {1,16,64,256,2048} x (K,N) in {(2048,2048),(2048,5632),(5632,2048)}; GOP/s per case, stopping at the budget."""
    orc = ob.Oracle()
    rng = np.random.default_rng(4)
    out, t_start = [], time.perf_counter()
    for (k, n) in ((2048, 2048), (2048, 5632), (5632, 2048)):
        w = rng.integers(-1, 2, (n, k)).astype(np.float32)
        tau = np.full(n, 0.05, np.float32)
        packed = orc.trit_pack(w * 0.1, tau)
        for m in (1, 16, 64, 256, 2048):
            if time.perf_counter() - t_start > budget_s:
                return out
            q, s = orc.act_quant_tm(rng.standard_normal((m, k), dtype=np.float32))
            t0 = time.perf_counter()
            orc.bitlinear_i8_tm(packed, tau, None, q, s, want_acc=False)
            dt = time.perf_counter() - t0
            out.append({"M": m, "K": k, "N": n, "ms": dt * 1e3, "gops": 2.0 * m * k * n / dt / 1e9})
    return out


class CpuArm:
    """The CPU restatement on a bounded sample of a workload, extrapolated per token to the workload's step."""

    def __init__(self, workload):
        self.cores = _cpu_threads()
        self.pkg, self.ob, self.ot = _cpu_imports()
        self.name, self.wl = workload, WORKLOADS[workload]
        wl = self.wl
        self.rng = np.random.default_rng(1)
        model = dict(wl["model"])
        self.layer_scale = 1.0
        if model["n_layer"] > 24:
            # 2 of the layers (a couple of GB of f32 weights instead of 10+ GB); the per-layer cost is scaled
            model["n_layer"] = 2
            self.layer_scale = wl["model"]["n_layer"] / 2.0
        self.cfg = self.pkg.GptConfig(exact=True, **model)
        self.flat = _cpu_flat(self.cfg)
        self.gpt = self.ob.OracleGpt(self.cfg, self.flat)
        self.tr = self.ot.OracleTrainer(self.cfg, self.flat) if wl["kind"] != "decode" else None

    def sample(self):
        wl, cfg, rng = self.wl, self.cfg, self.rng
        n_seq, P_s, G_s = min(self.cores, 16), 8, 8
        prompts = rng.integers(0, cfg.vocab, (n_seq, P_s)).astype(np.int32)
        t0 = time.perf_counter()
        self.gpt.rollout(prompts, G_s, wl["temperature"], wl["top_k"], seed=1)
        t_roll = time.perf_counter() - t0
        # the sample's time per token splits into the layers (scaled to the full depth) and the head (not scaled), by
        # their multiply-accumulate counts
        m = wl["model"]
        dm, Fm, Hm = m["d_model"], m["d_ff"], m["n_head"]
        dkv_m = (m.get("n_head_kv") or Hm) * (dm // Hm)
        layer_macs = 2 * dm * dm + 2 * dkv_m * dm + (3 if m["act"] >= 1 else 2) * dm * Fm
        head_frac = m["vocab"] * dm / (m["vocab"] * dm + cfg.n_layer * layer_macs)
        per_tok_decode = t_roll / (n_seq * (P_s + G_s - 1)) * ((1.0 - head_frac) * self.layer_scale + head_frac)
        S = wl["prompt_len"] + wl["max_new"]
        if wl["kind"] == "decode":
            N = wl["n_seq"]
            est = per_tok_decode * N * (S - 1)
            return {"step_s": est, "value": N * wl["max_new"] / est, "extrapolated": True,
                    "sample": f"C step-path rollout of {n_seq} seqs x {P_s + G_s} tokens on 2 of the {wl['model']['n_layer']} layers "
                              f"({t_roll:.1f} s), the layers scaled by {self.layer_scale:g}, and per token to {N} x {S - 1} token-steps (attention cost at "
                              f"the sample's short context; the head's share of the sample, {head_frac:.2f} by multiply-accumulates, is "
                              f"not scaled)"}
        if self.name == "tiny":  # small enough to run whole: a measured step, nothing extrapolated
            c1 = cpu_config1_step(self.pkg, self.ob, self.ot)
            return {"step_s": c1["step_s"], "value": 1.0 / c1["step_s"], "extrapolated": False,
                    "sample": f"the complete step, measured: C step-path rollout of 64 seqs x 96 tokens ({c1['rollout_s']:.1f} s), numpy "
                              "forward, objective, backward, AdamW"}
        # enough rows that the per-call fixed costs of the numpy restatement (weight conversions) do not dominate
        n_t, S_t = 4, 64
        toks = rng.integers(0, cfg.vocab, (n_t, S_t)).astype(np.int32)
        t0 = time.perf_counter()
        lp, ent, val = self.tr.forward(toks, 4)
        t_fwd = time.perf_counter() - t0
        kw = dict(value=val, returns=val, old_value=val, value_coef=0.5) if cfg.value_head else {}
        _, up_lp, up_ent, dv = self.tr.objective(lp, ent, np.ones_like(lp), lp, np.ones_like(lp), lp, kl_coef=0.04, **kw)
        t0 = time.perf_counter()
        self.tr.backward(up_lp, None, dv)
        t_bwd = time.perf_counter() - t0
        rows = n_t * S_t
        if wl["kind"] == "grpo":
            N = wl["groups"] * wl["group_size"]
            n_ref = 1 if wl["kl_coef"] != 0.0 else 0
            est = per_tok_decode * N * (S - 1) + self.layer_scale * ((t_fwd / rows) * N * S * (1 + n_ref) + (t_bwd / rows) * N * S)
        else:
            N = wl["n_seq"]
            est = per_tok_decode * N * (S - 1) + (t_fwd / rows) * N * S * (1 + wl["epochs"]) + (t_bwd / rows) * N * S * wl["epochs"]
        return {"step_s": est, "value": 1.0 / est, "extrapolated": True,
                "sample": f"C step-path rollout of {n_seq} seqs x {P_s + G_s} tokens ({t_roll:.1f} s), numpy forward+backward of {n_t} x {S_t} "
                          f"tokens ({t_fwd:.1f}+{t_bwd:.1f} s), extrapolated per token to the full step (attention cost at the "
                          "sample's short context)" + (f"; 2 of the {wl['model']['n_layer']} layers, scaled by {self.layer_scale:g}"
                                                       if self.layer_scale != 1.0 else "")}


def cpu_baseline(workload: str, gpu=None):
    """cpu_baseline of the bench line: the extrapolated sample of THIS workload (the line's unit), and beside it what was
    measured without extrapolation: a complete GRPO step of the tiny configuration on the CPU (and on the GPU when one
    is at hand) and the operator sweep of the ternary linear."""
    arm = CpuArm(workload)
    s = arm.sample()
    wl = WORKLOADS[workload]
    unit = {"grpo": "GRPO steps/s", "ppo": "PPO steps/s", "decode": "generated tokens/s"}[wl["kind"]]
    out = {"value": s["value"], "unit": unit, "cores": arm.cores, "kind": "port", "sample": s["sample"],
           "estimated_step_s": s["step_s"], "extrapolated": s["extrapolated"]}
    pkg, ob, ot = arm.pkg, arm.ob, arm.ot
    del arm
    c1 = cpu_config1_step(pkg, ob, ot)
    out["measured_tiny_grpo_step"] = {"cpu_step_s": c1["step_s"], "cpu_steps_per_s": 1.0 / c1["step_s"],
                                      "cpu_rollout_tok_per_s": c1["rollout_tok_per_s"], "extrapolated": False}
    if gpu is not None:
        torch, gpkg, eng = gpu
        job = GrpoJob(torch, gpkg, eng, WORKLOADS["tiny"], 0, 1)
        for _ in range(3):
            job.step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(5):
            job.step()
        torch.cuda.synchronize()
        g = (time.perf_counter() - t0) / 5
        out["measured_tiny_grpo_step"].update(gpu_step_s=g, gpu_over_cpu=c1["step_s"] / g)
    out["measured_ternary_linear_sweep"] = cpu_config2_sweep(ob)
    return out


def run_reference(args):
    """The CPU arm on this workload's configuration, metric and unit: every step is one bounded sample of the workload
    (see CpuArm.sample), W warm-up samples and K timed ones; rank 0 only."""
    rank, world, _ = _dist_env()
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    arm = CpuArm(args.workload)
    # one sample costs seconds: bound the run to a few minutes whatever K and W are
    budget = 150.0
    t0 = time.perf_counter()
    first = arm.sample()
    per = max(time.perf_counter() - t0, 1e-3)
    n_max = max(1, int(budget / per))
    W = min(args.warmup, max(0, n_max // 5))
    K = max(1, min(args.steps, n_max - W))
    samples = [arm.sample() for _ in range(W + K)][W:] if (W + K) > 1 else [first]
    est = float(np.mean([s["step_s"] for s in samples]))
    job = JOBS[wl["kind"]]
    value = (wl["n_seq"] * wl["max_new"] / est) if wl["kind"] == "decode" else 1.0 / est
    cb = {"value": value, "unit": job.unit, "cores": arm.cores, "kind": "port", "sample": samples[-1]["sample"],
          "estimated_step_s": est, "samples_timed": len(samples), "extrapolated": samples[-1]["extrapolated"]}
    out = {
        "impl": "reference", "metric": job.metric, "value": value, "unit": job.unit, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": est * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 x 2-bit -> int32 forward, f64 backward (CPU restatement)",
        "data": "synthetic",
        "config": {"workload": wl["text"] + "; CPU restatement of the reference CpuEngine semantics (the reference's own engine "
                               "source is an un-vendored submodule and cannot be built), bounded sample per step",
                   "name": args.workload},
        "cpu_baseline": cb,
        "e2e": {"value": value, "unit": job.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="grpo1b", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--groups", type=int, default=0,
                    help="GRPO workloads: prompt groups instead of the workload's own count (e.g. 8 = one GPU's share of "
                         "grpo1b at 8 GPUs); the line's config says so and is not the benchmark's")
    ap.add_argument("--micro-batch", type=int, default=0,
                    help="sequences per forward/backward instead of the workload's own micro-batch (a tuning knob: the "
                         "step's result is the same accumulation)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
