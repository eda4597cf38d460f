"""bench.py — hot-path benchmark of the nn-b200 engine: one GRPO step of the ~1B ternary policy.

python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload grpo1b|tiny]

Workload (default grpo1b): GRPO on a 24-layer, d 2048, 16-head, RoPE, SwiGLU 5632, vocab 32000 ternary
policy; 64 prompt groups x 16 samples, prompt 128 uniform-random ids, 512 generated tokens, top-k 50,
temperature 0.8; reward = seeded hash of the generated tokens -> {0,1} with p 0.3; clip 0.2, KL 0.04
against a frozen copy of the initial weights; AdamW.  Prompt groups are sharded over the ranks
(whole groups per rank, strong scaling); the policy gradient is all-reduced with NCCL.
A "step" = rollout + rewards/advantages + reference log-probs + forward/backward + optimizer.
Synthetic data, random-init weights.  Prints ONE JSON line on rank 0.
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
    # the configuration the metric is quoted on
    "grpo1b": dict(model=dict(n_layer=24, d_model=2048, n_head=16, d_ff=5632, vocab=32000, ctx=640, act=1, pos=1),
                   groups=64, group_size=16, prompt_len=128, max_new=512, temperature=0.8, top_k=50,
                   micro_batch=16, rollout_chunk=1024),
    # the CPU-runnable configuration (parity-test shape; selectable for quick checks)
    "tiny": dict(model=dict(n_layer=4, d_model=256, n_head=4, d_ff=1024, vocab=10000, ctx=256, act=0, pos=0),
                 groups=8, group_size=8, prompt_len=32, max_new=64, temperature=1.0, top_k=0,
                 micro_batch=64, rollout_chunk=64),
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
    """Times the dominant kernels alone (CUDA events on the launching stream, inputs larger than L2)."""
    m = wl["model"]
    d, F = m["d_model"], m["d_ff"]
    dev = eng.device
    out = {}
    # (1) backward dX GEMM of fc1 at one micro-batch (tcgen05, bf16 operands, f32 accumulation in TMEM): the
    # backward GEMMs are the largest single share of the step.  Operands are prepared once; the timed loop
    # launches the GEMM kernel only.
    T = wl["micro_batch"] * (wl["prompt_len"] + wl["max_new"])
    packed, tau = pol.linear(0, 4)  # fc1: (2F, d)
    O = packed.shape[0]
    w8, wb = eng.expand_weights(packed, d)
    dy = torch.randn((T, O), device=dev)
    dx = torch.empty((T, d), device=dev)
    x = torch.randn((T, d), device=dev)
    q, s, qsum = eng.act_quant_tm(x)
    dyb = torch.empty((T, O), device=dev, dtype=torch.bfloat16)
    eng.bitlinear_bwd_tc(dy, tau, wb, q, s, d, dx=dx, scratch=(dyb, None))
    ms = _time_loop(torch, lambda: eng.bitlinear_bwd_tc(dy, tau, wb, q, s, d, dx=dx, scratch=(dyb, None), prepared=True), 10)
    flops = 2.0 * T * d * O
    ach = flops / (ms * 1e-3) / 1e12
    out["roofline"] = {"bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                       "frac": ach / peaks["bf16_tflops_sustained"],
                       # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this shape
                       # (profiles/gemm_tc_kernel_bf16_dx_10240x11264x2048.md); algorithmic bytes 361 MB
                       "traffic": 557.7e6 if (T, O, d) == (10240, 11264, 2048) else None,
                       "peak_source": peaks["src"] + " (sustained)",
                       "kernel": "gemm_tc_kernel<bf16 dX>", "kernel_ms": ms, "shape": f"T={T} K={O} N={d}"}
    # (2) ternary forward GEMM at one micro-batch (tcgen05 kind::i8, int32 accumulation in TMEM)
    y = torch.empty((T, O), device=dev)
    ms = _time_loop(torch, lambda: eng.bitlinear_fwd_tc(w8, tau, None, q, s, y=y), 10)
    out["roofline_int8_gemm"] = {"bound": "tensor", "achieved": 2.0 * T * d * O / (ms * 1e-3) / 1e12, "unit": "TOP/s (int8)",
                                 "peak": None, "kernel": "gemm_tc_kernel<int8 forward>", "kernel_ms": ms,
                                 "shape": f"T={T} K={d} O={O}"}
    eng.check_device_errors()
    del w8, wb, dy, dx, dyb, y
    # (2b) decode attention of one step at a mid-rollout context: the HBM-bound kernel of the rollout
    H = m["n_head"]
    dk = d // H
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
    # (3) decode-sized ternary GEMV: packed-weight stream of a stack of fc1-shaped matrices (> L2)
    n_mats = 64
    wst = torch.randint(-2**31, 2**31 - 1, (n_mats, O, d // 16), device=dev, dtype=torch.int64)
    lo, hi = wst & 0x55555555, (wst >> 1) & 0x55555555
    wst = wst | ((~(lo | hi)) & 0x55555555) << 1
    wst = (wst & 0xFFFFFFFF)
    wst = torch.where(wst >= 2**31, wst - 2**32, wst).to(torch.int32).contiguous()
    taus = torch.rand((n_mats, O), device=dev) * 0.09 + 0.01
    for mtok in (1, 16):
        xq = torch.randn((mtok, d), device=dev)
        q1, s1, qs1 = eng.act_quant_tm(xq)
        ys = torch.empty((n_mats, mtok, O), device=dev)
        ms = _time_loop(torch, lambda: eng.bitlinear_fwd_tm_stack(wst, taus, None, q1, s1, qs1, ys), 20)
        alg = n_mats * (d * O / 4 + 4 * O + mtok * d + 4 * mtok + 4 * mtok * O)
        ach = alg / (ms * 1e-3) / 1e9
        out[f"roofline_gemv_m{mtok}"] = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                          "frac": ach / peaks["hbm_gbs"], "kernel": "bitlinear_skinny_kernel",
                                          "kernel_ms": ms, "shape": f"M={mtok} K={d} N={O} x{n_mats}"}
    return out


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
    cfg = pkg.GptConfig(exact=False, **wl["model"])
    assert wl["groups"] % world == 0, "prompt groups must divide over the ranks"
    groups_local = wl["groups"] // world
    pol = _init_policy_device(pkg, eng, cfg, seed=1)
    ref = _init_policy_device(pkg, eng, cfg, seed=1)  # frozen copy of the initial weights
    gcfg = pkg.GrpoConfig(group_size=wl["group_size"], prompt_len=wl["prompt_len"], max_new=wl["max_new"],
                          temperature=wl["temperature"], top_k=wl["top_k"], clip_eps=0.2, kl_coef=0.04, lr=1e-4,
                          micro_batch=wl["micro_batch"], rollout_chunk=wl["rollout_chunk"])
    trainer = pkg.GrpoTrainer(pol, ref, gcfg)
    P, G = gcfg.prompt_len, gcfg.max_new
    rng = np.random.default_rng(2)
    all_prompts = rng.integers(0, cfg.vocab, (wl["groups"], P)).astype(np.int32)
    h_prompts = torch.from_numpy(all_prompts[rank * groups_local:(rank + 1) * groups_local].copy()).pin_memory()
    d_prompts = h_prompts.to(dev)

    def reward_dev(tokens):
        return pkg.hash_reward(tokens[:, P:], 7)

    class Phases:
        def __init__(self):
            self.ev = []

        def mark(self, name):
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.ev.append((name, e))

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    step_no = [0]

    def step(prompts, reward_fn, phases=None):
        step_no[0] += 1
        return trainer.step(prompts, reward_fn, seed=step_no[0], timers=phases)

    W = max(args.warmup, 3)
    for _ in range(W):
        step(d_prompts, reward_dev)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.4)
    l0 = eng.launch_count()
    phases = Phases()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0 = time.time()
    ev0.record()
    last = None
    for _ in range(args.steps):
        last = step(d_prompts, reward_dev, phases)
    ev1.record()
    barrier()
    t1 = time.time()
    launches = eng.launch_count() - l0
    total_ms = ev0.elapsed_time(ev1)
    # phase breakdown (this rank)
    ph = {}
    for i in range(1, len(phases.ev)):
        nm = phases.ev[i][0]
        if nm != "start":
            ph[nm] = ph.get(nm, 0.0) + phases.ev[i - 1][1].elapsed_time(phases.ev[i][1]) / args.steps
    if world > 1:
        tt = torch.tensor([total_ms, ph.get("rollout", 0.0)], device=dev)
        torch.distributed.all_reduce(tt, op=torch.distributed.ReduceOp.MAX)
        total_ms, ph["rollout"] = float(tt[0]), float(tt[1])
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    ms_per_step = total_ms / args.steps
    value = 1000.0 / ms_per_step
    gen_tokens = wl["groups"] * wl["group_size"] * G
    rollout_tok_s = gen_tokens / (ph["rollout"] * 1e-3)

    # e2e: prompts start in pinned host memory, generated tokens go back to the host where the reward is
    # computed, rewards come back up, and the step's report is read on the host
    def reward_host(tokens):
        tk = tokens[:, P:].cpu().numpy().astype(np.int64)
        pos = (np.arange(1, G + 1, dtype=np.int64) * 2654435761) % 2147483647
        h = ((tk + 1) * pos).sum(1) + 7 * 97003
        h = (h * 1103515245 + 12345) % 2147483648
        h = ((h ^ (h >> 13)) * 1274126177) % 2147483648
        r = ((h % 1000003).astype(np.float32) / np.float32(1000003.0) < 0.3).astype(np.float32)
        return torch.from_numpy(r).pin_memory().to(dev, non_blocking=True)

    n_e2e = max(1, args.steps // 2)
    barrier()
    te0 = time.perf_counter()
    for _ in range(n_e2e):
        out = step(h_prompts.to(dev, non_blocking=True), reward_host)
        host_report = out["report"].cpu()
    barrier()
    te = time.perf_counter() - te0
    if world > 1:
        tt = torch.tensor([te], device=dev)
        torch.distributed.all_reduce(tt, op=torch.distributed.ReduceOp.MAX)
        te = float(tt[0])
    e2e_value = n_e2e / te
    N_local = groups_local * wl["group_size"]
    h2d = groups_local * P * 4 + N_local * 4
    d2h = N_local * G * 4 + 10 * 4

    res = {
        "metric": "grpo_steps_per_s", "value": value, "unit": "GRPO steps/s", "n_gpus": world, "steps": args.steps,
        "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 x 2-bit -> int32 forward, bf16 backward, f32 master weights", "data": "synthetic",
        "config": {"workload": "GRPO step, ~1B ternary Llama-style policy (24 layers, d 2048, 16 heads, RoPE, SwiGLU 5632, "
                               "vocab 32000), 64 prompts x group 16, prompt 128, 512 generated, top-k 50, T 0.8, clip 0.2, "
                               "KL 0.04 vs frozen initial policy" if args.workload == "grpo1b" else "tiny GRPO configuration",
                   "global_batch": wl["groups"] * wl["group_size"], "seq_len": P + G, "parallelism": f"dp{world} by prompt group",
                   "l2": "working set per step (weights 0.34 GB packed + 11 GB f32, KV cache, activations) far larger than L2"},
        "rollout_tok_per_s": rollout_tok_s,
        "phase_ms": {k: round(v, 2) for k, v in ph.items()},
        "e2e": {"value": e2e_value, "unit": "GRPO steps/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "steps": n_e2e},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "last_report": {k: float(v) for k, v in zip(
            ["policy_loss", "ratio_mean", "approx_kl", "clip_fraction", "kl_loss", "entropy_loss", "entropy", "units"],
            last["report"].cpu().tolist())},
    }
    del host_report
    if rank == 0 and world == 1:
        pol.release_workspaces()
        ref.release_workspaces()
        res.update(_kernel_rooflines(torch, pkg, eng, pol, wl, peaks))
        if not args.no_cpu_baseline:
            res["cpu_baseline"] = cpu_baseline(args.workload)
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        torch.distributed.destroy_process_group()


# ----------------------------------------------------------------------------- CPU arm
def cpu_baseline(workload: str, budget_s: float = 25.0):
    """The CPU restatement (oracle/) on the host cores, on a bounded sample of the same workload:
    a rollout of a few sequences and tokens through the C step path (OpenMP over sequences) and one
    teacher-forced forward/backward of one short sequence through the numpy restatement; the per-token
    costs are extrapolated to the full step."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    from __graft_entry__ import load_package
    from oracle_binding import OracleGpt
    import oracle_train as ot

    pkg = load_package()
    wl = WORKLOADS[workload]
    cfg = pkg.GptConfig(exact=True, **wl["model"])
    cores = os.cpu_count() or 1
    layout, n = cfg.param_layout()
    rng = np.random.default_rng(1)
    flat = (rng.standard_normal(n, dtype=np.float32) * np.float32(0.02))
    for name, off, shape in layout:
        size = int(np.prod(shape))
        if name.endswith("gamma"):
            flat[off:off + size] = 1.0
        elif name.endswith(".bias"):
            flat[off:off + size] = 0.0
    P_s, G_s, n_seq = 8, 8, min(cores, 16)
    m = OracleGpt(cfg, flat)
    prompts = rng.integers(0, cfg.vocab, (n_seq, P_s)).astype(np.int32)
    t0 = time.perf_counter()
    tokens, _, _ = m.rollout(prompts, G_s, wl["temperature"], wl["top_k"], seed=1)
    t_roll = time.perf_counter() - t0
    per_tok_decode = t_roll / (n_seq * (P_s + G_s - 1))
    del m
    tr = ot.OracleTrainer(cfg, flat)
    S_t = 32
    toks = rng.integers(0, cfg.vocab, (1, S_t)).astype(np.int32)
    t0 = time.perf_counter()
    lp, ent, _ = tr.forward(toks, 8)
    t_fwd = time.perf_counter() - t0
    rep, up_lp, up_ent, _ = tr.objective(lp, ent, np.ones_like(lp), lp, np.ones_like(lp), lp, kl_coef=0.04)
    t0 = time.perf_counter()
    tr.backward(up_lp)
    t_bwd = time.perf_counter() - t0
    N = wl["groups"] * wl["group_size"]
    S = wl["prompt_len"] + wl["max_new"]
    # full step: decode N*(S-1) token-steps, reference forward over N*S tokens, policy forward+backward over N*S
    est = per_tok_decode * N * (S - 1) + (t_fwd / S_t) * N * S * 2 + (t_bwd / S_t) * N * S
    return {"value": 1.0 / est, "unit": "GRPO steps/s", "cores": cores, "kind": "port",
            "sample": f"C step-path rollout of {n_seq} seqs x {P_s + G_s} tokens ({t_roll:.1f} s), numpy forward+backward of 1 x {S_t} "
                      f"tokens ({t_fwd:.1f}+{t_bwd:.1f} s), extrapolated per token to the full step (attention cost at the sample's short context)",
            "estimated_step_s": est}


def run_reference(args):
    rank, world, _ = _dist_env()
    if rank != 0:
        return
    cb = cpu_baseline(args.workload)
    wl = WORKLOADS[args.workload]
    out = {
        "impl": "reference", "metric": "grpo_steps_per_s", "value": cb["value"], "unit": "GRPO steps/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": cb["estimated_step_s"] * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int8 x 2-bit -> int32 forward, f64 backward (numpy restatement)",
        "data": "synthetic",
        "config": {"workload": "GRPO step, ~1B ternary Llama-style policy; CPU restatement of the reference CpuEngine semantics "
                               "(the reference's own engine source is an un-vendored submodule and cannot be built)",
                   "global_batch": wl["groups"] * wl["group_size"], "seq_len": wl["prompt_len"] + wl["max_new"]},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "GRPO steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
