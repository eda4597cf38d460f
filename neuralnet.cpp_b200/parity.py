"""How far the fast numeric mode (bf16 attention operands and KV cache, bf16 tensor-core backward GEMMs, hardware
exp) moves the results of the exact mode (f32 storage, f64-accumulated reductions) on the tiny GRPO configuration:
teacher-forced log-probs, the clipped-surrogate loss and every gradient tensor.  Both modes share the integer
forward of every ternary linear; the differences come from float roundings that occasionally flip an int8
activation.  Used by the benchmark (reported next to the throughput) and by the GPU tests, which also compare
the fast mode with the CPU restatement directly."""
from __future__ import annotations

import numpy as np
import torch

TINY = dict(n_layer=4, d_model=256, n_head=4, d_ff=1024, vocab=10000, ctx=256, act=0, pos=0)


def compare_gradients(cfg, g_fast: np.ndarray, g_ref: np.ndarray):
    """Per-tensor relative deviation: max |a-b| / max |b| and rms(a-b) / rms(b); returns the worst of each and
    the tensors they occur in."""
    worst_max, worst_rms, at_max, at_rms = 0.0, 0.0, "", ""
    # a tensor whose gradient vanishes analytically (the key bias: softmax is shift-invariant) holds rounding noise only;
    # deviations are measured against at least a thousandth of the largest gradient entry of the whole model
    floor = 1e-3 * float(np.abs(g_ref).max())
    for name, off, shape in cfg.param_layout()[0]:
        size = int(np.prod(shape))
        a, b = g_fast[off:off + size].astype(np.float64), g_ref[off:off + size].astype(np.float64)
        scale = max(np.abs(b).max(), floor)
        if scale < 1e-30:
            continue
        em = np.abs(a - b).max() / scale
        er = np.sqrt(((a - b) ** 2).mean()) / max(np.sqrt((b ** 2).mean()), floor)
        if em > worst_max:
            worst_max, at_max = em, name
        if er > worst_rms:
            worst_rms, at_rms = er, name
    return {"grad_rel_max": worst_max, "grad_rel_max_tensor": at_max, "grad_rel_rms": worst_rms, "grad_rel_rms_tensor": at_rms}


def fast_vs_exact(pkg, eng, groups: int = 2, group_size: int = 8, prompt_len: int = 32, max_new: int = 64, seed: int = 1):
    """Runs the same GRPO micro-batch (rollout by the exact policy, group advantages, clipped surrogate) through an
    exact and a fast policy holding the same weights."""
    cfg_e, cfg_f = pkg.GptConfig(exact=True, **TINY), pkg.GptConfig(exact=False, **TINY)
    flat = cfg_e.init_params(seed)
    pe, pf = pkg.Policy(eng, cfg_e), pkg.Policy(eng, cfg_f)
    pe.upload_params(flat)
    pf.upload_params(flat)
    rng = np.random.default_rng(seed + 1)
    n = groups * group_size
    prompts = torch.from_numpy(np.repeat(rng.integers(0, cfg_e.vocab, (groups, prompt_len)), group_size, axis=0).astype(np.int32)).to(eng.device)
    tokens, old_lp, _ = pe.rollout(prompts, max_new, temperature=1.0, seed=3)
    reward = (tokens[:, prompt_len:] < 5000).float().mean(1).contiguous()
    adv_seq = eng.group_advantage(reward, [(g * group_size, group_size) for g in range(groups)])
    adv = adv_seq[:, None].expand(n, max_new).contiguous()
    mask = torch.ones((n, max_new), device=eng.device)
    out = {}
    lps, grads, reps, acts = [], [], [], []
    for pol in (pe, pf):
        lp, _, _ = pol.logprobs(tokens, prompt_len)
        pol.zero_grad()
        rep = pol.train_step(tokens, prompt_len, mask, old_logp=old_lp, advantage=adv, clip_eps=0.2)
        lps.append(lp.cpu().numpy().astype(np.float64))
        grads.append(pol.grads_view().cpu().numpy())
        reps.append(rep.cpu().numpy().astype(np.float64))
        acts.append([[pol.cached_activation(l, w)[0] for w in range(4)] for l in range(cfg_e.n_layer)])
    eng.check_device_errors()
    # how many of the int8 activations that feed the linears differ between the modes (both keep them in the same
    # layout), over all layers; and by more than one quantisation step
    flipped = big = total = 0
    first = None
    for l in range(cfg_e.n_layer):
        for w in range(4):
            diff = (acts[0][l][w].to(torch.int16) - acts[1][l][w].to(torch.int16)).abs()
            flipped += int((diff > 0).sum())
            big += int((diff > 1).sum())
            total += diff.numel()
            if first is None:
                first = float((diff > 0).float().mean())  # layer 0's ln1 output: before any bf16 arithmetic
    out["int8_flip_fraction"] = flipped / total
    out["int8_flip_gt1_fraction"] = big / total
    out["int8_flip_fraction_first_input"] = first
    out["logp_max_abs"] = float(np.abs(lps[1] - lps[0]).max())
    out["logp_mean_abs"] = float(np.abs(lps[1] - lps[0]).mean())
    out["loss_abs"] = float(abs(reps[1][0] - reps[0][0]))
    out["loss_exact"] = float(reps[0][0])
    out.update(compare_gradients(cfg_e, grads[1], grads[0]))
    out["shape"] = f"tiny GRPO configuration, {groups} groups x {group_size}, prompt {prompt_len} + {max_new}"
    out["against"] = "the exact mode of the same engine (which the GPU tests hold within 1e-3 of the CPU restatement)"
    state = {"cfg": cfg_e, "flat": flat, "tokens": tokens, "old_lp": old_lp, "adv": adv, "mask": mask, "lp_fast": lps[1],
             "lp_exact": lps[0], "g_fast": grads[1], "g_exact": grads[0], "rep_fast": reps[1], "rep_exact": reps[0]}
    return out, state
