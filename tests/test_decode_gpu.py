"""Rollout parity: the batched CUDA decode path against the CPU restatement of
GPTModel::forward_step / generate.  In the exact mode logits are compared bitwise and greedy
(and top-k sampled) rollouts token by token."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(pkg, eng, cfg, seed=1, bias_std=0.01):
    from oracle_binding import OracleGpt

    flat = cfg.init_params(seed, bias_std=bias_std)
    pol = pkg.Policy(eng, cfg)
    pol.upload_params(flat)
    return pol, OracleGpt(cfg, flat), flat


def _prompts(cfg, n, p, seed):
    return np.random.default_rng(seed).integers(0, cfg.vocab, (n, p)).astype(np.int32)


def test_layout_matches_host_mirror(pkg, eng):
    cfg = pkg.GptConfig(n_layer=2, d_model=64, n_head=2, d_ff=128, vocab=97, ctx=24, act=1, pos=1, value_head=True)
    pol = pkg.Policy(eng, cfg)
    layout, n = cfg.param_layout()
    assert pol.n_params == n
    got = pol.tensors()
    assert [g[0] for g in got] == [l[0] for l in layout]
    assert [g[1] for g in got] == [l[1] for l in layout]
    for g, l in zip(got, layout):
        assert g[2] * g[3] == int(np.prod(l[2]))


@pytest.mark.parametrize("act,pos", [(0, 0), (1, 1)])
def test_requantisation_matches_oracle(pkg, eng, orc, act, pos):
    cfg = pkg.GptConfig(n_layer=2, d_model=64, n_head=2, d_ff=128, vocab=97, ctx=24, act=act, pos=pos)
    pol, m, flat = _setup(pkg, eng, cfg)
    for layer, which, rows, cols in [(0, 0, 64, 64), (1, 4, 128 * (2 if act else 1), 64), (1, 5, 64, 128), (-1, 0, 97, 64)]:
        packed, tau = pol.linear(layer, which)
        tau_ref, trit_ref = m.linear(layer, which, rows, cols)
        assert np.array_equal(tau.cpu().numpy(), tau_ref)
        assert np.array_equal(orc.trit_unpack(packed.cpu().numpy().view(np.uint32), cols), trit_ref)


@pytest.mark.parametrize("act,pos,heads,d", [(0, 0, 2, 64), (1, 1, 2, 64), (1, 1, 1, 128), (0, 1, 4, 256),
                                             (1, 1, 16, 1600),  # head dim 100, the 3B decode shape's
                                             (2, 1, 2, 128)])   # ReLU2GLU feed-forward
def test_greedy_rollout_token_identical_and_logits_bitwise(pkg, eng, act, pos, heads, d):
    cfg = pkg.GptConfig(n_layer=2, d_model=d, n_head=heads, d_ff=2 * d, vocab=211, ctx=40, act=act, pos=pos)
    pol, m, _ = _setup(pkg, eng, cfg)
    prompts = _prompts(cfg, 5, 7, seed=3)
    tok_ref, lp_ref, lg_ref = m.rollout(prompts, 12, 0.0, 0, seed=0, want_logits=True)
    tok, lp, lg = pol.rollout(torch.from_numpy(prompts).to(eng.device), 12, temperature=0.0, want_logits=True)
    torch.cuda.synchronize()
    assert np.array_equal(lg.cpu().numpy().view(np.uint32), lg_ref.view(np.uint32)), "logits differ bitwise"
    assert np.array_equal(tok.cpu().numpy(), tok_ref)
    assert np.abs(lp.cpu().numpy() - lp_ref).max() <= 1e-3 * np.abs(lp_ref).max()


@pytest.mark.parametrize("temperature,top_k", [(0.8, 50), (1.0, 5), (1.3, 1)])
def test_top_k_sampled_rollout_token_identical(pkg, eng, temperature, top_k):
    cfg = pkg.GptConfig(n_layer=2, d_model=64, n_head=2, d_ff=128, vocab=300, ctx=40, act=1, pos=1)
    pol, m, _ = _setup(pkg, eng, cfg)
    prompts = _prompts(cfg, 6, 5, seed=4)
    tok_ref, lp_ref, _ = m.rollout(prompts, 16, temperature, top_k, seed=99, seq0=10)
    tok, lp, _ = pol.rollout(torch.from_numpy(prompts).to(eng.device), 16, temperature=temperature, top_k=top_k,
                             seed=99, seq0=10)
    assert np.array_equal(tok.cpu().numpy(), tok_ref)
    assert np.abs(lp.cpu().numpy() - lp_ref).max() <= 1e-3 * np.abs(lp_ref).max()


@pytest.mark.parametrize("kw", [dict(temperature=0.9, top_k=40, top_p=0.7), dict(temperature=1.0, top_k=0, top_p=0.5),
                                dict(temperature=0.0, repeat_penalty=4.0), dict(temperature=0.8, top_k=20, repeat_penalty=1.5, repeat_window=6),
                                dict(temperature=1.0, top_k=30, top_p=0.9, repeat_penalty=1.3, bias=True),
                                dict(temperature=1.0, top_k=8, eos_token=5, min_new_tokens=2)])
def test_sampling_config_rollout_token_identical(pkg, eng, kw):
    """top-p, repeat penalty / window, the logit bias and end-of-sequence handling of SamplingConfig / generate, in the
    reference's order: rollouts token for token against the CPU restatement."""
    kw = dict(kw)
    cfg = pkg.GptConfig(n_layer=2, d_model=64, n_head=2, d_ff=128, vocab=300, ctx=40, act=1, pos=1)
    pol, m, _ = _setup(pkg, eng, cfg)
    prompts = _prompts(cfg, 12, 5, seed=4)
    bias = None
    if kw.pop("bias", False):
        bias = np.zeros(300, np.float32)
        bias[::3] = -np.inf  # a third of the vocabulary is forbidden
        bias[7] = 2.5
    eos, min_new = kw.pop("eos_token", -1), kw.pop("min_new_tokens", 0)
    if eos >= 0:  # an end-of-sequence id that the rollout does sample: the most frequent token of the unconstrained run
        free_run, _, _ = m.rollout_cfg(prompts, 20, seed=77, seq0=3, **kw)
        eos = int(np.bincount(free_run[:, 5 + min_new:5 + 12].ravel()).argmax())
    tok_ref, lp_ref, len_ref = m.rollout_cfg(prompts, 20, bias=bias, eos=eos, min_new=min_new, seed=77, seq0=3, **kw)
    sc = pkg.SamplingConfig(seed=77, eos_token=eos, min_new_tokens=min_new,
                            logit_bias=None if bias is None else torch.from_numpy(bias).to(eng.device), **kw)
    tok, lp, glen, _ = pol.rollout_sampled(torch.from_numpy(prompts).to(eng.device), 20, sc, seq0=3)
    assert np.array_equal(tok.cpu().numpy(), tok_ref)
    assert np.array_equal(glen.cpu().numpy(), len_ref)
    assert np.abs(lp.cpu().numpy() - lp_ref).max() <= 1e-3 * max(np.abs(lp_ref).max(), 1e-6)
    if bias is not None:
        assert not np.isin(tok_ref[:, 5:], np.arange(0, 300, 3)).any()
    if eos >= 0:
        assert (len_ref < 20).any()  # the case does exercise an early end


@pytest.mark.parametrize("pos,P,max_new,kw", [(0, 5, 14, dict(temperature=0.0)), (1, 5, 14, dict(temperature=0.9, top_k=12)),
                                              (1, 15, 6, dict(temperature=0.0)), (0, 12, 3, dict(temperature=1.0, top_k=5))])
def test_generation_past_the_context_slides_the_window_like_the_reference(pkg, eng, pos, P, max_new, kw):
    """GPTModel::generate beyond seq_len (compute_layer_gpt.hpp:768-818): a prompt longer than the context is cut to its
    tail, and once the cache is full every further token is sampled after rebuilding it from the last ctx-1 tokens at
    positions 0..ctx-2.  Context 12 here; tokens against the CPU restatement."""
    cfg = pkg.GptConfig(n_layer=2, d_model=64, n_head=2, d_ff=128, vocab=211, ctx=12, act=1, pos=pos)
    pol, m, _ = _setup(pkg, eng, cfg)
    prompts = _prompts(cfg, 4, P, seed=8)
    tok_ref, lp_ref, _ = m.rollout_cfg(prompts, max_new, seed=5, seq0=2, **kw)
    tok, lp, _, _ = pol.rollout_sampled(torch.from_numpy(prompts).to(eng.device), max_new, pkg.SamplingConfig(seed=5, **kw), seq0=2)
    assert np.array_equal(tok.cpu().numpy(), tok_ref)
    assert np.abs(lp.cpu().numpy() - lp_ref).max() <= 1e-3 * np.abs(lp_ref).max()
    # grouped prompts fall back to one window per sequence and give the same tokens
    rep = np.repeat(prompts[:2], 2, axis=0)
    a, _, _, _ = pol.rollout_sampled(torch.from_numpy(rep).to(eng.device), max_new, pkg.SamplingConfig(seed=5, **kw), group_size=2)
    b, _, _, _ = pol.rollout_sampled(torch.from_numpy(rep).to(eng.device), max_new, pkg.SamplingConfig(seed=5, **kw))
    assert torch.equal(a, b)


def test_top_p_over_a_large_vocabulary_without_top_k_is_refused(pkg, eng):
    cfg = pkg.GptConfig(n_layer=1, d_model=64, n_head=2, d_ff=128, vocab=2000, ctx=24, act=0, pos=0)
    pol, _, _ = _setup(pkg, eng, cfg)
    p = torch.from_numpy(_prompts(cfg, 2, 4, seed=6)).to(eng.device)
    with pytest.raises(pkg.NnbError):
        pol.rollout_sampled(p, 4, pkg.SamplingConfig(top_p=0.5))


@pytest.mark.parametrize("kw", [dict(temperature=0.0), dict(temperature=0.9, top_k=40), dict(temperature=1.0, top_k=0),
                                dict(temperature=0.8, top_k=64, top_p=0.8, repeat_penalty=1.2, repeat_window=6),
                                dict(temperature=0.0, repeat_penalty=3.0), dict(temperature=1.1, top_k=30, repeat_penalty=1.5, bias=True)])
def test_vocabulary_larger_than_a_ctas_shared_memory(pkg, eng, kw):
    """70 000 logits (280 KB) do not fit one CTA's shared memory: the sampler keeps its working row in a scratch buffer
    instead and must choose the same tokens"""
    cfg = pkg.GptConfig(n_layer=1, d_model=64, n_head=2, d_ff=128, vocab=70000, ctx=24, act=1, pos=1)
    pol, m, _ = _setup(pkg, eng, cfg)
    prompts = _prompts(cfg, 4, 5, seed=9)
    kw = dict(kw)
    bias = None
    if kw.pop("bias", False):
        bias = np.zeros(70000, np.float32)
        bias[::2] = -np.inf  # half of the vocabulary is forbidden
        bias[12345] = 1.5
    whole_vocab = kw.get("temperature", 1.0) > 0 and kw.get("top_k", 0) == 0
    n_new = 1 if whole_vocab else 10
    ref_tok, ref_lp, _ = m.rollout_cfg(prompts, n_new, seed=4, bias=bias, **kw)
    sc = pkg.SamplingConfig(seed=4, logit_bias=None if bias is None else torch.from_numpy(bias).to(eng.device), **kw)
    tok, lp, _, _ = pol.rollout_sampled(torch.from_numpy(prompts).to(eng.device), n_new, sc)
    if whole_vocab:
        # 70 000 nearly equal probabilities summed sequentially in f32 by the reference rule and in f64 by chunks here:
        # the draw lands within a few dozen entries of the same place in the cumulative distribution
        assert np.abs(tok.cpu().numpy()[:, -1].astype(np.int64) - ref_tok[:, -1]).max() <= 128
        return
    assert np.array_equal(tok.cpu().numpy(), ref_tok)
    assert np.abs(lp.cpu().numpy() - ref_lp).max() <= 1e-3 * np.abs(ref_lp).max()
    if bias is not None:
        assert not (ref_tok[:, 5:] % 2 == 0).any()


def test_full_vocab_sampled_rollout_agrees(pkg, eng):
    # without top-k the CDF is accumulated in f64 by chunks on the GPU and in f32 sequentially by the
    # reference rule: tokens agree except where the draw falls within rounding of a CDF step
    cfg = pkg.GptConfig(n_layer=1, d_model=64, n_head=2, d_ff=128, vocab=1000, ctx=24, act=0, pos=0)
    pol, m, _ = _setup(pkg, eng, cfg)
    prompts = _prompts(cfg, 64, 4, seed=5)
    tok_ref, _, _ = m.rollout(prompts, 1, 1.0, 0, seed=5)
    tok, _, _ = pol.rollout(torch.from_numpy(prompts).to(eng.device), 1, temperature=1.0, top_k=0, seed=5)
    agree = (tok.cpu().numpy() == tok_ref).mean()
    assert agree >= 0.999
    # and the draws are not degenerate
    assert len(np.unique(tok_ref[:, -1])) > 20


def test_seed_and_sequence_offset_semantics(pkg, eng):
    cfg = pkg.GptConfig(n_layer=1, d_model=64, n_head=2, d_ff=128, vocab=300, ctx=24, act=1, pos=1)
    pol, _, _ = _setup(pkg, eng, cfg)
    p = torch.from_numpy(_prompts(cfg, 8, 4, seed=6)).to(eng.device)
    a, _, _ = pol.rollout(p, 8, 1.0, 20, seed=1, seq0=0)
    b, _, _ = pol.rollout(p, 8, 1.0, 20, seed=1, seq0=0)
    c, _, _ = pol.rollout(p, 8, 1.0, 20, seed=2, seq0=0)
    assert torch.equal(a, b) and not torch.equal(a, c)
    # sharding by sequence: rows 4..7 rolled out alone with seq0=4 reproduce the same tokens
    d, _, _ = pol.rollout(p[4:].contiguous(), 8, 1.0, 20, seed=1, seq0=4)
    assert torch.equal(a[4:], d)


def test_tiny_grpo_policy_shape_greedy_rollout(pkg, eng):
    """The CPU-runnable configuration: 4 layers, d 256, 4 heads, GELU 1024, vocab 10000, ctx 256;
    8 prompts x group 8, prompt 32, 64 generated tokens — greedy rollouts must be token-identical."""
    cfg = pkg.GptConfig(n_layer=4, d_model=256, n_head=4, d_ff=1024, vocab=10000, ctx=256, act=0, pos=0)
    pol, m, _ = _setup(pkg, eng, cfg, seed=1, bias_std=0.0)
    base = np.random.default_rng(2).integers(0, 10000, (8, 32)).astype(np.int32)
    prompts = np.repeat(base, 8, axis=0)  # groups are contiguous rows
    tok_ref, lp_ref, _ = m.rollout(prompts[::8].copy(), 64, 0.0, 0, seed=0)
    tok, lp, _ = pol.rollout(torch.from_numpy(prompts).to(eng.device), 64, temperature=0.0)
    tok = tok.cpu().numpy()
    assert np.array_equal(tok[::8], tok_ref)
    for g in range(8):  # greedy: every member of a group is the same sequence
        assert np.array_equal(tok[8 * g:8 * g + 8], np.repeat(tok_ref[g:g + 1], 8, 0))
    assert np.abs(lp.cpu().numpy()[::8] - lp_ref).max() <= 1e-3 * np.abs(lp_ref).max()


def test_fast_mode_runs_and_is_close(pkg, eng):
    cfg_e = pkg.GptConfig(n_layer=2, d_model=128, n_head=2, d_ff=256, vocab=500, ctx=48, act=1, pos=1, exact=True)
    cfg_f = pkg.GptConfig(n_layer=2, d_model=128, n_head=2, d_ff=256, vocab=500, ctx=48, act=1, pos=1, exact=False)
    flat = cfg_e.init_params(3, bias_std=0.01)
    pe, pf = pkg.Policy(eng, cfg_e), pkg.Policy(eng, cfg_f)
    pe.upload_params(flat)
    pf.upload_params(flat)
    p = torch.from_numpy(_prompts(cfg_e, 4, 6, seed=8)).to(eng.device)
    _, _, lg_e = pe.rollout(p, 1, 0.0, want_logits=True)
    _, _, lg_f = pf.rollout(p, 1, 0.0, want_logits=True)
    err = (lg_e - lg_f).abs().max().item() / lg_e.abs().max().item()
    assert err < 0.05  # bf16 KV cache, f32 accumulation


@pytest.mark.parametrize("group_size", [1, 4])
def test_fast_mode_head_size_100(pkg, eng, group_size):
    """the 3B decode shape's head size in the fast mode: bf16 cache rows padded from 100 to 104 features, attention on the
    tensor-core streamer (tiles padded to 112 features in shared memory); logits after a prompt against the exact mode, and
    the rollout's log-probs against the teacher-forced pass; also with a prompt prefix shared by 4 sequences"""
    kw = dict(n_layer=2, d_model=1600, n_head=16, d_ff=3200, vocab=500, ctx=80, act=1, pos=1)
    cfg_e, cfg_f = pkg.GptConfig(exact=True, **kw), pkg.GptConfig(exact=False, **kw)
    flat = cfg_e.init_params(3, bias_std=0.01)
    pe, pf = pkg.Policy(eng, cfg_e), pkg.Policy(eng, cfg_f)
    pe.upload_params(flat)
    pf.upload_params(flat)
    prompts = np.repeat(_prompts(cfg_e, 8 // group_size, 37, seed=8), group_size, axis=0)
    p = torch.from_numpy(prompts).to(eng.device)
    _, _, lg_e = pe.rollout(p, 1, 0.0, want_logits=True, group_size=group_size)
    _, _, lg_f = pf.rollout(p, 1, 0.0, want_logits=True, group_size=group_size)
    assert (lg_e - lg_f).abs().max().item() <= 0.05 * lg_e.abs().max().item()
    toks, old_lp, _ = pf.rollout(p, 40, temperature=1.0, top_k=20, seed=1, group_size=group_size)
    lp2, _, _ = pf.logprobs(toks, 37)
    assert (lp2 - old_lp).abs().max().item() <= 2e-2 * max(old_lp.abs().max().item(), 1.0)
    eng.check_device_errors()


@pytest.mark.parametrize("d,heads,kv", [(256, 4, 0), (512, 4, 0), (1600, 16, 0), (512, 4, 2)])
@pytest.mark.parametrize("group_size", [1, 4])
def test_tensor_core_decode_attention_with_a_roomy_cache(pkg, eng, d, heads, kv, group_size):
    """from 512 cached positions of capacity on, the fast mode's decode attention runs on the tensor-core streamer for
    head sizes 64, 128 and 100, multi-head or grouped: logits after a prompt of 490 tokens against the exact mode, and the
    rollout's log-probs against the teacher-forced pass; also with the prompt shared by 4 sequences"""
    kw = dict(n_layer=2, d_model=d, n_head=heads, n_head_kv=kv, d_ff=2 * d, vocab=500, ctx=520, act=1, pos=1)
    cfg_e, cfg_f = pkg.GptConfig(exact=True, **kw), pkg.GptConfig(exact=False, **kw)
    flat = cfg_e.init_params(3, bias_std=0.01)
    pe, pf = pkg.Policy(eng, cfg_e), pkg.Policy(eng, cfg_f)
    pe.upload_params(flat)
    pf.upload_params(flat)
    prompts = np.repeat(_prompts(cfg_e, 8 // group_size, 490, seed=8), group_size, axis=0)
    p = torch.from_numpy(prompts).to(eng.device)
    _, _, lg_e = pe.rollout(p, 30, 0.0, want_logits=True, group_size=group_size)
    _, _, lg_f = pf.rollout(p, 30, 0.0, want_logits=True, group_size=group_size)
    # the first generated position: both modes have consumed the same tokens there
    assert (lg_e[:, 0] - lg_f[:, 0]).abs().max().item() <= 0.05 * lg_e[:, 0].abs().max().item()
    toks, old_lp, _ = pf.rollout(p, 30, temperature=1.0, top_k=20, seed=1, group_size=group_size)
    lp2, _, _ = pf.logprobs(toks, 490)
    assert (lp2 - old_lp).abs().max().item() <= 2e-2 * max(old_lp.abs().max().item(), 1.0)
    eng.check_device_errors()


@pytest.mark.parametrize("group_size,kw", [(1, dict(temperature=0.9, top_k=30)), (4, dict(temperature=1.0, top_k=12)),
                                           (4, dict(temperature=1.0, top_k=8, eos=True))])
def test_rollout_of_128_sequences_matches_the_restatement(pkg, eng, group_size, kw):
    """128 sequences, alone and in groups of 4 with a shared prompt prefix: tokens, log-probs, lengths and logits are those
    of the CPU restatement for every row, in the caller's order"""
    kw = dict(kw)
    use_eos = kw.pop("eos", False)
    cfg = pkg.GptConfig(n_layer=1, d_model=64, n_head=2, d_ff=128, vocab=300, ctx=32, act=1, pos=1)
    pol, m, _ = _setup(pkg, eng, cfg)
    prompts = np.repeat(_prompts(cfg, 128 // group_size, 6, seed=11), group_size, axis=0)
    eos = -1
    if use_eos:
        free_run, _, _ = m.rollout_cfg(prompts, 10, seed=5, seq0=7, **kw)
        eos = int(np.bincount(free_run[:, 6:].ravel()).argmax())
    tok_ref, lp_ref, len_ref = m.rollout_cfg(prompts, 10, eos=eos, seed=5, seq0=7, **kw)
    sc = pkg.SamplingConfig(seed=5, eos_token=eos, **kw)
    tok, lp, glen, _ = pol.rollout_sampled(torch.from_numpy(prompts).to(eng.device), 10, sc, seq0=7, group_size=group_size)
    assert np.array_equal(tok.cpu().numpy(), tok_ref)
    assert np.array_equal(glen.cpu().numpy(), len_ref)
    assert np.abs(lp.cpu().numpy() - lp_ref).max() <= 1e-3 * max(np.abs(lp_ref).max(), 1e-6)
    # greedy with logits: bitwise, row for row
    tok_g, _, lg_ref = m.rollout(prompts, 4, 0.0, 0, seed=0, want_logits=True)
    tok2, _, lg = pol.rollout(torch.from_numpy(prompts).to(eng.device), 4, temperature=0.0, want_logits=True, group_size=group_size)
    assert np.array_equal(tok2.cpu().numpy(), tok_g)
    assert np.array_equal(lg.cpu().numpy().view(np.uint32), lg_ref.view(np.uint32))


def test_host_rollout_entry_point(pkg, eng):
    cfg = pkg.GptConfig(n_layer=1, d_model=64, n_head=2, d_ff=128, vocab=300, ctx=24, act=0, pos=0)
    pol, m, _ = _setup(pkg, eng, cfg)
    prompts = _prompts(cfg, 3, 4, seed=9)
    h_p = torch.from_numpy(prompts).pin_memory()
    h_t = torch.empty((3, 10), dtype=torch.int32).pin_memory()
    h_l = torch.empty((3, 6), dtype=torch.float32).pin_memory()
    pol.rollout_host(h_p, 6, 0.0, 0, 0, 0, h_t, h_l)
    tok_ref, lp_ref, _ = m.rollout(prompts, 6, 0.0, 0, seed=0)
    assert np.array_equal(h_t.numpy(), tok_ref)


def test_context_overflow_slides_in_the_rollout_and_is_rejected_by_the_teacher_forced_pass(pkg, eng):
    cfg = pkg.GptConfig(n_layer=1, d_model=64, n_head=2, d_ff=128, vocab=300, ctx=8, act=0, pos=0)
    pol = pkg.Policy(eng, cfg)
    pol.upload_params(cfg.init_params(0))
    p = torch.zeros((2, 4), dtype=torch.int32, device=eng.device)
    tok, _, _ = pol.rollout(p, 8)  # 12 tokens through a window of 8, as GPTModel::generate does
    assert tok.shape == (2, 12)
    with pytest.raises(pkg.NnbError):
        pol.logprobs(tok, 4)  # the teacher-forced pass takes whole sequences within the context only


@pytest.mark.parametrize("exact", [True, False])
@pytest.mark.parametrize("P", [1, 2, 9])
def test_grouped_rollout_equals_ungrouped(pkg, eng, exact, P):
    """Sharing the prompt prefix inside a group changes where K/V are stored, not the arithmetic: bit-identical in
    the exact mode.  The fast mode attends to the shared prefix for all members of a group at once on tensor cores
    (queries rounded to bf16, the softmax merged from two parts), so there the logits agree to bf16 rounding."""
    cfg = pkg.GptConfig(n_layer=2, d_model=128, n_head=2, d_ff=256, vocab=300, ctx=48, act=1, pos=1, exact=exact)
    pol = pkg.Policy(eng, cfg)
    pol.upload_params(cfg.init_params(5, bias_std=0.01))
    base = _prompts(cfg, 3, P, seed=11)
    prompts = torch.from_numpy(np.repeat(base, 4, axis=0)).to(eng.device)  # 3 groups of 4
    a_tok, a_lp, a_lg = pol.rollout(prompts, 12, temperature=0.9, top_k=20, seed=5, seq0=7, want_logits=True)
    b_tok, b_lp, b_lg = pol.rollout(prompts, 12, temperature=0.9, top_k=20, seed=5, seq0=7, want_logits=True, group_size=4)
    if exact or P == 1:  # a one-token prompt leaves no prefix to share
        assert torch.equal(a_lg, b_lg) and torch.equal(a_tok, b_tok) and torch.equal(a_lp, b_lp)
    else:
        # first generated step: same inputs on both paths (later steps follow whichever tokens were sampled)
        assert (a_lg[:, 0] - b_lg[:, 0]).abs().max().item() <= 2e-2 * a_lg[:, 0].abs().max().item()
    with pytest.raises(pkg.NnbError):
        pol.rollout(prompts[:10].contiguous(), 4, group_size=4)
