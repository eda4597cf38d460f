// policy.cu — the ternary GPT policy object: parameter storage, requantisation, and the
// batched rollout (prefill + decode + sampling) that replaces per-sequence
// GPTModel::generate (include/neuralnet.cpp/compute_layer_gpt.hpp:740-852).
#include <math.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include <cstdlib>

#include "common.cuh"
#include "policy.cuh"

namespace nnb {

static void add_tensor(nnb_policy* p, const std::string& name, size_t off, size_t rows, size_t cols)
{
    p->tensors.push_back({name, off, rows, cols});
}

// Parameter order (one flat f32 buffer):
//   tok_emb (V,d) | pos_emb (ctx,d) if learned |
//   per layer: ln1_g | wq wk wv | bq bk bv | wo | bo | ln2_g | w1 | b1 | w2 | b2
//   lnf_g | head_w (V,d) | head_b | value_w (1,d) | value_b if value head
static void build_layout(nnb_policy* p)
{
    const nnb_gpt_config& c = p->cfg;
    const size_t d = c.d_model, F = c.d_ff, V = c.vocab;
    const size_t F1 = act_gated(c.act) ? 2 * F : F;
    const size_t dkv = cfg_kv_heads(c) * (d / c.n_head);
    size_t o = 0, po = 0, to = 0;
    auto lin = [&](LinW& l, const std::string& nm, size_t w_off, size_t b_off, size_t in, size_t out) {
        l.w_off = w_off;
        l.b_off = b_off;
        l.in = in;
        l.out = out;
        l.packed_off = po;
        l.tau_off = to;
        po += out * (in / 16);
        to += out;
        add_tensor(p, nm + ".weight", w_off, out, in);
        add_tensor(p, nm + ".bias", b_off, out, 1);
    };
    p->tok_emb = o;
    add_tensor(p, "tok_emb", o, V, d);
    o += V * d;
    p->pos_emb = (size_t)-1;
    if (c.pos == 0) {
        p->pos_emb = o;
        add_tensor(p, "pos_emb", o, c.ctx, d);
        o += (size_t)c.ctx * d;
    }
    p->layers.resize(c.n_layer);
    for (int l = 0; l < c.n_layer; ++l) {
        LayerW& L = p->layers[l];
        const std::string pre = "blocks." + std::to_string(l) + ".";
        L.ln1_g = o;
        add_tensor(p, pre + "ln1.gamma", o, d, 1);
        o += d;
        const size_t wq = o, wk = o + d * d, wv = wk + dkv * d;
        o += (d + 2 * dkv) * d;
        const size_t bq = o, bk = o + d, bv = bk + dkv;
        o += d + 2 * dkv;
        lin(L.q, pre + "attn.q", wq, bq, d, d);
        lin(L.k, pre + "attn.k", wk, bk, d, dkv);
        lin(L.v, pre + "attn.v", wv, bv, d, dkv);
        L.qkv = L.q;
        L.qkv.out = d + 2 * dkv;
        if (c.sub_ln) {
            L.attn_sub_g = o;
            add_tensor(p, pre + "attn.sub_norm.gamma", o, d, 1);
            o += d;
        }
        const size_t wo = o;
        o += d * d;
        const size_t bo = o;
        o += d;
        lin(L.o, pre + "attn.o", wo, bo, d, d);
        L.ln2_g = o;
        add_tensor(p, pre + "ln2.gamma", o, d, 1);
        o += d;
        const size_t w1 = o;
        o += F1 * d;
        const size_t b1 = o;
        o += F1;
        lin(L.fc1, pre + "ffn.fc1", w1, b1, d, F1);
        if (c.sub_ln) {
            L.ffn_sub_g = o;
            add_tensor(p, pre + "ffn.sub_norm.gamma", o, F, 1);
            o += F;
        }
        const size_t w2 = o;
        o += d * F;
        const size_t b2 = o;
        o += d;
        lin(L.fc2, pre + "ffn.fc2", w2, b2, F, d);
    }
    p->lnf_g = o;
    add_tensor(p, "ln_f.gamma", o, d, 1);
    o += d;
    if (!c.tie_embeddings) {
        const size_t hw = o;
        o += V * d;
        const size_t hb = o;
        o += V;
        lin(p->head, "lm_head", hw, hb, d, V);
    }
    p->value_w = p->value_b = (size_t)-1;
    if (c.value_head) {
        p->value_w = o;
        add_tensor(p, "value_head.weight", o, 1, d);
        o += d;
        p->value_b = o;
        add_tensor(p, "value_head.bias", o, 1, 1);
        o += 1;
    }
    std::sort(p->tensors.begin(), p->tensors.end(),
              [](const TensorInfo& a, const TensorInfo& b) { return a.offset < b.offset; });
    p->n_params = o;
    p->packed_words = po;
    p->tau_count = to;
}

static nnb_status requantize_linear(nnb_policy* p, const LinW& l)
{
    float* tau = p->tau + l.tau_off;
    NNB_TRY(launch_absmean_tau(p->e, p->params + l.w_off, l.out, l.in, tau));
    return launch_trit_pack(p->e, p->params + l.w_off, tau, l.out, l.in, p->packed + l.packed_off);
}

static nnb_status expand_all(nnb_policy* p, bool want_w8, bool want_wb)
{
    // one launch over the whole container arena: every matrix starts on a 64-feature block boundary
    return launch_expand_weights(p->e, p->packed, 1, p->packed_words * 16, want_w8 ? p->w8 : nullptr,
                                 want_wb ? p->wb : nullptr);
}

nnb_status policy_ensure_wb(nnb_policy* p)
{
    if (p->cfg.exact) return NNB_OK;
    if (!p->wb) {
        cudaError_t er = cudaMalloc((void**)&p->wb, p->packed_words * 16 * sizeof(__nv_bfloat16));
        if (er != cudaSuccess) {
            cudaGetLastError();
            NNB_FAIL(NNB_ERR_OOM, "out of device memory for the bf16 weight copy");
        }
        p->wb_valid = false;
    }
    if (!p->wb_valid) {
        NNB_TRY(expand_all(p, false, true));
        p->wb_valid = true;
    }
    return NNB_OK;
}

nnb_status policy_linear_fwd(nnb_policy* p, const LinW& l, size_t n_mats, const int8_t* q, const float* s,
                             const int32_t* qsum, size_t T, const float* residual, float* y, size_t y_stride, bool y_bf16)
{
    NNB_REQUIRE(!y_bf16 || policy_linear_can_bf16(p, T), "linear: a bf16 result needs the tensor-core forward");
    // from 64 tokens up the tcgen05 kernel wins (its tile width follows the shape; measured 1.7-1.9x over the
    // mma.sync kernel at 128 tokens); below that the persistent mma.sync kernels stream the 2-bit container,
    // a quarter of the int8 copy's bytes
    if (!p->cfg.exact && p->w8 && T >= 64)
        return launch_tc_forward(p->e, q, p->w8 + l.packed_off * 16, p->tau + l.tau_off, s, p->params + l.b_off, residual, T,
                                 l.in, l.out, y_bf16 ? nullptr : y, n_mats, y_stride,
                                 y_bf16 ? reinterpret_cast<__nv_bfloat16*>(y) : nullptr);
    return launch_bitlinear_fwd_tm(p->e, p->packed + l.packed_off, n_mats > 1 ? l.out * (l.in / 16) : 0, p->tau + l.tau_off,
                                   p->params + l.b_off, residual, q, s, qsum, n_mats, T, l.in, l.out, y, y_stride, NNB_F32,
                                   nullptr);
}

bool policy_h1_bf16(const nnb_policy* p, size_t T, size_t F, size_t F1)
{
    static const bool on = [] { const char* ev = getenv("NNB_H1_BF16"); return !(ev && ev[0] == '0'); }();
    return on && policy_linear_can_bf16(p, T) && F1 % 8 == 0 && F % 8 == 0;
}

// seeded = true: tau and the containers were just written from a model file and are authoritative (the first forward
// then reproduces the saved model bit for bit, compute_layer_bitlinear.hpp:276-300); only the derived copies are rebuilt
nnb_status policy_requantize(nnb_policy* p, bool seeded)
{
    p->wb_valid = false;
    if (!seeded) {
        for (auto& L : p->layers) {
            NNB_TRY(requantize_linear(p, L.q));
            NNB_TRY(requantize_linear(p, L.k));
            NNB_TRY(requantize_linear(p, L.v));
            NNB_TRY(requantize_linear(p, L.o));
            NNB_TRY(requantize_linear(p, L.fc1));
            NNB_TRY(requantize_linear(p, L.fc2));
        }
        if (!p->cfg.tie_embeddings) NNB_TRY(requantize_linear(p, p->head));
    }
    if (!p->cfg.exact) {
        if (!p->w8) {
            cudaError_t er = cudaMalloc((void**)&p->w8, p->packed_words * 16);
            if (er != cudaSuccess) {
                cudaGetLastError();
                NNB_FAIL(NNB_ERR_OOM, "out of device memory for the int8 weight copy");
            }
        }
        NNB_TRY(expand_all(p, true, p->wb != nullptr));
        p->wb_valid = p->wb != nullptr;
        if (p->cfg.tie_embeddings) {
            const size_t n = (size_t)p->cfg.vocab * p->cfg.d_model;
            if (!p->eb) {
                cudaError_t er = cudaMalloc((void**)&p->eb, n * sizeof(__nv_bfloat16));
                if (er != cudaSuccess) {
                    cudaGetLastError();
                    NNB_FAIL(NNB_ERR_OOM, "out of device memory for the bf16 embedding copy");
                }
            }
            NNB_TRY(launch_f32_to_bf16(p->e, p->params + p->tok_emb, n, p->eb));
        }
    }
    return NNB_OK;
}

nnb_status policy_tied_head_fwd(nnb_policy* p, const float* hn, __nv_bfloat16* hnb, size_t T, float* logits)
{
    const size_t d = p->cfg.d_model, V = p->cfg.vocab;
    if (p->cfg.exact) return launch_dense_nt(p->e, true, hn, p->params + p->tok_emb, T, V, d, logits);
    NNB_REQUIRE(p->eb && hnb, "tied head: the bf16 embedding copy is missing");
    NNB_TRY(launch_f32_to_bf16(p->e, hn, T * d, hnb));
    if (T >= 64 && d % 8 == 0 && V % 4 == 0) return launch_tc_nt(p->e, hnb, p->eb, T, d, V, logits);
    return launch_dense_nt_bf16(p->e, hnb, p->eb, T, V, d, logits);
}

static void free_decode(nnb_policy* p)
{
    DecodeWs& w = p->dec;
    void* ptrs[] = {w.k, w.v, w.k_pre, w.v_pre, w.tokens_pre, w.x, w.qkv, w.att, w.pre_ml, w.h1, w.logits, w.q8, w.s, w.qsum, w.d_pos,
                    w.tokens, w.logp, w.done, w.gen_len, w.qkv_raw, w.act, w.hn, w.hnb, w.sample_rows};
    for (void* q : ptrs)
        if (q) cudaFree(q);
    w = DecodeWs();
}

void policy_free_decode(nnb_policy* p) { free_decode(p); }

// total positions = pre_len (shared prefix, one copy per group) + ctx_alloc (per sequence)
// tok_cols: columns of the token / log-prob buffers (the whole sequence, which outgrows the cache once the
// context window slides)
static nnb_status ensure_decode(nnb_policy* p, size_t B, size_t ctx_alloc, size_t group, size_t pre_len, size_t tok_cols)
{
    DecodeWs& w = p->dec;
    if (w.B == B && w.ctx_alloc == ctx_alloc && w.group == group && w.pre_len == pre_len && w.tok_cols == tok_cols) return NNB_OK;
    NNB_CUDA(cudaStreamSynchronize(p->e->stream));
    free_decode(p);
    const nnb_gpt_config& c = p->cfg;
    const size_t d = c.d_model, F = c.d_ff, V = c.vocab, F1 = act_gated(c.act) ? 2 * F : F;
    const size_t kv_elem = c.exact ? 4 : 2;
    const size_t dkv = cfg_kv_heads(c) * attn_decode_kv_pitch(c.exact != 0, d / c.n_head);  // cached features per position
    const size_t kv_bytes = (size_t)c.n_layer * B * dkv * ctx_alloc * kv_elem;
    const size_t pre_bytes = (size_t)c.n_layer * (B / group) * dkv * pre_len * kv_elem;
    const size_t total = tok_cols;
    size_t free_b = 0, total_b = 0;
    NNB_CUDA(cudaMemGetInfo(&free_b, &total_b));
    const size_t need = 2 * (kv_bytes + pre_bytes) + B * (d * 4 * 5 + F1 * 4 + V * 4 + (F > d ? F : d) + total * 8) + (64u << 20);
    if (need > free_b)
        NNB_FAIL(NNB_ERR_OOM, "rollout of %zu sequences x %zu positions needs %.1f GB (KV cache %.1f GB), %.1f GB free",
                 B, total, need / 1e9, 2 * (kv_bytes + pre_bytes) / 1e9, free_b / 1e9);
#define NNB_ALLOC(ptr, bytes)                                                          \
    do {                                                                               \
        cudaError_t er__ = cudaMalloc((void**)&(ptr), (bytes));                        \
        if (er__ != cudaSuccess) {                                                     \
            cudaGetLastError();                                                        \
            free_decode(p);                                                            \
            NNB_FAIL(NNB_ERR_OOM, "cudaMalloc(%zu) failed: %s", (size_t)(bytes), cudaGetErrorString(er__)); \
        }                                                                              \
    } while (0)
    NNB_ALLOC(w.k, kv_bytes);
    NNB_ALLOC(w.v, kv_bytes);
    if (pre_len > 0) {
        NNB_ALLOC(w.k_pre, pre_bytes);
        NNB_ALLOC(w.v_pre, pre_bytes);
        NNB_ALLOC(w.tokens_pre, (B / group) * pre_len * 4);
    }
    NNB_ALLOC(w.x, B * d * 4);
    NNB_ALLOC(w.qkv, 3 * B * d * 4);
    NNB_ALLOC(w.att, B * d * 4);
    NNB_ALLOC(w.pre_ml, B * c.n_head * 2 * 4);
    NNB_ALLOC(w.h1, B * F1 * 4);
    NNB_ALLOC(w.logits, B * V * 4);
    NNB_ALLOC(w.q8, B * (F > d ? F : d));
    NNB_ALLOC(w.s, B * 4);
    NNB_ALLOC(w.qsum, B * 4);
    NNB_ALLOC(w.d_pos, 16);
    NNB_ALLOC(w.tokens, B * total * 4);
    NNB_ALLOC(w.logp, B * total * 4);
    NNB_ALLOC(w.done, B * 4);
    NNB_ALLOC(w.gen_len, B * 4);
    if (cfg_gqa(c)) NNB_ALLOC(w.qkv_raw, B * (d + 2 * cfg_kv_heads(c) * (d / c.n_head)) * 4);
    if (!sample_row_in_smem(V)) NNB_ALLOC(w.sample_rows, B * ((V + 3) & ~(size_t)3) * 4);
    if (c.tie_embeddings) {
        NNB_ALLOC(w.hn, B * d * 4);
        NNB_ALLOC(w.hnb, B * d * 2);
    }
#undef NNB_ALLOC
    w.B = B;
    w.ctx_alloc = ctx_alloc;
    w.group = group;
    w.pre_len = pre_len;
    w.tok_cols = tok_cols;
    return NNB_OK;
}

// What one decode step runs on: either all sequences (own caches + shared prefix) or, while the shared
// prompt prefix is being filled, one representative per group writing the prefix cache.
struct StepView {
    size_t B;
    const int32_t* tokens;
    size_t tok_stride;
    void *k, *v;          // cache written by this step, per layer stride = layer_bytes
    size_t own_alloc, layer_bytes;
    const void *k_pre, *v_pre;
    size_t pre_len, pre_alloc, pre_layer_bytes, group;
};

// NNB_PDL=0 in the environment turns the programmatic launches of the decode step off (for A/B timing)
static bool pdl_enabled()
{
    static int v = -1;
    if (v < 0) {
        const char* s = getenv("NNB_PDL");
        v = (s && s[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

// one decode step at the position stored in d_pos: consumes tokens[:, pos], appends to the KV
// cache and, when with_head, samples tokens[:, pos+1]
static nnb_status decode_step(nnb_policy* p, const StepView& sv, bool with_head, const SampleOpts& so,
                              unsigned long long seed, unsigned seq0, int prompt_len, bool want_logp)
{
    nnb_engine* e = p->e;
    const nnb_gpt_config& c = p->cfg;
    DecodeWs& w = p->dec;
    const size_t B = sv.B, d = c.d_model, F = c.d_ff, V = c.vocab, H = c.n_head, dk = d / H;
    const size_t F1 = act_gated(c.act) ? 2 * F : F;
    const size_t Hkv = cfg_kv_heads(c);
    const bool gqa = cfg_gqa(c);
    const bool exact = c.exact != 0;
    const float* P = p->params;
    // The fast mode's step is ~200 short kernels, each of which waits for the one before it (pdl_wait) before
    // touching memory: let each become resident while its predecessor drains.
    struct PdlScope {
        nnb_engine* e;
        bool prev;
        PdlScope(nnb_engine* en, bool on) : e(en), prev(en->pdl) { e->pdl = on; }
        ~PdlScope() { e->pdl = prev; }
    } pdl_scope(e, !exact && pdl_enabled());

    NNB_TRY(launch_embed(e, P + p->tok_emb, c.pos == 0 ? P + p->pos_emb : nullptr, sv.tokens, sv.tok_stride, w.d_pos, B, d,
                         V, w.x));
    for (int l = 0; l < c.n_layer; ++l) {
        const LayerW& L = p->layers[l];
        NNB_TRY(launch_row_quant(e, 0, exact, w.x, P + L.ln1_g, B, d, d, w.q8, w.s, w.qsum, nullptr));
        AttnIn ain = attn_in_or_planes(nullptr, w.qkv, B, d);
        if (gqa) {
            // one matrix of d + 2 dkv rows; the attention kernels map query head h to KV head h / (H / Hkv) themselves and
            // the cache holds the Hkv heads only (the reference expands K and V to H heads instead: same numbers)
            const size_t wq = d + 2 * Hkv * dk;
            NNB_TRY(policy_linear_fwd(p, L.qkv, 1, w.q8, w.s, w.qsum, B, nullptr, w.qkv_raw, 0));
            ain = AttnIn{w.qkv_raw, w.qkv_raw + d, w.qkv_raw + d + Hkv * dk, (int)wq, (int)(H / Hkv)};
        } else {
            // q, k, v projections: three equally shaped matrices stored back to back, one launch
            NNB_TRY(policy_linear_fwd(p, L.q, 3, w.q8, w.s, w.qsum, B, nullptr, w.qkv, B * d));
        }
        void* kl = (char*)sv.k + (size_t)l * sv.layer_bytes;
        void* vl = (char*)sv.v + (size_t)l * sv.layer_bytes;
        const void* kpl = sv.k_pre ? (const char*)sv.k_pre + (size_t)l * sv.pre_layer_bytes : nullptr;
        const void* vpl = sv.v_pre ? (const char*)sv.v_pre + (size_t)l * sv.pre_layer_bytes : nullptr;
        // The attention kernel lives on memory-level parallelism through L1; overlapped with a kernel that claims
        // the whole shared-memory carve-out (the GEMMs) it loses a third of its bandwidth (measured).  So it and the
        // projection after it are launched the plain way: each starts on a drained GPU.
        const bool pdl_saved = e->pdl;
        e->pdl = false;
        // One CTA per sequence needs a few hundred sequences to fill the GPU.  Below about one wave of per-head CTAs
        // (16 resident per SM) the kernel with one CTA per (sequence, head), four warps splitting the keys, has
        // several times the loads in flight and wins, the separate quantisation launch included.
        static int few_ctas = -1;  // NNB_FEW_CTAS in the environment: (sequence, head) CTAs per SM up to which the per-head path runs
        if (few_ctas < 0) {
            const char* ev = getenv("NNB_FEW_CTAS");
            few_ctas = ev ? atoi(ev) : 16;
            if (few_ctas < 0) few_ctas = 0;
        }
        const bool few = B * H <= (size_t)e->sm_count * (size_t)few_ctas;
        if (!exact && !few && !c.sub_ln && !gqa && attn_decode_fused_supported(H, dk) && d % 64 == 0) {
            // all heads of a sequence in one CTA, attention output quantised in the same launch.  (Not with SubLN, which
            // normalises the row first, nor with grouped queries: measured on the 2B4T shape, the warps of a KV group drift
            // apart and re-read their cache rows through L2, 0.0059 ms per position against 0.0051 for per-head CTAs.)
            NNB_TRY(launch_attn_decode_fused(e, w.qkv, kl, vl, sv.own_alloc, kpl, vpl, sv.pre_len, sv.pre_alloc, sv.group,
                                             c.pos == 1 ? p->rope_cos : nullptr, c.pos == 1 ? p->rope_sin : nullptr, w.d_pos, B, H,
                                             dk, nullptr, w.q8, w.s, w.qsum, w.att, w.pre_ml, &ain));
        } else {
            NNB_TRY(launch_attn_decode(e, exact, w.qkv, kl, vl, sv.own_alloc, kpl, vpl, sv.pre_len, sv.pre_alloc, sv.group,
                                       p->rope_cos, p->rope_sin, w.d_pos, B, H, dk, w.att, attn_decode_kv_pitch(exact, dk), &ain));
            // SubLN: the heads' output is normalised before it is quantised for the o projection
            NNB_TRY(launch_row_quant(e, c.sub_ln ? 0 : 3, exact, w.att, c.sub_ln ? P + L.attn_sub_g : nullptr, B, d, d, w.q8, w.s,
                                     w.qsum, nullptr));
        }
        {
            const nnb_status so = policy_linear_fwd(p, L.o, 1, w.q8, w.s, w.qsum, B, w.x, w.x, 0);
            e->pdl = pdl_saved;
            NNB_TRY(so);
        }
        NNB_TRY(launch_row_quant(e, 0, exact, w.x, P + L.ln2_g, B, d, d, w.q8, w.s, w.qsum, nullptr));
        const bool h1_b16 = policy_h1_bf16(p, B, F, F1);  // the buffer keeps its f32 size
        NNB_TRY(policy_linear_fwd(p, L.fc1, 1, w.q8, w.s, w.qsum, B, nullptr, w.h1, 0, h1_b16));
        // SubLN: the activated hidden is normalised, then quantised for fc2, in the same launch
        NNB_TRY(launch_row_quant(e, act_quant_mode(c.act), exact, w.h1, c.sub_ln ? P + L.ffn_sub_g : nullptr, B, F, F1, w.q8, w.s,
                                 w.qsum, nullptr, c.sub_ln != 0, h1_b16));
        NNB_TRY(policy_linear_fwd(p, L.fc2, 1, w.q8, w.s, w.qsum, B, w.x, w.x, 0));
    }
    if (with_head) {
        const size_t total = w.tok_cols;  // row pitch of the token / log-prob buffers
        NNB_TRY(launch_row_quant(e, 0, exact, w.x, P + p->lnf_g, B, d, d, w.q8, w.s, w.qsum, c.tie_embeddings ? w.hn : nullptr));
        if (c.tie_embeddings) NNB_TRY(policy_tied_head_fwd(p, w.hn, w.hnb, B, w.logits));
        else NNB_TRY(policy_linear_fwd(p, p->head, 1, w.q8, w.s, w.qsum, B, nullptr, w.logits, 0));
        SampleOpts so_rows = so;
        so_rows.row_scratch = w.sample_rows;
        NNB_TRY(launch_sample_opts(e, exact, w.logits, B, V, so_rows, seed, seq0, w.d_pos, prompt_len, w.tokens, total,
                                   want_logp ? w.logp : nullptr, total, nullptr));
    }
    return launch_add_int(e, w.d_pos, 1);  // the position lives on the device so a captured step can be replayed
}

// One decode step is ~10 launches per layer; at decode sizes the host cannot issue them as fast as the
// GPU retires them.  The first step of each kind runs eagerly, the second is captured into a CUDA
// graph, and every later step of that kind replays the graph.
struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    unsigned long long launches = 0;
    int seen = 0;
};

static nnb_status run_step(nnb_policy* p, StepGraph& g, bool allow_graph, const StepView& sv, bool with_head, const SampleOpts& so,
                           unsigned long long seed, unsigned seq0, int prompt_len, bool want_logp)
{
    nnb_engine* e = p->e;
    if (g.exec) {
        NNB_CUDA(cudaGraphLaunch(g.exec, e->stream));
        e->launches += g.launches;
        return NNB_OK;
    }
    if (g.seen == 0 || !allow_graph) {
        g.seen = 1;
        return decode_step(p, sv, with_head, so, seed, seq0, prompt_len, want_logp);
    }
    NNB_CUDA(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
    const unsigned long long l0 = e->launches;
    const nnb_status cs = decode_step(p, sv, with_head, so, seed, seq0, prompt_len, want_logp);
    cudaGraph_t graph = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(e->stream, &graph);
    if (cs != NNB_OK) {
        if (graph) cudaGraphDestroy(graph);
        return cs;
    }
    if (ce != cudaSuccess) NNB_FAIL(NNB_ERR_CUDA, "stream capture of a decode step failed: %s", cudaGetErrorString(ce));
    g.launches = e->launches - l0;
    const cudaError_t ie = cudaGraphInstantiate(&g.exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) NNB_FAIL(NNB_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(ie));
    NNB_CUDA(cudaGraphLaunch(g.exec, e->stream));
    return NNB_OK;
}

// group > 1: sequences [g*group, (g+1)*group) were given the same prompt.  Their first P-1 prompt
// positions are computed once per group (batch B/group) into a prefix cache that all members read;
// from position P-1 on every sequence runs on its own.  The arithmetic per sequence is unchanged.
nnb_status policy_rollout(nnb_policy* p, const int32_t* d_prompts, size_t B, size_t P, size_t max_new, size_t group,
                          const SampleOpts& so_in, unsigned long long seed, unsigned seq0,
                          int32_t* d_tokens, float* d_logp, float* d_logits, int32_t* d_gen_len)
{
    NNB_REQUIRE(p && d_prompts && d_tokens, "rollout: NULL argument");
    NNB_REQUIRE(B > 0 && P > 0 && max_new > 0, "rollout: empty shape");
    NNB_REQUIRE(group >= 1 && B % group == 0, "rollout: %zu sequences do not divide into groups of %zu", B, group);
    NNB_REQUIRE(p->cfg.ctx >= 2 || P + max_new <= (size_t)p->cfg.ctx, "rollout: a context of %d cannot slide", p->cfg.ctx);
    nnb_engine* e = p->e;
    const nnb_gpt_config& c = p->cfg;
    const size_t total = P + max_new;
    // A sequence that outgrows the context is generated the way GPTModel::generate does it
    // (include/neuralnet.cpp/compute_layer_gpt.hpp:768-818): the window keeps the last ctx-1 tokens and is rebuilt
    // from position 0 before every further token.  Positions then differ between the members of a group only by
    // their tokens, but the shared prefix cache assumes fixed positions, so it is not used in that case.
    const size_t ctx = (size_t)c.ctx;
    const bool windowed = total > ctx;
    if (windowed) group = 1;
    const size_t pre_len = (group > 1 && P > 1) ? P - 1 : 0;
    const size_t own = (windowed ? ctx : total) - pre_len;
    NNB_TRY(ensure_decode(p, B, own, group, pre_len, total));
    DecodeWs& w = p->dec;
    SampleOpts so = so_in;
    if (so.eos >= 0 || d_gen_len) {
        so.done = w.done;
        so.gen_len = w.gen_len;
    }
    const size_t V = c.vocab, d = c.d_model;
    const size_t kv_elem = c.exact ? 4 : 2;
    const size_t dkv = cfg_kv_heads(c) * attn_decode_kv_pitch(c.exact != 0, d / c.n_head);
    const size_t Bg = B / group;
    StepView main_view{B, w.tokens, total, w.k, w.v, own, B * dkv * own * kv_elem, w.k_pre, w.v_pre, pre_len, pre_len,
                       Bg * dkv * pre_len * kv_elem, group};
    StepView pre_view{Bg, w.tokens_pre, pre_len, w.k_pre, w.v_pre, pre_len, Bg * dkv * pre_len * kv_elem, nullptr, nullptr, 0, 0, 0, 1};

    // the steps run on the engine's own stream (graph capture is not possible on the legacy default
    // stream); it is ordered after and before the caller's stream with events
    cudaStream_t user = e->stream;
    const bool swap = user != e->own_stream;
    cudaEvent_t ev = nullptr;
    if (swap) {
        NNB_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        NNB_CUDA(cudaEventRecord(ev, user));
        NNB_CUDA(cudaStreamWaitEvent(e->own_stream, ev, 0));
        e->stream = e->own_stream;
    }
    StepGraph graphs[3];  // prefix fill, own steps without head, own steps with head
    auto run = [&]() -> nnb_status {
        NNB_CUDA(cudaMemcpy2DAsync(w.tokens, total * 4, d_prompts, P * 4, P * 4, B, cudaMemcpyDeviceToDevice, e->stream));
        if (pre_len > 0)  // prompt of the first member of every group, without its last token
            NNB_CUDA(cudaMemcpy2DAsync(w.tokens_pre, pre_len * 4, d_prompts, group * P * 4, pre_len * 4, Bg,
                                       cudaMemcpyDeviceToDevice, e->stream));
        NNB_TRY(launch_set_int(e, w.d_pos, 0));
        if (so.done) {
            NNB_CUDA(cudaMemsetAsync(w.done, 0, B * 4, e->stream));
            NNB_TRY(launch_fill_int(e, w.gen_len, B, (int)max_new));
        }
        const bool allow_graph = total >= 8;
        size_t t0 = 0;
        if (pre_len > 0 && policy_can_prefill(p)) {
            // fast mode: the shared prompt prefixes go through one teacher-forced forward (all positions at once)
            // that leaves every layer's keys and values in the prefix cache, instead of pre_len decode steps
            NNB_TRY(policy_prefill_prefix(p, w.tokens_pre, Bg, pre_len, w.k_pre, w.v_pre, pre_len, Bg * dkv * pre_len * kv_elem));
            NNB_TRY(launch_set_int(e, w.d_pos, (int)pre_len));
            t0 = pre_len;
        }
        auto mark = [&](size_t t) -> nnb_status {
            cudaEvent_t evt = nullptr;
            NNB_CUDA(cudaEventCreate(&evt));
            p->time_events.push_back(evt);
            p->time_pos.push_back((int)t);
            NNB_CUDA(cudaEventRecord(evt, e->stream));
            return NNB_OK;
        };
        if (p->time_stride) {
            for (cudaEvent_t evt : p->time_events) cudaEventDestroy(evt);
            p->time_events.clear();
            p->time_pos.clear();
        }
        if (windowed) {
            size_t cur = 0;  // tokens in the window = position of the next one
            const size_t col0 = P > ctx ? P - ctx : 0;  // a prompt longer than the context is cut to its tail
            NNB_TRY(launch_set_int2(e, w.d_pos, 0, (int)col0));
            for (size_t col = col0; col + 1 < total; ++col) {
                const bool with_head = col + 1 >= P;
                if (with_head && cur + 1 >= ctx) {
                    // the window is full: it becomes the ctx-1 tokens that end at this column, from position 0
                    const size_t start = col + 1 - (ctx - 1);
                    NNB_TRY(launch_set_int2(e, w.d_pos, 0, (int)start));
                    cur = 0;
                    for (size_t i = start; i < col; ++i, ++cur)
                        NNB_TRY(run_step(p, graphs[1], allow_graph, main_view, false, so, seed, seq0, (int)P, false));
                }
                NNB_TRY(run_step(p, graphs[with_head ? 2 : 1], allow_graph, main_view, with_head, so, seed, seq0, (int)P,
                                 d_logp != nullptr));
                ++cur;
                if (with_head && d_logits) {
                    const size_t gi = col + 1 - P;
                    NNB_CUDA(cudaMemcpy2DAsync(d_logits + gi * V, max_new * V * 4, w.logits, V * 4, V * 4, B,
                                               cudaMemcpyDeviceToDevice, e->stream));
                }
            }
            return NNB_OK;
        }
        for (size_t t = t0; t + 1 < total; ++t) {
            if (p->time_stride && (t - t0) % p->time_stride == 0) NNB_TRY(mark(t));
            if (t < pre_len) {
                NNB_TRY(run_step(p, graphs[0], allow_graph, pre_view, false, so, seed, seq0, (int)P, false));
                continue;
            }
            const bool with_head = t + 1 >= P;
            NNB_TRY(run_step(p, graphs[with_head ? 2 : 1], allow_graph, main_view, with_head, so, seed, seq0,
                             (int)P, d_logp != nullptr));
            if (with_head && d_logits) {
                const size_t gi = t + 1 - P;
                NNB_CUDA(cudaMemcpy2DAsync(d_logits + gi * V, max_new * V * 4, w.logits, V * 4, V * 4, B,
                                           cudaMemcpyDeviceToDevice, e->stream));
            }
        }
        if (p->time_stride) NNB_TRY(mark(total - 1));
        return NNB_OK;
    };
    const nnb_status st = run();
    for (auto& g : graphs)
        if (g.exec) {
            cudaStreamSynchronize(e->stream);
            cudaGraphExecDestroy(g.exec);
        }
    if (st != NNB_OK) {
        if (swap) {
            cudaStreamSynchronize(e->own_stream);
            e->stream = user;
            cudaEventDestroy(ev);
        }
        return st;
    }
    NNB_CUDA(cudaMemcpyAsync(d_tokens, w.tokens, B * total * 4, cudaMemcpyDeviceToDevice, e->stream));
    if (d_logp)
        NNB_CUDA(cudaMemcpy2DAsync(d_logp, max_new * 4, w.logp, total * 4, max_new * 4, B,
                                   cudaMemcpyDeviceToDevice, e->stream));
    if (d_gen_len) NNB_CUDA(cudaMemcpyAsync(d_gen_len, w.gen_len, B * 4, cudaMemcpyDeviceToDevice, e->stream));
    if (swap) {
        NNB_CUDA(cudaEventRecord(ev, e->own_stream));
        NNB_CUDA(cudaStreamWaitEvent(user, ev, 0));
        e->stream = user;
        NNB_CUDA(cudaEventDestroy(ev));
    }
    return NNB_OK;
}

}  // namespace nnb

using namespace nnb;

extern "C" {

nnb_status nnb_policy_create(nnb_engine* e, const nnb_gpt_config* cfg, nnb_policy** out)
{
    NNB_REQUIRE(e && cfg && out, "policy_create: NULL argument");
    *out = nullptr;
    const nnb_gpt_config& c = *cfg;
    NNB_REQUIRE(c.n_layer > 0 && c.d_model > 0 && c.n_head > 0 && c.d_ff > 0 && c.vocab > 0 && c.ctx > 0,
                "policy_create: non-positive dimension");
    NNB_REQUIRE(c.d_model % c.n_head == 0, "policy_create: d_model %d not divisible by n_head %d", c.d_model, c.n_head);
    NNB_REQUIRE(c.d_model % 64 == 0 && c.d_ff % 64 == 0,
                "policy_create: d_model and d_ff must be multiples of 64 (got %d, %d)", c.d_model, c.d_ff);
    const int dk = c.d_model / c.n_head;
    NNB_REQUIRE(dk % 4 == 0 && dk <= 128, "policy_create: head dim %d unsupported (multiple of 4, <= 128)", dk);
    NNB_REQUIRE(c.act >= 0 && c.act <= 2, "policy_create: act must be 0 (QuickGELU), 1 (SwiGLU) or 2 (ReLU2GLU)");
    NNB_REQUIRE(c.pos == 0 || c.pos == 1, "policy_create: pos must be 0 (learned) or 1 (RoPE)");
    NNB_REQUIRE(c.pos == 0 || dk % 2 == 0, "policy_create: RoPE needs an even head dim");
    NNB_REQUIRE(c.n_head_kv >= 0 && (c.n_head_kv == 0 || (c.n_head_kv <= c.n_head && c.n_head % c.n_head_kv == 0)),
                "policy_create: n_head_kv %d must divide n_head %d", c.n_head_kv, c.n_head);
    nnb_policy* p = new nnb_policy();
    p->e = e;
    p->cfg = c;
    build_layout(p);
    auto fail = [&](nnb_status st) {
        nnb_policy_destroy(p);
        return st;
    };
    if (cudaMalloc((void**)&p->params, p->n_params * 4) != cudaSuccess ||
        cudaMalloc((void**)&p->packed, p->packed_words * 4) != cudaSuccess ||
        cudaMalloc((void**)&p->tau, p->tau_count * 4) != cudaSuccess) {
        cudaGetLastError();
        nnb::set_error("policy_create: out of device memory for %zu parameters", p->n_params);
        return fail(NNB_ERR_OOM);
    }
    cudaMemsetAsync(p->params, 0, p->n_params * 4, e->stream);
    if (c.pos == 1) {
        // RotaryEmbedding::fill_pos_column_ (compute_position_encoding.hpp:64-80): f32 host tables
        const int half = dk / 2;
        std::vector<float> cs((size_t)c.ctx * half), sn((size_t)c.ctx * half);
        for (int pos = 0; pos < c.ctx; ++pos)
            for (int j = 0; j < half; ++j) {
                const float theta = (float)pos / powf(10000.0f, (float)(2 * j) / (float)dk);
                cs[(size_t)pos * half + j] = cosf(theta);
                sn[(size_t)pos * half + j] = sinf(theta);
            }
        if (cudaMalloc((void**)&p->rope_cos, cs.size() * 4) != cudaSuccess ||
            cudaMalloc((void**)&p->rope_sin, sn.size() * 4) != cudaSuccess) {
            cudaGetLastError();
            nnb::set_error("policy_create: out of device memory for RoPE tables");
            return fail(NNB_ERR_OOM);
        }
        cudaMemcpyAsync(p->rope_cos, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, e->stream);
        cudaMemcpyAsync(p->rope_sin, sn.data(), sn.size() * 4, cudaMemcpyHostToDevice, e->stream);
        cudaStreamSynchronize(e->stream);
    }
    *out = p;
    return NNB_OK;
}

void nnb_policy_destroy(nnb_policy* p)
{
    if (!p) return;
    cudaStreamSynchronize(p->e->stream);
    for (cudaEvent_t evt : p->time_events) cudaEventDestroy(evt);
    free_decode(p);
    policy_free_train(p);
    void* ptrs[] = {p->params, p->grads, p->adam_m, p->adam_v, p->packed, p->tau, p->rope_cos, p->rope_sin, p->w8, p->wb, p->eb};
    for (void* q : ptrs)
        if (q) cudaFree(q);
    delete p;
}

size_t nnb_policy_param_count(const nnb_policy* p) { return p ? p->n_params : 0; }
float* nnb_policy_params(nnb_policy* p) { return p ? p->params : nullptr; }
size_t nnb_policy_tensor_count(const nnb_policy* p) { return p ? p->tensors.size() : 0; }

nnb_status nnb_policy_tensor_info(const nnb_policy* p, size_t index, char* name, size_t name_len,
                                  size_t* offset, size_t* rows, size_t* cols)
{
    NNB_REQUIRE(p && index < p->tensors.size(), "policy_tensor_info: index out of range");
    const TensorInfo& t = p->tensors[index];
    if (name && name_len) snprintf(name, name_len, "%s", t.name.c_str());
    if (offset) *offset = t.offset;
    if (rows) *rows = t.rows;
    if (cols) *cols = t.cols;
    return NNB_OK;
}

nnb_status nnb_policy_upload_params(nnb_policy* p, const float* h_params)
{
    NNB_REQUIRE(p && h_params, "policy_upload_params: NULL argument");
    NNB_CUDA(cudaMemcpyAsync(p->params, h_params, p->n_params * 4, cudaMemcpyHostToDevice, p->e->stream));
    NNB_TRY(policy_requantize(p));
    NNB_CUDA(cudaStreamSynchronize(p->e->stream));
    return NNB_OK;
}

nnb_status nnb_policy_requantize(nnb_policy* p)
{
    NNB_REQUIRE(p, "policy is NULL");
    return policy_requantize(p);
}

nnb_status nnb_policy_linear(nnb_policy* p, int layer, int which, uint32_t** d_packed, float** d_tau,
                             size_t* in, size_t* out)
{
    NNB_REQUIRE(p, "policy is NULL");
    const LinW* l = nullptr;
    if (layer < 0) {
        NNB_REQUIRE(!p->cfg.tie_embeddings, "policy_linear: a policy with tied embeddings has no head linear");
        l = &p->head;
    } else {
        NNB_REQUIRE(layer < p->cfg.n_layer && which >= 0 && which < 6, "policy_linear: bad index");
        LayerW& L = p->layers[layer];
        const LinW* all[6] = {&L.q, &L.k, &L.v, &L.o, &L.fc1, &L.fc2};
        l = all[which];
    }
    if (d_packed) *d_packed = p->packed + l->packed_off;
    if (d_tau) *d_tau = p->tau + l->tau_off;
    if (in) *in = l->in;
    if (out) *out = l->out;
    return NNB_OK;
}

nnb_status nnb_rollout_set_step_timing(nnb_policy* p, size_t stride)
{
    NNB_REQUIRE(p, "policy is NULL");
    p->time_stride = stride;
    return NNB_OK;
}

nnb_status nnb_rollout_step_times(nnb_policy* p, float* h_ms, int32_t* h_pos, size_t cap, size_t* n_out)
{
    NNB_REQUIRE(p && n_out, "rollout_step_times: NULL argument");
    const size_t n = p->time_events.size() > 1 ? p->time_events.size() - 1 : 0;
    *n_out = n;
    if (!h_ms || n == 0) return NNB_OK;
    NNB_CUDA(cudaEventSynchronize(p->time_events.back()));
    for (size_t i = 0; i < n && i < cap; ++i) {
        NNB_CUDA(cudaEventElapsedTime(&h_ms[i], p->time_events[i], p->time_events[i + 1]));
        if (h_pos) h_pos[i] = p->time_pos[i];
    }
    return NNB_OK;
}

nnb_status nnb_rollout(nnb_policy* p, const int32_t* d_prompts, size_t n_seq, size_t prompt_len,
                       size_t max_new, float temperature, int top_k, uint64_t seed, uint32_t seq0,
                       int32_t* d_tokens, float* d_logp, float* d_logits)
{
    SampleOpts so;
    so.temperature = temperature;
    so.top_k = top_k;
    return policy_rollout(p, d_prompts, n_seq, prompt_len, max_new, 1, so, seed, seq0, d_tokens, d_logp, d_logits, nullptr);
}

nnb_status nnb_rollout_sampled(nnb_policy* p, const int32_t* d_prompts, size_t n_seq, size_t prompt_len, size_t max_new,
                               size_t group_size, const nnb_sampling_config* cfg, uint32_t seq0, int32_t* d_tokens,
                               float* d_logp, float* d_logits, int32_t* d_gen_len)
{
    NNB_REQUIRE(cfg, "rollout_sampled: sampling configuration is NULL");
    NNB_REQUIRE(cfg->top_k >= 0 && cfg->repeat_window >= 0 && cfg->min_new_tokens >= 0, "rollout_sampled: negative count");
    SampleOpts so;
    so.temperature = cfg->temperature;
    so.top_k = cfg->top_k;
    so.top_p = cfg->top_p;
    so.repeat_penalty = cfg->repeat_penalty;
    so.repeat_window = cfg->repeat_window;
    so.logit_bias = cfg->d_logit_bias;
    so.eos = cfg->eos_token;
    so.min_new = cfg->min_new_tokens;
    return policy_rollout(p, d_prompts, n_seq, prompt_len, max_new, group_size ? group_size : 1, so, cfg->seed, seq0, d_tokens,
                          d_logp, d_logits, d_gen_len);
}

nnb_status nnb_rollout_grouped(nnb_policy* p, const int32_t* d_prompts, size_t n_seq, size_t prompt_len, size_t max_new,
                               size_t group_size, float temperature, int top_k, uint64_t seed, uint32_t seq0,
                               int32_t* d_tokens, float* d_logp, float* d_logits)
{
    SampleOpts so;
    so.temperature = temperature;
    so.top_k = top_k;
    return policy_rollout(p, d_prompts, n_seq, prompt_len, max_new, group_size, so, seed, seq0, d_tokens, d_logp, d_logits,
                          nullptr);
}

nnb_status nnb_rollout_host(nnb_policy* p, const int32_t* h_prompts, size_t n_seq, size_t prompt_len,
                            size_t max_new, float temperature, int top_k, uint64_t seed, uint32_t seq0,
                            int32_t* h_tokens, float* h_logp)
{
    NNB_REQUIRE(p && h_prompts && h_tokens, "rollout_host: NULL argument");
    nnb_engine* e = p->e;
    const size_t total = prompt_len + max_new;
    auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
    const size_t pb = al(n_seq * prompt_len * 4), tb = al(n_seq * total * 4), lb = al(n_seq * max_new * 4);
    NNB_TRY(e->ensure_scratch(pb + tb + lb));
    char* base = (char*)e->scratch;
    int32_t* d_prompts = (int32_t*)base;
    int32_t* d_tokens = (int32_t*)(base + pb);
    float* d_logp = (float*)(base + pb + tb);
    NNB_CUDA(cudaMemcpyAsync(d_prompts, h_prompts, n_seq * prompt_len * 4, cudaMemcpyHostToDevice, e->stream));
    SampleOpts so;
    so.temperature = temperature;
    so.top_k = top_k;
    NNB_TRY(policy_rollout(p, d_prompts, n_seq, prompt_len, max_new, 1, so, seed, seq0, d_tokens, h_logp ? d_logp : nullptr,
                           nullptr, nullptr));
    NNB_CUDA(cudaMemcpyAsync(h_tokens, d_tokens, n_seq * total * 4, cudaMemcpyDeviceToHost, e->stream));
    if (h_logp)
        NNB_CUDA(cudaMemcpyAsync(h_logp, d_logp, n_seq * max_new * 4, cudaMemcpyDeviceToHost, e->stream));
    NNB_CUDA(cudaStreamSynchronize(e->stream));
    return NNB_OK;
}

}  // extern "C"
