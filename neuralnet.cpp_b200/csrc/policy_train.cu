// policy_train.cu — teacher-forced forward, objective and backward of the ternary GPT policy,
// and the optimizer step.  Replaces the reference's
//   GPTModel::forward / backward            include/neuralnet.cpp/compute_layer_gpt.hpp:460-636
//   PpoObjective / GrpoObjective::evaluate  include/neuralnet.cpp/rl_policy.hpp:799-953
//   TrainingSession::train_named_step, finish_update_  include/neuralnet.cpp/training_session.hpp:322-467,599-638
// for one micro-batch of whole sequences.  Gradients accumulate (+=) into the policy's flat
// gradient buffer, as the reference's layers accumulate into their grad tensors; the caller
// runs as many micro-batches as it likes before nnb_policy_optimizer_step.
//
// Decisions: sequence b of length S with a prompt of P tokens has G = S - P decisions; decision g
// is taken at position P-1+g and its action is token P+g.  All per-decision vectors are (n_seq, G).
#include <utility>
#include <vector>

#include "common.cuh"
#include "policy.cuh"

namespace nnb {

struct LayerSave {
    float *x_in = nullptr, *qkv = nullptr, *att = nullptr, *lse = nullptr, *x_mid = nullptr, *h1 = nullptr;
    int8_t *q1 = nullptr, *q2 = nullptr, *q3 = nullptr, *q4 = nullptr;
    float *s1 = nullptr, *s2 = nullptr, *s3 = nullptr, *s4 = nullptr;
    __nv_bfloat16* qkvb = nullptr;  // fast mode: rotated q, k and v as bf16 (3, T, d), the attention operands
};

struct TrainWs {
    size_t n_seq = 0, S = 0, P = 0;
    // row layout of the micro-batch: with group > 1 the prompt rows of a group are stored and computed once
    SeqMap map{0, 0, 0, 1};
    size_t rows = 0;
    int32_t *row_tok = nullptr, *row_pos = nullptr;  // token and position of every row
    float* part = nullptr;                           // per-member share of the prefix rows' dK, dV (grouped backward)
    bool saved_layers = false;
    bool with_head = true;  // false: layers only (prompt prefill), no decision / logits buffers
    char* arena = nullptr;
    size_t arena_bytes = 0;
    std::vector<LayerSave> L;
    float* x_last = nullptr;  // output of the last block (T,d)
    int32_t* qsum = nullptr;
    // head
    int32_t* actions = nullptr;
    float *xd = nullptr, *hn = nullptr, *sh = nullptr, *logits = nullptr, *logp = nullptr, *ent = nullptr,
          *value = nullptr, *up_lp = nullptr, *up_ent = nullptr, *dvalue = nullptr, *dhn = nullptr, *report = nullptr,
          *vreport = nullptr;
    int8_t* qh = nullptr;
    // backward temporaries
    float *g = nullptr, *g2 = nullptr, *dn = nullptr, *datt = nullptr, *dqkv = nullptr, *da = nullptr, *dh1 = nullptr,
          *delta = nullptr;
    __nv_bfloat16 *dyb = nullptr, *xs = nullptr;  // bf16 operand scratch of the tcgen05 backward GEMMs
    __nv_bfloat16* dob = nullptr;                 // bf16 copy of the attention output gradient
    bool b16_attn = false;
    // fast mode: the LM head's GEMM computes log-prob / entropy in its epilogue and its backward operand is recomputed
    // from the same integer GEMM, so the (decisions x vocabulary) f32 logits do not exist
    bool fused_head = false;
    bool h1_b16 = false;  // the saved fc1 outputs hold bf16 elements
    float *lse = nullptr, *head_scratch = nullptr;
    ColsumSink bias_sink;  // bias-gradient partial sums of a whole backward pass, finished by one launch
    // structure switches
    float* qkv_raw = nullptr;  // grouped-query attention: (T, d + 2 dkv) projections (forward) / their gradients (backward)
    float *act = nullptr, *dact = nullptr;  // SubLN: (T, d_ff) activated hidden before its norm, and its gradient
    __nv_bfloat16* hnb = nullptr;           // tied embeddings, fast mode: bf16 copy of the head's input (Td, d)
};

static void free_ws(void*& slot)
{
    TrainWs* w = (TrainWs*)slot;
    if (!w) return;
    if (w->arena) cudaFree(w->arena);
    delete w;
    slot = nullptr;
}

void policy_free_train(nnb_policy* p)
{
    free_ws(p->train);
    free_ws(p->prefill);
}

static nnb_status ensure_train(nnb_policy* p, size_t n_seq, size_t S, size_t P, bool save_layers, size_t group,
                               bool with_head = true)
{
    TrainWs* w = (TrainWs*)p->train;
    {
        // sharing the prompt rows needs the bf16 attention kernels (they take the row map) and whole 64-row
        // key tiles inside the prompt; otherwise every sequence keeps its own copy, which is always valid
        const nnb_gpt_config& c0 = p->cfg;
        const bool can = !c0.exact && attn_b16_supported(c0.d_model / c0.n_head, c0.d_model) && P % 64 == 0 && group > 1 &&
                         n_seq % group == 0;
        if (!can) group = 1;
    }
    if (w && w->n_seq == n_seq && w->S == S && w->P == P && (size_t)w->map.group == group && w->with_head == with_head &&
        (w->saved_layers || !save_layers))
        return NNB_OK;
    NNB_CUDA(cudaStreamSynchronize(p->e->stream));
    free_ws(p->train);
    w = new TrainWs();
    p->train = w;
    const nnb_gpt_config& c = p->cfg;
    const size_t d = c.d_model, F = c.d_ff, F1 = act_gated(c.act) ? 2 * F : F, V = c.vocab, H = c.n_head;
    const size_t G = S - P, Td = with_head ? n_seq * G : 0;
    const size_t wqkv = d + 2 * cfg_kv_heads(c) * (d / H);
    const bool tie = c.tie_embeddings != 0;
    w->with_head = with_head;
    w->map = SeqMap{(int)S, (int)P, (int)G, (int)group};
    w->rows = map_rows_total(w->map, n_seq);
    const size_t T = w->rows;
    const size_t n_save = save_layers ? (size_t)c.n_layer : 1;
    // fast mode: attention runs on bf16 copies of q, k, v; those are what a layer keeps for its backward,
    // and the f32 projections become one buffer shared by all layers
    w->b16_attn = !c.exact && attn_b16_supported(d / H, d);
    w->h1_b16 = policy_h1_bf16(p, T, F, F1);
    w->fused_head = with_head && !tie && !c.exact && p->w8 != nullptr && V % 8 == 0 && Td >= 64;
    // carve one arena: first pass measures, second assigns
    for (int pass = 0; pass < 2; ++pass) {
        size_t off = 0;
        auto take = [&](size_t bytes) -> char* {
            char* ptr = w->arena ? w->arena + off : nullptr;
            off += (bytes + 255) & ~(size_t)255;
            return ptr;
        };
        w->L.assign(c.n_layer, LayerSave());
        for (size_t l = 0; l < n_save; ++l) {
            LayerSave s;
            s.x_in = (float*)take(T * d * 4);
            if (w->b16_attn) {
                s.qkv = l == 0 ? (float*)take(3 * T * d * 4) : w->L[0].qkv;
                s.qkvb = (__nv_bfloat16*)take(3 * T * d * 2);
            } else {
                s.qkv = (float*)take(3 * T * d * 4);
            }
            s.att = (float*)take(T * d * 4);
            s.lse = (float*)take(n_seq * H * S * 4);
            s.x_mid = (float*)take(T * d * 4);
            s.h1 = (float*)take(T * F1 * (w->h1_b16 ? 2 : 4));
            s.q1 = (int8_t*)take(T * d);
            s.q2 = (int8_t*)take(T * d);
            s.q3 = (int8_t*)take(T * d);
            s.q4 = (int8_t*)take(T * F);
            s.s1 = (float*)take(T * 4);
            s.s2 = (float*)take(T * 4);
            s.s3 = (float*)take(T * 4);
            s.s4 = (float*)take(T * 4);
            w->L[l] = s;
        }
        if (!save_layers)
            for (int l = 1; l < c.n_layer; ++l) w->L[l] = w->L[0];
        w->x_last = (float*)take(T * d * 4);
        if (cfg_gqa(c)) w->qkv_raw = (float*)take(T * wqkv * 4);
        if (c.sub_ln) w->act = (float*)take(T * F * 4);
        if (tie && !c.exact) w->hnb = (__nv_bfloat16*)take(Td * d * 2);
        w->qsum = (int32_t*)take(T * 4);
        w->row_tok = (int32_t*)take(T * 4);
        w->row_pos = (int32_t*)take(T * 4);
        w->actions = (int32_t*)take(Td * 4);
        w->xd = (float*)take(Td * d * 4);
        w->hn = (float*)take(Td * d * 4);
        w->qh = (int8_t*)take(Td * d);
        w->sh = (float*)take(Td * 4);
        if (w->fused_head) {
            w->lse = (float*)take(Td * 4);
            w->head_scratch = (float*)take(tc_lmhead_scratch_floats(Td, V) * 4);
        } else {
            w->logits = (float*)take(Td * V * 4);
        }
        w->logp = (float*)take(Td * 4);
        w->ent = (float*)take(Td * 4);
        w->value = (float*)take(Td * 4);
        w->up_lp = (float*)take(Td * 4);
        w->up_ent = (float*)take(Td * 4);
        w->dvalue = (float*)take(Td * 4);
        w->report = (float*)take(64);
        w->vreport = (float*)take(64);
        if (save_layers) {
            w->dhn = (float*)take(Td * d * 4);
            w->g = (float*)take(T * d * 4);
            w->g2 = (float*)take(T * d * 4);
            w->dn = (float*)take(T * d * 4);
            w->datt = (float*)take(T * d * 4);
            w->dqkv = (float*)take(3 * T * d * 4);
            w->da = (float*)take(T * F * 4);
            w->dh1 = (float*)take(T * F1 * 4);
            w->delta = (float*)take(n_seq * H * S * 4);
            if (c.sub_ln) w->dact = (float*)take(T * F * 4);
            if (!c.exact) {
                // widest operand written into dyb: fc1's (T, F1), the merged q|k|v gradient (T, 3d), the head's (Td, V)
                const size_t wide = F1 > 3 * d ? F1 : 3 * d;
                const size_t dyb_elems = T * wide > Td * V ? T * wide : Td * V;
                w->dyb = (__nv_bfloat16*)take(dyb_elems * 2);
                w->xs = (__nv_bfloat16*)take(T * (F > d ? F : d) * 2);
                if (w->b16_attn) w->dob = (__nv_bfloat16*)take(T * d * 2);
                if (group > 1) w->part = (float*)take(2 * n_seq * P * d * 4);
                // per linear: ceil(T / 128) chunks x out partial sums (q|k|v, o, fc1, fc2 of every layer)
                const size_t chunks = (T + 127) / 128;
                w->bias_sink.cap = chunks * (size_t)c.n_layer * (3 * d + d + F1 + d) + 64;
                w->bias_sink.buf = (float*)take(w->bias_sink.cap * 4);
                w->bias_sink.desc_cap = (size_t)c.n_layer * 6 + 8;
                w->bias_sink.d_descs = (ColsumDesc*)take(w->bias_sink.desc_cap * sizeof(ColsumDesc));
            }
        }
        if (pass == 0) {
            size_t free_b = 0, total_b = 0;
            NNB_CUDA(cudaMemGetInfo(&free_b, &total_b));
            if (off + (256u << 20) > free_b) {
                free_ws(p->train);
                NNB_FAIL(NNB_ERR_OOM, "training workspace for %zu sequences x %zu needs %.1f GB, %.1f GB free: use smaller micro-batches",
                         n_seq, S, off / 1e9, free_b / 1e9);
            }
            cudaError_t er = cudaMalloc((void**)&w->arena, off);
            if (er != cudaSuccess) {
                cudaGetLastError();
                free_ws(p->train);
                NNB_FAIL(NNB_ERR_OOM, "cudaMalloc(%zu) for the training workspace failed: %s", off, cudaGetErrorString(er));
            }
            w->arena_bytes = off;
        }
    }
    w->n_seq = n_seq;
    w->S = S;
    w->P = P;
    w->saved_layers = save_layers;
    return NNB_OK;
}

__global__ void gather_actions_kernel(const int32_t* __restrict__ tokens, int S, int P, int G, size_t n,
                                      int32_t* __restrict__ actions)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t b = i / G, g = i % G;
    actions[i] = tokens[b * S + P + g];
}

static nnb_status lin_fwd(nnb_policy* p, const LinW& l, size_t n_mats, const int8_t* q, const float* s,
                          const int32_t* qsum, size_t T, const float* residual, float* y, size_t y_stride)
{
    return policy_linear_fwd(p, l, n_mats, q, s, qsum, T, residual, y, y_stride);
}

// where the prompt prefill stores every layer's keys and values
struct KvSink {
    void *k, *v;
    size_t alloc, layer_bytes;
};

// teacher-forced forward of n_seq sequences; fills w->logp / w->ent / w->value for the decisions
static nnb_status forward(nnb_policy* p, const int32_t* tokens, size_t n_seq, size_t S, size_t P, bool want_entropy,
                          const KvSink* sink = nullptr)
{
    nnb_engine* e = p->e;
    const nnb_gpt_config& c = p->cfg;
    TrainWs* w = (TrainWs*)p->train;
    const size_t d = c.d_model, F = c.d_ff, F1 = act_gated(c.act) ? 2 * F : F, V = c.vocab, H = c.n_head, dk = d / H;
    const size_t T = w->rows, G = S - P, Td = n_seq * G;
    const bool exact = c.exact != 0;
    const bool grouped = w->map.group > 1;
    const size_t Hkv = cfg_kv_heads(c);
    const bool gqa = cfg_gqa(c);
    const float* PP = p->params;
    NNB_TRY(launch_build_rows(e, tokens, w->map, n_seq, w->row_tok, w->row_pos));
    NNB_TRY(launch_embed_rows_fwd(e, PP + p->tok_emb, c.pos == 0 ? PP + p->pos_emb : nullptr, w->row_tok, w->row_pos, T, d, V,
                                  w->L[0].x_in));
    for (int l = 0; l < c.n_layer; ++l) {
        const LayerW& LW = p->layers[l];
        LayerSave& s = w->L[l];
        float* x_out = (l + 1 < c.n_layer) ? w->L[l + 1].x_in : w->x_last;
        if (!w->saved_layers) x_out = (l % 2 == 0) ? w->x_last : w->L[0].x_in;  // ping-pong when nothing is kept
        const float* x_in = (!w->saved_layers) ? ((l % 2 == 0) ? w->L[0].x_in : w->x_last) : s.x_in;
        NNB_TRY(launch_row_quant(e, 0, exact, x_in, PP + LW.ln1_g, T, d, d, s.q1, s.s1, w->qsum, nullptr));
        if (gqa) {
            // one matrix of d + 2 dkv rows, then the KV heads are replicated: attention below is plain multi-head
            NNB_TRY(lin_fwd(p, LW.qkv, 1, s.q1, s.s1, w->qsum, T, nullptr, w->qkv_raw, 0));
            NNB_TRY(launch_gqa_expand(e, w->qkv_raw, T, H, Hkv, dk, s.qkv));
        } else {
            NNB_TRY(lin_fwd(p, LW.q, 3, s.q1, s.s1, w->qsum, T, nullptr, s.qkv, T * d));
        }
        if (w->b16_attn) {
            NNB_TRY(launch_rope_pack_b16(e, s.qkv, s.qkv + T * d, s.qkv + 2 * T * d, c.pos == 1 ? p->rope_cos : nullptr,
                                         c.pos == 1 ? p->rope_sin : nullptr, T, S, H, dk, s.qkvb, w->row_pos));
            if (sink)
                NNB_TRY(launch_kv_to_cache(e, s.qkvb + T * d, s.qkvb + 2 * T * d, n_seq, S, H, dk,
                                           (__nv_bfloat16*)((char*)sink->k + (size_t)l * sink->layer_bytes),
                                           (__nv_bfloat16*)((char*)sink->v + (size_t)l * sink->layer_bytes), sink->alloc, H / Hkv));
            NNB_TRY(launch_attn_fwd_b16(e, s.qkvb, s.qkvb + T * d, s.qkvb + 2 * T * d, n_seq, S, H, dk, s.att, s.lse, &w->map));
        } else {
            if (c.pos == 1) {
                NNB_TRY(launch_rope(e, s.qkv, p->rope_cos, p->rope_sin, T, S, H, dk, false));
                NNB_TRY(launch_rope(e, s.qkv + T * d, p->rope_cos, p->rope_sin, T, S, H, dk, false));
            }
            NNB_TRY(launch_attn_fwd(e, exact, s.qkv, s.qkv + T * d, s.qkv + 2 * T * d, n_seq, S, H, dk, s.att, s.lse));
        }
        // SubLN: the heads' output is normalised before it is quantised for the o projection
        NNB_TRY(launch_row_quant(e, c.sub_ln ? 0 : 3, exact, s.att, c.sub_ln ? PP + LW.attn_sub_g : nullptr, T, d, d, s.q2, s.s2,
                                 w->qsum, nullptr));
        NNB_TRY(lin_fwd(p, LW.o, 1, s.q2, s.s2, w->qsum, T, x_in, s.x_mid, 0));
        NNB_TRY(launch_row_quant(e, 0, exact, s.x_mid, PP + LW.ln2_g, T, d, d, s.q3, s.s3, w->qsum, nullptr));
        NNB_TRY(policy_linear_fwd(p, LW.fc1, 1, s.q3, s.s3, w->qsum, T, nullptr, s.h1, 0, w->h1_b16));
        // SubLN: the activated hidden is normalised, then quantised for fc2, in the same launch
        NNB_TRY(launch_row_quant(e, act_quant_mode(c.act), exact, s.h1, c.sub_ln ? PP + LW.ffn_sub_g : nullptr, T, F, F1, s.q4, s.s4,
                                 w->qsum, nullptr, c.sub_ln != 0, w->h1_b16));
        NNB_TRY(lin_fwd(p, LW.fc2, 1, s.q4, s.s4, w->qsum, T, s.x_mid, x_out, 0));
    }
    if (!w->with_head) return NNB_OK;
    const float* x_final = w->x_last;
    if (!w->saved_layers) x_final = (c.n_layer % 2 == 1) ? w->x_last : w->L[0].x_in;
    if (grouped) NNB_TRY(launch_gather_decisions_map(e, x_final, w->map, n_seq, d, w->xd));
    else NNB_TRY(launch_gather_decisions(e, x_final, n_seq, S, P, G, d, w->xd));
    gather_actions_kernel<<<(unsigned)ceil_div(Td, 256), 256, 0, e->stream>>>(tokens, (int)S, (int)P, (int)G, Td, w->actions);
    e->launches++;
    NNB_TRY(launch_row_quant(e, 0, exact, w->xd, PP + p->lnf_g, Td, d, d, w->qh, w->sh, w->qsum, w->hn));
    if (w->fused_head) {
        NNB_TRY(launch_tc_lmhead_fwd(e, w->qh, p->w8 + p->head.packed_off * 16, p->tau + p->head.tau_off, w->sh, PP + p->head.b_off,
                                     w->actions, Td, d, V, w->head_scratch, w->lse, w->logp, want_entropy ? w->ent : nullptr));
    } else {
        if (c.tie_embeddings) NNB_TRY(policy_tied_head_fwd(p, w->hn, w->hnb, Td, w->logits));
        else NNB_TRY(lin_fwd(p, p->head, 1, w->qh, w->sh, w->qsum, Td, nullptr, w->logits, 0));
        NNB_TRY(launch_categorical_fwd(e, w->logits, w->actions, Td, V, w->logp, want_entropy ? w->ent : nullptr));
    }
    if (c.value_head) NNB_TRY(launch_value_fwd(e, w->hn, PP + p->value_w, PP + p->value_b, Td, d, w->value));
    return NNB_OK;
}

// whether the tcgen05 backward serves a linear of `out` outputs at T tokens
static bool tc_bwd_ok(const nnb_policy* p, size_t out, size_t T)
{
    return !p->cfg.exact && p->wb && p->wb_valid && out % 8 == 0 && T >= 64;
}

// the layers' linears (T rows) park their bias-gradient partial sums in the workspace; the head (Td rows) finishes its own
static ColsumSink* sink_of(TrainWs* w, size_t rows) { return (w->bias_sink.buf && rows == w->rows) ? &w->bias_sink : nullptr; }

// the two GEMMs of a linear's backward on operands already prepared in the workspace: w->dyb (T, out) =
// bf16(dy*tau).  `out` may span several matrices stored one after the other (their weights, and so their
// weight gradients, are contiguous): one dX over the concatenated contraction, one dW for all rows.
static nnb_status lin_bwd_gemms(nnb_policy* p, const LinW& l, size_t out, const int8_t* q, const float* s, size_t T, float* dx,
                                bool accumulate_dx)
{
    nnb_engine* e = p->e;
    TrainWs* w = (TrainWs*)p->train;
    if (dx) NNB_TRY(launch_tc_dx(e, w->dyb, p->wb + l.packed_off * 16, T, l.in, out, dx, accumulate_dx));
    NNB_TRY(launch_dequant_to_bf16(e, q, s, T, l.in, w->xs));
    return launch_tc_dw(e, w->dyb, w->xs, T, l.in, out, p->grads + l.w_off);
}

static nnb_status lin_bwd(nnb_policy* p, const LinW& l, const float* dy, const int8_t* q, const float* s, size_t T,
                          float* dx, bool accumulate_dx)
{
    nnb_engine* e = p->e;
    const bool exact = p->cfg.exact != 0;
    TrainWs* w = (TrainWs*)p->train;
    if (tc_bwd_ok(p, l.out, T)) {
        // tcgen05 path: dyb = bf16(dy*tau) serves both GEMMs, xs = bf16(s*q) in natural feature order
        NNB_TRY(launch_scale_colsum(e, dy, p->tau + l.tau_off, T, l.out, w->dyb, p->grads + l.b_off, 0, sink_of(w, T)));
        return lin_bwd_gemms(p, l, l.out, q, s, T, dx, accumulate_dx);
    }
    if (dx) NNB_TRY(launch_bitlinear_dx(e, exact, dy, p->packed + l.packed_off, p->tau + l.tau_off, T, l.in, l.out, dx, accumulate_dx));
    NNB_TRY(launch_bitlinear_dw(e, exact, dy, q, s, p->tau + l.tau_off, T, l.in, l.out, p->grads + l.w_off));
    return launch_colsum_add(e, dy, T, l.out, p->grads + l.b_off);
}

static nnb_status backward(nnb_policy* p, const int32_t* tokens, size_t n_seq, size_t S, size_t P)
{
    nnb_engine* e = p->e;
    const nnb_gpt_config& c = p->cfg;
    TrainWs* w = (TrainWs*)p->train;
    const size_t d = c.d_model, F = c.d_ff, V = c.vocab, H = c.n_head, dk = d / H;
    const size_t T = w->rows, G = S - P, Td = n_seq * G;
    const bool grouped = w->map.group > 1;
    const float* PP = p->params;
    float* GG = p->grads;
    w->bias_sink.descs.clear();
    w->bias_sink.used = 0;
    const size_t Hkv = cfg_kv_heads(c), F1 = act_gated(c.act) ? 2 * F : F;
    const bool gqa = cfg_gqa(c), exact = c.exact != 0;
    if (c.tie_embeddings) {
        // the logits buffer holds d loss / d logits (Td, V).  dX = g . E and dE += g^T . hn, into the gradient that the
        // embedding lookup's backward adds to as well (compute_layer_gpt.hpp:556-575)
        if (!exact && p->eb && Td >= 64 && V % 8 == 0) {
            NNB_TRY(launch_f32_to_bf16(e, w->logits, Td * V, w->dyb));
            NNB_TRY(launch_tc_dx(e, w->dyb, p->eb, Td, d, V, w->dhn, false));
            NNB_TRY(launch_tc_dw(e, w->dyb, w->hnb, Td, d, V, GG + p->tok_emb));
        } else {
            NNB_TRY(launch_dense_nn(e, exact, w->logits, PP + p->tok_emb, Td, V, d, w->dhn));
            NNB_TRY(launch_dense_tn_acc(e, exact, w->logits, w->hn, Td, V, d, GG + p->tok_emb));
        }
    } else if (w->fused_head) {
        // w->dyb already holds bf16(dlogits * tau) and the bias gradient is done (launch_tc_lmhead_bwd)
        NNB_REQUIRE(tc_bwd_ok(p, V, Td), "fused LM head: the tensor-core backward is not available");
        NNB_TRY(lin_bwd_gemms(p, p->head, V, w->qh, w->sh, Td, w->dhn, false));
    } else {
        // head: logits buffer now holds dlogits
        NNB_TRY(lin_bwd(p, p->head, w->logits, w->qh, w->sh, Td, w->dhn, false));
    }
    if (c.value_head)
        // w->dn (T, d) is free until the layers' backward: scratch for the partial sums
        NNB_TRY(launch_value_bwd(e, w->hn, PP + p->value_w, w->dvalue, Td, d, w->dhn, GG + p->value_w, GG + p->value_b, w->dn, T * d));
    NNB_TRY(launch_rmsnorm_bwd(e, w->xd, PP + p->lnf_g, w->dhn, nullptr, Td, d, w->xd, GG + p->lnf_g));
    if (grouped) NNB_TRY(launch_scatter_decisions_map(e, w->xd, w->map, n_seq, d, w->g));
    else NNB_TRY(launch_scatter_decisions(e, w->xd, n_seq, S, P, G, d, w->g));
    for (int l = c.n_layer - 1; l >= 0; --l) {
        const LayerW& LW = p->layers[l];
        LayerSave& s = w->L[l];
        // feed-forward branch
        NNB_TRY(lin_bwd(p, LW.fc2, w->g, s.q4, s.s4, T, w->da, false));
        const float* da = w->da;
        if (c.sub_ln) {
            // SubLN: the activated hidden is recomputed from h1 (fc2's operands q4 / s4 are spent by now and serve as the
            // quantiser's scratch), the norm's backward turns d(normed) into d(activated)
            NNB_TRY(launch_row_quant(e, act_quant_mode(c.act), exact, s.h1, nullptr, T, F, F1, s.q4, s.s4, w->qsum, w->act,
                                     false, w->h1_b16));
            NNB_TRY(launch_rmsnorm_bwd(e, w->act, PP + LW.ffn_sub_g, w->da, nullptr, T, F, w->dact, GG + LW.ffn_sub_g));
            da = w->dact;
        }
        if (tc_bwd_ok(p, LW.fc1.out, T) && F % 2 == 0) {
            // the activation's backward writes the GEMM operand directly (no f32 round trip of dh1)
            NNB_TRY(launch_act_bwd_scale_colsum(e, act_bwd_mode(c.act), s.h1, da, p->tau + LW.fc1.tau_off, T, F, w->dyb,
                                                GG + LW.fc1.b_off, sink_of(w, T), w->h1_b16));
            NNB_TRY(lin_bwd_gemms(p, LW.fc1, LW.fc1.out, s.q3, s.s3, T, w->dn, false));
        } else {
            NNB_REQUIRE(!w->h1_b16, "backward: the bf16 fc1 output needs the tensor-core backward");
            NNB_TRY(launch_act_bwd(e, act_bwd_mode(c.act), s.h1, da, T, F, w->dh1));
            NNB_TRY(lin_bwd(p, LW.fc1, w->dh1, s.q3, s.s3, T, w->dn, false));
        }
        NNB_TRY(launch_rmsnorm_bwd(e, s.x_mid, PP + LW.ln2_g, w->dn, w->g, T, d, w->g2, GG + LW.ln2_g));
        // attention branch
        NNB_TRY(lin_bwd(p, LW.o, w->g2, s.q2, s.s2, T, w->datt, false));
        const float* datt = w->datt;
        if (c.sub_ln) {
            // SubLN: d(normed heads' output) -> d(heads' output); w->dn is free between the two branches
            NNB_TRY(launch_rmsnorm_bwd(e, s.att, PP + LW.attn_sub_g, w->datt, nullptr, T, d, w->dn, GG + LW.attn_sub_g));
            datt = w->dn;
        }
        if (w->b16_attn) {
            // the inverse rotation of dq and dk is part of the kernels' epilogues
            NNB_TRY(launch_attn_bwd_b16(e, s.qkvb, s.qkvb + T * d, s.qkvb + 2 * T * d, s.att, datt, s.lse, w->delta, w->dob,
                                        c.pos == 1 ? p->rope_cos : nullptr, c.pos == 1 ? p->rope_sin : nullptr, n_seq, S, H, dk,
                                        w->dqkv, w->dqkv + T * d, w->dqkv + 2 * T * d, &w->map, w->part));
        } else {
            NNB_TRY(launch_attn_bwd(e, c.exact != 0, s.qkv, s.qkv + T * d, s.qkv + 2 * T * d, s.att, datt, s.lse, w->delta, n_seq,
                                    S, H, dk, w->dqkv, w->dqkv + T * d, w->dqkv + 2 * T * d));
            if (c.pos == 1) {
                NNB_TRY(launch_rope(e, w->dqkv, p->rope_cos, p->rope_sin, T, S, H, dk, true));
                NNB_TRY(launch_rope(e, w->dqkv + T * d, p->rope_cos, p->rope_sin, T, S, H, dk, true));
            }
        }
        if (gqa) {
            // fold the replicas' dK, dV onto their KV heads; q | k | v then go back as one matrix of d + 2 dkv rows
            NNB_TRY(launch_gqa_reduce(e, w->dqkv, T, H, Hkv, dk, w->qkv_raw));
            NNB_TRY(lin_bwd(p, LW.qkv, w->qkv_raw, s.q1, s.s1, T, w->dn, false));
        } else if (tc_bwd_ok(p, 3 * d, T)) {
            // q, k, v share their input: their gradients go side by side into one (T, 3d) operand, so the
            // backward is one dX GEMM over the concatenated contraction and one dW GEMM for all three
            for (int m = 0; m < 3; ++m)
                NNB_TRY(launch_scale_colsum(e, w->dqkv + m * T * d, p->tau + LW.q.tau_off + m * d, T, d, w->dyb + m * d,
                                            GG + LW.q.b_off + m * d, 3 * d, sink_of(w, T)));
            NNB_TRY(lin_bwd_gemms(p, LW.q, 3 * d, s.q1, s.s1, T, w->dn, false));
        } else {
            NNB_TRY(lin_bwd(p, LW.q, w->dqkv, s.q1, s.s1, T, w->dn, false));
            NNB_TRY(lin_bwd(p, LW.k, w->dqkv + T * d, s.q1, s.s1, T, w->dn, true));
            NNB_TRY(lin_bwd(p, LW.v, w->dqkv + 2 * T * d, s.q1, s.s1, T, w->dn, true));
        }
        NNB_TRY(launch_rmsnorm_bwd(e, s.x_in, PP + LW.ln1_g, w->dn, w->g2, T, d, w->g, GG + LW.ln1_g));
    }
    NNB_TRY(launch_colsum_finish_all(e, &w->bias_sink));
    return launch_embed_rows_bwd(e, w->g, w->row_tok, w->row_pos, T, d, V, GG + p->tok_emb, c.pos == 0 ? GG + p->pos_emb : nullptr);
}

}  // namespace nnb

bool nnb::policy_can_prefill(const nnb_policy* p)
{
    return !p->cfg.exact && attn_b16_supported((size_t)p->cfg.d_model / p->cfg.n_head, (size_t)p->cfg.d_model);
}

nnb_status nnb::policy_prefill_prefix(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t L, void* k_pre, void* v_pre,
                                      size_t alloc, size_t layer_bytes)
{
    NNB_REQUIRE(policy_can_prefill(p) && n_seq > 0 && L > 0 && L <= alloc, "prefill: unsupported configuration");
    // the prefill keeps a workspace of its own, so that the training workspace survives a rollout
    std::swap(p->train, p->prefill);
    nnb_status st = ensure_train(p, n_seq, L, 0, false, 1, /*with_head=*/false);
    if (st == NNB_OK) {
        const KvSink sink{k_pre, v_pre, alloc, layer_bytes};
        st = forward(p, d_tokens, n_seq, L, 0, false, &sink);
    }
    std::swap(p->train, p->prefill);
    return st;
}

namespace nnb {

static nnb_status check_shape(nnb_policy* p, const int32_t* tokens, size_t n_seq, size_t S, size_t P)
{
    NNB_REQUIRE(p && tokens, "policy or tokens is NULL");
    NNB_REQUIRE(n_seq > 0 && S >= 2 && P >= 1 && P < S, "bad sequence shape (n_seq=%zu, seq_len=%zu, prompt_len=%zu)", n_seq, S, P);
    NNB_REQUIRE(S <= (size_t)p->cfg.ctx, "sequence length %zu exceeds the context %d", S, p->cfg.ctx);
    return NNB_OK;
}

}  // namespace nnb

using namespace nnb;

extern "C" {

nnb_status nnb_policy_logprobs(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t seq_len, size_t prompt_len,
                               float* d_logp, float* d_entropy, float* d_value)
{
    return nnb_policy_logprobs_grouped(p, d_tokens, n_seq, seq_len, prompt_len, 1, d_logp, d_entropy, d_value);
}

nnb_status nnb_policy_logprobs_grouped(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t seq_len, size_t prompt_len,
                                       size_t group, float* d_logp, float* d_entropy, float* d_value)
{
    NNB_TRY(check_shape(p, d_tokens, n_seq, seq_len, prompt_len));
    NNB_REQUIRE(d_value == nullptr || p->cfg.value_head, "policy has no value head");
    NNB_REQUIRE(group >= 1 && n_seq % group == 0, "logprobs: %zu sequences are not whole groups of %zu", n_seq, group);
    NNB_TRY(ensure_train(p, n_seq, seq_len, prompt_len, false, group));
    NNB_TRY(forward(p, d_tokens, n_seq, seq_len, prompt_len, d_entropy != nullptr));
    TrainWs* w = (TrainWs*)p->train;
    const size_t Td = n_seq * (seq_len - prompt_len);
    cudaStream_t st = p->e->stream;
    if (d_logp) NNB_CUDA(cudaMemcpyAsync(d_logp, w->logp, Td * 4, cudaMemcpyDeviceToDevice, st));
    if (d_entropy) NNB_CUDA(cudaMemcpyAsync(d_entropy, w->ent, Td * 4, cudaMemcpyDeviceToDevice, st));
    if (d_value) NNB_CUDA(cudaMemcpyAsync(d_value, w->value, Td * 4, cudaMemcpyDeviceToDevice, st));
    return NNB_OK;
}

float* nnb_policy_grads(nnb_policy* p)
{
    if (!p) return nullptr;
    if (!p->grads) {
        if (cudaMalloc((void**)&p->grads, p->n_params * 4) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        cudaMemsetAsync(p->grads, 0, p->n_params * 4, p->e->stream);
    }
    return p->grads;
}

nnb_status nnb_policy_zero_grad(nnb_policy* p)
{
    NNB_REQUIRE(p, "policy is NULL");
    NNB_REQUIRE(nnb_policy_grads(p), "out of device memory for the gradient buffer");
    NNB_CUDA(cudaMemsetAsync(p->grads, 0, p->n_params * 4, p->e->stream));
    return NNB_OK;
}

nnb_status nnb_policy_train_step(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t seq_len,
                                 size_t prompt_len, const nnb_objective* obj, float* d_report)
{
    return nnb_policy_train_step_grouped(p, d_tokens, n_seq, seq_len, prompt_len, 1, obj, d_report);
}

nnb_status nnb_policy_train_step_grouped(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t seq_len,
                                         size_t prompt_len, size_t group, const nnb_objective* obj, float* d_report)
{
    NNB_TRY(check_shape(p, d_tokens, n_seq, seq_len, prompt_len));
    NNB_REQUIRE(group >= 1 && n_seq % group == 0, "train_step: %zu sequences are not whole groups of %zu", n_seq, group);
    NNB_REQUIRE(obj && obj->d_mask, "train_step: objective or mask is NULL");
    NNB_REQUIRE(nnb_policy_grads(p), "out of device memory for the gradient buffer");
    const bool use_value = obj->value_coef != 0.0f;
    NNB_REQUIRE(!use_value || (p->cfg.value_head && obj->d_returns && obj->d_old_value),
                "train_step: the value term needs a value head, returns and old values");
    NNB_TRY(ensure_train(p, n_seq, seq_len, prompt_len, true, group));
    NNB_TRY(policy_ensure_wb(p));
    nnb_engine* e = p->e;
    TrainWs* w = (TrainWs*)p->train;
    const size_t Td = n_seq * (seq_len - prompt_len), V = p->cfg.vocab;
    const bool use_ent = obj->entropy_coef != 0.0f;
    NNB_TRY(forward(p, d_tokens, n_seq, seq_len, prompt_len, true));
    NNB_TRY(launch_token_objective(e, w->logp, w->ent, obj->d_old_logp, obj->d_ref_logp, obj->d_advantage, obj->d_mask,
                                   Td, obj->units, obj->clip_eps, obj->kl_coef, obj->entropy_coef, w->up_lp, w->up_ent,
                                   w->report));
    if (use_value) {
        NNB_TRY(launch_clipped_value(e, w->value, obj->d_returns, obj->d_old_value, obj->d_mask, Td, obj->units,
                                     obj->value_clip_eps, obj->value_coef, w->dvalue, w->vreport));
    } else if (p->cfg.value_head) {
        NNB_CUDA(cudaMemsetAsync(w->dvalue, 0, Td * 4, e->stream));
        NNB_CUDA(cudaMemsetAsync(w->vreport, 0, 8, e->stream));
    }
    if (w->fused_head) {
        NNB_TRY(launch_tc_lmhead_bwd(e, w->qh, p->w8 + p->head.packed_off * 16, p->tau + p->head.tau_off, w->sh,
                                     p->params + p->head.b_off, w->actions, w->lse, w->ent, w->up_lp, use_ent ? w->up_ent : nullptr, Td,
                                     (size_t)p->cfg.d_model, V, w->head_scratch, w->dyb, p->grads + p->head.b_off));
    } else {
        NNB_TRY(launch_categorical_bwd(e, w->logits, w->actions, w->up_lp, use_ent ? w->up_ent : nullptr, Td, V, w->logits));
    }
    NNB_TRY(backward(p, d_tokens, n_seq, seq_len, prompt_len));
    if (d_report) {
        NNB_CUDA(cudaMemcpyAsync(d_report, w->report, 8 * 4, cudaMemcpyDeviceToDevice, e->stream));
        if (p->cfg.value_head)
            NNB_CUDA(cudaMemcpyAsync(d_report + 8, w->vreport, 2 * 4, cudaMemcpyDeviceToDevice, e->stream));
        else
            NNB_CUDA(cudaMemsetAsync(d_report + 8, 0, 8, e->stream));
    }
    return NNB_OK;
}

nnb_status nnb_policy_cached_activation(nnb_policy* p, int layer, int which, int8_t* d_q, float* d_s, size_t* rows, size_t* cols)
{
    NNB_REQUIRE(p, "policy is NULL");
    TrainWs* w = (TrainWs*)p->train;
    NNB_REQUIRE(w && w->saved_layers, "cached_activation: no training micro-batch has run on this policy");
    NNB_REQUIRE(layer >= 0 && layer < p->cfg.n_layer && which >= 0 && which < 4, "cached_activation: bad index");
    const LayerSave& s = w->L[layer];
    const int8_t* qs[4] = {s.q1, s.q2, s.q3, s.q4};
    const float* ss[4] = {s.s1, s.s2, s.s3, s.s4};
    const size_t k = which == 3 ? (size_t)p->cfg.d_ff : (size_t)p->cfg.d_model;
    if (rows) *rows = w->rows;
    if (cols) *cols = k;
    if (d_q) NNB_CUDA(cudaMemcpyAsync(d_q, qs[which], w->rows * k, cudaMemcpyDeviceToDevice, p->e->stream));
    if (d_s) NNB_CUDA(cudaMemcpyAsync(d_s, ss[which], w->rows * 4, cudaMemcpyDeviceToDevice, p->e->stream));
    return NNB_OK;
}

nnb_status nnb_policy_sft_step(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t seq_len, size_t prompt_len,
                               size_t group, const float* d_mask, float units, float* d_report)
{
    NNB_TRY(check_shape(p, d_tokens, n_seq, seq_len, prompt_len));
    NNB_REQUIRE(d_mask, "sft_step: mask is NULL");
    NNB_REQUIRE(group >= 1 && n_seq % group == 0, "sft_step: %zu sequences are not whole groups of %zu", n_seq, group);
    // -sum mask * logp / units is the sampled-KL term against a reference log-prob of zero with coefficient -1
    NNB_TRY(ensure_train(p, n_seq, seq_len, prompt_len, true, group));
    TrainWs* w = (TrainWs*)p->train;
    const size_t Td = n_seq * (seq_len - prompt_len);
    NNB_CUDA(cudaMemsetAsync(w->dvalue, 0, Td * 4, p->e->stream));  // read by the objective before anything rewrites it
    const nnb_objective obj{d_mask, nullptr, nullptr, w->dvalue, nullptr, nullptr, units, 0.0f, -1.0f, 0.0f, 0.0f, 0.0f};
    NNB_TRY(nnb_policy_train_step_grouped(p, d_tokens, n_seq, seq_len, prompt_len, group, &obj, d_report));
    if (d_report) NNB_CUDA(cudaMemcpyAsync(d_report, d_report + 4, 4, cudaMemcpyDeviceToDevice, p->e->stream));
    return NNB_OK;
}

nnb_status nnb_policy_optimizer_step(nnb_policy* p, float lr, float beta1, float beta2, float eps, float weight_decay,
                                     float max_grad_norm, float* d_norm_out)
{
    NNB_REQUIRE(p && p->grads, "optimizer_step: no gradients have been computed");
    nnb_engine* e = p->e;
    if (!p->adam_m) {
        if (cudaMalloc((void**)&p->adam_m, p->n_params * 4) != cudaSuccess ||
            cudaMalloc((void**)&p->adam_v, p->n_params * 4) != cudaSuccess) {
            cudaGetLastError();
            NNB_FAIL(NNB_ERR_OOM, "out of device memory for the AdamW moments");
        }
        NNB_CUDA(cudaMemsetAsync(p->adam_m, 0, p->n_params * 4, e->stream));
        NNB_CUDA(cudaMemsetAsync(p->adam_v, 0, p->n_params * 4, e->stream));
    }
    // a tensor-core GEMM that gave up on a bounded wait left garbage in the gradients: report it before
    // anything is applied to the weights
    if (!p->cfg.exact) NNB_TRY(tc_check_errors(e));
    if (max_grad_norm > 0.0f || d_norm_out) NNB_TRY(launch_clip_grad_norm(e, p->grads, p->n_params, max_grad_norm, d_norm_out));
    p->adam_t += 1;
    NNB_TRY(launch_adamw(e, p->params, p->grads, p->adam_m, p->adam_v, p->n_params, lr, beta1, beta2, eps, weight_decay,
                         p->adam_t));
    NNB_CUDA(cudaMemsetAsync(p->grads, 0, p->n_params * 4, e->stream));
    return policy_requantize(p);
}

nnb_status nnb_policy_release_workspaces(nnb_policy* p)
{
    NNB_REQUIRE(p, "policy is NULL");
    NNB_CUDA(cudaStreamSynchronize(p->e->stream));
    policy_free_train(p);
    policy_free_decode(p);
    return NNB_OK;
}

}  // extern "C"
