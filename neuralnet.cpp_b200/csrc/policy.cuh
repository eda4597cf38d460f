// policy.cuh — the policy object behind the opaque nnb_policy handle.
#pragma once
#include <string>
#include <vector>

#include "common.cuh"

namespace nnb {

struct LinW {
    size_t w_off = 0, b_off = 0;  // offsets (floats) of latent weight (out,in) and bias (out) in params
    size_t in = 0, out = 0;
    size_t packed_off = 0;        // offset (words) of the 2-bit container in `packed`
    size_t tau_off = 0;           // offset of the per-row scales in `tau`
};

struct LayerW {
    size_t ln1_g = 0, ln2_g = 0;
    size_t attn_sub_g = 0, ffn_sub_g = 0;  // SubLN gains (d_model), (d_ff); only with cfg.sub_ln
    LinW q, k, v, o, fc1, fc2;
    LinW qkv;  // q, k and v as one matrix of d + 2 * dkv rows (their weights, scales and biases are contiguous)
};

struct TensorInfo {
    std::string name;
    size_t offset, rows, cols;
};

struct DecodeWs {
    size_t B = 0, ctx_alloc = 0;     // sequences; positions held by the per-sequence cache
    size_t tok_cols = 0;             // columns of tokens / logp: the whole sequence
    size_t group = 1, pre_len = 0;   // sequences per shared prompt; positions held by the shared prefix cache
    void *k = nullptr, *v = nullptr;  // (L, B, H, ctx_alloc, dk), f32 in the exact mode else bf16
    void *k_pre = nullptr, *v_pre = nullptr;  // (L, B/group, H, pre_len, dk): prompt prefix, one per group
    int32_t* tokens_pre = nullptr;            // (B/group, pre_len) prompt tokens of the group representatives
    float *x = nullptr, *qkv = nullptr, *att = nullptr, *h1 = nullptr, *logits = nullptr;
    float* qkv_raw = nullptr;  // grouped-query attention: (B, d + 2 dkv) projections before the KV heads are replicated
    float* act = nullptr;      // (unused: the feed-forward SubLN is applied inside the quantiser launch)
    float* sample_rows = nullptr;  // (B, V) the sampler's working rows when a row does not fit shared memory
    float* hn = nullptr;       // tied embeddings: (B, d) final-norm output, the dense head's operand
    __nv_bfloat16* hnb = nullptr;
    float* pre_ml = nullptr;  // (B, H, 2): partial softmax (max, sum) over the shared prefix; its values go to att
    int8_t* q8 = nullptr;
    float* s = nullptr;
    int32_t* qsum = nullptr;
    int* d_pos = nullptr;
    int32_t* tokens = nullptr;  // (B, tok_cols)
    float* logp = nullptr;      // (B, tok_cols), generated index
    int32_t *done = nullptr, *gen_len = nullptr;  // (B) end-of-sequence flags and generated lengths
};

}  // namespace nnb

struct nnb_policy {
    nnb_engine* e = nullptr;
    nnb_gpt_config cfg{};
    size_t n_params = 0, packed_words = 0, tau_count = 0;
    float* params = nullptr;  // f32 master weights, flat
    float* grads = nullptr;   // allocated on first training use
    float* adam_m = nullptr;
    float* adam_v = nullptr;
    int adam_t = 0;  // optimizer steps taken
    uint32_t* packed = nullptr;
    int8_t* w8 = nullptr;           // fast mode: int8 trits, K permuted like the activations (tcgen05 forward)
    __nv_bfloat16* wb = nullptr;    // fast mode, trainable policies: bf16 trits (tcgen05 dX)
    bool wb_valid = false;
    __nv_bfloat16* eb = nullptr;    // fast mode, tied embeddings: bf16 copy of tok_emb, the dense head's weight
    float* tau = nullptr;
    float *rope_cos = nullptr, *rope_sin = nullptr;  // (ctx, dk/2)
    size_t tok_emb = 0, pos_emb = 0, lnf_g = 0, value_w = 0, value_b = 0;
    std::vector<nnb::LayerW> layers;
    nnb::LinW head;
    std::vector<nnb::TensorInfo> tensors;
    nnb::DecodeWs dec;
    // optional timing of the rollout: a CUDA event every time_stride decode steps (0 = off)
    size_t time_stride = 0;
    std::vector<cudaEvent_t> time_events;
    std::vector<int> time_pos;  // position consumed by the step that follows each event
    void* train = nullptr;    // workspace of the teacher-forced passes (policy_train.cu)
    void* prefill = nullptr;  // a second one, for the batched prompt prefill of the rollout
};

namespace nnb {
// nnb_gpt_config.act: 0 QuickGELU, 1 SwiGLU, 2 ReLU2GLU.  The gated ones take fc1 rows (gate | up), 2 * d_ff wide.
inline bool act_gated(int act) { return act >= 1; }
inline size_t cfg_kv_heads(const nnb_gpt_config& c) { return c.n_head_kv > 0 ? (size_t)c.n_head_kv : (size_t)c.n_head; }
inline bool cfg_gqa(const nnb_gpt_config& c) { return cfg_kv_heads(c) != (size_t)c.n_head; }
inline int act_quant_mode(int act) { return act == 0 ? 1 : (act == 1 ? 2 : 4); }  // mode of launch_row_quant
inline int act_bwd_mode(int act) { return act == 0 ? 1 : (act == 1 ? 2 : 3); }    // mode of launch_act_bwd[_scale_colsum]
nnb_status policy_requantize(nnb_policy* p, bool seeded = false);
void policy_free_train(nnb_policy* p);
// Fast mode: run the teacher-forced forward over n_seq prompts of L tokens and store every layer's rotated keys
// and values as the (layer, n_seq, head, alloc, dk) bf16 prefix cache of a rollout, instead of L decode steps.
bool policy_can_prefill(const nnb_policy* p);
nnb_status policy_prefill_prefix(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t L, void* k_pre, void* v_pre,
                                 size_t alloc, size_t layer_bytes);
void policy_free_decode(nnb_policy* p);
nnb_status policy_ensure_wb(nnb_policy* p);
// tied embeddings: logits (T, V) = hn (T, d) . tok_emb^T.  Exact mode: f64-accumulated CUDA-core product of the f32
// operands.  Fast mode: bf16 operands (hnb is scratch for T * d elements), tcgen05 from 64 rows up.
nnb_status policy_tied_head_fwd(nnb_policy* p, const float* hn, __nv_bfloat16* hnb, size_t T, float* logits);
// y = [residual +] linear(q) through the fastest kernel for this mode and token count
nnb_status policy_linear_fwd(nnb_policy* p, const LinW& l, size_t n_mats, const int8_t* q, const float* s,
                             const int32_t* qsum, size_t T, const float* residual, float* y, size_t y_stride,
                             bool y_bf16 = false);
// y_bf16: the tensor-core forward rounds its result to bf16 and y points at bf16 elements (one matrix, no residual);
// allowed where policy_linear_can_bf16 holds
inline bool policy_linear_can_bf16(const nnb_policy* p, size_t T) { return !p->cfg.exact && p->w8 != nullptr && T >= 64; }
// fast mode: fc1's output (T, F1) is kept as bf16; it is read once by the activation quantiser and once by the
// activation's backward.  NNB_H1_BF16=0 keeps it f32, for A/B runs (read once per process).
bool policy_h1_bf16(const nnb_policy* p, size_t T, size_t F, size_t F1);
}  // namespace nnb
