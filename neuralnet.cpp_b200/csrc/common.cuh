// common.cuh — shared declarations of the engine's translation units.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <string>
#include <vector>

#include "nn_b200.h"

namespace nnb {

// thread-local error text behind nnb_last_error()
void set_error(const char* fmt, ...);
const char* get_error();

#define NNB_FAIL(code, ...)           \
    do {                              \
        ::nnb::set_error(__VA_ARGS__); \
        return (code);                \
    } while (0)

#define NNB_CUDA(call)                                                                       \
    do {                                                                                     \
        cudaError_t err__ = (call);                                                          \
        if (err__ != cudaSuccess)                                                            \
            NNB_FAIL(NNB_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(err__), \
                     __FILE__, __LINE__);                                                    \
    } while (0)

#define NNB_CHECK_LAUNCH(name)                                                              \
    do {                                                                                    \
        cudaError_t err__ = cudaGetLastError();                                             \
        if (err__ != cudaSuccess)                                                           \
            NNB_FAIL(NNB_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(err__)); \
    } while (0)

#define NNB_REQUIRE(cond, ...)                         \
    do {                                               \
        if (!(cond)) NNB_FAIL(NNB_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define NNB_TRY(expr)                  \
    do {                               \
        nnb_status st__ = (expr);      \
        if (st__ != NNB_OK) return st__; \
    } while (0)

inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

}  // namespace nnb

// The engine object behind the opaque C handle.
struct nnb_engine {
    int device = 0;
    int sm_count = 0;
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;  // the stream in use (own_stream or the caller's)
    // grow-only scratch arena for operators that need temporaries
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    // pinned staging for the *_host entry points
    void* pinned = nullptr;
    size_t pinned_bytes = 0;
    // counts kernel launches issued through this engine (reported by the benchmark)
    unsigned long long launches = 0;
    int* dev_flags = nullptr;  // small device block: [0] error flag raised by bounded device-side waits
    // partial products of the weight-gradient GEMM when it splits the token axis (allocated at first use)
    float* dw_part = nullptr;
    size_t dw_part_floats = 0;
    // While set, launch_ex marks its launches for programmatic dependent launch: the next kernel may become
    // resident and run its prologue while this one drains.  Only kernels that call pdl_wait() before their
    // first global-memory access go through launch_ex.
    bool pdl = false;
    std::string describe_text;

    nnb_status ensure_scratch(size_t bytes);
    nnb_status ensure_pinned(size_t bytes);
};

namespace nnb {

// Launch on the engine's stream; with e->pdl the launch carries the programmatic-stream-serialization
// attribute (it is recorded as a programmatic edge when the stream is being captured into a graph).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_ex(nnb_engine* e, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = e->stream;
    cudaLaunchAttribute attr[1];
    if (e->pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ---- no_alloc.cu: resolves, once per device, the device address of the fixed scratch array of
// nnb_group_advantage_noalloc; leaves the caller's current device as it found it
nnb_status noalloc_prepare(int device);

// ---- ternary.cu: launchers (all enqueue on e->stream)
nnb_status launch_absmean_tau(nnb_engine* e, const float* latent, size_t rows, size_t k, float* tau);
nnb_status launch_trit_pack(nnb_engine* e, const float* latent, const float* tau, size_t rows,
                            size_t k, uint32_t* packed);
nnb_status launch_col_absmax_scale(nnb_engine* e, const float* x, size_t k, size_t n, float* s);
nnb_status launch_quantize_i8(nnb_engine* e, const float* x, size_t m, size_t n, const float* scale,
                              int col_scale, uint32_t* out);
nnb_status launch_unpack_i8(nnb_engine* e, const uint32_t* packed, size_t m, size_t n, float* out);
nnb_status launch_matmul_q_i8_ref(nnb_engine* e, const uint32_t* wq, const float* tau,
                                  const uint32_t* xq, const float* s, size_t rows, size_t k,
                                  size_t n, float* y, int32_t* acc);
nnb_status launch_matmul_q_ref(nnb_engine* e, const uint32_t* wq, const float* tau, const float* x,
                               size_t rows, size_t k, size_t n, float* c);
nnb_status launch_matmul_q_t_ref(nnb_engine* e, const uint32_t* wq, const float* tau,
                                 const float* b, size_t rows, size_t mcols, size_t n, float* c);
nnb_status launch_act_quant_tm(nnb_engine* e, const void* x, nnb_dtype dtype, size_t t, size_t k,
                               int8_t* q, float* s, int32_t* qsum);
nnb_status launch_actq_to_plain(nnb_engine* e, const int8_t* q, size_t t, size_t k, int8_t* plain);
// y = [residual +] (tau*s)*acc [+ bias]; residual (t,out) f32 and acc (t,out) may be NULL
nnb_status launch_bitlinear_fwd_tm(nnb_engine* e, const uint32_t* wq, size_t wq_stride_words,
                                   const float* tau, const float* bias, const float* residual,
                                   const int8_t* q, const float* s, const int32_t* qsum,
                                   size_t n_mats, size_t t, size_t k, size_t out, void* y,
                                   size_t y_stride_elems, nnb_dtype dtype, int32_t* acc);

// ---- decode.cu
// mode 0 RMSNorm*gamma, 1 QuickGELU, 2 SwiGLU (row = gate|up, in_stride = 2k), 3 identity;
// quantises the transformed row; f_out (t,k) optional copy of the transformed row
nnb_status launch_row_quant(nnb_engine* e, int mode, bool exact, const float* in, const float* gamma,
                            size_t t, size_t k, size_t in_stride, int8_t* q, float* s,
                            int32_t* qsum, float* f_out, bool norm_after = false, bool in_bf16 = false /* modes 1, 2, 4 */);
// Where a decode step's new projections live and how the heads map: q, k, v point at sequence 0 (rows `stride` floats
// apart); kv_rep query heads read one key / value head (grouped-query attention; 1 = multi-head), the caches then hold
// H / kv_rep heads.  Without it the launchers take qkv as three (B, d) planes.
struct AttnIn {
    const float *q, *k, *v;
    int stride, kv_rep;
};
inline AttnIn attn_in_or_planes(const AttnIn* in, const float* qkv, size_t B, size_t d)
{
    return in ? *in : AttnIn{qkv, qkv + B * d, qkv + 2 * B * d, (int)d, 1};
}
nnb_status launch_attn_decode(nnb_engine* e, bool exact, const float* qkv, void* kcache, void* vcache,
                              size_t own_alloc, const void* kpre, const void* vpre, size_t pre_len, size_t pre_alloc,
                              size_t group, const float* rope_cos, const float* rope_sin, const int* d_pos, size_t B,
                              size_t H, size_t dk, float* out, size_t kv_pitch = 0 /* elements per cached key; 0 = dk */,
                              const AttnIn* in = nullptr);
size_t attn_decode_kv_pitch(bool exact, size_t dk);
bool attn_decode_fused_supported(size_t H, size_t dk);
nnb_status launch_attn_decode_fused(nnb_engine* e, const float* qkv, void* kcache, void* vcache, size_t own_alloc,
                                    const void* kpre, const void* vpre, size_t pre_len, size_t pre_alloc, size_t group,
                                    const float* rope_cos, const float* rope_sin, const int* d_pos, size_t B, size_t H,
                                    size_t dk, float* att, int8_t* q8, float* s, int32_t* qsum, float* pre_o = nullptr,
                                    float* pre_ml = nullptr, const AttnIn* in = nullptr);
// what the sampler applies beyond temperature and top-k (defaults = off); see sample_kernel
struct SampleOpts {
    float temperature = 1.0f;
    int top_k = 0;
    float top_p = 1.0f;
    float repeat_penalty = 1.0f;
    int repeat_window = 0;
    const float* logit_bias = nullptr;  // (V) added to the raw logits before everything else
    int eos = -1, min_new = 0;
    int32_t* done = nullptr;     // (B) set once a sequence has sampled eos; NULL = no end-of-sequence handling
    int32_t* gen_len = nullptr;  // (B) tokens generated before eos
    // Working copy of the logits, (B, V rounded up to 4) f32, for vocabularies whose row does not fit a CTA's shared
    // memory (sample_row_in_smem(V) false); the kernel then keeps the row there (L2) instead
    float* row_scratch = nullptr;
};
bool sample_row_in_smem(size_t V);
nnb_status launch_sample_opts(nnb_engine* e, bool exact, const float* logits, size_t B, size_t V, const SampleOpts& o,
                              unsigned long long seed, unsigned seq0, const int* d_pos, int prompt_len, int32_t* tokens,
                              size_t tokens_stride, float* logp, size_t logp_stride, float* entropy);
nnb_status launch_sample(nnb_engine* e, bool exact, const float* logits, size_t B, size_t V,
                         float temperature, int top_k, unsigned long long seed, unsigned seq0,
                         const int* d_pos, int prompt_len, int32_t* tokens, size_t tokens_stride,
                         float* logp, size_t logp_stride, float* entropy);
nnb_status launch_set_int(nnb_engine* e, int* p, int v);
nnb_status launch_set_int2(nnb_engine* e, int* p, int v, int v1);
nnb_status launch_fill_int(nnb_engine* e, int* p, size_t n, int v);
nnb_status launch_add_int(nnb_engine* e, int* p, int v);
nnb_status launch_embed(nnb_engine* e, const float* tok_emb, const float* pos_emb, const int32_t* tokens,
                        size_t tokens_stride, const int* d_pos, size_t B, size_t d, size_t vocab, float* x);

// ---- rl.cu
nnb_status launch_gae(nnb_engine* e, const float* rewards, const float* values, const float* done,
                      const float* mask, const float* bootstrap, size_t steps, size_t batch, float gamma,
                      float lambda, float* adv, float* ret);
nnb_status launch_group_advantage(nnb_engine* e, const float* returns, const int32_t* first, const int32_t* count,
                                  size_t n_spans, float eps, float* out);
nnb_status launch_masked_normalize(nnb_engine* e, const float* x, const float* mask, size_t n, float eps, float* out);
nnb_status launch_categorical_fwd(nnb_engine* e, const float* logits, const int32_t* actions, size_t t, size_t v,
                                  float* logp, float* entropy);
nnb_status launch_categorical_bwd(nnb_engine* e, const float* logits, const int32_t* actions, const float* up_lp,
                                  const float* up_ent, size_t t, size_t v, float* dlogits);
nnb_status launch_token_objective(nnb_engine* e, const float* logp, const float* entropy, const float* old_logp,
                                  const float* ref_logp, const float* adv, const float* mask, size_t n,
                                  float units_override, float clip_eps, float kl_coef, float ent_coef,
                                  float* up_lp, float* up_ent, float* report);
nnb_status launch_clipped_value(nnb_engine* e, const float* value, const float* returns, const float* old_value,
                                const float* mask, size_t n, float units_override, float clip_eps, float coef,
                                float* grad, float* report);
nnb_status launch_clip_grad_norm(nnb_engine* e, float* g, size_t n, float max_norm, float* norm_out);
nnb_status launch_scale(nnb_engine* e, float* x, size_t n, float sc);
nnb_status launch_adamw(nnb_engine* e, float* p, const float* g, float* m, float* v, size_t n, float lr,
                        float beta1, float beta2, float eps, float wd, int t);

// ---- gemm_float.cu
// dx (t,k) (+)= (dy (t,out) * tau) . trit (out,k)
nnb_status launch_bitlinear_dx(nnb_engine* e, bool exact, const float* dy, const uint32_t* wq, const float* tau,
                               size_t t, size_t k, size_t out, float* dx, bool accumulate);
// dw (out,k) += tau * ((dy * s)^T . q)
nnb_status launch_bitlinear_dw(nnb_engine* e, bool exact, const float* dy, const int8_t* q, const float* s,
                               const float* tau, size_t t, size_t k, size_t out, float* dw);
// ---- gemm_bf16.cu (bf16 tensor-core versions of the two above)
nnb_status launch_bitlinear_dx_bf16(nnb_engine* e, const float* dy, const uint32_t* wq, const float* tau, size_t t,
                                    size_t k, size_t out, float* dx, bool accumulate);
nnb_status launch_bitlinear_dw_bf16(nnb_engine* e, const float* dy, const int8_t* q, const float* s, const float* tau,
                                    size_t t, size_t k, size_t out, float* dw);
nnb_status launch_colsum_add(nnb_engine* e, const float* dy, size_t t, size_t out, float* db);

// ---- train.cu
nnb_status launch_embed_fwd(nnb_engine* e, const float* tok_emb, const float* pos_emb, const int32_t* tokens,
                            size_t n_rows, size_t S, size_t d, size_t vocab, float* x);
nnb_status launch_embed_bwd(nnb_engine* e, const float* g, const int32_t* tokens, size_t n_rows, size_t S, size_t d,
                            size_t vocab, float* g_tok, float* g_pos);
nnb_status launch_rope(nnb_engine* e, float* x, const float* rope_cos, const float* rope_sin, size_t n_rows,
                       size_t S, size_t H, size_t dk, bool backward);
nnb_status launch_attn_fwd(nnb_engine* e, bool exact, const float* q, const float* k, const float* v, size_t n_seq,
                           size_t S, size_t H, size_t dk, float* out, float* lse);
nnb_status launch_attn_bwd(nnb_engine* e, bool exact, const float* q, const float* k, const float* v, const float* out,
                           const float* dout, const float* lse, float* delta, size_t n_seq, size_t S, size_t H,
                           size_t dk, float* dq, float* dkk, float* dvv);
nnb_status launch_rmsnorm_bwd(nnb_engine* e, const float* x, const float* gamma, const float* dy,
                              const float* residual, size_t T, size_t F, float* dx, float* dgamma);
nnb_status launch_act_bwd(nnb_engine* e, int mode, const float* h, const float* da, size_t T, size_t F, float* dh);
// Row layout of a micro-batch of n_seq sequences of S = P + G tokens.  group == 1: sequence b owns rows
// [b*S, (b+1)*S).  group > 1: the `group` consecutive sequences of a prompt group share their first P
// tokens, which are stored (and computed) once: a group owns P + group*G rows, its prefix first, then the
// G generated rows of each member.  Position r of sequence b lives in row map_row(m, b, r).
struct SeqMap {
    int S, P, G, group;
};
__host__ __device__ inline size_t map_row(const SeqMap& m, int b, int r)
{
    if (m.group <= 1) return (size_t)b * m.S + r;
    const int grp = b / m.group, mm = b % m.group;
    const size_t base = (size_t)grp * ((size_t)m.P + (size_t)m.group * m.G);
    return r < m.P ? base + r : base + m.P + (size_t)mm * m.G + (r - m.P);
}
inline size_t map_rows_total(const SeqMap& m, size_t n_seq)
{
    return m.group <= 1 ? n_seq * m.S : (n_seq / m.group) * ((size_t)m.P + (size_t)m.group * m.G);
}
// per-(sequence, head, position) vectors (lse, delta): (n_seq, H, S) when group == 1, (H, rows) by row otherwise
__host__ __device__ inline size_t map_vec(const SeqMap& m, int b, int h, int r, int H, size_t rows)
{
    return m.group <= 1 ? ((size_t)b * H + h) * m.S + r : (size_t)h * rows + map_row(m, b, r);
}

nnb_status launch_build_rows(nnb_engine* e, const int32_t* tokens, const SeqMap& map, size_t n_seq, int32_t* row_tok,
                             int32_t* row_pos);
nnb_status launch_embed_rows_fwd(nnb_engine* e, const float* tok_emb, const float* pos_emb, const int32_t* row_tok,
                                 const int32_t* row_pos, size_t n_rows, size_t d, size_t vocab, float* x);
nnb_status launch_embed_rows_bwd(nnb_engine* e, const float* g, const int32_t* row_tok, const int32_t* row_pos, size_t n_rows,
                                 size_t d, size_t vocab, float* g_tok, float* g_pos);
nnb_status launch_gather_decisions_map(nnb_engine* e, const float* src, const SeqMap& map, size_t n_seq, size_t d, float* dst);
nnb_status launch_scatter_decisions_map(nnb_engine* e, const float* src, const SeqMap& map, size_t n_seq, size_t d, float* dst);
nnb_status launch_gather_decisions(nnb_engine* e, const float* src, size_t n_seq, size_t S, size_t P, size_t G,
                                   size_t d, float* dst);
nnb_status launch_scatter_decisions(nnb_engine* e, const float* src, size_t n_seq, size_t S, size_t P, size_t G,
                                    size_t d, float* dst);
nnb_status launch_value_fwd(nnb_engine* e, const float* x, const float* w, const float* b, size_t n, size_t d,
                            float* value);
nnb_status launch_value_bwd(nnb_engine* e, const float* x, const float* w, const float* dv, size_t n, size_t d,
                            float* dx, float* dw, float* db, float* scratch, size_t scratch_floats);
nnb_status launch_add(nnb_engine* e, float* dst, const float* src, size_t n);

// ---- gemm_tc.cu (tcgen05 / TMEM / TMA GEMMs)
nnb_status launch_tc_forward(nnb_engine* e, const int8_t* q, const int8_t* w8, const float* tau, const float* s,
                             const float* bias, const float* residual, size_t t, size_t k, size_t out, float* y,
                             size_t n_mats = 1, size_t y_stride = 0, __nv_bfloat16* y_bf16 = nullptr /* instead of y */);
nnb_status launch_tc_dx(nnb_engine* e, const __nv_bfloat16* dyb, const __nv_bfloat16* wb, size_t t, size_t k, size_t out,
                        float* dx, bool accumulate);
nnb_status launch_tc_dw(nnb_engine* e, const __nv_bfloat16* dyb, const __nv_bfloat16* xs, size_t t, size_t k, size_t out,
                        float* dw);
// LM head fused with log-softmax (fast mode): forward leaves log-prob / entropy / log-sum-exp per row, backward the
// bf16 operand of the head's backward GEMMs and the bias gradient; scratch holds tc_lmhead_scratch_floats floats
size_t tc_lmhead_scratch_floats(size_t t, size_t v);
nnb_status launch_tc_lmhead_fwd(nnb_engine* e, const int8_t* q, const int8_t* w8, const float* tau, const float* s, const float* bias,
                                const int32_t* actions, size_t t, size_t k, size_t v, float* scratch, float* lse, float* logp, float* ent);
nnb_status launch_tc_lmhead_bwd(nnb_engine* e, const int8_t* q, const int8_t* w8, const float* tau, const float* s, const float* bias,
                                const int32_t* actions, const float* lse, const float* ent, const float* up_lp, const float* up_ent,
                                size_t t, size_t k, size_t v, float* scratch, __nv_bfloat16* dyb, float* db);
nnb_status tc_check_errors(nnb_engine* e);
nnb_status tc_set_forward_tile(int bn);
nnb_status launch_expand_weights(nnb_engine* e, const uint32_t* wq, size_t rows, size_t k, int8_t* w8, __nv_bfloat16* wb);
nnb_status launch_scale_to_bf16(nnb_engine* e, const float* dy, const float* tau, size_t t, size_t out, __nv_bfloat16* dyb);
// Where the per-token-chunk column sums of several launches wait to be added to their bias gradients by ONE
// finishing launch (launch_colsum_finish_all) instead of one small launch each.  buf / d_descs are device memory owned
// by the caller; the partial sums stay valid until the finishing launch.
struct ColsumDesc {
    const float* part;
    float* db;
    int n_chunks, out;
};
struct ColsumSink {
    float* buf = nullptr;
    size_t cap = 0, used = 0;  // floats
    ColsumDesc* d_descs = nullptr;
    size_t desc_cap = 0;
    std::vector<ColsumDesc> descs;
};
nnb_status launch_colsum_finish_all(nnb_engine* e, ColsumSink* sink);
// sink == NULL: the bias gradient is finished by the call itself
nnb_status launch_scale_colsum(nnb_engine* e, const float* dy, const float* tau, size_t t, size_t out, __nv_bfloat16* dyb,
                               float* db, size_t dyb_ld = 0, ColsumSink* sink = nullptr);
nnb_status launch_act_bwd_scale_colsum(nnb_engine* e, int mode, const float* h, const float* da, const float* tau, size_t t,
                                       size_t F, __nv_bfloat16* dyb, float* db, ColsumSink* sink = nullptr, bool h_bf16 = false);
nnb_status launch_dequant_to_bf16(nnb_engine* e, const int8_t* q, const float* s, size_t t, size_t k, __nv_bfloat16* xs);
// c (T, N) f32 = a (T, K) bf16 . b (N, K)^T bf16 on tcgen05 (T >= 64, K % 8 == 0, N % 4 == 0)
nnb_status launch_tc_nt(nnb_engine* e, const __nv_bfloat16* a, const __nv_bfloat16* b, size_t t, size_t k, size_t n, float* c);
// struct_ops.cu: grouped-query attention (replicate the KV heads of (T, d + 2 dkv) into planes (3, T, d); fold the
// replicas' gradients back) and the dense products of the tied head
nnb_status launch_gqa_expand(nnb_engine* e, const float* raw, size_t T, size_t H, size_t Hkv, size_t dk, float* planes);
nnb_status launch_gqa_reduce(nnb_engine* e, const float* planes, size_t T, size_t H, size_t Hkv, size_t dk, float* raw);
nnb_status launch_f32_to_bf16(nnb_engine* e, const float* x, size_t n, __nv_bfloat16* y);
nnb_status launch_dense_nt(nnb_engine* e, bool exact, const float* A, const float* B, size_t T, size_t N, size_t K, float* C);
nnb_status launch_dense_nt_bf16(nnb_engine* e, const __nv_bfloat16* A, const __nv_bfloat16* B, size_t T, size_t N, size_t K, float* C);
nnb_status launch_dense_nn(nnb_engine* e, bool exact, const float* G, const float* B, size_t T, size_t N, size_t K, float* C);
nnb_status launch_dense_tn_acc(nnb_engine* e, bool exact, const float* G, const float* X, size_t T, size_t N, size_t K, float* D);

// ---- attn_b16.cu (bf16 tensor-core attention of the teacher-forced pass, head dims 64 and 128)
bool attn_b16_supported(size_t dk, size_t d);
nnb_status launch_rope_pack_b16(nnb_engine* e, const float* q, const float* k, const float* v, const float* rope_cos,
                                const float* rope_sin, size_t T, size_t S, size_t H, size_t dk, __nv_bfloat16* out,
                                const int* row_pos = nullptr);
nnb_status launch_kv_to_cache(nnb_engine* e, const __nv_bfloat16* k, const __nv_bfloat16* v, size_t n_seq, size_t S, size_t H,
                              size_t dk, __nv_bfloat16* kc, __nv_bfloat16* vc, size_t alloc, size_t kv_rep = 1);
nnb_status launch_attn_fwd_b16(nnb_engine* e, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                               size_t n_seq, size_t S, size_t H, size_t dk, float* out, float* lse, const SeqMap* map = nullptr);
// with a grouped map, part (2 * n_seq * P * H*dk floats) receives every member's share of the prefix rows'
// dK and dV before they are summed
nnb_status launch_attn_bwd_b16(nnb_engine* e, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                               const float* out, const float* dout, const float* lse, float* delta, __nv_bfloat16* dob,
                               const float* rope_cos, const float* rope_sin, size_t n_seq, size_t S, size_t H, size_t dk,
                               float* dq, float* dkk, float* dvv, const SeqMap* map = nullptr, float* part = nullptr);

}  // namespace nnb
