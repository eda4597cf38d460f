/*
 * nn_b200.h — C-ABI of libnn-b200.so, a CUDA (sm_100a) engine for neuralnet.cpp's
 * RL step on ternary (BitNet b1.58) GPT policies.
 *
 * The reference reaches its engines through C++ virtual calls on
 * nn::ComputeEngine obtained from nn::create_cpu_engine()/create_gpu_engine()
 * (include/neuralnet.cpp/cli/cli_engine_factory.hpp:51-77).  This header is the
 * plain-C surface a third engine object exposes for the same operators: opaque
 * handles, device pointers, sizes, a status code and a thread-local error string
 * (the reference's Result<T>/last_error() convention,
 * docs/internal/34-engine-link-abi-boundary.md:36-74,173-185).
 *
 * Conventions
 *  - every function returns NNB_OK (0) or a negative nnb_status; on failure
 *    nnb_last_error() describes it.  Nothing falls back to the CPU.
 *  - pointers named d_* are device pointers on the engine's device, h_* are host.
 *  - work is enqueued on the engine's stream; call nnb_engine_sync before
 *    reading results on the host (the *_host entry points synchronise themselves).
 *  - "reference layout": row-major, activations (features, tokens), weights
 *    (out_features, in_features)  (AGENTS.md:256-265).
 *  - "token-major": activations (tokens, features) row-major — the layout the
 *    engine's own kernels use between operators.
 */
#ifndef NN_B200_H
#define NN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int nnb_status;
enum {
    NNB_OK = 0,
    NNB_ERR_INVALID = -1,     /* bad argument / shape / alignment */
    NNB_ERR_CUDA = -2,        /* a CUDA runtime call failed */
    NNB_ERR_UNSUPPORTED = -3, /* operator or shape outside what the engine implements */
    NNB_ERR_OOM = -4,
    NNB_ERR_TIMEOUT = -5      /* a bounded device-side wait gave up */
};

typedef enum { NNB_F32 = 0, NNB_BF16 = 1 } nnb_dtype;

typedef struct nnb_engine nnb_engine;

/* ---- engine lifetime; replaces nn::create_gpu_engine(device) / nn::last_error()
 *      (include/neuralnet.cpp/cli/cli_engine_factory.hpp:51-77) */
nnb_status nnb_engine_create(int device, nnb_engine** out);
void nnb_engine_destroy(nnb_engine* e);
const char* nnb_last_error(void);
/* ComputeEngine::describe() -> EngineInfo text (src/ternary_gemm_test.cpp:176-185) */
nnb_status nnb_engine_describe(nnb_engine* e, char* buf, size_t buf_len);
/* end_batch()/flush_batch() equivalent: wait for everything enqueued so far */
nnb_status nnb_engine_sync(nnb_engine* e);
/* use a caller-owned cudaStream_t (as void*) for all later launches.  NULL is the legacy
 * default stream (what torch uses unless told otherwise); NNB_STREAM_OWN restores the engine's
 * own non-blocking stream. */
#define NNB_STREAM_OWN ((void*)(intptr_t)-1)
nnb_status nnb_engine_set_stream(nnb_engine* e, void* cuda_stream);
void* nnb_engine_stream(nnb_engine* e);
/* number of kernel launches issued through this engine so far (for benchmarks) */
unsigned long long nnb_engine_launch_count(nnb_engine* e);

/* ---- device memory; replaces create_tensor / upload_span / download_span */
nnb_status nnb_alloc(nnb_engine* e, size_t bytes, void** d_out);
nnb_status nnb_free(nnb_engine* e, void* d_ptr);
nnb_status nnb_upload(nnb_engine* e, void* d_dst, const void* h_src, size_t bytes);
nnb_status nnb_download(nnb_engine* e, void* h_dst, const void* d_src, size_t bytes);
nnb_status nnb_zero(nnb_engine* e, void* d_ptr, size_t bytes);

/* ================= tensors and engine primitives, reference layout ========
 * The reference's Tensor is a value over refcounted storage with a write epoch that every writing engine
 * entry bumps (AGENTS.md:158-164; BitLinear's quantisation cache compares it,
 * include/neuralnet.cpp/compute_layer_bitlinear.hpp:607-615).  nnb_tensor is that storage: row-major
 * (rows, cols) f32 on the engine's device (ternary and int8 containers are uint32 words bit-cast into f32
 * tensors, as in the reference).  Functions that return a tensor create it; the caller destroys every
 * handle it received.  Operands of one call must belong to the same engine (NNB_ERR_INVALID otherwise:
 * the reference's cross-domain rule, docs/development/07-engine-ownership.md:14-24).  The verbs are those
 * of docs/usage/03-compute-engine-usage.md:1080-1187 (candidate C list:
 * docs/internal/34-engine-link-abi-boundary.md:36-74). */
typedef struct nnb_tensor nnb_tensor;
nnb_status nnb_tensor_create(nnb_engine* e, size_t rows, size_t cols, nnb_tensor** out); /* zero-filled */
void nnb_tensor_destroy(nnb_tensor* t);
size_t nnb_tensor_rows(const nnb_tensor* t);
size_t nnb_tensor_cols(const nnb_tensor* t);
float* nnb_tensor_data(nnb_tensor* t); /* device pointer; after writing through it call nnb_tensor_mark_written */
unsigned long long nnb_tensor_write_epoch(const nnb_tensor* t);
nnb_status nnb_tensor_mark_written(nnb_tensor* t);
nnb_status nnb_tensor_upload(nnb_tensor* t, const float* h_src, size_t count);   /* upload_span / copy_from */
nnb_status nnb_tensor_download(const nnb_tensor* t, float* h_dst, size_t count); /* download_span / to_matrix */
nnb_status nnb_t_zero(nnb_tensor* t);
nnb_status nnb_t_clone(const nnb_tensor* src, nnb_tensor** out);
nnb_status nnb_t_copy_into(nnb_tensor* dst, const nnb_tensor* src);
nnb_status nnb_t_transpose(const nnb_tensor* src, nnb_tensor** out);
/* rows [start_row, start_row + count) as a new (count, cols) tensor / all rows of src written at dst_start_row */
nnb_status nnb_t_slice_rows(const nnb_tensor* src, size_t start_row, size_t count, nnb_tensor** out);
nnb_status nnb_t_insert_rows(nnb_tensor* dst, size_t dst_start_row, const nnb_tensor* src);
/* out[i] = table[indices[i]] (indices are f32 values, any shape; out of range -> zero row) and its adjoint
 * dst[indices[i]] += grad[i] (repeated indices accumulate) */
nnb_status nnb_t_gather_rows(const nnb_tensor* table, const nnb_tensor* indices, nnb_tensor** out);
nnb_status nnb_t_scatter_add_rows(nnb_tensor* dst, const nnb_tensor* indices, const nnb_tensor* grad);
/* (M, B*N) -> (B*M, N): out[b*M + m, n] = in[m, b*N + n]; inverse != 0 the other way */
nnb_status nnb_t_rearrange_3d(const nnb_tensor* x, size_t M, size_t B, size_t N, int inverse, nnb_tensor** out);
nnb_status nnb_t_scale_inplace(nnb_tensor* t, float s);
nnb_status nnb_t_accumulate(nnb_tensor* dst, const nnb_tensor* src);
nnb_status nnb_t_col_reduce_max(const nnb_tensor* t, nnb_tensor** out); /* (1, cols): max over the rows */
nnb_status nnb_t_row_reduce_sum(const nnb_tensor* t, nnb_tensor** out); /* (rows, 1) */
/* the ternary primitives BitLinear calls (compute_layer_bitlinear.hpp:443-464,494,516,637-650) on tensors */
nnb_status nnb_t_absmean_tau(const nnb_tensor* latent, nnb_tensor** tau);
nnb_status nnb_t_trit_pack(const nnb_tensor* latent, const nnb_tensor* tau, nnb_tensor** packed);
nnb_status nnb_t_trit_pack_into(const nnb_tensor* latent, const nnb_tensor* tau, nnb_tensor* packed);
nnb_status nnb_t_matmul_q(const nnb_tensor* packed, const nnb_tensor* tau, const nnb_tensor* x, nnb_tensor** out);
nnb_status nnb_t_matmul_q_t(const nnb_tensor* packed, const nnb_tensor* tau, const nnb_tensor* b, size_t m_cols, nnb_tensor** out);
nnb_status nnb_t_quantize_i8(const nnb_tensor* x, const nnb_tensor* scale, int col_scale, nnb_tensor** out);
nnb_status nnb_t_unpack_i8(const nnb_tensor* packed, size_t cols, nnb_tensor** out);
nnb_status nnb_t_matmul_q_i8(const nnb_tensor* packed, const nnb_tensor* tau, const nnb_tensor* xq, const nnb_tensor* s, nnb_tensor** out);
/* the three expression-DSL compositions of BitLinear::forward / backward, one kernel each (the expression JIT
 * itself is not part of this engine): |x| (:441), y + row_broadcast(b) (:455), and
 * grad_w + ((dy o col_broadcast(s)) . x^T) o row_broadcast(tau) (:518-534; s may be NULL) */
nnb_status nnb_t_abs(const nnb_tensor* src, nnb_tensor** out);
nnb_status nnb_t_add_row_broadcast(nnb_tensor* y, const nnb_tensor* b);
nnb_status nnb_t_bitlinear_dw_accumulate(nnb_tensor* grad_w, const nnb_tensor* dy, const nnb_tensor* s, const nnb_tensor* x,
                                         const nnb_tensor* tau);

/* ---- standalone RMSNorm and rotary embedding, token-major (rows = tokens).
 * RMSNorm::forward / backward (include/neuralnet.cpp/compute_layer_mlp.hpp:686-746): y = x * rsqrt(mean(x^2) + 1e-5) * gamma;
 * the backward writes d_dx and ADDS the gain gradient to d_dgamma.  f must be a multiple of 64 in the forward.
 * RotaryEmbedding (compute_position_encoding.hpp:64-80,126-168): tables (ctx, dk/2) of cos / sin of pos / 10000^(2j/dk);
 * apply rotates, in place, rows of n_head blocks of dk features, row r being at position r % seq_len (backward != 0: the
 * inverse rotation, which is the gradient); step rotates every row as position `pos` (apply_step). */
nnb_status nnb_rmsnorm_fwd(nnb_engine* e, const float* d_x, const float* d_gamma, size_t t, size_t f, float* d_y);
nnb_status nnb_rmsnorm_bwd(nnb_engine* e, const float* d_x, const float* d_gamma, const float* d_dy, size_t t, size_t f, float* d_dx,
                           float* d_dgamma);
nnb_status nnb_rope_tables(nnb_engine* e, size_t dk, size_t ctx, float* d_cos, float* d_sin);
nnb_status nnb_rope_apply(nnb_engine* e, float* d_x, const float* d_cos, const float* d_sin, size_t n_rows, size_t seq_len, size_t n_head,
                          size_t dk, int backward);
nnb_status nnb_rope_step(nnb_engine* e, float* d_x, const float* d_cos, const float* d_sin, size_t n_seq, size_t pos, size_t n_head, size_t dk);

/* ================= ternary linear, reference layout =======================
 * One entry per ComputeEngine primitive that BitLinear calls
 * (include/neuralnet.cpp/compute_layer_bitlinear.hpp:443-464,494,516,637-650). */

/* tau = row_reduce_sum(|W| * (1/K)); compute_layer_bitlinear.hpp:637-640 */
nnb_status nnb_absmean_tau(nnb_engine* e, const float* d_latent, size_t rows, size_t k, float* d_tau);
/* ComputeEngine::trit_pack_into(latent, tau, dst); compute_layer_bitlinear.hpp:650.
 * d_packed is (rows, ceil(k/16)) uint32 words, 2 bits per weight, code = trit+2. */
nnb_status nnb_trit_pack(nnb_engine* e, const float* d_latent, const float* d_tau, size_t rows,
                         size_t k, uint32_t* d_packed);
/* ComputeEngine::col_reduce_max(|X|) followed by scale_inplace(1/127);
 * compute_layer_bitlinear.hpp:443-446.  x is (k, n), s is (n). */
nnb_status nnb_col_absmax_scale(nnb_engine* e, const float* d_x, size_t k, size_t n, float* d_s);
/* ComputeEngine::quantize_i8(x, scale, col_scale); compute_layer_bitlinear.hpp:447.
 * x (m, n) f32; scale (n) if col_scale else (m); out (m, ceil(n/4)) words. */
nnb_status nnb_quantize_i8(nnb_engine* e, const float* d_x, size_t m, size_t n, const float* d_scale,
                           int col_scale, uint32_t* d_out);
/* ComputeEngine::unpack_i8(packed, cols); compute_layer_bitlinear.hpp:516 */
nnb_status nnb_unpack_i8(nnb_engine* e, const uint32_t* d_packed, size_t m, size_t n, float* d_out);
/* ComputeEngine::matmul_q_i8(wq, tau, xq, s); compute_layer_bitlinear.hpp:454.
 * wq (rows, ceil(k/16)), tau (rows), xq (k, ceil(n/4)) words, s (n);
 * y (rows, n) f32 = (tau*s)*float(acc); d_acc (rows, n) int32 optional (NULL to skip). */
nnb_status nnb_matmul_q_i8(nnb_engine* e, const uint32_t* d_wq, const float* d_tau,
                           const uint32_t* d_xq, const float* d_s, size_t rows, size_t k, size_t n,
                           float* d_y, int32_t* d_acc);
/* ComputeEngine::matmul_q(wq, tau, X); compute_layer_bitlinear.hpp:464.  X (k, n) f32, C (rows, n). */
nnb_status nnb_matmul_q(nnb_engine* e, const uint32_t* d_wq, const float* d_tau, const float* d_x,
                        size_t rows, size_t k, size_t n, float* d_c);
/* ComputeEngine::matmul_q_t(wq, tau, dY, M); compute_layer_bitlinear.hpp:494.
 * wq stored (rows, ceil(mcols/16)), tau (rows), B (rows, n); C (mcols, n). */
nnb_status nnb_matmul_q_t(nnb_engine* e, const uint32_t* d_wq, const float* d_tau, const float* d_b,
                          size_t rows, size_t mcols, size_t n, float* d_c);

/* ================= ternary linear, token-major (the fast path) ============
 * The same arithmetic as quantize_i8 + matmul_q_i8 + bias
 * (BitLinear::forward with activation quantisation,
 * compute_layer_bitlinear.hpp:443-455), on the engine's private layouts. */

/* bytes of the engine's quantised-activation buffer for t tokens of k features */
size_t nnb_actq_bytes(size_t t, size_t k);
/* x (t, k) of dtype -> d_q (engine-private int8 layout, nnb_actq_bytes), d_s (t) f32 scale
 * = absmax*(1/127), d_qsum (t) int32 row sums of q. */
nnb_status nnb_act_quant_tm(nnb_engine* e, const void* d_x, nnb_dtype dtype, size_t t, size_t k,
                            int8_t* d_q, float* d_s, int32_t* d_qsum);
/* engine-private q layout -> plain (t, k) int8 rows (for checking / interop) */
nnb_status nnb_actq_to_plain(nnb_engine* e, const int8_t* d_q, size_t t, size_t k, int8_t* d_plain);
/* y (t, out) of dtype = (tau*s)*float(acc) + bias; d_bias and d_acc (t, out) int32 may be NULL.
 * Requires k % 64 == 0. */
nnb_status nnb_bitlinear_fwd_tm(nnb_engine* e, const uint32_t* d_wq, const float* d_tau,
                                const float* d_bias, const int8_t* d_q, const float* d_s,
                                const int32_t* d_qsum, size_t t, size_t k, size_t out, void* d_y,
                                nnb_dtype dtype, int32_t* d_acc);
/* the same over a stack of n_mats equally-shaped independent linears sharing the
 * activations: matrix i uses d_wq + i*wq_stride_words, d_tau + i*out, d_bias + i*out and
 * writes d_y + i*y_stride_elems (one launch; this is how Q/K/V or a layer stack streams). */
nnb_status nnb_bitlinear_fwd_tm_stack(nnb_engine* e, const uint32_t* d_wq, size_t wq_stride_words,
                                      const float* d_tau, const float* d_bias, const int8_t* d_q,
                                      const float* d_s, const int32_t* d_qsum, size_t n_mats,
                                      size_t t, size_t k, size_t out, void* d_y,
                                      size_t y_stride_elems, nnb_dtype dtype);

/* BitLinear::backward, token-major (compute_layer_bitlinear.hpp:475-544).
 * dX (matmul_q_t, :494): d_dx (t,k) (+)= (d_dy (t,out) * tau) . trit (out,k).
 * dW (:514-534): d_dw (out,k) += tau * ((d_dy * s)^T . q) with q, s from nnb_act_quant_tm.
 * exact = 1: f32 operands on CUDA cores; 0: bf16 operands on tensor cores, f32 accumulation. */
nnb_status nnb_bitlinear_dx_tm(nnb_engine* e, const float* d_dy, const uint32_t* d_wq, const float* d_tau, size_t t,
                               size_t k, size_t out, float* d_dx, int accumulate, int exact);
nnb_status nnb_bitlinear_dw_tm(nnb_engine* e, const float* d_dy, const int8_t* d_q, const float* d_s,
                               const float* d_tau, size_t t, size_t k, size_t out, float* d_dw, int exact);

/* ---- the tcgen05 (tensor memory) versions for large token counts.  The ternary container is
 * expanded once per requantisation: d_w8 (rows,k) int8 trits with k permuted like the engine's
 * activation layout, d_wb (rows,k) bf16 trits; either may be NULL. */
nnb_status nnb_expand_weights(nnb_engine* e, const uint32_t* d_wq, size_t rows, size_t k, int8_t* d_w8, void* d_wb);
/* same result as nnb_bitlinear_fwd_tm (bit-exact), f32 output, optional bias and residual (t,out) */
nnb_status nnb_bitlinear_fwd_tc(nnb_engine* e, const int8_t* d_w8, const float* d_tau, const float* d_bias,
                                const float* d_residual, const int8_t* d_q, const float* d_s, size_t t, size_t k,
                                size_t out, float* d_y);
/* The LM head fused with CategoricalDistribution::log_prob / entropy and their gradients
 * (include/neuralnet.cpp/rl_policy.hpp:92-187): the logits x = (tau*s)*acc + bias of nnb_bitlinear_fwd_tc are consumed in
 * the GEMM's epilogue and never stored, as the reference's sparse cross-entropy folds its log-sum-exp online instead of
 * re-reading (V, T) logits (include/neuralnet.cpp/compute_loss.hpp:315-429).
 * fwd: d_logp[t] = x[t, action] - lse, d_entropy[t] = -sum p log p (may be NULL), d_lse[t] = log sum exp(x[t, :]).
 * bwd: d logits = (onehot - p) * up_logp + (-p * (log p + H)) * up_entropy, recomputed from the same integer GEMM;
 * d_dyb (t, v) bf16 receives d logits * tau, the operand nnb_bitlinear_bwd_tc takes with d_dy == NULL, and d_dbias (v)
 * is incremented by the column sums of d logits.  d_up_entropy may be NULL.  Requires v % 4 == 0 in the backward. */
nnb_status nnb_lmhead_logprob_entropy_fwd(nnb_engine* e, const int8_t* d_w8, const float* d_tau, const float* d_bias, const int8_t* d_q,
                                          const float* d_s, const int32_t* d_actions, size_t t, size_t k, size_t v, float* d_logp,
                                          float* d_entropy, float* d_lse);
nnb_status nnb_lmhead_logprob_entropy_bwd(nnb_engine* e, const int8_t* d_w8, const float* d_tau, const float* d_bias, const int8_t* d_q,
                                          const float* d_s, const int32_t* d_actions, const float* d_lse, const float* d_entropy,
                                          const float* d_up_logp, const float* d_up_entropy, size_t t, size_t k, size_t v, void* d_dyb,
                                          float* d_dbias);
/* Tuning knob, process-wide: width of the 128 x bn output tile of nnb_bitlinear_fwd_tc (64, 128, 192 or
 * 256); 0 restores the automatic choice from the problem shape.  Results do not depend on it. */
nnb_status nnb_tc_set_forward_tile(int bn);
/* BitLinear::backward on bf16 tensor cores: d_dyb (t,out) and d_xs (t,k) are bf16 scratch buffers the
 * call fills (dy*tau and s*q); d_dx (t,k) and/or d_dw (out,k) may be NULL to skip that half.  With
 * d_dy == NULL the scratch buffers are taken as already filled by an earlier call and only the GEMMs run. */
nnb_status nnb_bitlinear_bwd_tc(nnb_engine* e, const float* d_dy, const float* d_tau, const void* d_wb,
                                const int8_t* d_q, const float* d_s, size_t t, size_t k, size_t out, void* d_dyb,
                                void* d_xs, float* d_dx, int accumulate_dx, float* d_dw);
/* Causal multi-head self-attention over whole sequences, token-major: q, k, v, out, dout and the
 * gradients are (n_seq*seq_len, n_head*dk) f32 (q, k already rotated), lse and delta (n_seq, n_head, seq_len).
 * AttentionBase::forward core (include/neuralnet.cpp/compute_layer_attention.hpp:752-828: scale folded into
 * Q, online-softmax fold) and backward core (:873-960).  exact = 1: f64/f32 CUDA-core path; 0: bf16
 * tensor cores (head dims 64 and 128, else the CUDA-core path). */
nnb_status nnb_attention_fwd(nnb_engine* e, const float* d_q, const float* d_k, const float* d_v, size_t n_seq,
                             size_t seq_len, size_t n_head, size_t dk, int exact, float* d_out, float* d_lse);
nnb_status nnb_attention_bwd(nnb_engine* e, const float* d_q, const float* d_k, const float* d_v, const float* d_out,
                             const float* d_dout, const float* d_lse, size_t n_seq, size_t seq_len, size_t n_head,
                             size_t dk, int exact, float* d_delta, float* d_dq, float* d_dk, float* d_dv);
/* The same operators with the rotary embedding inside (AttentionBase with rope,
 * include/neuralnet.cpp/compute_layer_attention.hpp:698-750 applies it to q and k before the core): q and k
 * are un-rotated, d_rope_cos / d_rope_sin are (seq_len, dk/2) tables indexed by the position in the
 * sequence, and d_dq / d_dk are gradients with respect to the un-rotated q and k. */
nnb_status nnb_attention_rope_fwd(nnb_engine* e, const float* d_q, const float* d_k, const float* d_v,
                                  const float* d_rope_cos, const float* d_rope_sin, size_t n_seq, size_t seq_len,
                                  size_t n_head, size_t dk, int exact, float* d_out, float* d_lse);
nnb_status nnb_attention_rope_bwd(nnb_engine* e, const float* d_q, const float* d_k, const float* d_v,
                                  const float* d_rope_cos, const float* d_rope_sin, const float* d_out, const float* d_dout,
                                  const float* d_lse, size_t n_seq, size_t seq_len, size_t n_head, size_t dk, int exact,
                                  float* d_delta, float* d_dq, float* d_dk, float* d_dv);
/* Attention of one new token per sequence against the KV cache: the attention part of
 * GPTModel::forward_step (include/neuralnet.cpp/compute_layer_gpt.hpp:520-560 drives
 * AttentionBase::forward_step, compute_layer_attention.hpp:990-1080).  d_qkv (3, n_seq, d) f32 holds the
 * new token's un-rotated projections; the position *d_pos lives on the device.  The call rotates q and k
 * (tables (ctx, dk/2), or NULL for none), appends k and v at row *d_pos - pre_len of the per-sequence
 * caches (n_seq, n_head, ctx_alloc, dk) — f32 when exact = 1, bf16 when 0 — and attends over positions
 * 0..*d_pos, the first pre_len of them read from the prefix caches (n_seq / group, n_head, pre_alloc, dk)
 * shared by `group` consecutive sequences (pre_len = 0, group = 1: none).  Outputs: d_out (n_seq, d) f32,
 * and/or, in the fast mode, the int8 quantisation of that row in the engine's activation layout (d_q8,
 * d_s, d_qsum as nnb_act_quant_tm would give), produced by the same launch. */
nnb_status nnb_attention_decode(nnb_engine* e, const float* d_qkv, void* d_kcache, void* d_vcache, size_t ctx_alloc,
                                const void* d_kpre, const void* d_vpre, size_t pre_len, size_t pre_alloc, size_t group,
                                const float* d_rope_cos, const float* d_rope_sin, const int* d_pos, size_t n_seq,
                                size_t n_head, size_t dk, int exact, float* d_out, int8_t* d_q8, float* d_s, int32_t* d_qsum);
/* synchronises and reports NNB_ERR_TIMEOUT if a kernel gave up on a bounded device-side wait */
nnb_status nnb_engine_check(nnb_engine* e);

/* Host-buffer convenience: quantise h_x (t,k) f32, run the linear, return h_y (t,out) f32.
 * Copies host->device and device->host inside the call and synchronises. */
nnb_status nnb_bitlinear_fwd_host(nnb_engine* e, const uint32_t* d_wq, const float* d_tau,
                                  const float* d_bias, const float* h_x, size_t t, size_t k,
                                  size_t out, float* h_y);

/* ================= GPT policy with ternary linears ========================
 * The model the reference builds with build_gpt_model(engine, GptConfig)
 * (include/neuralnet.cpp/domain_gpt.hpp:59-77): token embedding, learned or rotary positions,
 * pre-norm blocks (RMSNorm, causal MHA, QuickGELU or SwiGLU feed-forward), final RMSNorm and an
 * untied BitLinear head; every linear is a BitLinear with bias and int8 activations. */
typedef struct nnb_gpt_config {
    int32_t n_layer, d_model, n_head, d_ff, vocab, ctx;
    int32_t act;        /* 0 = QuickGELU (GeLU layer of the reference), 1 = SwiGLU, 2 = ReLU2GLU: relu(gate)^2 * up
                           (include/neuralnet.cpp/compute_layer_mlp.hpp:384-440, the BitNet 2B4T feed-forward) */
    int32_t pos;        /* 0 = learned additive positions, 1 = RoPE */
    int32_t value_head; /* 1 adds a Linear(d_model -> 1) port on the final-norm output */
    int32_t exact;      /* 1: f32 activations and KV cache, f64-accumulated reductions (the mode
                           compared token by token with the CPU restatement); 0: bf16 KV cache */
    /* The structure switches of BitNet b1.58 2B4T (all 0: the layout above, bit for bit). */
    int32_t sub_ln;     /* 1: an RMSNorm inside each sub-layer, between the heads' output and the o projection
                           (include/neuralnet.cpp/compute_layer_attention.hpp:482-489,820-826) and between the activated
                           hidden and fc2 (include/neuralnet.cpp/compute_layer_feedforward.hpp:37-47,201-206); adds the
                           tensors blocks.N.attn.sub_norm.gamma (d_model) and blocks.N.ffn.sub_norm.gamma (d_ff) */
    int32_t n_head_kv;  /* grouped-query attention: key / value heads (0 = n_head); must divide n_head; query head h reads
                           KV head h / (n_head / n_head_kv) (include/neuralnet.cpp/compute_layer_attention.hpp:444-454);
                           the k and v projections are (n_head_kv * d_k, d_model) */
    int32_t tie_embeddings; /* 1: logits = tok_emb . ln_f(x), a dense product without bias; no lm_head tensors; the
                           head's weight gradient adds into tok_emb's (include/neuralnet.cpp/compute_layer_gpt.hpp:286-297,
                           556-575) */
} nnb_gpt_config;

typedef struct nnb_policy nnb_policy;

nnb_status nnb_policy_create(nnb_engine* e, const nnb_gpt_config* cfg, nnb_policy** out);
void nnb_policy_destroy(nnb_policy* p);
/* the f32 master parameters live in one flat device buffer; tensors are described by name */
size_t nnb_policy_param_count(const nnb_policy* p);
float* nnb_policy_params(nnb_policy* p);
size_t nnb_policy_tensor_count(const nnb_policy* p);
nnb_status nnb_policy_tensor_info(const nnb_policy* p, size_t index, char* name, size_t name_len,
                                  size_t* offset, size_t* rows, size_t* cols);
/* Layer::import_param for every tensor at once: copy host parameters in and requantise */
nnb_status nnb_policy_upload_params(nnb_policy* p, const float* h_params);
/* BitLinear::quantize_weights_ for every linear (compute_layer_bitlinear.hpp:627-674):
 * call after the master weights changed */
nnb_status nnb_policy_requantize(nnb_policy* p);
/* Model files in the reference's two roles (include/neuralnet.cpp/model_serialization.hpp:40-89; parameter entries
 * :581-589 byte for byte).  role 0 = model (.nnmodel): ternary weights as TernaryPacked3 (base-3, 1.6 bits per weight)
 * plus tau; role 1 = checkpoint (.nnckpt): ternary weights as their f32 latent.  Loading a model-role file restores a
 * trainable policy the way WeightLoadIntent::Trainable does (compute_layer_bitlinear.hpp:262-300): latent = trit *
 * (tau * K / n), the quantiser's fixed point, with the file's tau and trits seeding the packed weights, so the first
 * forward reproduces the saved model bit for bit.  The spec record's byte layout and the base-3 digit order live in
 * modules absent from the reference tree and are this library's own.  The file is verified (tail marker, SHA-256)
 * before anything is read from it. */
nnb_status nnb_policy_save(nnb_policy* p, const char* path, int role);
nnb_status nnb_policy_load(nnb_policy* p, const char* path);
/* nn::trit_pack row codecs on the host: base-3 disk form <-> 2-bit container, and the dequantisation
 * L = trit * latent_row_scale, latent_row_scale = tau * K / n (0 for an all-zero row) (src/ternary_gemm_test.cpp:658-735) */
size_t nnb_trit_base3_bytes_per_row(size_t k);
void nnb_trit_pack_row_base3(const uint32_t* words, size_t k, uint8_t* out);
void nnb_trit_unpack_row_base3(const uint8_t* in, size_t k, uint32_t* words);
float nnb_trit_latent_row_scale(const uint32_t* words, size_t k, float tau);
void nnb_trit_dequant_row(const uint32_t* words, size_t k, float tau, float* latent);
/* device pointers of one linear's container and scales; layer < 0 selects the head,
 * which in 0..5 = q, k, v, o, fc1, fc2 */
nnb_status nnb_policy_linear(nnb_policy* p, int layer, int which, uint32_t** d_packed, float** d_tau,
                             size_t* in, size_t* out);

/* Batched GPTModel::generate (include/neuralnet.cpp/compute_layer_gpt.hpp:740-852) with
 * sample_next_token_ (compute_layer_base.hpp:1025-1163; temperature and top-k): n_seq prompts of
 * prompt_len ids each, max_new sampled tokens.  temperature <= 0 is greedy.  The uniform draw of
 * sequence b at generated step t is Philox4x32-10 keyed by seed with counter (seq0 + b, t).
 * d_tokens (n_seq, prompt_len + max_new); d_logp (n_seq, max_new) log-prob of each sampled token
 * under softmax(raw logits), may be NULL; d_logits (n_seq, max_new, vocab) may be NULL. */
nnb_status nnb_rollout(nnb_policy* p, const int32_t* d_prompts, size_t n_seq, size_t prompt_len,
                       size_t max_new, float temperature, int top_k, uint64_t seed, uint32_t seq0,
                       int32_t* d_tokens, float* d_logp, float* d_logits);
/* The same when every `group_size` consecutive sequences were given the same prompt (the GRPO sampling
 * pattern): the shared prompt prefix is decoded once per group into a prefix KV cache that all members
 * read, so prompt positions cost 1/group_size of the work and of the cache traffic.  Per-sequence
 * results are identical to nnb_rollout.  n_seq must be a multiple of group_size. */
nnb_status nnb_rollout_grouped(nnb_policy* p, const int32_t* d_prompts, size_t n_seq, size_t prompt_len, size_t max_new,
                               size_t group_size, float temperature, int top_k, uint64_t seed, uint32_t seq0,
                               int32_t* d_tokens, float* d_logp, float* d_logits);
/* SamplingConfig of the reference (include/neuralnet.cpp/compute_layer_base.hpp:1002-1022) for the batched
 * rollout; the sampler applies its fields in the reference's order (compute_layer_base.hpp:1025-1163):
 * logit bias -> repeat penalty over the distinct tokens of the last repeat_window tokens of the sequence so far
 * (0 = all of it; positive logits are divided by the penalty, the others multiplied) -> temperature -> top-k ->
 * softmax over the candidates -> top-p -> greedy (temperature <= 0) or inverse CDF.
 * d_logit_bias (vocab) f32, optional, is added to the raw logits first: the device-side form of the reference's
 * host hook logits_transform (-inf forbids a token).  top_p < 1 needs at most 1024 candidates (top_k in 1..1024,
 * or a vocabulary of at most 1024), otherwise NNB_ERR_UNSUPPORTED.  eos_token >= 0: a sequence that samples it
 * at a generated index >= min_new_tokens is finished (GPTModel::generate, compute_layer_gpt.hpp:826-828); its
 * later tokens are eos_token with log-prob 0, and d_gen_len[b] = tokens generated before it (max_new if never). */
typedef struct nnb_sampling_config {
    float temperature; /* <= 0: greedy */
    int32_t top_k;     /* 0: off */
    float top_p;       /* >= 1: off */
    float repeat_penalty; /* <= 0 or 1: off */
    int32_t repeat_window;
    uint64_t seed;
    const float* d_logit_bias;
    int32_t eos_token; /* < 0: none */
    int32_t min_new_tokens;
} nnb_sampling_config;
/* nnb_rollout_grouped with the full sampling configuration; d_gen_len (n_seq) may be NULL */
nnb_status nnb_rollout_sampled(nnb_policy* p, const int32_t* d_prompts, size_t n_seq, size_t prompt_len, size_t max_new,
                               size_t group_size, const nnb_sampling_config* cfg, uint32_t seq0, int32_t* d_tokens,
                               float* d_logp, float* d_logits, int32_t* d_gen_len);
/* the same with host buffers: copies prompts in and tokens / log-probs out, and synchronises */
nnb_status nnb_rollout_host(nnb_policy* p, const int32_t* h_prompts, size_t n_seq, size_t prompt_len,
                            size_t max_new, float temperature, int top_k, uint64_t seed, uint32_t seq0,
                            int32_t* h_tokens, float* h_logp);

/* Measurement aid for the rollout (the reference times its decode loop per token on the host,
 * src/layer_bench.cpp:702-715).  With stride > 0 every later rollout of this policy records a CUDA event
 * on its stream before every stride-th decode step and after the last one; stride = 0 turns it off.
 * nnb_rollout_step_times waits for the last rollout and returns, for segment i, h_ms[i] = device time of
 * the steps between events i and i+1 and h_pos[i] = the position the first of those steps consumed
 * (either array may be NULL; *n_out = number of segments, at most cap of them are written). */
nnb_status nnb_rollout_set_step_timing(nnb_policy* p, size_t stride);
nnb_status nnb_rollout_step_times(nnb_policy* p, float* h_ms, int32_t* h_pos, size_t cap, size_t* n_out);

/* ---- training of the policy on micro-batches of whole sequences.
 * A sequence of seq_len tokens whose first prompt_len are the prompt has G = seq_len - prompt_len
 * decisions; decision g is taken at position prompt_len-1+g and its action is token prompt_len+g.
 * Per-decision vectors are (n_seq, G) f32 on the device. */

/* teacher-forced GPTModel::forward (include/neuralnet.cpp/compute_layer_gpt.hpp:460-543) followed by
 * CategoricalDistribution::log_prob / entropy; d_entropy and d_value may be NULL.  No gradients:
 * this is how a frozen reference policy (TrainingGroupSession readonly role,
 * include/neuralnet.cpp/training_group_session.hpp:102-110) is evaluated. */
nnb_status nnb_policy_logprobs(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t seq_len, size_t prompt_len,
                               float* d_logp, float* d_entropy, float* d_value);

/* the objective of one training micro-batch: PpoObjective / GrpoObjective with explicit advantages
 * (include/neuralnet.cpp/rl_policy.hpp:799-953) plus a sampled-KL term against a reference policy */
typedef struct nnb_objective {
    const float* d_mask;       /* action mask, required */
    const float* d_old_logp;   /* with d_advantage: clipped policy term; both NULL to skip */
    const float* d_advantage;
    const float* d_ref_logp;   /* KL term (kl_coef != 0): kl_coef * mean(logp - ref_logp).  An addition of this engine
                                  for a frozen reference policy: the reference's GrpoObjective has no KL term
                                  (rl_policy.hpp:934-951) and its SampledKlObjective (:503-530) penalises
                                  logp - old_log_prob, which is d_ref_logp = d_old_logp here; kl_coef = 0 is the
                                  reference's GRPO preset */
    const float* d_returns;    /* value term (value_coef != 0): returns and old values */
    const float* d_old_value;
    float units;               /* normalisation count; <= 0 = sum of this micro-batch's mask.  Pass the
                                  count of the whole (global) batch when it is split into micro-batches
                                  or across GPUs (normalization_units, training_session.hpp:102-109) */
    float clip_eps, kl_coef, entropy_coef, value_coef, value_clip_eps;
} nnb_objective;

/* The ten floats a training call reports, named after the reference's report structs (PpoReport / GrpoReport and
 * PpoPolicyMetrics, include/neuralnet.cpp/rl_policy.hpp:787-797,858-864): PpoReport.policy_loss =
 * [NNB_REPORT_CLIPPED_POLICY_LOSS] + [NNB_REPORT_ENTROPY_LOSS], PpoReport.value_loss = [NNB_REPORT_VALUE_LOSS],
 * PpoReport.loss = their sum (+ [NNB_REPORT_KL_LOSS], this engine's addition), PpoReport.entropy =
 * [NNB_REPORT_ENTROPY], approx_kl, policy_clip_fraction and value_clip_fraction as named. */
enum {
    NNB_REPORT_CLIPPED_POLICY_LOSS = 0, /* ClippedPolicyObjective loss */
    NNB_REPORT_RATIO_MEAN = 1,          /* PpoPolicyMetrics.ratio_mean */
    NNB_REPORT_APPROX_KL = 2,
    NNB_REPORT_POLICY_CLIP_FRACTION = 3,
    NNB_REPORT_KL_LOSS = 4,     /* kl_coef * mean(logp - ref_logp) */
    NNB_REPORT_ENTROPY_LOSS = 5, /* -entropy_coef * mean entropy */
    NNB_REPORT_ENTROPY = 6,
    NNB_REPORT_UNITS = 7,        /* the normalisation count */
    NNB_REPORT_VALUE_LOSS = 8,
    NNB_REPORT_VALUE_CLIP_FRACTION = 9,
    NNB_REPORT_COUNT = 10
};
/* forward + objective + GPTModel::backward (compute_layer_gpt.hpp:545-636): gradients are ADDED to the
 * policy's gradient buffer.  d_report[NNB_REPORT_COUNT] (may be NULL) as named above.
 * The activations kept for the backward live in one workspace sized at the first call of a shape (n_seq, seq_len,
 * prompt_len, group).  A workspace that does not fit the free device memory is refused with NNB_ERR_OOM before any
 * kernel runs and before the gradient buffer is touched: call again with fewer sequences (gradients accumulate over
 * calls, so the split does not change the update). */
nnb_status nnb_policy_train_step(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t seq_len,
                                 size_t prompt_len, const nnb_objective* obj, float* d_report);
/* The same two calls for a batch whose sequences come in groups of `group` consecutive rows that share
 * their first prompt_len tokens (the completions of one prompt, as nnb_rollout_grouped produces them; the
 * caller vouches for it).  Results per sequence are those of the plain calls; the prompt's rows are
 * stored and computed once per group instead of once per sequence, and their gradient contributions are
 * summed before the weight-gradient GEMMs.  Applies in the fast mode when prompt_len is a multiple of 64;
 * otherwise the calls fall back to one copy per sequence.  No counterpart in the reference, which runs
 * every sequence in full. */
nnb_status nnb_policy_logprobs_grouped(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t seq_len, size_t prompt_len,
                                       size_t group, float* d_logp, float* d_entropy, float* d_value);
nnb_status nnb_policy_train_step_grouped(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t seq_len,
                                         size_t prompt_len, size_t group, const nnb_objective* obj, float* d_report);
/* Supervised step on the same machinery: sparse cross-entropy of the next token
 * (CrossEntropyLoss::fused_forward_sparse_, include/neuralnet.cpp/compute_loss.hpp:315-429): with the
 * decisions and actions defined above (prompt_len = 1 covers every position of a sequence),
 * loss = -sum mask * log softmax(logits)[label] / units, units <= 0 meaning the sum of the mask (the
 * reference's num_valid); gradients are ADDED to the gradient buffer.  d_report[10] as in
 * nnb_policy_train_step with the loss in d_report[0] and the units in d_report[7].  group as above. */
nnb_status nnb_policy_sft_step(nnb_policy* p, const int32_t* d_tokens, size_t n_seq, size_t seq_len, size_t prompt_len,
                               size_t group, const float* d_mask, float units, float* d_report);

/* After a training micro-batch (nnb_policy_train_step* / nnb_policy_sft_step): the int8 activations that layer `layer`
 * kept for its backward pass, in the engine's K-permuted layout, and their per-token scales.  which: 0 = input of
 * q|k|v (ln1 output), 1 = input of o, 2 = input of fc1 (ln2 output), 3 = input of fc2.  *rows / *cols receive the
 * shape; d_q (rows * cols bytes) and d_s (rows floats) may be NULL to query the shape only.  Two policies in
 * different numeric modes given the same tokens can be compared entry by entry with it (how many int8 activations
 * the fast mode flips). */
nnb_status nnb_policy_cached_activation(nnb_policy* p, int layer, int which, int8_t* d_q, float* d_s, size_t* rows,
                                        size_t* cols);
/* flat f32 gradient buffer, same layout as the parameters (allocated and zeroed on first use) */
float* nnb_policy_grads(nnb_policy* p);
nnb_status nnb_policy_zero_grad(nnb_policy* p);
/* TrainingSession::finish_update_ (include/neuralnet.cpp/training_session.hpp:599-638): global-norm clip
 * (max_grad_norm <= 0 disables), AdamW step, zero_grad, and requantisation of every BitLinear.  The
 * gradient norm before clipping goes to d_norm_out (may be NULL).  With several GPUs, all-reduce
 * nnb_policy_grads before calling this. */
nnb_status nnb_policy_optimizer_step(nnb_policy* p, float lr, float beta1, float beta2, float eps, float weight_decay,
                                     float max_grad_norm, float* d_norm_out);
/* frees the rollout (KV cache) and training workspaces; they are re-created on demand */
nnb_status nnb_policy_release_workspaces(nnb_policy* p);

/* ================= advantages, objectives, optimizer ======================
 * Per-decision vectors are plain f32 arrays of length n (the reference's (1,T) tensors);
 * logits are token-major (t, vocab).  Nothing here synchronises with the host. */

/* GaeAdvantage::apply (include/neuralnet.cpp/rl_experience.hpp:273-380).  rewards, values,
 * done, mask, outputs are (steps, batch) with row = time; done, mask, bootstrap (batch) may be NULL. */
nnb_status nnb_gae(nnb_engine* e, const float* d_rewards, const float* d_values, const float* d_done,
                   const float* d_mask, const float* d_bootstrap, size_t steps, size_t batch, float gamma,
                   float lambda, float* d_advantage, float* d_returns);
/* MonteCarloReturn::apply (rl_experience.hpp:395-440): ret_t = r_t + gamma * ret_{t+1} * (1 - done_t), each
 * row multiplied by the mask before it is carried to the previous step; same layout as nnb_gae. */
nnb_status nnb_monte_carlo_return(nnb_engine* e, const float* d_rewards, const float* d_done, const float* d_mask,
                                  size_t steps, size_t batch, float gamma, float* d_returns);
/* GroupAdvantage::apply (rl_experience.hpp:516-545): spans (first_row, row_count) given on the
 * host must be contiguous and cover all n rows, else NNB_ERR_INVALID. */
nnb_status nnb_group_advantage(nnb_engine* e, const float* d_returns, size_t n, const int32_t* h_first,
                               const int32_t* h_count, size_t n_spans, float eps, float* d_out);
/* nnb_group_advantage for callers that cannot allocate device memory (a host whose own pool owns the
 * whole GPU, a step running where the CUDA allocator must not be entered, a fixed start-up budget).
 * It has no counterpart in the reference.  Same arguments and result as nnb_group_advantage; the
 * device copy of the span table lives in a fixed 128 KiB array inside the library (held by every GPU
 * that loads it, until exit), so the call does no cudaMalloc / cudaFree.  Limit: n_spans <= 16384,
 * larger requests are rejected with NNB_ERR_INVALID.  The array's device address is looked up once per
 * device (cudaGetSymbolAddress, with that device current; the caller's current device is put back):
 * nnb_engine_create does it, and a call on a device where that has not happened yet does it first, so
 * create the engine before any stream capture begins.  h_first / h_count are read during the call and
 * may be reused once it returns.  All calls share the one array, which keeps the last call's table:
 * the entries a call reads are rewritten by that call, nothing has to start at zero.  Calls whose GPU
 * work can overlap (different streams or engines on the same device) race on it and must be serialised
 * by the caller. */
nnb_status nnb_group_advantage_noalloc(nnb_engine* e, const float* d_returns, size_t n, const int32_t* h_first,
                                       const int32_t* h_count, size_t n_spans, float eps, float* d_out);
/* MaskedNormalizer::apply (rl_experience.hpp:456-498); mask may be NULL (all ones) */
nnb_status nnb_masked_normalize(nnb_engine* e, const float* d_values, const float* d_mask, size_t n, float eps,
                                float* d_out);
/* CategoricalDistribution::log_prob / entropy (include/neuralnet.cpp/rl_policy.hpp:92-143) */
nnb_status nnb_categorical_logp_entropy(nnb_engine* e, const float* d_logits, const int32_t* d_actions, size_t t,
                                        size_t v, float* d_logp, float* d_entropy);
/* log_prob_with_gradient + entropy_with_gradient (rl_policy.hpp:145-187):
 * dlogits = (onehot - p)*up_logp + (-p*(log p + H))*up_entropy; either upstream may be NULL */
nnb_status nnb_categorical_backward(nnb_engine* e, const float* d_logits, const int32_t* d_actions,
                                    const float* d_up_logp, const float* d_up_entropy, size_t t, size_t v,
                                    float* d_dlogits);
/* ClippedPolicyObjective + SampledKlObjective + EntropyBonusObjective in one pass
 * (rl_policy.hpp:564-661, 503-530, 460-481; the PPO / GRPO presets :799-953 sum them).
 * units <= 0 means sum(mask); pass the global count when the batch is sharded.
 * d_old_logp/d_advantage (clipped term), d_ref_logp (KL term) and d_entropy may be NULL.
 * Outputs: d_up_logp = d loss/d logp, d_up_entropy = d loss/d entropy (may be NULL),
 * d_report[8] = policy_loss, ratio_mean, approx_kl, clip_fraction, kl_loss, entropy_loss,
 * mean entropy, units (may be NULL). */
nnb_status nnb_token_objective(nnb_engine* e, const float* d_logp, const float* d_entropy, const float* d_old_logp,
                               const float* d_ref_logp, const float* d_advantage, const float* d_mask, size_t n,
                               float units, float clip_eps, float kl_coef, float entropy_coef, float* d_up_logp,
                               float* d_up_entropy, float* d_report);
/* ClippedValueObjective (rl_policy.hpp:670-773); d_report[2] = value_loss, clip_fraction */
nnb_status nnb_clipped_value(nnb_engine* e, const float* d_value, const float* d_returns, const float* d_old_value,
                             const float* d_mask, size_t n, float units, float clip_eps, float coef, float* d_grad,
                             float* d_report);
/* ValueRegressionObjective (rl_policy.hpp:393-439): loss = coef * sum (V-R)^2 mask / units,
 * d_grad = (V-R) * mask * (2*coef/units); d_report[2] = loss, units (may be NULL) */
nnb_status nnb_value_regression(nnb_engine* e, const float* d_value, const float* d_returns, const float* d_mask, size_t n,
                                float units, float coef, float* d_grad, float* d_report);
/* Optimizer::clip_grad_norm (include/neuralnet.cpp/compute_optimizer.hpp:134-187); the norm
 * before clipping is written to d_norm_out (may be NULL) */
nnb_status nnb_clip_grad_norm(nnb_engine* e, float* d_grads, size_t n, float max_norm, float* d_norm_out);
/* ComputeEngine::scale_inplace */
nnb_status nnb_scale_inplace(nnb_engine* e, float* d_x, size_t n, float scale);
/* AdamW::step (compute_optimizer.hpp:384-436,563-597) at 1-based step t */
nnb_status nnb_adamw_step(nnb_engine* e, float* d_params, const float* d_grads, float* d_m, float* d_v, size_t n,
                          float lr, float beta1, float beta2, float eps, float weight_decay, int t);

#ifdef __cplusplus
}
#endif
#endif /* NN_B200_H */
