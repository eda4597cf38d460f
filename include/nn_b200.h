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

/* Host-buffer convenience: quantise h_x (t,k) f32, run the linear, return h_y (t,out) f32.
 * Copies host->device and device->host inside the call and synchronises. */
nnb_status nnb_bitlinear_fwd_host(nnb_engine* e, const uint32_t* d_wq, const float* d_tau,
                                  const float* d_bias, const float* h_x, size_t t, size_t k,
                                  size_t out, float* h_y);

#ifdef __cplusplus
}
#endif
#endif /* NN_B200_H */
