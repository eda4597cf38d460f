/*
 * oracle.c — CPU restatement of the reference's ternary-linear semantics.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA engine: it is
 * compiled into oracle/liboracle.so and may be loaded only by tests, by the smoke
 * check and by the CPU-baseline leg of the benchmark.  Nothing in the product
 * library links, loads or calls it, and the product has no CPU fallback.
 *
 * Why a restatement: the reference's CPU engine (CpuEngine, ternary_pack.hpp,
 * int8_pack.hpp) lives in the un-vendored submodule
 * neuralnet-cpp-dev/compute.neuralnet.cpp (pinned commit not recoverable), so it
 * cannot be compiled.  Each function below follows the reference's own call
 * sites and the host reference loops of its tests, cited per function, and is
 * pinned by the golden vectors those tests contain (tests/test_oracle_pins.py).
 * Float accumulation order of matmul_q / matmul_q_t is not pinned bitwise by any
 * reference test ("parity unpinned" for those two: tolerance-gated only);
 * integer paths are order-independent and pinned bit-exactly.
 *
 * Layouts are the reference's: row-major 2-D, activations (features, tokens),
 * weights (out_features, in_features).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- trit codec
 * nn::trit_pack — 2 bits per weight, 16 per uint32 word, code = trit + 2,
 * weight j of a row at bits (word >> 2j) & 3, tail padded with code 2.
 * Pinned by src/ternary_gemm_test.cpp:69-99.  Threshold rule (strict compares,
 * |w| == 0.5*tau -> 0): include/neuralnet.cpp/compute_layer_bitlinear.hpp:657-667.
 */
ORC_API uint32_t orc_trit_code_of(float w, float tau)
{
    const float hi = tau * 0.5f;
    const float lo = tau * -0.5f;
    if (w > hi) return 3u;
    if (w < lo) return 1u;
    return 2u;
}

ORC_API float orc_trit_value_of(uint32_t code) { return (float)((int)code - 2); }

ORC_API size_t orc_trit_words_per_row(size_t k) { return (k + 15) / 16; }

ORC_API size_t orc_trit_bytes_per_row(size_t k) { return orc_trit_words_per_row(k) * 4; }

ORC_API void orc_trit_pack_row(const float* w, size_t k, float tau, uint32_t* words)
{
    const size_t wpr = orc_trit_words_per_row(k);
    for (size_t i = 0; i < wpr; ++i) words[i] = 0u;
    for (size_t i = 0; i < wpr * 16; ++i) {
        const uint32_t code = (i < k) ? orc_trit_code_of(w[i], tau) : 2u;
        words[i / 16] |= code << (2 * (i % 16));
    }
}

ORC_API float orc_trit_at(const uint32_t* words, size_t i)
{
    return orc_trit_value_of((words[i / 16] >> (2 * (i % 16))) & 3u);
}

/* tau_o = sum_k |W[o,k]| * (1/K)  (compute_layer_bitlinear.hpp:637-640).  The terms are
 * f32 products as in the reference; the order of the reference's f32 row sum is
 * engine-defined (tau is tolerance-level there: 1e-6 in src/t1_58_test.cpp:291), so the
 * sum is taken in double and rounded once, which makes it independent of the order. */
ORC_API void orc_absmean_tau(const float* latent, size_t rows, size_t k, float* tau)
{
    const float inv = 1.0f / (float)k;
    for (size_t r = 0; r < rows; ++r) {
        double s = 0.0;
        for (size_t c = 0; c < k; ++c) s += (double)(fabsf(latent[r * k + c]) * inv);
        tau[r] = (float)s;
    }
}

/* ComputeEngine::trit_pack(latent, tau): (rows,K) f32 + (rows,1) -> (rows, ceil(K/16)) words.
 * src/ternary_gemm_test.cpp:223-251. */
ORC_API void orc_trit_pack(const float* latent, const float* tau, size_t rows, size_t k,
                           uint32_t* packed)
{
    const size_t wpr = orc_trit_words_per_row(k);
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r)
        orc_trit_pack_row(latent + r * k, k, tau[r], packed + r * wpr);
}

/* ------------------------------------------------------------------ i8 codec
 * nn::i8_pack — q = round_half_away(clamp(x/s, -127, 127)); NaN -> 0; s == 0 -> 0.
 * 4 int8 per word, little-endian bytes within a word, tail bytes 0.
 * docs/internal/21-quantized-weights.md:966-982; src/int8_act_test.cpp:86-137.
 */
ORC_API int8_t orc_i8_quantize(float x, float s)
{
    if (s == 0.0f) return 0;
    float v = x / s;
    if (v != v) return 0;
    if (v > 127.0f) v = 127.0f;
    if (v < -127.0f) v = -127.0f;
    return (int8_t)roundf(v);
}

ORC_API size_t orc_i8_words_per_row(size_t n) { return (n + 3) / 4; }

ORC_API int8_t orc_i8_at(const uint32_t* words, size_t i)
{
    return (int8_t)((words[i / 4] >> (8 * (i % 4))) & 0xFFu);
}

/* ComputeEngine::quantize_i8(x (M,N), scale, col_scale): scale is (1,N) when
 * col_scale (per-token activations) else (M,1).  Output (M, ceil(N/4)) words. */
ORC_API void orc_quantize_i8(const float* x, size_t m, size_t n, const float* scale, int col_scale,
                             uint32_t* out)
{
    const size_t wpr = orc_i8_words_per_row(n);
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < m; ++r) {
        for (size_t wi = 0; wi < wpr; ++wi) out[r * wpr + wi] = 0u;
        for (size_t c = 0; c < n; ++c) {
            const float s = col_scale ? scale[c] : scale[r];
            const uint8_t q = (uint8_t)orc_i8_quantize(x[r * n + c], s);
            out[r * wpr + c / 4] |= (uint32_t)q << (8 * (c % 4));
        }
    }
}

/* ComputeEngine::unpack_i8(packed, cols) -> f32 integers, no scale applied. */
ORC_API void orc_unpack_i8(const uint32_t* packed, size_t m, size_t n, float* out)
{
    const size_t wpr = orc_i8_words_per_row(n);
    for (size_t r = 0; r < m; ++r)
        for (size_t c = 0; c < n; ++c) out[r * n + c] = (float)orc_i8_at(packed + r * wpr, c);
}

/* BitLinear's per-token scale: s_n = max_k |X[k,n]| * (1/127)
 * (col_reduce_max then scale_inplace(1/127), compute_layer_bitlinear.hpp:443-446). */
ORC_API void orc_col_absmax_scale(const float* x, size_t k, size_t n, float* s)
{
    const float inv = 1.0f / 127.0f;
    for (size_t c = 0; c < n; ++c) {
        float mx = 0.0f;
        for (size_t r = 0; r < k; ++r) {
            const float a = fabsf(x[r * n + c]);
            if (a > mx) mx = a;
        }
        s[c] = mx * inv;
    }
}

/* ------------------------------------------------------------------- matmuls
 * matmul_q: C[m,n] = sum_k (tau_m * trit[m,k]) * X[k,n]; the reference test's
 * host loop accumulates in double (src/ternary_gemm_test.cpp:141-156). */
ORC_API void orc_matmul_q(const uint32_t* packed, const float* tau, const float* x, size_t rows,
                          size_t k, size_t n, float* c)
{
    const size_t wpr = orc_trit_words_per_row(k);
#pragma omp parallel for schedule(static)
    for (size_t m = 0; m < rows; ++m) {
        for (size_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (size_t kk = 0; kk < k; ++kk) {
                const float t = orc_trit_at(packed + m * wpr, kk);
                acc += (double)(tau[m] * t) * (double)x[kk * n + j];
            }
            c[m * n + j] = (float)acc;
        }
    }
}

/* matmul_q_t: A stored (K=rows, M=cols) packed along M; C[m,n] = sum_k (tau_k * trit[k,m]) * B[k,n],
 * tau indexed by storage row, inside the sum (src/ternary_gemm_test.cpp:157-169). */
ORC_API void orc_matmul_q_t(const uint32_t* packed, const float* tau, const float* b, size_t rows,
                            size_t mcols, size_t n, float* c)
{
    const size_t wpr = orc_trit_words_per_row(mcols);
#pragma omp parallel for schedule(static)
    for (size_t m = 0; m < mcols; ++m) {
        for (size_t j = 0; j < n; ++j) {
            double acc = 0.0;
            for (size_t kk = 0; kk < rows; ++kk) {
                const float t = orc_trit_at(packed + kk * wpr, m);
                acc += (double)(tau[kk] * t) * (double)b[kk * n + j];
            }
            c[m * n + j] = (float)acc;
        }
    }
}

/* matmul_q_i8: acc = sum_k trit(m,k) * q(k,n) in int32, k ascending;
 * Y[m,n] = tau_m * s_n * float(acc) evaluated left to right in f32, i.e.
 * (tau*s)*float(acc) (src/int8_act_test.cpp:210-236).  xq is the reference
 * container (K, ceil(N/4)).  acc_out (rows,n) is optional. */
ORC_API void orc_matmul_q_i8(const uint32_t* packed, const float* tau, const uint32_t* xq,
                             const float* s, size_t rows, size_t k, size_t n, float* y,
                             int32_t* acc_out)
{
    const size_t wpr_w = orc_trit_words_per_row(k);
    const size_t wpr_q = orc_i8_words_per_row(n);
#pragma omp parallel for schedule(static)
    for (size_t m = 0; m < rows; ++m) {
        for (size_t j = 0; j < n; ++j) {
            int32_t acc = 0;
            for (size_t kk = 0; kk < k; ++kk) {
                const uint32_t code = (packed[m * wpr_w + kk / 16] >> (2 * (kk % 16))) & 3u;
                const int32_t trit = (int32_t)code - 2;
                acc += trit * (int32_t)orc_i8_at(xq + kk * wpr_q, j);
            }
            if (y) y[m * n + j] = tau[m] * s[j] * (float)acc;
            if (acc_out) acc_out[m * n + j] = acc;
        }
    }
}

/* --------------------------------------------------------------- fast variants
 * Token-major ternary linear used for large parity cases and as the timed CPU
 * baseline.  Same arithmetic as orc_matmul_q_i8 (integer sums are
 * order-independent), organised the way the reference documents its CPU kernel:
 * decode a block of packed weight rows to a scratch tile, then run a dense
 * kernel over it (docs/internal/21-quantized-weights.md:794-798, row block 64).
 *   q   (T, K) int8 token-major, s (T), packed (OUT, ceil(K/16)), tau (OUT), bias (OUT) or NULL
 *   y   (T, OUT) f32 = (tau*s)*float(acc) [+ bias], acc_out (T, OUT) optional. */
ORC_API void orc_bitlinear_i8_tm(const uint32_t* packed, const float* tau, const float* bias,
                                 const int8_t* q, const float* s, size_t t, size_t k, size_t out,
                                 float* y, int32_t* acc_out)
{
    const size_t wpr = orc_trit_words_per_row(k);
    enum { RB = 64 };
#pragma omp parallel
    {
        int8_t* tile = (int8_t*)__builtin_malloc((size_t)RB * k);
#pragma omp for schedule(dynamic, 1)
        for (size_t r0 = 0; r0 < out; r0 += RB) {
            const size_t rb = (out - r0 < RB) ? (out - r0) : RB;
            for (size_t r = 0; r < rb; ++r) {
                const uint32_t* row = packed + (r0 + r) * wpr;
                for (size_t kk = 0; kk < k; ++kk)
                    tile[r * k + kk] = (int8_t)((int)((row[kk / 16] >> (2 * (kk % 16))) & 3u) - 2);
            }
            for (size_t ti = 0; ti < t; ++ti) {
                const int8_t* qr = q + ti * k;
                for (size_t r = 0; r < rb; ++r) {
                    const int8_t* wr = tile + r * k;
                    int32_t acc = 0;
                    for (size_t kk = 0; kk < k; ++kk) acc += (int32_t)wr[kk] * (int32_t)qr[kk];
                    const size_t o = r0 + r;
                    if (acc_out) acc_out[ti * out + o] = acc;
                    if (y) {
                        float v = tau[o] * s[ti] * (float)acc;
                        if (bias) v += bias[o];
                        y[ti * out + o] = v;
                    }
                }
            }
        }
        __builtin_free(tile);
    }
}

/* Token-major activation quantisation: s_t = max_k |x[t,k]| * (1/127), q per orc_i8_quantize. */
ORC_API void orc_act_quant_tm(const float* x, size_t t, size_t k, int8_t* q, float* s)
{
    const float inv = 1.0f / 127.0f;
#pragma omp parallel for schedule(static)
    for (size_t ti = 0; ti < t; ++ti) {
        float mx = 0.0f;
        for (size_t kk = 0; kk < k; ++kk) {
            const float a = fabsf(x[ti * k + kk]);
            if (a > mx) mx = a;
        }
        const float sc = mx * inv;
        s[ti] = sc;
        for (size_t kk = 0; kk < k; ++kk) q[ti * k + kk] = orc_i8_quantize(x[ti * k + kk], sc);
    }
}
