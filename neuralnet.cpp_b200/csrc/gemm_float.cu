// gemm_float.cu — the two float GEMMs of BitLinear::backward
// (include/neuralnet.cpp/compute_layer_bitlinear.hpp:475-544), token-major:
//
//   dX  (matmul_q_t, :494):       dX[t,k]  (+)= sum_o (dY[t,o] * tau_o) * trit[o,k]
//   dW  (STE, int8 path :514-534): dW[o,k] += tau_o * sum_t (dY[t,o] * s_t) * q[t,k]
//
// trit is decoded on the fly from the 2-bit container (out, K/16); q is the engine's permuted
// int8 activation cache written by the forward pass.  This file holds the f32 CUDA-core
// versions (the "exact" numeric mode: f32 operands, f32 accumulation).
#include "common.cuh"
#include "device_math.cuh"

namespace nnb {

// actual feature index of byte position c inside a permuted 64-byte block (inverse of qperm_pos)
__host__ __device__ __forceinline__ int qperm_src(int c)
{
    return 16 * ((c & 15) >> 2) + 4 * (c & 3) + (c >> 4);
}

constexpr int BM = 128, BN = 128, BK = 16, THREADS = 256;

// C[M,N] (+)= A[M,Kc] * B[Kc,N] with tile loaders specialised per mode; 8x8 outputs per thread.
// MODE 0 (dX): M = tokens, N = in features, Kc = out features.
// MODE 1 (dW): M = out features, N = in features, Kc = tokens.
template <int MODE>
__global__ void __launch_bounds__(THREADS)
gemm_f32_kernel(const float* __restrict__ dy, const float* __restrict__ tau, const float* __restrict__ s,
                const uint32_t* __restrict__ wq, const int8_t* __restrict__ q, int T, int O, int K,
                float* c, int accumulate)
{
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int M = MODE == 0 ? T : O;
    const int N = K;
    const int KC = MODE == 0 ? O : T;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;  // 16 x 16 threads, each 8 x 8 outputs (strided by 16)

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < KC; k0 += BK) {
        // ---- A tile -> As[kk][m]
        if (MODE == 0) {
            // dy (T, O): rows m = tokens, contraction along o (contiguous)
            for (int i = tid; i < BM * BK; i += THREADS) {
                const int m = i / BK, kk = i % BK;
                const int gm = m0 + m, go = k0 + kk;
                float v = 0.0f;
                if (gm < M && go < KC) v = __fmul_rn(dy[(size_t)gm * O + go], tau[go]);
                As[kk][m] = v;
            }
        } else {
            // dy (T, O): rows m = out features (contiguous), contraction along tokens
            for (int i = tid; i < BM * BK; i += THREADS) {
                const int kk = i / BM, m = i % BM;
                const int gt = k0 + kk, gm = m0 + m;
                float v = 0.0f;
                if (gm < M && gt < KC) v = __fmul_rn(dy[(size_t)gt * O + gm], s[gt]);
                As[kk][m] = v;
            }
        }
        // ---- B tile -> Bs[kk][n]
        if (MODE == 0) {
            // decoded weights: row o = k0+kk, columns n0..n0+BN of the container
            for (int i = tid; i < BK * (BN / 16); i += THREADS) {
                const int kk = i / (BN / 16), w = i % (BN / 16);
                const int go = k0 + kk, gk = n0 + w * 16;
                uint32_t word = 0xAAAAAAAAu;  // sixteen codes 2 = trit 0
                if (go < KC && gk < N) word = wq[(size_t)go * (K / 16) + gk / 16];
#pragma unroll
                for (int j = 0; j < 16; ++j) Bs[kk][w * 16 + j] = (float)((int)((word >> (2 * j)) & 3u) - 2);
            }
        } else {
            // q (T, K) permuted int8: row t = k0+kk; column c of the tile is permuted position n0+c
            for (int i = tid; i < BK * (BN / 4); i += THREADS) {
                const int kk = i / (BN / 4), w = i % (BN / 4);
                const int gt = k0 + kk, gc = n0 + w * 4;
                uint32_t word = 0;
                if (gt < KC && gc < N) word = *reinterpret_cast<const uint32_t*>(q + (size_t)gt * K + gc);
#pragma unroll
                for (int j = 0; j < 4; ++j) Bs[kk][w * 4 + j] = (float)(int8_t)((word >> (8 * j)) & 0xFFu);
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[8], b[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = As[kk][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < 8; ++j) b[j] = Bs[kk][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int gm = m0 + ty + 16 * i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int gn = n0 + tx + 16 * j;
            if (gn >= N) continue;
            if (MODE == 0) {
                float* dst = c + (size_t)gm * N + gn;
                *dst = accumulate ? __fadd_rn(*dst, acc[i][j]) : acc[i][j];
            } else {
                const int col = (gn & ~63) + qperm_src(gn & 63);
                float* dst = c + (size_t)gm * N + col;
                *dst = __fadd_rn(*dst, __fmul_rn(acc[i][j], tau[gm]));
            }
        }
    }
}

nnb_status launch_bitlinear_dx(nnb_engine* e, bool exact, const float* dy, const uint32_t* wq, const float* tau,
                               size_t t, size_t k, size_t out, float* dx, bool accumulate)
{
    NNB_REQUIRE(dy && wq && tau && dx && t > 0 && out > 0, "bitlinear_dx: bad arguments");
    NNB_REQUIRE(k > 0 && k % 64 == 0, "bitlinear_dx: k=%zu must be a multiple of 64", k);
    if (!exact) return launch_bitlinear_dx_bf16(e, dy, wq, tau, t, k, out, dx, accumulate);
    dim3 grid((unsigned)ceil_div(k, BN), (unsigned)ceil_div(t, BM));
    NNB_REQUIRE(grid.y <= 65535, "bitlinear_dx: too many tokens (%zu)", t);
    gemm_f32_kernel<0><<<grid, THREADS, 0, e->stream>>>(dy, tau, nullptr, wq, nullptr, (int)t, (int)out, (int)k, dx,
                                                        accumulate ? 1 : 0);
    e->launches++;
    NNB_CHECK_LAUNCH("gemm_f32_kernel<dX>");
    return NNB_OK;
}

nnb_status launch_bitlinear_dw(nnb_engine* e, bool exact, const float* dy, const int8_t* q, const float* s,
                               const float* tau, size_t t, size_t k, size_t out, float* dw)
{
    NNB_REQUIRE(dy && q && s && tau && dw && t > 0 && out > 0, "bitlinear_dw: bad arguments");
    NNB_REQUIRE(k > 0 && k % 64 == 0, "bitlinear_dw: k=%zu must be a multiple of 64", k);
    if (!exact) return launch_bitlinear_dw_bf16(e, dy, q, s, tau, t, k, out, dw);
    dim3 grid((unsigned)ceil_div(k, BN), (unsigned)ceil_div(out, BM));
    NNB_REQUIRE(grid.y <= 65535, "bitlinear_dw: too many rows (%zu)", out);
    gemm_f32_kernel<1><<<grid, THREADS, 0, e->stream>>>(dy, tau, s, nullptr, q, (int)t, (int)out, (int)k, dw, 1);
    e->launches++;
    NNB_CHECK_LAUNCH("gemm_f32_kernel<dW>");
    return NNB_OK;
}

// db[o] += sum_t dy[t,o]: one thread column, coalesced over o, f64 accumulation split over token chunks
__global__ void colsum_kernel(const float* __restrict__ dy, int T, int O, int chunk, float* __restrict__ db)
{
    const int o = blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= O) return;
    const int t0 = blockIdx.y * chunk, t1 = min(T, t0 + chunk);
    float sacc = 0.0f;
    for (int t = t0; t < t1; ++t) sacc += dy[(size_t)t * O + o];
    atomicAdd(db + o, sacc);
}

nnb_status launch_colsum_add(nnb_engine* e, const float* dy, size_t t, size_t out, float* db)
{
    NNB_REQUIRE(dy && db && t > 0 && out > 0, "colsum: bad arguments");
    const int chunk = 256;
    dim3 grid((unsigned)ceil_div(out, 128), (unsigned)ceil_div(t, chunk));
    NNB_REQUIRE(grid.y <= 65535, "colsum: too many tokens (%zu)", t);
    colsum_kernel<<<grid, 128, 0, e->stream>>>(dy, (int)t, (int)out, chunk, db);
    e->launches++;
    NNB_CHECK_LAUNCH("colsum_kernel");
    return NNB_OK;
}

}  // namespace nnb
