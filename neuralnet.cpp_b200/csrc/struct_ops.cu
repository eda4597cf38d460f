// struct_ops.cu — the small operators behind the structure switches of BitNet b1.58 2B4T:
//   grouped-query attention   include/neuralnet.cpp/compute_layer_attention.hpp:444-454 (head map h / (H / Hkv); the
//                             reference expands K, V with gather_rows and folds dK, dV with scatter_add_rows)
//   tied embeddings           include/neuralnet.cpp/compute_layer_gpt.hpp:286-297,556-575 (logits = E . x, dX = E^T . g,
//                             dE += g . x^T: dense products, no quantiser)
// The dense products here run on CUDA cores: they serve the exact mode (f64 accumulation of f32 operands, the mode
// compared with the CPU restatement) and token counts below the tensor-core kernels' 64 rows.
#include "common.cuh"

namespace nnb {

// raw (T, d + 2 dkv) = [q | k | v] per token  ->  planes (3, T, d): q, K and V with every KV head repeated rep times
__global__ void __launch_bounds__(256)
gqa_expand_kernel(const float* __restrict__ raw, size_t T, int H, int Hkv, int dk, float* __restrict__ planes)
{
    const int d = H * dk, dkv = Hkv * dk, rep = H / Hkv, w = d + 2 * dkv;
    const size_t n = 3 * T * (size_t)d;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
        const int m = (int)(i / (T * (size_t)d));
        const size_t r = i % (T * (size_t)d);
        const size_t t = r / d;
        const int c = (int)(r % d);
        int src = c;
        if (m > 0) src = d + (m - 1) * dkv + (c / dk / rep) * dk + c % dk;
        planes[i] = raw[t * w + src];
    }
}

// planes (3, T, d) of gradients -> raw (T, d + 2 dkv): dq copied, the rep replicas of each KV head summed in head order
__global__ void __launch_bounds__(256)
gqa_reduce_kernel(const float* __restrict__ planes, size_t T, int H, int Hkv, int dk, float* __restrict__ raw)
{
    const int d = H * dk, dkv = Hkv * dk, rep = H / Hkv, w = d + 2 * dkv;
    const size_t n = T * (size_t)w;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
        const size_t t = i / w;
        const int c = (int)(i % w);
        float v;
        if (c < d) {
            v = planes[t * d + c];
        } else {
            const int m = (c - d) / dkv + 1, cc = (c - d) % dkv;
            const int g = cc / dk, j = cc % dk;
            const float* src = planes + (size_t)m * T * d + t * d + (size_t)g * rep * dk + j;
            v = 0.0f;
            for (int q = 0; q < rep; ++q) v = __fadd_rn(v, src[(size_t)q * dk]);
        }
        raw[i] = v;
    }
}

nnb_status launch_gqa_expand(nnb_engine* e, const float* raw, size_t T, size_t H, size_t Hkv, size_t dk, float* planes)
{
    NNB_REQUIRE(raw && planes && T > 0 && Hkv > 0 && H % Hkv == 0, "gqa_expand: bad arguments");
    const size_t n = 3 * T * H * dk;
    const unsigned grid = (unsigned)std::min<size_t>(ceil_div(n, 256), (size_t)e->sm_count * 16);
    gqa_expand_kernel<<<grid, 256, 0, e->stream>>>(raw, T, (int)H, (int)Hkv, (int)dk, planes);
    e->launches++;
    NNB_CHECK_LAUNCH("gqa_expand_kernel");
    return NNB_OK;
}

nnb_status launch_gqa_reduce(nnb_engine* e, const float* planes, size_t T, size_t H, size_t Hkv, size_t dk, float* raw)
{
    NNB_REQUIRE(raw && planes && T > 0 && Hkv > 0 && H % Hkv == 0, "gqa_reduce: bad arguments");
    const size_t n = T * (H + 2 * Hkv) * dk;
    const unsigned grid = (unsigned)std::min<size_t>(ceil_div(n, 256), (size_t)e->sm_count * 16);
    gqa_reduce_kernel<<<grid, 256, 0, e->stream>>>(planes, T, (int)H, (int)Hkv, (int)dk, raw);
    e->launches++;
    NNB_CHECK_LAUNCH("gqa_reduce_kernel");
    return NNB_OK;
}

__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* __restrict__ x, size_t n, __nv_bfloat16* __restrict__ y)
{
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) y[i] = __float2bfloat16_rn(x[i]);
}

nnb_status launch_f32_to_bf16(nnb_engine* e, const float* x, size_t n, __nv_bfloat16* y)
{
    NNB_REQUIRE(x && y && n > 0, "f32_to_bf16: bad arguments");
    const unsigned grid = (unsigned)std::min<size_t>(ceil_div(n, 256), (size_t)e->sm_count * 32);
    f32_to_bf16_kernel<<<grid, 256, 0, e->stream>>>(x, n, y);
    e->launches++;
    NNB_CHECK_LAUNCH("f32_to_bf16_kernel");
    return NNB_OK;
}

// ------------------------------------------------------------------ dense products
template <typename T>
__device__ __forceinline__ float ld_f(const T* p);
template <>
__device__ __forceinline__ float ld_f<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename ACC>
__device__ __forceinline__ ACC warp_sum_acc(ACC v)
{
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// C (T, N) = A (T, K) . B (N, K)^T.  One warp per row of B and TT rows of A at a time: the lanes split K, every element
// of B's row is used for TT tokens.  grid.x walks N in blocks of 8 rows (one per warp), grid.y walks T in blocks of TT.
constexpr int DENSE_TT = 4;
template <typename OP, typename ACC>
__global__ void __launch_bounds__(256)
dense_nt_kernel(const OP* __restrict__ A, const OP* __restrict__ B, int T, int N, int K, float* __restrict__ C)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    const int t0 = blockIdx.y * DENSE_TT;
    if (n >= N) return;
    ACC acc[DENSE_TT];
#pragma unroll
    for (int j = 0; j < DENSE_TT; ++j) acc[j] = 0;
    const OP* br = B + (size_t)n * K;
    for (int i = lane; i < K; i += 32) {
        const ACC b = (ACC)ld_f<OP>(br + i);
#pragma unroll
        for (int j = 0; j < DENSE_TT; ++j)
            if (t0 + j < T) acc[j] += (ACC)ld_f<OP>(A + (size_t)(t0 + j) * K + i) * b;
    }
#pragma unroll
    for (int j = 0; j < DENSE_TT; ++j) {
        const ACC s = warp_sum_acc<ACC>(acc[j]);
        if (lane == 0 && t0 + j < T) C[(size_t)(t0 + j) * N + n] = (float)s;
    }
}

// C (T, K) = G (T, N) . B (N, K): one thread per output, N walked in order
template <typename ACC>
__global__ void __launch_bounds__(256)
dense_nn_kernel(const float* __restrict__ G, const float* __restrict__ B, int T, int N, int K, float* __restrict__ C)
{
    const int i = blockIdx.y * 256 + threadIdx.x, t = blockIdx.x;
    if (i >= K) return;
    ACC acc = 0;
    const float* g = G + (size_t)t * N;
    for (int n = 0; n < N; ++n) acc += (ACC)g[n] * (ACC)B[(size_t)n * K + i];
    C[(size_t)t * K + i] = (float)acc;
}

// D (N, K) += G (T, N)^T . X (T, K): one thread per output, T walked in order
template <typename ACC>
__global__ void __launch_bounds__(256)
dense_tn_acc_kernel(const float* __restrict__ G, const float* __restrict__ X, int T, int N, int K, float* __restrict__ D)
{
    const int i = blockIdx.y * 256 + threadIdx.x, n = blockIdx.x;
    if (i >= K) return;
    ACC acc = 0;
    for (int t = 0; t < T; ++t) acc += (ACC)G[(size_t)t * N + n] * (ACC)X[(size_t)t * K + i];
    D[(size_t)n * K + i] = __fadd_rn(D[(size_t)n * K + i], (float)acc);
}

static nnb_status dense_shape_ok(size_t T, size_t N, size_t K)
{
    NNB_REQUIRE(T > 0 && N > 0 && K > 0 && T <= 0x7fffffff && N <= 0x7fffffff && K <= 0x7fffffff, "dense product: bad shape");
    NNB_REQUIRE(ceil_div(T, DENSE_TT) <= 65535 && ceil_div(K, 256) <= 65535, "dense product: %zu x %zu x %zu exceeds the grid", T, N, K);
    return NNB_OK;
}

nnb_status launch_dense_nt(nnb_engine* e, bool exact, const float* A, const float* B, size_t T, size_t N, size_t K, float* C)
{
    NNB_TRY(dense_shape_ok(T, N, K));
    const dim3 grid((unsigned)ceil_div(N, 8), (unsigned)ceil_div(T, DENSE_TT));
    if (exact) dense_nt_kernel<float, double><<<grid, 256, 0, e->stream>>>(A, B, (int)T, (int)N, (int)K, C);
    else dense_nt_kernel<float, float><<<grid, 256, 0, e->stream>>>(A, B, (int)T, (int)N, (int)K, C);
    e->launches++;
    NNB_CHECK_LAUNCH("dense_nt_kernel");
    return NNB_OK;
}

nnb_status launch_dense_nt_bf16(nnb_engine* e, const __nv_bfloat16* A, const __nv_bfloat16* B, size_t T, size_t N, size_t K, float* C)
{
    NNB_TRY(dense_shape_ok(T, N, K));
    const dim3 grid((unsigned)ceil_div(N, 8), (unsigned)ceil_div(T, DENSE_TT));
    dense_nt_kernel<__nv_bfloat16, float><<<grid, 256, 0, e->stream>>>(A, B, (int)T, (int)N, (int)K, C);
    e->launches++;
    NNB_CHECK_LAUNCH("dense_nt_kernel");
    return NNB_OK;
}

nnb_status launch_dense_nn(nnb_engine* e, bool exact, const float* G, const float* B, size_t T, size_t N, size_t K, float* C)
{
    NNB_TRY(dense_shape_ok(T, N, K));
    const dim3 grid((unsigned)T, (unsigned)ceil_div(K, 256));
    if (exact) dense_nn_kernel<double><<<grid, 256, 0, e->stream>>>(G, B, (int)T, (int)N, (int)K, C);
    else dense_nn_kernel<float><<<grid, 256, 0, e->stream>>>(G, B, (int)T, (int)N, (int)K, C);
    e->launches++;
    NNB_CHECK_LAUNCH("dense_nn_kernel");
    return NNB_OK;
}

nnb_status launch_dense_tn_acc(nnb_engine* e, bool exact, const float* G, const float* X, size_t T, size_t N, size_t K, float* D)
{
    NNB_TRY(dense_shape_ok(T, N, K));
    const dim3 grid((unsigned)N, (unsigned)ceil_div(K, 256));
    if (exact) dense_tn_acc_kernel<double><<<grid, 256, 0, e->stream>>>(G, X, (int)T, (int)N, (int)K, D);
    else dense_tn_acc_kernel<float><<<grid, 256, 0, e->stream>>>(G, X, (int)T, (int)N, (int)K, D);
    e->launches++;
    NNB_CHECK_LAUNCH("dense_tn_acc_kernel");
    return NNB_OK;
}

}  // namespace nnb
