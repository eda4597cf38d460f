// device_math.cuh — small device helpers shared by the kernels: quantisation rules, warp
// reductions, a bit-reproducible exp, and the counter-based Philox generator.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace nnb {

// Programmatic dependent launch (no-ops for a kernel launched without the attribute):
// pdl_launch lets the next kernel in the stream become resident; pdl_wait returns once every kernel this one
// depends on has completed and its writes are visible.  Nothing in global memory may be touched before it.
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

// code = trit + 2; strict compares so |w| == 0.5*tau -> 0
// (include/neuralnet.cpp/compute_layer_bitlinear.hpp:657-667)
__device__ __forceinline__ uint32_t trit_code_of(float w, float tau)
{
    const float hi = __fmul_rn(tau, 0.5f);
    const float lo = __fmul_rn(tau, -0.5f);
    return w > hi ? 3u : (w < lo ? 1u : 2u);
}

// q = round_half_away(clamp(x / s, -127, 127)), NaN -> 0, s == 0 -> 0
// (docs/internal/21-quantized-weights.md:966-982)
__device__ __forceinline__ int i8_quantize(float x, float s)
{
    if (s == 0.0f) return 0;
    float v = __fdiv_rn(x, s);
    if (v != v) return 0;
    v = fminf(fmaxf(v, -127.0f), 127.0f);
    return (int)roundf(v);
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum_d(double v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float shfl_xor_t(float v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }
__device__ __forceinline__ double shfl_xor_t(double v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }
__device__ __forceinline__ float warp_sum_t(float v) { return warp_sum(v); }
__device__ __forceinline__ double warp_sum_t(double v) { return warp_sum_d(v); }

// accumulator type of a numeric mode: f64 in the exact mode, f32 otherwise
template <bool EXACT>
struct AccT { typedef float type; };
template <>
struct AccT<true> { typedef double type; };

// exp as a fixed sequence of fmaf steps (Cephes-style range reduction, degree-5 polynomial):
// the same sequence evaluated on any IEEE machine gives the same bits.  x < -86 -> 0.
__device__ __forceinline__ float nnb_expf(float x)
{
    if (x < -86.0f) return 0.0f;
    if (x > 88.0f) x = 88.0f;
    const float t = fmaf(x, 1.44269504088896341f, 12582912.0f);
    const float n = __fsub_rn(t, 12582912.0f);
    float r = fmaf(n, -0.693359375f, x);
    r = fmaf(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    const float r2 = __fmul_rn(r, r);
    const float res = __fadd_rn(fmaf(p, r2, r), 1.0f);
    return __int_as_float(__float_as_int(res) + (((int)n) << 23));
}

// Philox4x32-10 (Salmon et al., SC'11).  One uniform in [0,1) with 24 bits from the counter
// (sequence, step, 0, 0) and the 64-bit seed as key.
__device__ __forceinline__ float philox_uniform(unsigned long long seed, unsigned sequence, unsigned step)
{
    uint32_t c0 = sequence, c1 = step, c2 = 0u, c3 = 0u;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int i = 0; i < 10; ++i) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
    return (float)(c0 >> 8) * (1.0f / 16777216.0f);
}

}  // namespace nnb
