// gemm_bf16.cu — tensor-core versions (bf16 operands, f32 accumulation) of the two float GEMMs of
// BitLinear::backward (include/neuralnet.cpp/compute_layer_bitlinear.hpp:475-544), used when the
// policy is not in the exact numeric mode:
//   dX[t,k] (+)= sum_o (dY[t,o]*tau_o) * trit[o,k]        trits decoded from the 2-bit container
//   dW[o,k] += tau_o * sum_t (dY[t,o]*s_t) * q[t,k]       q = permuted int8 activation cache
// Trits and int8 values are exact in bf16; only dY*tau / dY*s are rounded to bf16.
// Operand tiles are converted while they are staged into shared memory in their global
// orientation; ldmatrix(.trans) produces the mma.sync fragments.
#include "common.cuh"
#include "device_math.cuh"

namespace nnb {

__host__ __device__ __forceinline__ int qperm_src_b(int c) { return 16 * ((c & 15) >> 2) + 4 * (c & 3) + (c >> 4); }

namespace bf {
constexpr int BM = 128, BN = 128, BK = 32, THREADS = 256;
constexpr int A0_STRIDE = BK + 8;   // MODE 0: A_s[m][k]
constexpr int A1_STRIDE = BM + 8;   // MODE 1: A_s[k][m]
constexpr int B_STRIDE = BN + 8;    // B_s[k][n]
constexpr int A_ELEMS = BM * A0_STRIDE > BK * A1_STRIDE ? BM * A0_STRIDE : BK * A1_STRIDE;
constexpr int B_ELEMS = BK * B_STRIDE;
}  // namespace bf

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p)
{
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p)
{
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// 16 consecutive floats of a row starting at column c0 (zero beyond `cols`), scaled
template <bool VEC>
__device__ __forceinline__ void load16(const float* row, int c0, int cols, float (&v)[16])
{
    if (VEC && c0 + 16 <= cols) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 t = *reinterpret_cast<const float4*>(row + c0 + 4 * i);
            v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = (c0 + i < cols) ? row[c0 + i] : 0.0f;
    }
}

// MODE 0: dX.  M = T, N = K, contraction over O.   MODE 1: dW.  M = O, N = K, contraction over T.
template <int MODE, bool VEC>
__global__ void __launch_bounds__(bf::THREADS)
gemm_bf16_kernel(const float* __restrict__ dy, const float* __restrict__ tau, const float* __restrict__ s,
                 const uint32_t* __restrict__ wq, const int8_t* __restrict__ q, int T, int O, int K, float* c,
                 int accumulate)
{
    using namespace bf;
    __shared__ __align__(16) __nv_bfloat16 As[2][A_ELEMS];
    __shared__ __align__(16) __nv_bfloat16 Bs[2][B_ELEMS];
    const int M = MODE == 0 ? T : O;
    const int N = K;
    const int KC = MODE == 0 ? O : T;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 2, wn = warp & 3;  // 2 x 4 warps, warp tile 64 x 32
    const int g = lane >> 2, t4 = lane & 3;

    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0f;

    // staging registers
    uint32_t a_st[8], b_st[8];
    auto fetch = [&](int k0) {
        float v[16];
        if (MODE == 0) {
            const int m = tid >> 1, kh = (tid & 1) * 16;
            const int gm = m0 + m, go = k0 + kh;
            if (gm < M && go < KC) {
                load16<VEC>(dy + (size_t)gm * O, go, O, v);
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = (go + i < KC) ? v[i] * tau[go + i] : 0.0f;
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) a_st[i] = pack_bf16(v[2 * i], v[2 * i + 1]);
            // B: one packed word -> 16 trits
            const int kr = tid >> 3, w = tid & 7;
            const int gk = n0 + w * 16;
            uint32_t word = 0xAAAAAAAAu;
            if (k0 + kr < KC && gk < N) word = wq[(size_t)(k0 + kr) * (K / 16) + gk / 16];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t c0 = (word >> (4 * i)) & 3u, c1 = (word >> (4 * i + 2)) & 3u;
                // bf16 bits of code-2: 1 -> -1 (0xBF80), 2 -> 0, 3 -> +1 (0x3F80)
                const uint32_t lo = c0 == 3u ? 0x3F80u : (c0 == 1u ? 0xBF80u : 0u);
                const uint32_t hi = c1 == 3u ? 0x3F80u : (c1 == 1u ? 0xBF80u : 0u);
                b_st[i] = lo | (hi << 16);
            }
        } else {
            const int kr = tid >> 3, ch = (tid & 7) * 16;
            const int gt = k0 + kr, gm = m0 + ch;
            if (gt < KC && gm < M) {
                load16<VEC>(dy + (size_t)gt * O, gm, O, v);
                const float sc = s[gt];
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] *= sc;
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = 0.0f;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) a_st[i] = pack_bf16(v[2 * i], v[2 * i + 1]);
            const int gc = n0 + ch;
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (gt < KC && gc < N) raw = *reinterpret_cast<const uint4*>(q + (size_t)gt * K + gc);
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float f0 = (float)(int8_t)(words[i] & 0xFF), f1 = (float)(int8_t)((words[i] >> 8) & 0xFF);
                const float f2 = (float)(int8_t)((words[i] >> 16) & 0xFF), f3 = (float)(int8_t)((words[i] >> 24) & 0xFF);
                b_st[2 * i] = pack_bf16(f0, f1);
                b_st[2 * i + 1] = pack_bf16(f2, f3);
            }
        }
    };
    auto stage = [&](int buf) {
        uint4* pa;
        uint4* pb;
        if (MODE == 0) {
            const int m = tid >> 1, kh = (tid & 1) * 16;
            pa = reinterpret_cast<uint4*>(&As[buf][m * A0_STRIDE + kh]);
            const int kr = tid >> 3, w = tid & 7;
            pb = reinterpret_cast<uint4*>(&Bs[buf][kr * B_STRIDE + w * 16]);
        } else {
            const int kr = tid >> 3, ch = (tid & 7) * 16;
            pa = reinterpret_cast<uint4*>(&As[buf][kr * A1_STRIDE + ch]);
            pb = reinterpret_cast<uint4*>(&Bs[buf][kr * B_STRIDE + ch]);
        }
        pa[0] = make_uint4(a_st[0], a_st[1], a_st[2], a_st[3]);
        pa[1] = make_uint4(a_st[4], a_st[5], a_st[6], a_st[7]);
        pb[0] = make_uint4(b_st[0], b_st[1], b_st[2], b_st[3]);
        pb[1] = make_uint4(b_st[4], b_st[5], b_st[6], b_st[7]);
    };

    const int ktiles = (KC + BK - 1) / BK;
    fetch(0);
    stage(0);
    __syncthreads();
    for (int kt = 0; kt < ktiles; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < ktiles) fetch((kt + 1) * BK);
#pragma unroll
        for (int ks = 0; ks < BK; ks += 16) {
            uint32_t af[4][4];
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                const int mb = wm * 64 + mt * 16;
                if (MODE == 0) {
                    const int r = mb + (lane & 7) + 8 * ((lane >> 3) & 1), kc = ks + 8 * (lane >> 4);
                    ldsm_x4(af[mt], &As[buf][r * A0_STRIDE + kc]);
                } else {
                    const int kr = ks + (lane & 7) + 8 * (lane >> 4), mc = mb + 8 * ((lane >> 3) & 1);
                    ldsm_x4_t(af[mt], &As[buf][kr * A1_STRIDE + mc]);
                }
            }
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t bfr[4];
                const int kr = ks + (lane & 7) + 8 * ((lane >> 3) & 1), nc = wn * 32 + np * 16 + 8 * (lane >> 4);
                ldsm_x4_t(bfr, &Bs[buf][kr * B_STRIDE + nc]);
#pragma unroll
                for (int mt = 0; mt < 4; ++mt) {
                    mma_bf16(acc[mt][np * 2], af[mt], bfr[0], bfr[1]);
                    mma_bf16(acc[mt][np * 2 + 1], af[mt], bfr[2], bfr[3]);
                }
            }
        }
        if (kt + 1 < ktiles) {
            stage(buf ^ 1);
        }
        __syncthreads();
    }

#pragma unroll
    for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int gm = m0 + wm * 64 + mt * 16 + g + 8 * h;
            if (gm >= M) continue;
            const float tm = MODE == 1 ? tau[gm] : 1.0f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int gn = n0 + wn * 32 + nt * 8 + t4 * 2 + cc;
                    if (gn >= N) continue;
                    const float v = acc[mt][nt][h * 2 + cc];
                    if (MODE == 0) {
                        float* dst = c + (size_t)gm * N + gn;
                        *dst = accumulate ? *dst + v : v;
                    } else {
                        float* dst = c + (size_t)gm * N + (gn & ~63) + qperm_src_b(gn & 63);
                        *dst += v * tm;
                    }
                }
            }
        }
    }
}

nnb_status launch_bitlinear_dx_bf16(nnb_engine* e, const float* dy, const uint32_t* wq, const float* tau, size_t t,
                                    size_t k, size_t out, float* dx, bool accumulate)
{
    using namespace bf;
    dim3 grid((unsigned)ceil_div(k, BN), (unsigned)ceil_div(t, BM));
    NNB_REQUIRE(grid.y <= 65535, "bitlinear_dx: too many tokens (%zu)", t);
    const bool vec = (out % 4 == 0) && (((uintptr_t)dy & 15) == 0);
    if (vec)
        gemm_bf16_kernel<0, true><<<grid, THREADS, 0, e->stream>>>(dy, tau, nullptr, wq, nullptr, (int)t, (int)out, (int)k, dx, accumulate);
    else
        gemm_bf16_kernel<0, false><<<grid, THREADS, 0, e->stream>>>(dy, tau, nullptr, wq, nullptr, (int)t, (int)out, (int)k, dx, accumulate);
    e->launches++;
    NNB_CHECK_LAUNCH("gemm_bf16_kernel<dX>");
    return NNB_OK;
}

nnb_status launch_bitlinear_dw_bf16(nnb_engine* e, const float* dy, const int8_t* q, const float* s, const float* tau,
                                    size_t t, size_t k, size_t out, float* dw)
{
    using namespace bf;
    dim3 grid((unsigned)ceil_div(k, BN), (unsigned)ceil_div(out, BM));
    NNB_REQUIRE(grid.y <= 65535, "bitlinear_dw: too many rows (%zu)", out);
    const bool vec = (out % 4 == 0) && (((uintptr_t)dy & 15) == 0);
    if (vec)
        gemm_bf16_kernel<1, true><<<grid, THREADS, 0, e->stream>>>(dy, tau, s, nullptr, q, (int)t, (int)out, (int)k, dw, 1);
    else
        gemm_bf16_kernel<1, false><<<grid, THREADS, 0, e->stream>>>(dy, tau, s, nullptr, q, (int)t, (int)out, (int)k, dw, 1);
    e->launches++;
    NNB_CHECK_LAUNCH("gemm_bf16_kernel<dW>");
    return NNB_OK;
}

}  // namespace nnb
