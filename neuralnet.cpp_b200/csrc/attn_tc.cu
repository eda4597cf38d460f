// attn_tc.cu — causal self-attention of the teacher-forced pass on tensor cores (bf16 operands, f32
// accumulation, online softmax), used when the policy is not in the exact numeric mode.
//   forward   O = softmax(Qs K^T) V, Qs = q * 1/sqrt(dk)          compute_layer_attention.hpp:698-828
//   backward  P = exp(S - lse); dV = P^T dO; dS = P o (dO V^T - D); dQ = scale * dS K; dK = dS^T Qs
//             (the reference recomputes W from Q, K and forms R = rowsum(W o P), X = W o (P - R)) :830-988
// (paths under include/neuralnet.cpp/ of the reference).  q, k, v, dO are f32 token-major (n*S, H*dk)
// and are converted to bf16 while they are staged into shared memory.  Head dims 64 and 128.
#include "common.cuh"
#include "device_math.cuh"

namespace nnb {
namespace att {

__device__ __forceinline__ void ldsm(uint32_t (&r)[4], const void* p)
{
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_t(uint32_t (&r)[4], const void* p)
{
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi)
{
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// stage `rows` rows x DK features of a (n*S, d) f32 matrix into bf16 shared memory (row stride LD),
// rows beyond S are zero; optional scale
template <int DK, int LD, int THREADS>
__device__ __forceinline__ void stage_tile(const float* __restrict__ src, size_t base_row, int row0, int S, int d,
                                           int col0, float scale, __nv_bfloat16* dst)
{
    constexpr int CH = DK / 4;  // float4 chunks per row
    for (int i = threadIdx.x; i < 64 * CH; i += THREADS) {
        const int r = i / CH, c = (i % CH) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < S) v = *reinterpret_cast<const float4*>(src + (base_row + row0 + r) * d + col0 + c);
        uint2 o;
        o.x = pack2(v.x * scale, v.y * scale);
        o.y = pack2(v.z * scale, v.w * scale);
        *reinterpret_cast<uint2*>(dst + r * LD + c) = o;
    }
}

// ------------------------------------------------------------------ forward
// grid (n*H, ceil(S/64)), 128 threads: warp w owns query rows 16w..16w+15 of the tile
template <int DK>
__global__ void __launch_bounds__(128)
attn_fwd_tc_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int S, int H,
                   float scale, float* __restrict__ out, float* __restrict__ lse)
{
    constexpr int LD = DK + 8;
    extern __shared__ __align__(16) unsigned char smraw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);
    __nv_bfloat16* Ks = Qs + 64 * LD;
    __nv_bfloat16* Vs = Ks + 64 * LD;
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int d = H * DK;
    const int q0 = blockIdx.y * 64;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const size_t base = (size_t)b * S;
    const int col0 = h * DK;

    stage_tile<DK, LD, 128>(q, base, q0, S, d, col0, scale, Qs);
    __syncthreads();
    uint32_t qf[DK / 16][4];
#pragma unroll
    for (int ks = 0; ks < DK / 16; ++ks) {
        const int r = warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = ks * 16 + 8 * (lane >> 4);
        ldsm(qf[ks], Qs + r * LD + c);
    }
    float o[DK / 8][4];
#pragma unroll
    for (int i = 0; i < DK / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
    const int last_key_tile = min(q0 + 63, S - 1) / 64;
    for (int jt = 0; jt <= last_key_tile; ++jt) {
        const int j0 = jt * 64;
        __syncthreads();
        stage_tile<DK, LD, 128>(k, base, j0, S, d, col0, 1.0f, Ks);
        stage_tile<DK, LD, 128>(v, base, j0, S, d, col0, 1.0f, Vs);
        __syncthreads();
        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t bfr[4];
                const int kr = np * 16 + (lane & 7) + 8 * (lane >> 4), c = ks * 16 + 8 * ((lane >> 3) & 1);
                ldsm(bfr, Ks + kr * LD + c);
                mma16816(s[np * 2], qf[ks], bfr[0], bfr[1]);
                mma16816(s[np * 2 + 1], qf[ks], bfr[2], bfr[3]);
            }
        }
        // causal mask + online softmax (rows g and g+8 of the warp's 16)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = j0 + nt * 8 + 2 * t4 + (c & 1);
                const int row = (c < 2) ? row_a : row_b;
                if (key > row || key >= S) s[nt][c] = -INFINITY;
                mx[c >> 1] = fmaxf(mx[c >> 1], s[nt][c]);
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        }
        float corr[2], mnew[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mnew[r] = fmaxf(m[r], mx[r]);
            corr[r] = (mnew[r] == -INFINITY) ? 1.0f : __expf(m[r] - mnew[r]);
            m[r] = mnew[r];
            l[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < DK / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float mr = mnew[c >> 1];
                const float p = (mr == -INFINITY) ? 0.0f : __expf(s[nt][c] - mr);
                s[nt][c] = p;
                l[c >> 1] += p;
            }
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t pa[4];
            pa[0] = pack2(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack2(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < DK / 16; ++np) {
                uint32_t bfr[4];
                const int kr = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = np * 16 + 8 * (lane >> 4);
                ldsm_t(bfr, Vs + kr * LD + c);
                mma16816(o[np * 2], pa, bfr[0], bfr[1]);
                mma16816(o[np * 2 + 1], pa, bfr[2], bfr[3]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    const float inv_a = 1.0f / l[0], inv_b = 1.0f / l[1];
#pragma unroll
    for (int i = 0; i < DK / 8; ++i) {
        const int c = col0 + i * 8 + 2 * t4;
        if (row_a < S) *reinterpret_cast<float2*>(out + (base + row_a) * d + c) = make_float2(o[i][0] * inv_a, o[i][1] * inv_a);
        if (row_b < S) *reinterpret_cast<float2*>(out + (base + row_b) * d + c) = make_float2(o[i][2] * inv_b, o[i][3] * inv_b);
    }
    if (t4 == 0) {
        if (row_a < S) lse[((size_t)b * H + h) * S + row_a] = m[0] + logf(l[0]);
        if (row_b < S) lse[((size_t)b * H + h) * S + row_b] = m[1] + logf(l[1]);
    }
}

// ------------------------------------------------------------------ backward
// grid (n*H, ceil(S/64)) over key tiles, 256 threads: warp (wr, wc), wr = warp & 3 row group of 16,
// wc = warp >> 2 column half.  dQ is accumulated with atomics (zero it before the launch).
template <int DK>
__global__ void __launch_bounds__(256)
attn_bwd_tc_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                   const float* __restrict__ dout, const float* __restrict__ lse, const float* __restrict__ delta, int S,
                   int H, float scale, float* __restrict__ dq, float* __restrict__ dk, float* __restrict__ dv)
{
    constexpr int LD = DK + 8, LP = 64 + 8, HALF = DK / 2;
    extern __shared__ __align__(16) unsigned char smraw[];
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smraw);
    __nv_bfloat16* Vs = Ks + 64 * LD;
    __nv_bfloat16* Qs = Vs + 64 * LD;
    __nv_bfloat16* Gs = Qs + 64 * LD;   // dO
    __nv_bfloat16* Ps = Gs + 64 * LD;   // [q][key]
    __nv_bfloat16* Ds = Ps + 64 * LP;   // dS [q][key]
    float* Ls = reinterpret_cast<float*>(Ds + 64 * LP);
    float* Dl = Ls + 64;
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int d = H * DK;
    const int k0 = blockIdx.y * 64;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int wr = warp & 3, wc = warp >> 2;
    const size_t base = (size_t)b * S;
    const int col0 = h * DK;

    stage_tile<DK, LD, 256>(k, base, k0, S, d, col0, 1.0f, Ks);
    stage_tile<DK, LD, 256>(v, base, k0, S, d, col0, 1.0f, Vs);
    float adk[HALF / 8][4], adv[HALF / 8][4];
#pragma unroll
    for (int i = 0; i < HALF / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) adk[i][j] = adv[i][j] = 0.0f;

    for (int i0 = k0; i0 < S; i0 += 64) {
        __syncthreads();
        stage_tile<DK, LD, 256>(q, base, i0, S, d, col0, scale, Qs);
        stage_tile<DK, LD, 256>(dout, base, i0, S, d, col0, 1.0f, Gs);
        if (threadIdx.x < 64) {
            const int qi = i0 + threadIdx.x;
            Ls[threadIdx.x] = qi < S ? lse[((size_t)b * H + h) * S + qi] : 0.0f;
            Dl[threadIdx.x] = qi < S ? delta[((size_t)b * H + h) * S + qi] : 0.0f;
        }
        __syncthreads();
        // ---- phase A: S = Qs K^T and dP = dO V^T for q rows 16wr.., keys 32wc..32wc+31
        float s[4][4], dp[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = dp[i][j] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
            uint32_t aq[4], ag[4];
            const int r = wr * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = ks * 16 + 8 * (lane >> 4);
            ldsm(aq, Qs + r * LD + c);
            ldsm(ag, Gs + r * LD + c);
#pragma unroll
            for (int np = 0; np < 2; ++np) {
                uint32_t bk[4], bv[4];
                const int kr = wc * 32 + np * 16 + (lane & 7) + 8 * (lane >> 4), cc = ks * 16 + 8 * ((lane >> 3) & 1);
                ldsm(bk, Ks + kr * LD + cc);
                ldsm(bv, Vs + kr * LD + cc);
                mma16816(s[np * 2], aq, bk[0], bk[1]);
                mma16816(s[np * 2 + 1], aq, bk[2], bk[3]);
                mma16816(dp[np * 2], ag, bv[0], bv[1]);
                mma16816(dp[np * 2 + 1], ag, bv[2], bv[3]);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int rl = wr * 16 + g + 8 * hh;       // row inside the q tile
                const int row = i0 + rl;
                const float lr = Ls[rl], dr = Dl[rl];
                float pv[2], dsv[2];
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int key = k0 + wc * 32 + nt * 8 + 2 * t4 + c;
                    const bool ok = key <= row && row < S && key < S;
                    const float p = ok ? __expf(s[nt][hh * 2 + c] - lr) : 0.0f;
                    pv[c] = p;
                    dsv[c] = p * (dp[nt][hh * 2 + c] - dr);
                }
                const int cidx = wc * 32 + nt * 8 + 2 * t4;
                *reinterpret_cast<uint32_t*>(Ps + rl * LP + cidx) = pack2(pv[0], pv[1]);
                *reinterpret_cast<uint32_t*>(Ds + rl * LP + cidx) = pack2(dsv[0], dsv[1]);
            }
        }
        __syncthreads();
        // ---- phase B: dV[key][d] += P^T dO, dK[key][d] += dS^T Qs; key rows 16wr.., features HALF*wc..
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {  // contraction over the 64 queries of the tile
            uint32_t ap[4], ad[4];
            const int qr = ks * 16 + (lane & 7) + 8 * (lane >> 4), kc = wr * 16 + 8 * ((lane >> 3) & 1);
            ldsm_t(ap, Ps + qr * LP + kc);
            ldsm_t(ad, Ds + qr * LP + kc);
#pragma unroll
            for (int np = 0; np < HALF / 16; ++np) {
                uint32_t bg[4], bq[4];
                const int rr = ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), cc = wc * HALF + np * 16 + 8 * (lane >> 4);
                ldsm_t(bg, Gs + rr * LD + cc);
                ldsm_t(bq, Qs + rr * LD + cc);
                mma16816(adv[np * 2], ap, bg[0], bg[1]);
                mma16816(adv[np * 2 + 1], ap, bg[2], bg[3]);
                mma16816(adk[np * 2], ad, bq[0], bq[1]);
                mma16816(adk[np * 2 + 1], ad, bq[2], bq[3]);
            }
        }
        // ---- phase C: dQ[q][d] += scale * dS K; q rows 16wr.., features HALF*wc..
        float aq2[HALF / 8][4];
#pragma unroll
        for (int i = 0; i < HALF / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) aq2[i][j] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {  // contraction over the 64 keys
            uint32_t ads[4];
            const int r = wr * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = ks * 16 + 8 * (lane >> 4);
            ldsm(ads, Ds + r * LP + c);
#pragma unroll
            for (int np = 0; np < HALF / 16; ++np) {
                uint32_t bk[4];
                const int rr = ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), cc = wc * HALF + np * 16 + 8 * (lane >> 4);
                ldsm_t(bk, Ks + rr * LD + cc);
                mma16816(aq2[np * 2], ads, bk[0], bk[1]);
                mma16816(aq2[np * 2 + 1], ads, bk[2], bk[3]);
            }
        }
#pragma unroll
        for (int i = 0; i < HALF / 8; ++i) {
            const int c = col0 + wc * HALF + i * 8 + 2 * t4;
            const int ra = i0 + wr * 16 + g, rb = ra + 8;
            if (ra < S) {
                atomicAdd(dq + (base + ra) * d + c, aq2[i][0] * scale);
                atomicAdd(dq + (base + ra) * d + c + 1, aq2[i][1] * scale);
            }
            if (rb < S) {
                atomicAdd(dq + (base + rb) * d + c, aq2[i][2] * scale);
                atomicAdd(dq + (base + rb) * d + c + 1, aq2[i][3] * scale);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < HALF / 8; ++i) {
        const int c = col0 + wc * HALF + i * 8 + 2 * t4;
        const int ra = k0 + wr * 16 + g, rb = ra + 8;
        if (ra < S) {
            *reinterpret_cast<float2*>(dk + (base + ra) * d + c) = make_float2(adk[i][0], adk[i][1]);
            *reinterpret_cast<float2*>(dv + (base + ra) * d + c) = make_float2(adv[i][0], adv[i][1]);
        }
        if (rb < S) {
            *reinterpret_cast<float2*>(dk + (base + rb) * d + c) = make_float2(adk[i][2], adk[i][3]);
            *reinterpret_cast<float2*>(dv + (base + rb) * d + c) = make_float2(adv[i][2], adv[i][3]);
        }
    }
}

}  // namespace att

bool attn_tc_supported(size_t dk, size_t d) { return (dk == 64 || dk == 128) && d % 4 == 0; }

nnb_status launch_attn_fwd_tc(nnb_engine* e, const float* q, const float* k, const float* v, size_t n_seq, size_t S,
                              size_t H, size_t dk, float* out, float* lse)
{
    using namespace att;
    const float scale = 1.0f / sqrtf((float)dk);
    dim3 grid((unsigned)(n_seq * H), (unsigned)ceil_div(S, 64));
    const size_t smem = 3 * 64 * (dk + 8) * 2;
    if (dk == 128) {
        static bool cfg = false;
        if (!cfg) {
            NNB_CUDA(cudaFuncSetAttribute(attn_fwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            cfg = true;
        }
        attn_fwd_tc_kernel<128><<<grid, 128, smem, e->stream>>>(q, k, v, (int)S, (int)H, scale, out, lse);
    } else {
        attn_fwd_tc_kernel<64><<<grid, 128, smem, e->stream>>>(q, k, v, (int)S, (int)H, scale, out, lse);
    }
    e->launches++;
    NNB_CHECK_LAUNCH("attn_fwd_tc_kernel");
    return NNB_OK;
}

nnb_status launch_attn_bwd_tc(nnb_engine* e, const float* q, const float* k, const float* v, const float* dout,
                              const float* lse, const float* delta, size_t n_seq, size_t S, size_t H, size_t dk,
                              float* dq, float* dkk, float* dvv)
{
    using namespace att;
    const float scale = 1.0f / sqrtf((float)dk);
    dim3 grid((unsigned)(n_seq * H), (unsigned)ceil_div(S, 64));
    const size_t smem = 4 * 64 * (dk + 8) * 2 + 2 * 64 * 72 * 2 + 128 * 4;
    NNB_CUDA(cudaMemsetAsync(dq, 0, n_seq * S * H * dk * sizeof(float), e->stream));
    if (dk == 128) {
        static bool cfg = false;
        if (!cfg) {
            NNB_CUDA(cudaFuncSetAttribute(attn_bwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            cfg = true;
        }
        attn_bwd_tc_kernel<128><<<grid, 256, smem, e->stream>>>(q, k, v, dout, lse, delta, (int)S, (int)H, scale, dq, dkk, dvv);
    } else {
        static bool cfg = false;
        if (!cfg) {
            NNB_CUDA(cudaFuncSetAttribute(attn_bwd_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            cfg = true;
        }
        attn_bwd_tc_kernel<64><<<grid, 256, smem, e->stream>>>(q, k, v, dout, lse, delta, (int)S, (int)H, scale, dq, dkk, dvv);
    }
    e->launches++;
    NNB_CHECK_LAUNCH("attn_bwd_tc_kernel");
    return NNB_OK;
}

}  // namespace nnb
