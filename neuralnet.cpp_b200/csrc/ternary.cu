// ternary.cu — ternary (BitNet b1.58) linear: codecs, activation quantisation and the
// int8 x 2-bit GEMM with int32 accumulation.
//
// Arithmetic contract (reference: include/neuralnet.cpp/compute_layer_bitlinear.hpp:443-455,
// 637-667; src/int8_act_test.cpp:210-236; src/ternary_gemm_test.cpp:69-99):
//   code = trit + 2 in {1,2,3}, weight j of a row at bits (word >> 2j) & 3, tail = code 2
//   q = round_half_away(clamp(x / s, -127, 127)), NaN -> 0, s == 0 -> 0
//   acc = sum_k trit * q in int32;  y = (tau * s) * float(acc) [+ bias], no FMA contraction
//
// Fast path layouts (token-major):
//   weights  : the reference container itself, (out, K/16) words
//   q        : (T, K) int8 where every 64-byte block along K is permuted so that a
//              2-bit weight word needs only shift+mask to become tensor-core operands:
//              dest[16*(j%4) + 4*(j/16) + (j/4)%4] = src[j], j in 0..63
//   qsum     : (T) int32 row sums of q.  The kernel multiplies unsigned codes (0..3)
//              with q on the tensor cores (u8 x s8) and subtracts 2*qsum afterwards:
//              sum (code-2)*q = sum code*q - 2*sum q, exact in int32.
#include "common.cuh"
#include "device_math.cuh"

namespace nnb {

// position of source byte j (0..63) inside a permuted 64-byte block
__host__ __device__ __forceinline__ int qperm_pos(int j)
{
    return 16 * (j & 3) + 4 * (j >> 4) + ((j >> 2) & 3);
}

// ------------------------------------------------- reference-layout kernels
// tau_r = sum_k |W[r,k]| * (1/K): one warp per row.  Terms are f32 products; they are summed
// in double and rounded once so the value does not depend on the reduction order.
__global__ void absmean_tau_kernel(const float* __restrict__ latent, size_t rows, size_t k,
                                   float* __restrict__ tau)
{
    const size_t row = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const float inv = 1.0f / (float)k;
    const float* p = latent + row * k;
    double s = 0.0;
    for (size_t c = lane; c < k; c += 32) s += (double)__fmul_rn(fabsf(p[c]), inv);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) tau[row] = (float)s;
}

// one thread per packed word
__global__ void trit_pack_kernel(const float* __restrict__ latent, const float* __restrict__ tau,
                                 size_t rows, size_t k, uint32_t* __restrict__ packed)
{
    const size_t wpr = (k + 15) / 16;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * wpr) return;
    const size_t r = idx / wpr, wi = idx % wpr;
    const float t = tau[r];
    const float* p = latent + r * k + wi * 16;
    const size_t left = k - wi * 16;
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const uint32_t code = ((size_t)j < left) ? trit_code_of(p[j], t) : 2u;
        word |= code << (2 * j);
    }
    packed[idx] = word;
}

// s_n = max_k |x[k,n]| * (1/127); x is (k, n): one thread per column, coalesced over n
__global__ void col_absmax_scale_kernel(const float* __restrict__ x, size_t k, size_t n,
                                        float* __restrict__ s)
{
    const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n) return;
    float mx = 0.0f;
    for (size_t r = 0; r < k; ++r) {
        const float a = fabsf(x[r * n + c]);
        if (a > mx) mx = a;
    }
    s[c] = __fmul_rn(mx, 1.0f / 127.0f);
}

__global__ void quantize_i8_kernel(const float* __restrict__ x, size_t m, size_t n,
                                   const float* __restrict__ scale, int col_scale,
                                   uint32_t* __restrict__ out)
{
    const size_t wpr = (n + 3) / 4;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= m * wpr) return;
    const size_t r = idx / wpr, wi = idx % wpr;
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const size_t c = wi * 4 + b;
        if (c < n) {
            const float sc = col_scale ? scale[c] : scale[r];
            word |= (uint32_t)(uint8_t)(int8_t)i8_quantize(x[r * n + c], sc) << (8 * b);
        }
    }
    out[idx] = word;
}

__global__ void unpack_i8_kernel(const uint32_t* __restrict__ packed, size_t m, size_t n,
                                 float* __restrict__ out)
{
    const size_t wpr = (n + 3) / 4;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= m * n) return;
    const size_t r = idx / n, c = idx % n;
    out[idx] = (float)(int8_t)((packed[r * wpr + c / 4] >> (8 * (c % 4))) & 0xFFu);
}

// Any-shape matmul_q_i8 on the reference containers: one thread per output, k ascending.
__global__ void matmul_q_i8_ref_kernel(const uint32_t* __restrict__ wq,
                                       const float* __restrict__ tau,
                                       const uint32_t* __restrict__ xq, const float* __restrict__ s,
                                       size_t rows, size_t k, size_t n, float* __restrict__ y,
                                       int32_t* __restrict__ acc_out)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * n) return;
    const size_t m = idx / n, j = idx % n;
    const size_t wpr_w = (k + 15) / 16, wpr_q = (n + 3) / 4;
    int acc = 0;
    for (size_t kk = 0; kk < k; ++kk) {
        const int trit = (int)((wq[m * wpr_w + kk / 16] >> (2 * (kk % 16))) & 3u) - 2;
        const int q = (int)(int8_t)((xq[kk * wpr_q + j / 4] >> (8 * (j % 4))) & 0xFFu);
        acc += trit * q;
    }
    if (y) y[idx] = __fmul_rn(__fmul_rn(tau[m], s[j]), (float)acc);
    if (acc_out) acc_out[idx] = acc;
}

// Any-shape matmul_q: C[m,n] = sum_k (tau_m * trit) * X[k,n], f32 accumulate, k ascending.
__global__ void matmul_q_ref_kernel(const uint32_t* __restrict__ wq, const float* __restrict__ tau,
                                    const float* __restrict__ x, size_t rows, size_t k, size_t n,
                                    float* __restrict__ c)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * n) return;
    const size_t m = idx / n, j = idx % n;
    const size_t wpr = (k + 15) / 16;
    const float t = tau[m];
    float acc = 0.0f;
    for (size_t kk = 0; kk < k; ++kk) {
        const float trit = (float)((int)((wq[m * wpr + kk / 16] >> (2 * (kk % 16))) & 3u) - 2);
        acc = fmaf(__fmul_rn(t, trit), x[kk * n + j], acc);
    }
    c[idx] = acc;
}

// Any-shape matmul_q_t: C[m,n] = sum_k (tau_k * trit[k,m]) * B[k,n]
__global__ void matmul_q_t_ref_kernel(const uint32_t* __restrict__ wq,
                                      const float* __restrict__ tau, const float* __restrict__ b,
                                      size_t rows, size_t mcols, size_t n, float* __restrict__ c)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= mcols * n) return;
    const size_t m = idx / n, j = idx % n;
    const size_t wpr = (mcols + 15) / 16;
    float acc = 0.0f;
    for (size_t kk = 0; kk < rows; ++kk) {
        const float trit = (float)((int)((wq[kk * wpr + m / 16] >> (2 * (m % 16))) & 3u) - 2);
        acc = fmaf(__fmul_rn(tau[kk], trit), b[kk * n + j], acc);
    }
    c[idx] = acc;
}

// ------------------------------------------------ token-major activation quant
// One CTA per token: stage the row in shared memory, block absmax, quantise, write the
// permuted int8 row and the int32 row sum.
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__global__ void __launch_bounds__(256)
act_quant_tm_kernel(const T* __restrict__ x, int k, int8_t* __restrict__ q, float* __restrict__ s,
                    int32_t* __restrict__ qsum)
{
    extern __shared__ float row[];
    __shared__ float red_f[8];
    __shared__ int red_i[8];
    const size_t tok = blockIdx.x;
    const T* xr = x + tok * (size_t)k;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float mx = 0.0f;
    for (int i = tid; i < k; i += 256) {
        const float v = to_f32<T>(xr[i]);
        row[i] = v;
        const float a = fabsf(v);
        if (a > mx) mx = a;
    }
    mx = warp_max(mx);
    if (lane == 0) red_f[warp] = mx;
    __syncthreads();
    mx = red_f[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red_f[w]);
    const float sc = __fmul_rn(mx, 1.0f / 127.0f);
    // each thread writes whole 32-bit words of the permuted row
    uint32_t* qrow = reinterpret_cast<uint32_t*>(q + tok * (size_t)k);
    int local = 0;
    for (int w = tid; w < k / 4; w += 256) {
        const int blk = w >> 4, wd = w & 15;  // word wd of 64-byte block blk
        const int i = wd >> 2, t = wd & 3;    // dest word = 4*i + t holds src 16t + 4b + i
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int qi = i8_quantize(row[blk * 64 + 16 * t + 4 * b + i], sc);
            local += qi;
            word |= (uint32_t)(uint8_t)(int8_t)qi << (8 * b);
        }
        qrow[w] = word;
    }
    local = warp_sum_i(local);
    if (lane == 0) red_i[warp] = local;
    __syncthreads();
    if (tid == 0) {
        int tot = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += red_i[w];
        qsum[tok] = tot;
        s[tok] = sc;
    }
}

__global__ void actq_to_plain_kernel(const int8_t* __restrict__ q, size_t total,
                                     int8_t* __restrict__ plain)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t blk = idx >> 6;
    const int j = (int)(idx & 63);
    plain[idx] = q[(blk << 6) + qperm_pos(j)];
}

// ------------------------------------------------------- tensor-core GEMM
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid)
{
    const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
    const int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(sa), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem)
{
    const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(sa));
}

// D += A(u8 codes, 16x32) * B(s8, 32x8)
__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename OutT>
__device__ __forceinline__ void store_out(OutT* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v)
{
    *p = __float2bfloat16_rn(v);
}

// CTA tile: BM output rows x BN tokens, BK features per pipeline stage.
// Warps: WM x WN over the tile, WK ways over the 64-feature blocks of a stage
// (WK > 1 gives a small matrix enough warps; partial sums meet in shared memory).
template <int BM, int BN, int BK, int STAGES, int WM, int WN, int WK, typename OutT>
__global__ void __launch_bounds__(WM* WN* WK * 32)
bitlinear_mma_kernel(const uint32_t* __restrict__ wq, size_t wq_stride_words,
                     const float* __restrict__ tau, const float* __restrict__ bias,
                     const float* __restrict__ residual, const int8_t* __restrict__ q, const float* __restrict__ s,
                     const int32_t* __restrict__ qsum, int T, int K, int OUT, OutT* __restrict__ y,
                     size_t y_stride_elems, int32_t* __restrict__ acc_out)
{
    constexpr int THREADS = WM * WN * WK * 32;
    constexpr int A_ROW_BYTES = BK / 4;          // 2 bits per feature
    constexpr int A_UNITS = BK / 64;             // 16-byte units per A row
    constexpr int B_UNITS = BK / 16;             // 16-byte units per B row
    constexpr int A_STAGE = BM * A_ROW_BYTES;
    constexpr int B_STAGE = BN * BK;
    constexpr int TM = BM / WM, TN = BN / WN;    // warp tile
    constexpr int MT = TM / 16, NT = TN / 8;
    constexpr int NBLK = BK / 64;
    static_assert(BK % 128 == 0, "B swizzle needs 8 units per row");
    static_assert(TM % 16 == 0 && TN % 8 == 0, "warp tile");
    static_assert(NBLK % WK == 0, "k split");

    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* As = smem;
    unsigned char* Bs = smem + STAGES * A_STAGE;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wk = warp % WK, wn = (warp / WK) % WN, wm = warp / (WK * WN);
    const int g = lane >> 2, t4 = lane & 3;
    const int row0 = blockIdx.x * BM, tok0 = blockIdx.y * BN;
    const int mat = blockIdx.z;
    wq += (size_t)mat * wq_stride_words;
    tau += (size_t)mat * OUT;
    if (bias) bias += (size_t)mat * OUT;
    y += (size_t)mat * y_stride_elems;

    const int words_per_row = K / 16;
    const int ktiles = (K + BK - 1) / BK;

    auto load_stage = [&](int slot, int kt) {
        const int k0 = kt * BK;
        unsigned char* as = As + slot * A_STAGE;
        unsigned char* bs = Bs + slot * B_STAGE;
        for (int i = tid; i < BM * A_UNITS; i += THREADS) {
            const int r = i / A_UNITS, u = i % A_UNITS;
            const int grow = row0 + r;
            const bool ok = grow < OUT && (k0 + u * 64) < K;
            const uint32_t* src =
                wq + (size_t)(ok ? grow : 0) * words_per_row + (ok ? (k0 / 16 + u * 4) : 0);
            int pu = u;
            if (A_UNITS == 4) pu = u ^ ((r >> 1) & 3);
            if (A_UNITS == 2) pu = u ^ ((r >> 2) & 1);
            cp_async16(as + r * A_ROW_BYTES + pu * 16, src, ok);
        }
        for (int i = tid; i < BN * B_UNITS; i += THREADS) {
            const int r = i / B_UNITS, u = i % B_UNITS;
            const int gt = tok0 + r;
            const bool ok = gt < T && (k0 + u * 16) < K;
            const int8_t* src = q + (size_t)(ok ? gt : 0) * K + (ok ? (k0 + u * 16) : 0);
            cp_async16(bs + r * BK + ((u ^ (r & 7)) * 16), src, ok);
        }
    };

    int acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[i][j][c] = 0;

#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (st < ktiles) load_stage(st, st);
        cp_async_commit();
    }

    for (int kt = 0; kt < ktiles; ++kt) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int nk = kt + STAGES - 1;
            if (nk < ktiles) load_stage(nk % STAGES, nk);
            cp_async_commit();
        }
        const unsigned char* as = As + (kt % STAGES) * A_STAGE;
        const unsigned char* bs = Bs + (kt % STAGES) * B_STAGE;
#pragma unroll
        for (int bi = 0; bi < NBLK / WK; ++bi) {
            const int blk = bi * WK + wk;
            uint32_t bf[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int r = wn * TN + nt * 8 + (lane & 7);
                const int u = blk * 4 + (lane >> 3);
                ldmatrix_x4(bf[nt], bs + r * BK + ((u ^ (r & 7)) * 16));
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int r_lo = wm * TM + mt * 16 + g, r_hi = r_lo + 8;
                int pu_lo = blk, pu_hi = blk;
                if (A_UNITS == 4) {
                    pu_lo = blk ^ ((r_lo >> 1) & 3);
                    pu_hi = blk ^ ((r_hi >> 1) & 3);
                }
                if (A_UNITS == 2) {
                    pu_lo = blk ^ ((r_lo >> 2) & 1);
                    pu_hi = blk ^ ((r_hi >> 2) & 1);
                }
                const uint32_t w_lo =
                    *reinterpret_cast<const uint32_t*>(as + r_lo * A_ROW_BYTES + pu_lo * 16 + t4 * 4);
                const uint32_t w_hi =
                    *reinterpret_cast<const uint32_t*>(as + r_hi * A_ROW_BYTES + pu_hi * 16 + t4 * 4);
                constexpr uint32_t MSK = 0x03030303u;
                const uint32_t a0 = w_lo & MSK, a1 = w_hi & MSK;
                const uint32_t a2 = (w_lo >> 2) & MSK, a3 = (w_hi >> 2) & MSK;
                const uint32_t c0 = (w_lo >> 4) & MSK, c1 = (w_hi >> 4) & MSK;
                const uint32_t c2 = (w_lo >> 6) & MSK, c3 = (w_hi >> 6) & MSK;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma_u8s8(acc[mt][nt], a0, a1, a2, a3, bf[nt][0], bf[nt][1]);
                    mma_u8s8(acc[mt][nt], c0, c1, c2, c3, bf[nt][2], bf[nt][3]);
                }
            }
        }
    }
    cp_async_wait<0>();

    if (WK > 1) {
        // partial sums of the k-split warps meet in shared memory (pipeline buffers are free now)
        __syncthreads();
        int* red = reinterpret_cast<int*>(smem);
        constexpr int PER_THREAD = MT * NT * 4;
        const int group = warp / WK;  // (wm, wn) pair
        if (wk > 0) {
            int* dst = red + ((size_t)(group * (WK - 1) + (wk - 1)) * 32 + lane) * PER_THREAD;
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) dst[(i * NT + j) * 4 + c] = acc[i][j][c];
        }
        __syncthreads();
        if (wk > 0) return;
#pragma unroll
        for (int o = 1; o < WK; ++o) {
            const int* src = red + ((size_t)(group * (WK - 1) + (o - 1)) * 32 + lane) * PER_THREAD;
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[i][j][c] += src[(i * NT + j) * 4 + c];
        }
    }

    // epilogue: acc - 2*qsum, scale, bias, store token-major
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
            const int tok = tok0 + wn * TN + nt * 8 + t4 * 2 + cc;
            if (tok >= T) continue;
            const int qs2 = 2 * qsum[tok];
            const float st = s[tok];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = row0 + wm * TM + mt * 16 + g + h * 8;
                    if (row >= OUT) continue;
                    const int a = acc[mt][nt][h * 2 + cc] - qs2;
                    float v = __fmul_rn(__fmul_rn(tau[row], st), (float)a);
                    if (bias) v = __fadd_rn(v, bias[row]);
                    if (residual) v = __fadd_rn(residual[(size_t)tok * OUT + row], v);
                    store_out<OutT>(y + (size_t)tok * OUT + row, v);
                    if (acc_out) acc_out[(size_t)tok * OUT + row] = a;
                }
            }
        }
    }
}

// ----------------------------------------------------------- skinny (decode) kernel
// Few tokens (<= 8*NT), many output rows: the packed weights are the only real traffic, so the
// kernel is a persistent weight streamer.  The activations of all tokens stay resident in
// shared memory for the CTA's lifetime; every group of WK warps owns MS 16-row slabs at a
// time and splits K between its warps; weights go straight from global memory to the
// tensor-core operand registers (two 32-bit loads per slab per 64 features per lane, register
// double-buffered), no shared-memory staging and no barrier inside the K loop.  An activation
// fragment read from shared memory serves all MS slabs: with one slab per warp the shared-memory
// pipe, not HBM, bounds the kernel (2 to 4 bytes of activations per byte of weights).
template <int NT, int WK, int MS, typename OutT>
__global__ void __launch_bounds__(256)
bitlinear_skinny_kernel(const uint32_t* __restrict__ wq, size_t wq_stride_words,
                        const float* __restrict__ tau, const float* __restrict__ bias,
                        const float* __restrict__ residual, const int8_t* __restrict__ q,
                        const float* __restrict__ s, const int32_t* __restrict__ qsum, int T, int K,
                        int OUT, int n_mats, OutT* __restrict__ y, size_t y_stride_elems,
                        int32_t* __restrict__ acc_out)
{
    constexpr int GROUPS = 8 / WK;
    constexpr int UNROLL = MS == 1 ? 4 : 2;  // 64-feature blocks per register buffer
    extern __shared__ __align__(128) unsigned char smem[];
    const int row_stride = K + 16;  // +16 bytes: conflict-free ldmatrix across tokens
    unsigned char* Bs = smem;
    int* red = reinterpret_cast<int*>(smem + (size_t)NT * 8 * row_stride);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = warp / WK, wk = warp % WK;
    const int g = lane >> 2, t4 = lane & 3;

    // stage the activations once
    {
        const int units_per_row = K / 16;
        const int total = NT * 8 * units_per_row;
        for (int i = tid; i < total; i += 256) {
            const int r = i / units_per_row, u = i - r * units_per_row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < T) v = *reinterpret_cast<const uint4*>(q + (size_t)r * K + u * 16);
            *reinterpret_cast<uint4*>(Bs + (size_t)r * row_stride + u * 16) = v;
        }
    }
    __syncthreads();

    const int words_per_row = K / 16;
    const int nblk = K / 64;
    const int mtiles = (OUT + 16 * MS - 1) / (16 * MS);
    const int n_items = mtiles * n_mats;
    const int blk_lo = (int)(((long long)nblk * wk) / WK);
    const int blk_hi = (int)(((long long)nblk * (wk + 1)) / WK);
    // ldmatrix row address of this lane (token lane&7 of each n-tile, 16-byte unit lane>>3)
    const unsigned char* b_lane = Bs + (size_t)(lane & 7) * row_stride + (lane >> 3) * 16;

    for (int item = blockIdx.x * GROUPS + group; item < n_items; item += gridDim.x * GROUPS) {
        const int mat = item / mtiles, mt = item - mat * mtiles;
        const uint32_t* wm = wq + (size_t)mat * wq_stride_words;
        int r_lo[MS], r_hi[MS];
        bool ok_lo[MS], ok_hi[MS];
        const uint32_t *p_lo[MS], *p_hi[MS];
#pragma unroll
        for (int ms = 0; ms < MS; ++ms) {
            r_lo[ms] = (mt * MS + ms) * 16 + g;
            r_hi[ms] = r_lo[ms] + 8;
            ok_lo[ms] = r_lo[ms] < OUT;
            ok_hi[ms] = r_hi[ms] < OUT;
            p_lo[ms] = wm + (size_t)(ok_lo[ms] ? r_lo[ms] : 0) * words_per_row + t4;
            p_hi[ms] = wm + (size_t)(ok_hi[ms] ? r_hi[ms] : 0) * words_per_row + t4;
        }

        int acc[MS][NT][4];
#pragma unroll
        for (int ms = 0; ms < MS; ++ms)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[ms][j][c] = 0;

        uint32_t cur_lo[MS][UNROLL], cur_hi[MS][UNROLL], nxt_lo[MS][UNROLL], nxt_hi[MS][UNROLL];
        auto fetch = [&](int b0, uint32_t (&lo)[MS][UNROLL], uint32_t (&hi)[MS][UNROLL]) {
#pragma unroll
            for (int ms = 0; ms < MS; ++ms)
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    const int b = b0 + u;
                    const bool in = b < blk_hi;
                    lo[ms][u] = (in && ok_lo[ms]) ? __ldg(p_lo[ms] + 4 * b) : 0u;
                    hi[ms][u] = (in && ok_hi[ms]) ? __ldg(p_hi[ms] + 4 * b) : 0u;
                }
        };
        fetch(blk_lo, cur_lo, cur_hi);
        for (int b0 = blk_lo; b0 < blk_hi; b0 += UNROLL) {
            fetch(b0 + UNROLL, nxt_lo, nxt_hi);
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int b = b0 + u;
                if (b < blk_hi) {
                    constexpr uint32_t MSK = 0x03030303u;
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        uint32_t bf[4];
                        ldmatrix_x4(bf, b_lane + (size_t)nt * 8 * row_stride + b * 64);
#pragma unroll
                        for (int ms = 0; ms < MS; ++ms) {
                            const uint32_t w_lo = cur_lo[ms][u], w_hi = cur_hi[ms][u];
                            mma_u8s8(acc[ms][nt], w_lo & MSK, w_hi & MSK, (w_lo >> 2) & MSK, (w_hi >> 2) & MSK, bf[0], bf[1]);
                            mma_u8s8(acc[ms][nt], (w_lo >> 4) & MSK, (w_hi >> 4) & MSK, (w_lo >> 6) & MSK, (w_hi >> 6) & MSK, bf[2],
                                     bf[3]);
                        }
                    }
                }
            }
#pragma unroll
            for (int ms = 0; ms < MS; ++ms)
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) {
                    cur_lo[ms][u] = nxt_lo[ms][u];
                    cur_hi[ms][u] = nxt_hi[ms][u];
                }
        }

        if (WK > 1) {
            // items are assigned per group, so the WK warps of a group always iterate together;
            // they meet on a named barrier of their own (id group+1), never on the CTA barrier
            int* slot = red + ((size_t)(group * WK + wk) * 32 + lane) * (MS * NT * 4);
            if (wk > 0) {
#pragma unroll
                for (int ms = 0; ms < MS; ++ms)
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int c = 0; c < 4; ++c) slot[(ms * NT + j) * 4 + c] = acc[ms][j][c];
            }
            // named barrier per group: only the WK warps of this group take part
            asm volatile("bar.sync %0, %1;\n" ::"r"(group + 1), "r"(WK * 32));
            if (wk == 0) {
#pragma unroll
                for (int o = 1; o < WK; ++o) {
                    const int* src = red + ((size_t)(group * WK + o) * 32 + lane) * (MS * NT * 4);
#pragma unroll
                    for (int ms = 0; ms < MS; ++ms)
#pragma unroll
                        for (int j = 0; j < NT; ++j)
#pragma unroll
                            for (int c = 0; c < 4; ++c) acc[ms][j][c] += src[(ms * NT + j) * 4 + c];
                }
            }
            asm volatile("bar.sync %0, %1;\n" ::"r"(group + 1), "r"(WK * 32));
        }
        if (wk == 0) {
            const float* tau_m = tau + (size_t)mat * OUT;
            const float* bias_m = bias ? bias + (size_t)mat * OUT : nullptr;
            OutT* y_m = y + (size_t)mat * y_stride_elems;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int tok = nt * 8 + t4 * 2 + cc;
                    if (tok >= T) continue;
                    const int qs2 = 2 * qsum[tok];
                    const float st = s[tok];
#pragma unroll
                    for (int ms = 0; ms < MS; ++ms) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int row = h ? r_hi[ms] : r_lo[ms];
                            if (row >= OUT) continue;
                            const int a = acc[ms][nt][h * 2 + cc] - qs2;
                            float v = __fmul_rn(__fmul_rn(tau_m[row], st), (float)a);
                            if (bias_m) v = __fadd_rn(v, bias_m[row]);
                            if (residual) v = __fadd_rn(residual[(size_t)tok * OUT + row], v);
                            store_out<OutT>(y_m + (size_t)tok * OUT + row, v);
                            if (acc_out) acc_out[(size_t)tok * OUT + row] = a;
                        }
                    }
                }
            }
        }
    }
}

template <int NT, int WK, int MS, typename OutT>
static nnb_status launch_skinny(nnb_engine* e, const uint32_t* wq, size_t wq_stride,
                                const float* tau, const float* bias, const float* residual,
                                const int8_t* q, const float* s, const int32_t* qsum, size_t n_mats,
                                size_t t, size_t k, size_t out, OutT* y, size_t y_stride,
                                int32_t* acc)
{
    constexpr int GROUPS = 8 / WK;
    const size_t smem = (size_t)NT * 8 * (k + 16) + (size_t)8 * 32 * MS * NT * 4 * sizeof(int);
    auto kern = bitlinear_skinny_kernel<NT, WK, MS, OutT>;
    static size_t cfg_dev[64] = {}; size_t& configured = cfg_dev[e->device & 63];  // the attribute is per device
    if (smem > configured) {
        NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    const size_t n_items = ceil_div(out, 16 * MS) * n_mats;
    size_t ctas_per_sm = (200 * 1024) / (smem + 1024);
    if (ctas_per_sm > 4) ctas_per_sm = 4;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    size_t grid = ceil_div(n_items, GROUPS);
    const size_t cap = (size_t)e->sm_count * ctas_per_sm;
    if (grid > cap) grid = cap;
    kern<<<(unsigned)grid, 256, smem, e->stream>>>(wq, wq_stride, tau, bias, residual, q, s, qsum,
                                                   (int)t, (int)k, (int)out, (int)n_mats, y, y_stride,
                                                   acc);
    e->launches++;
    NNB_CHECK_LAUNCH("bitlinear_skinny_kernel");
    return NNB_OK;
}

template <int BM, int BN, int BK, int STAGES, int WM, int WN, int WK, typename OutT>
static nnb_status launch_cfg(nnb_engine* e, const uint32_t* wq, size_t wq_stride,
                             const float* tau, const float* bias, const float* residual,
                             const int8_t* q, const float* s,
                             const int32_t* qsum, size_t n_mats, size_t t, size_t k, size_t out,
                             OutT* y, size_t y_stride, int32_t* acc)
{
    constexpr int THREADS = WM * WN * WK * 32;
    constexpr size_t pipe = (size_t)STAGES * (BM * (BK / 4) + BN * BK);
    constexpr size_t red = WK > 1 ? (size_t)(WM * WN) * (WK - 1) * 32 * ((BM / WM / 16) * (BN / WN / 8) * 4) * 4 : 0;
    constexpr size_t smem = pipe > red ? pipe : red;
    auto kern = bitlinear_mma_kernel<BM, BN, BK, STAGES, WM, WN, WK, OutT>;
    static bool cfg_dev[64] = {}; bool& configured = cfg_dev[e->device & 63];  // the attribute is per device
    if (!configured) {
        NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = true;
    }
    dim3 grid((unsigned)ceil_div(out, BM), (unsigned)ceil_div(t, BN), (unsigned)n_mats);
    NNB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "bitlinear_fwd: grid too large (t=%zu, n_mats=%zu)",
                t, n_mats);
    kern<<<grid, THREADS, smem, e->stream>>>(wq, wq_stride, tau, bias, residual, q, s, qsum, (int)t,
                                             (int)k, (int)out, y, y_stride, acc);
    e->launches++;
    NNB_CHECK_LAUNCH("bitlinear_mma_kernel");
    return NNB_OK;
}


// ------------------------------------------------------- weight streamer with register-resident activations
// The skinny kernel above reads an activation fragment from shared memory for every weight word it multiplies, which
// makes the shared-memory pipe its bound (measured 90 % busy at half of the HBM rate).  Here the eight warps of a CTA
// split K once and for all: a warp owns at most BPW 64-feature blocks and keeps their activation fragments (4
// registers per block and token tile) for the CTA's lifetime, loaded once through the same shared-memory staging and
// ldmatrix addressing.  Inside the loop nothing but packed weights moves: every lane fetches the two words per block and
// 16-row slab it needs for the next item while the tensor cores work on the current one; the warps' partial sums meet in
// shared memory once per item (MS slabs of 16 rows).
template <int NT, int BPW, int MS, typename OutT>
__global__ void __launch_bounds__(256)
bitlinear_stream_kernel(const uint32_t* __restrict__ wq, size_t wq_stride_words, const float* __restrict__ tau,
                        const float* __restrict__ bias, const float* __restrict__ residual, const int8_t* __restrict__ q,
                        const float* __restrict__ s, const int32_t* __restrict__ qsum, int T, int K, int OUT, int n_mats,
                        OutT* __restrict__ y, size_t y_stride_elems, int32_t* __restrict__ acc_out)
{
    extern __shared__ __align__(128) unsigned char smem[];
    const int row_stride = K + 16;
    unsigned char* Bs = smem;
    const int tid = threadIdx.x, lane = tid & 31, wk = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    {
        const int units_per_row = K / 16;
        const int total = NT * 8 * units_per_row;
        for (int i = tid; i < total; i += 256) {
            const int r = i / units_per_row, u = i - r * units_per_row;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < T) v = *reinterpret_cast<const uint4*>(q + (size_t)r * K + u * 16);
            *reinterpret_cast<uint4*>(Bs + (size_t)r * row_stride + u * 16) = v;
        }
    }
    __syncthreads();
    const int words_per_row = K / 16;
    const int nblk = K / 64;
    const int blk_lo = (int)(((long long)nblk * wk) / 8);
    const int blk_hi = (int)(((long long)nblk * (wk + 1)) / 8);
    uint32_t frag[BPW][NT][4];
    {
        const unsigned char* b_lane = Bs + (size_t)(lane & 7) * row_stride + (lane >> 3) * 16;
#pragma unroll
        for (int u = 0; u < BPW; ++u)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                if (blk_lo + u < blk_hi) {
                    ldmatrix_x4(frag[u][nt], b_lane + (size_t)nt * 8 * row_stride + (size_t)(blk_lo + u) * 64);
                } else {
                    frag[u][nt][0] = frag[u][nt][1] = frag[u][nt][2] = frag[u][nt][3] = 0u;
                }
            }
    }
    __syncthreads();
    // the staging area is free now: it holds the warps' partial sums
    int* red = reinterpret_cast<int*>(smem);

    const int mtiles = (OUT + 16 * MS - 1) / (16 * MS);
    const int n_items = mtiles * n_mats;
    uint32_t cur[MS][BPW][2], nxt[MS][BPW][2];
    auto fetch = [&](int item, uint32_t(&dst)[MS][BPW][2]) {
        const int mat = item / mtiles, mt = item - mat * mtiles;
        const uint32_t* wm = wq + (size_t)mat * wq_stride_words;
#pragma unroll
        for (int ms = 0; ms < MS; ++ms) {
            const int r_lo = (mt * MS + ms) * 16 + g, r_hi = r_lo + 8;
            const uint32_t* p_lo = wm + (size_t)(r_lo < OUT ? r_lo : 0) * words_per_row + t4;
            const uint32_t* p_hi = wm + (size_t)(r_hi < OUT ? r_hi : 0) * words_per_row + t4;
#pragma unroll
            for (int u = 0; u < BPW; ++u) {
                const int b = blk_lo + u;
                const bool in = b < blk_hi && item < n_items;
                dst[ms][u][0] = (in && r_lo < OUT) ? __ldg(p_lo + 4 * b) : 0u;
                dst[ms][u][1] = (in && r_hi < OUT) ? __ldg(p_hi + 4 * b) : 0u;
            }
        }
    };
    int item = blockIdx.x;
    fetch(item, cur);
    for (; item < n_items; item += gridDim.x) {
        fetch(item + gridDim.x, nxt);
        int acc[MS][NT][4];
#pragma unroll
        for (int ms = 0; ms < MS; ++ms)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[ms][j][c] = 0;
        constexpr uint32_t MSK = 0x03030303u;
#pragma unroll
        for (int u = 0; u < BPW; ++u)
#pragma unroll
            for (int ms = 0; ms < MS; ++ms) {
                const uint32_t w_lo = cur[ms][u][0], w_hi = cur[ms][u][1];
                const uint32_t a0 = w_lo & MSK, a1 = w_hi & MSK, a2 = (w_lo >> 2) & MSK, a3 = (w_hi >> 2) & MSK;
                const uint32_t c0 = (w_lo >> 4) & MSK, c1 = (w_hi >> 4) & MSK, c2 = (w_lo >> 6) & MSK, c3 = (w_hi >> 6) & MSK;
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma_u8s8(acc[ms][nt], a0, a1, a2, a3, frag[u][nt][0], frag[u][nt][1]);
                    mma_u8s8(acc[ms][nt], c0, c1, c2, c3, frag[u][nt][2], frag[u][nt][3]);
                }
            }
        // warps 1..7 park their partial sums, warp 0 adds them up and writes the rows
        constexpr int PER = MS * NT * 4;
        if (wk > 0) {
            int* slot = red + ((size_t)(wk - 1) * 32 + lane) * PER;
#pragma unroll
            for (int ms = 0; ms < MS; ++ms)
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) slot[(ms * NT + j) * 4 + c] = acc[ms][j][c];
        }
        __syncthreads();
        if (wk == 0) {
#pragma unroll
            for (int o = 0; o < 7; ++o) {
                const int* src = red + ((size_t)o * 32 + lane) * PER;
#pragma unroll
                for (int ms = 0; ms < MS; ++ms)
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[ms][j][c] += src[(ms * NT + j) * 4 + c];
            }
            const int mat = item / mtiles, mt = item - mat * mtiles;
            const float* tau_m = tau + (size_t)mat * OUT;
            const float* bias_m = bias ? bias + (size_t)mat * OUT : nullptr;
            OutT* y_m = y + (size_t)mat * y_stride_elems;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    const int tok = nt * 8 + t4 * 2 + cc;
                    if (tok >= T) continue;
                    const int qs2 = 2 * qsum[tok];
                    const float st = s[tok];
#pragma unroll
                    for (int ms = 0; ms < MS; ++ms) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int row = (mt * MS + ms) * 16 + g + h * 8;
                            if (row >= OUT) continue;
                            const int a = acc[ms][nt][h * 2 + cc] - qs2;
                            float v = __fmul_rn(__fmul_rn(tau_m[row], st), (float)a);
                            if (bias_m) v = __fadd_rn(v, bias_m[row]);
                            if (residual) v = __fadd_rn(residual[(size_t)tok * OUT + row], v);
                            store_out<OutT>(y_m + (size_t)tok * OUT + row, v);
                            if (acc_out) acc_out[(size_t)tok * OUT + row] = a;
                        }
                    }
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int ms = 0; ms < MS; ++ms)
#pragma unroll
            for (int u = 0; u < BPW; ++u) {
                cur[ms][u][0] = nxt[ms][u][0];
                cur[ms][u][1] = nxt[ms][u][1];
            }
    }
}

// NNB_STREAM=0 in the environment turns the register-resident streamer off (for A/B timing)
static bool stream_enabled()
{
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("NNB_STREAM");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

template <int NT, int BPW, int MS, typename OutT>
static nnb_status launch_stream(nnb_engine* e, const uint32_t* wq, size_t wq_stride, const float* tau, const float* bias,
                                const float* residual, const int8_t* q, const float* s, const int32_t* qsum, size_t n_mats,
                                size_t t, size_t k, size_t out, OutT* y, size_t y_stride, int32_t* acc)
{
    const size_t stage = (size_t)NT * 8 * (k + 16), red = (size_t)7 * 32 * MS * NT * 4 * sizeof(int);
    const size_t smem = stage > red ? stage : red;
    auto kern = bitlinear_stream_kernel<NT, BPW, MS, OutT>;
    static size_t cfg_dev[64] = {}; size_t& configured = cfg_dev[e->device & 63];  // the attribute is per device
    if (smem > configured) {
        NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    const size_t n_items = ceil_div(out, 16 * MS) * n_mats;
    // persistent CTAs: as many as are resident together (registers and shared memory decide), each walks the items
    int resident = 0;
    NNB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kern, 256, smem));
    if (resident < 1) resident = 1;
    if (resident > 4) resident = 4;
    size_t grid = n_items;
    if (grid > (size_t)e->sm_count * resident) grid = (size_t)e->sm_count * resident;
    kern<<<(unsigned)grid, 256, smem, e->stream>>>(wq, wq_stride, tau, bias, residual, q, s, qsum, (int)t, (int)k, (int)out,
                                                   (int)n_mats, y, y_stride, acc);
    e->launches++;
    NNB_CHECK_LAUNCH("bitlinear_stream_kernel");
    return NNB_OK;
}

// picks the streamer's shape: eight warps split the K / 64 blocks, at most BPW each
template <int NT, typename OutT>
static bool try_stream(nnb_engine* e, const uint32_t* wq, size_t wq_stride, const float* tau, const float* bias,
                       const float* residual, const int8_t* q, const float* s, const int32_t* qsum, size_t n_mats, size_t t,
                       size_t k, size_t out, OutT* y, size_t y_stride, int32_t* acc, nnb_status* st)
{
    if (!stream_enabled()) return false;
    const size_t bpw = ceil_div(k / 64, 8);
    // enough items to give every CTA a few rounds; small problems stay on the kernels that split K less
    if (ceil_div(out, 32) * n_mats < (size_t)e->sm_count * 4) return false;
    // measured on stacks of 64 matrices at 1 to 8 tokens: K 5632 (11 blocks per warp) 80-86 us against 108-111 us for the
    // skinny kernel; at K 2048-3200 (4 to 7 blocks per warp) the two barriers per 32-row item cost more than the saved
    // shared-memory reads (160-210 us against 115-142 us), so those shapes stay on the skinny kernel
    if (bpw > 8 && bpw <= 12 && NT == 1)
        *st = launch_stream<NT, 12, 1, OutT>(e, wq, wq_stride, tau, bias, residual, q, s, qsum, n_mats, t, k, out, y, y_stride, acc);
    else return false;
    return true;
}

// ------------------------------------------------------- CUDA-core GEMV (one to four tokens)
// At a handful of tokens the tensor-core kernels spend their shared-memory bandwidth on activation fragments that are
// mostly padding (token tiles of 8): the shared-memory pipe, not HBM, bounds them.  Here nothing but the packed weights
// moves inside the loop.  A warp owns a slab of output rows; its 32 lanes split K in 64-feature blocks; a lane keeps
// the int8 activations of its block in registers (16 words per token), reads its 16 bytes of every row (the warp reads
// 512 contiguous bytes of a row), unpacks the 2-bit codes with shift + mask (the activation layout pairs
// (w >> 2c) & 0x03030303 of word i with activation word 4c + i of the block) and multiplies with dp4a, unsigned codes x
// signed activations; 2 * rowsum comes off afterwards, as in the mma kernels.  Eight rows are in flight per lane while
// the previous eight are multiplied; their partial sums are folded across the lanes by a reduce-scatter (9 shuffles per
// token for 8 rows).  K beyond 2048 is walked in chunks of 32 blocks, the rows' totals waiting in shared memory.
__device__ __forceinline__ int dp4a_us(uint32_t a_u8, uint32_t b_s8, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a_u8), "r"(b_s8), "r"(c));
    return d;
}

constexpr int GEMV_SR_MAX = 256;  // rows per work item at most (totals kept per warp in shared memory)

template <int MT, typename OutT>
__global__ void __launch_bounds__(256)
bitlinear_gemv_kernel(const uint32_t* __restrict__ wq, size_t wq_stride_words, const float* __restrict__ tau,
                      const float* __restrict__ bias, const float* __restrict__ residual, const int8_t* __restrict__ q,
                      const float* __restrict__ s, const int32_t* __restrict__ qsum, int T, int K, int OUT, int n_mats, int SR,
                      OutT* __restrict__ y, size_t y_stride_elems, int32_t* __restrict__ acc_out)
{
    __shared__ int tot_s[8][MT][GEMV_SR_MAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nblk = K / 64, NC = (nblk + 31) / 32;
    const int rstride = K / 64;  // 16-byte units per row
    const int slabs = (OUT + SR - 1) / SR;
    const int n_items = slabs * n_mats;
    int(*tot)[GEMV_SR_MAX] = tot_s[warp];
    // which of a group's 8 rows this lane ends up holding after the reduce-scatter
    const int b0 = lane & 1, b1 = (lane >> 1) & 1, b2 = (lane >> 2) & 1;
    const int myrow = 4 * b0 + 2 * b1 + b2;
    constexpr uint32_t MSK = 0x03030303u;

    for (int item = blockIdx.x * 8 + warp; item < n_items; item += gridDim.x * 8) {
        const int mat = item / slabs, sl = item - mat * slabs;
        const int row0 = sl * SR;
        const int nrows = min(SR, OUT - row0);
        const int ngroups = (nrows + 7) >> 3;
        const uint4* wm = reinterpret_cast<const uint4*>(wq + (size_t)mat * wq_stride_words) + (size_t)row0 * rstride;
        for (int c = 0; c < NC; ++c) {
            const int bi = c * 32 + lane;
            const bool bok = bi < nblk;
            uint32_t A[MT][16];
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (bok && m < T) {
                    const uint4* ap = reinterpret_cast<const uint4*>(q + (size_t)m * K + (size_t)bi * 64);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint4 a4 = __ldg(ap + u);
                        A[m][4 * u + 0] = a4.x; A[m][4 * u + 1] = a4.y; A[m][4 * u + 2] = a4.z; A[m][4 * u + 3] = a4.w;
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < 16; ++u) A[m][u] = 0u;
                }
            }
            const uint4* wp = wm + bi;
            uint4 cur[8], nxt[8];
            auto fetch = [&](int g, uint4(&dst)[8]) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int r = g * 8 + j;
                    dst[j] = (bok && r < nrows) ? __ldg(wp + (size_t)r * rstride) : make_uint4(0u, 0u, 0u, 0u);
                }
            };
            fetch(0, cur);
            for (int g = 0; g < ngroups; ++g) {
                if (g + 1 < ngroups) fetch(g + 1, nxt);
                int v[MT][8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const uint32_t w[4] = {cur[j].x, cur[j].y, cur[j].z, cur[j].w};
                    uint32_t f[16];  // f[4c + i] = codes c, c+4, c+8, c+12 of word i
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        f[i] = w[i] & MSK;
                        f[4 + i] = (w[i] >> 2) & MSK;
                        f[8 + i] = (w[i] >> 4) & MSK;
                        f[12 + i] = (w[i] >> 6) & MSK;
                    }
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        int a = 0;
#pragma unroll
                        for (int u = 0; u < 16; ++u) a = dp4a_us(f[u], A[m][u], a);
                        v[m][j] = a;
                    }
                }
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    // reduce-scatter over lane bits 0..2 (8 -> 4 -> 2 -> 1 values), then a plain sum over bits 3, 4
                    int u4[4], u2[2], u1;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int send = b0 ? v[m][i] : v[m][i + 4], keep = b0 ? v[m][i + 4] : v[m][i];
                        u4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int send = b1 ? u4[i] : u4[i + 2], keep = b1 ? u4[i + 2] : u4[i];
                        u2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
                    }
                    {
                        const int send = b2 ? u2[0] : u2[1], keep = b2 ? u2[1] : u2[0];
                        u1 = keep + __shfl_xor_sync(0xffffffffu, send, 4);
                    }
                    u1 += __shfl_xor_sync(0xffffffffu, u1, 8);
                    u1 += __shfl_xor_sync(0xffffffffu, u1, 16);
                    if (lane < 8) {
                        if (c == 0) tot[m][g * 8 + myrow] = u1;
                        else tot[m][g * 8 + myrow] += u1;
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
            }
        }
        __syncwarp();
        const float* tau_m = tau + (size_t)mat * OUT;
        const float* bias_m = bias ? bias + (size_t)mat * OUT : nullptr;
        OutT* y_m = y + (size_t)mat * y_stride_elems;
        for (int i = lane; i < nrows; i += 32) {
            const int row = row0 + i;
            const float tr = tau_m[row];
            const float br = bias_m ? bias_m[row] : 0.0f;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m >= T) break;
                const int a = tot[m][i] - 2 * qsum[m];
                float val = __fmul_rn(__fmul_rn(tr, s[m]), (float)a);
                if (bias_m) val = __fadd_rn(val, br);
                if (residual) val = __fadd_rn(residual[(size_t)m * OUT + row], val);
                store_out<OutT>(y_m + (size_t)m * OUT + row, val);
                if (acc_out) acc_out[(size_t)m * OUT + row] = a;
            }
        }
        __syncwarp();
    }
}

// NNB_GEMV_MAX_T in the environment: largest token count served by the CUDA-core GEMV (0 turns it off; for A/B timing)
static int gemv_max_tokens()
{
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("NNB_GEMV_MAX_T");
        v = e ? atoi(e) : 1;
        if (v < 0) v = 0;
        if (v > 4) v = 4;
    }
    return v;
}

template <int MT, typename OutT>
static nnb_status launch_gemv(nnb_engine* e, const uint32_t* wq, size_t wq_stride, const float* tau, const float* bias,
                              const float* residual, const int8_t* q, const float* s, const int32_t* qsum, size_t n_mats,
                              size_t t, size_t k, size_t out, OutT* y, size_t y_stride, int32_t* acc)
{
    // register budget (125 registers at one token, about 180 beyond): 2 CTAs of 256 threads per SM, or 1
    const size_t ctas_per_sm = MT == 1 ? 2 : 1;
    const size_t warps = (size_t)e->sm_count * ctas_per_sm * 8;
    // rows per work item: about four items per warp, whole groups of 8 rows, at most GEMV_SR_MAX
    size_t sr = (out * n_mats) / (warps * 4);
    sr = (sr + 7) & ~(size_t)7;
    if (sr < 8) sr = 8;
    if (sr > GEMV_SR_MAX) sr = GEMV_SR_MAX;
    const size_t items = ceil_div(out, sr) * n_mats;
    size_t grid = ceil_div(items, 8);
    if (grid > (size_t)e->sm_count * ctas_per_sm) grid = (size_t)e->sm_count * ctas_per_sm;
    bitlinear_gemv_kernel<MT, OutT><<<(unsigned)grid, 256, 0, e->stream>>>(wq, wq_stride, tau, bias, residual, q, s, qsum, (int)t,
                                                                           (int)k, (int)out, (int)n_mats, (int)sr, y, y_stride, acc);
    e->launches++;
    NNB_CHECK_LAUNCH("bitlinear_gemv_kernel");
    return NNB_OK;
}

template <int NT, typename OutT>
static nnb_status dispatch_skinny(nnb_engine* e, const uint32_t* wq, size_t wq_stride,
                                  const float* tau, const float* bias, const float* residual,
                                  const int8_t* q, const float* s, const int32_t* qsum,
                                  size_t n_mats, size_t t, size_t k, size_t out, OutT* y,
                                  size_t y_stride, int32_t* acc)
{
    // pick the rows per warp and the K split so that the slabs fill the machine's warp slots: two 16-row slabs
    // per warp (half the shared-memory reads per weight byte) whenever that still leaves enough items
    const size_t smem = (size_t)NT * 8 * (k + 16) + 8192 * NT;
    size_t ctas_per_sm = (200 * 1024) / (smem + 1024);
    if (ctas_per_sm > 4) ctas_per_sm = 4;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    const size_t slots = (size_t)e->sm_count * ctas_per_sm * 8;
    const size_t nblk = k / 64;
#define NNB_SKINNY(WK_, MS_)                                                                            \
    return launch_skinny<NT, WK_, MS_, OutT>(e, wq, wq_stride, tau, bias, residual, q, s, qsum, n_mats, \
                                             t, k, out, y, y_stride, acc)
    // (four slabs per warp were measured too: 6 to 8 % slower than two at 1 to 8 tokens)
    const size_t items2 = ceil_div(out, 32) * n_mats;
    // (measured on 2048 x 11264 stacks: 0.51-0.53 of the copy bandwidth at 1-8 tokens against 0.49-0.50 with
    // one slab, 0.35 against 0.30 at 32 tokens; at 9-16 tokens the extra registers cost more occupancy than the
    // shared-memory reads they save: 0.39 against 0.43)
    if (NT != 2 && items2 * 2 >= slots) {
        if (items2 >= slots || nblk < 2) NNB_SKINNY(1, 2);
        NNB_SKINNY(2, 2);
    }
    const size_t items = ceil_div(out, 16) * n_mats;
    if (items >= slots || nblk < 2) NNB_SKINNY(1, 1);
    if (items * 2 >= slots || nblk < 4) NNB_SKINNY(2, 1);
    if (items * 4 >= slots || nblk < 8) NNB_SKINNY(4, 1);
    NNB_SKINNY(8, 1);
#undef NNB_SKINNY
}

template <typename OutT>
static nnb_status dispatch_fwd(nnb_engine* e, const uint32_t* wq, size_t wq_stride, const float* tau,
                               const float* bias, const float* residual, const int8_t* q,
                               const float* s, const int32_t* qsum, size_t n_mats, size_t t,
                               size_t k, size_t out, OutT* y, size_t y_stride, int32_t* acc)
{
    const size_t skinny_limit = 200 * 1024;
    // CUDA-core GEMV: measured against the tensor-core kernels on stacks of 64 matrices it wins at one token when K fills
    // the lanes (K 2048: 84 against 114 us, K 5632: 55 against 106 us) and loses from two tokens on (ALU-bound)
    if ((int)t <= gemv_max_tokens() && (k / 64) * 4 >= ceil_div(k / 64, 32) * 32 * 3) {
        if (t == 1) return launch_gemv<1, OutT>(e, wq, wq_stride, tau, bias, residual, q, s, qsum, n_mats, t, k, out, y, y_stride, acc);
        if (t == 2) return launch_gemv<2, OutT>(e, wq, wq_stride, tau, bias, residual, q, s, qsum, n_mats, t, k, out, y, y_stride, acc);
        return launch_gemv<4, OutT>(e, wq, wq_stride, tau, bias, residual, q, s, qsum, n_mats, t, k, out, y, y_stride, acc);
    }
    {
        nnb_status st = NNB_OK;
        if (t <= 8 && 8 * (k + 16) <= skinny_limit &&
            try_stream<1, OutT>(e, wq, wq_stride, tau, bias, residual, q, s, qsum, n_mats, t, k, out, y, y_stride, acc, &st))
            return st;
        if (t > 8 && t <= 16 && 16 * (k + 16) <= skinny_limit &&
            try_stream<2, OutT>(e, wq, wq_stride, tau, bias, residual, q, s, qsum, n_mats, t, k, out, y, y_stride, acc, &st))
            return st;
    }
    if (t <= 8 && 8 * (k + 16) + 4096 <= skinny_limit)
        return dispatch_skinny<1, OutT>(e, wq, wq_stride, tau, bias, residual, q, s, qsum, n_mats, t,
                                        k, out, y, y_stride, acc);
    if (t <= 16 && 16 * (k + 16) + 8192 <= skinny_limit)
        return dispatch_skinny<2, OutT>(e, wq, wq_stride, tau, bias, residual, q, s, qsum, n_mats, t,
                                        k, out, y, y_stride, acc);
    if (t <= 32 && 32 * (k + 16) + 16384 <= skinny_limit)
        return dispatch_skinny<4, OutT>(e, wq, wq_stride, tau, bias, residual, q, s, qsum, n_mats, t,
                                        k, out, y, y_stride, acc);
    if (t <= 64)
        return launch_cfg<64, 64, 128, 4, 2, 2, 1, OutT>(e, wq, wq_stride, tau, bias, residual, q, s,
                                                          qsum, n_mats, t, k, out, y, y_stride, acc);
    if (t <= 1024)  // few token tiles: narrower token tiles give the machine more CTAs
        return launch_cfg<128, 64, 128, 4, 4, 2, 1, OutT>(e, wq, wq_stride, tau, bias, residual, q, s,
                                                           qsum, n_mats, t, k, out, y, y_stride, acc);
    return launch_cfg<128, 128, 128, 4, 2, 4, 1, OutT>(e, wq, wq_stride, tau, bias, residual, q, s,
                                                        qsum, n_mats, t, k, out, y, y_stride, acc);
}

// ------------------------------------------------------------------ launchers
static inline unsigned blocks_for(size_t n, int threads) { return (unsigned)ceil_div(n, (size_t)threads); }

nnb_status launch_absmean_tau(nnb_engine* e, const float* latent, size_t rows, size_t k, float* tau)
{
    NNB_REQUIRE(latent && tau && rows > 0 && k > 0, "absmean_tau: bad arguments");
    absmean_tau_kernel<<<blocks_for(rows, 8), 256, 0, e->stream>>>(latent, rows, k, tau);
    e->launches++;
    NNB_CHECK_LAUNCH("absmean_tau_kernel");
    return NNB_OK;
}

nnb_status launch_trit_pack(nnb_engine* e, const float* latent, const float* tau, size_t rows,
                            size_t k, uint32_t* packed)
{
    NNB_REQUIRE(latent && tau && packed && rows > 0 && k > 0, "trit_pack: bad arguments");
    const size_t words = rows * ceil_div(k, 16);
    trit_pack_kernel<<<blocks_for(words, 256), 256, 0, e->stream>>>(latent, tau, rows, k, packed);
    e->launches++;
    NNB_CHECK_LAUNCH("trit_pack_kernel");
    return NNB_OK;
}

nnb_status launch_col_absmax_scale(nnb_engine* e, const float* x, size_t k, size_t n, float* s)
{
    NNB_REQUIRE(x && s && k > 0 && n > 0, "col_absmax_scale: bad arguments");
    col_absmax_scale_kernel<<<blocks_for(n, 128), 128, 0, e->stream>>>(x, k, n, s);
    e->launches++;
    NNB_CHECK_LAUNCH("col_absmax_scale_kernel");
    return NNB_OK;
}

nnb_status launch_quantize_i8(nnb_engine* e, const float* x, size_t m, size_t n, const float* scale,
                              int col_scale, uint32_t* out)
{
    NNB_REQUIRE(x && scale && out && m > 0 && n > 0, "quantize_i8: bad arguments");
    const size_t words = m * ceil_div(n, 4);
    quantize_i8_kernel<<<blocks_for(words, 256), 256, 0, e->stream>>>(x, m, n, scale, col_scale, out);
    e->launches++;
    NNB_CHECK_LAUNCH("quantize_i8_kernel");
    return NNB_OK;
}

nnb_status launch_unpack_i8(nnb_engine* e, const uint32_t* packed, size_t m, size_t n, float* out)
{
    NNB_REQUIRE(packed && out && m > 0 && n > 0, "unpack_i8: bad arguments");
    unpack_i8_kernel<<<blocks_for(m * n, 256), 256, 0, e->stream>>>(packed, m, n, out);
    e->launches++;
    NNB_CHECK_LAUNCH("unpack_i8_kernel");
    return NNB_OK;
}

nnb_status launch_matmul_q_i8_ref(nnb_engine* e, const uint32_t* wq, const float* tau,
                                  const uint32_t* xq, const float* s, size_t rows, size_t k,
                                  size_t n, float* y, int32_t* acc)
{
    NNB_REQUIRE(wq && tau && xq && s && (y || acc) && rows > 0 && k > 0 && n > 0,
                "matmul_q_i8: bad arguments");
    matmul_q_i8_ref_kernel<<<blocks_for(rows * n, 128), 128, 0, e->stream>>>(wq, tau, xq, s, rows, k,
                                                                             n, y, acc);
    e->launches++;
    NNB_CHECK_LAUNCH("matmul_q_i8_ref_kernel");
    return NNB_OK;
}

nnb_status launch_matmul_q_ref(nnb_engine* e, const uint32_t* wq, const float* tau, const float* x,
                               size_t rows, size_t k, size_t n, float* c)
{
    NNB_REQUIRE(wq && tau && x && c && rows > 0 && k > 0 && n > 0, "matmul_q: bad arguments");
    matmul_q_ref_kernel<<<blocks_for(rows * n, 128), 128, 0, e->stream>>>(wq, tau, x, rows, k, n, c);
    e->launches++;
    NNB_CHECK_LAUNCH("matmul_q_ref_kernel");
    return NNB_OK;
}

nnb_status launch_matmul_q_t_ref(nnb_engine* e, const uint32_t* wq, const float* tau,
                                 const float* b, size_t rows, size_t mcols, size_t n, float* c)
{
    NNB_REQUIRE(wq && tau && b && c && rows > 0 && mcols > 0 && n > 0, "matmul_q_t: bad arguments");
    matmul_q_t_ref_kernel<<<blocks_for(mcols * n, 128), 128, 0, e->stream>>>(wq, tau, b, rows, mcols,
                                                                             n, c);
    e->launches++;
    NNB_CHECK_LAUNCH("matmul_q_t_ref_kernel");
    return NNB_OK;
}

nnb_status launch_act_quant_tm(nnb_engine* e, const void* x, nnb_dtype dtype, size_t t, size_t k,
                               int8_t* q, float* s, int32_t* qsum)
{
    NNB_REQUIRE(x && q && s && qsum && t > 0, "act_quant_tm: bad arguments");
    NNB_REQUIRE(k > 0 && k % 64 == 0, "act_quant_tm: k=%zu must be a positive multiple of 64", k);
    NNB_REQUIRE(k * 4 <= 96 * 1024, "act_quant_tm: k=%zu too large", k);
    NNB_REQUIRE(((uintptr_t)q & 15) == 0, "act_quant_tm: q must be 16-byte aligned");
    const size_t smem = k * sizeof(float);
    if (dtype == NNB_F32) {
        static bool cfg_dev[64] = {}; bool& cfg = cfg_dev[e->device & 63];  // the attribute is per device
        if (!cfg) {
            NNB_CUDA(cudaFuncSetAttribute(act_quant_tm_kernel<float>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
            cfg = true;
        }
        act_quant_tm_kernel<float><<<(unsigned)t, 256, smem, e->stream>>>((const float*)x, (int)k, q, s, qsum);
    } else if (dtype == NNB_BF16) {
        static bool cfg_dev[64] = {}; bool& cfg = cfg_dev[e->device & 63];  // the attribute is per device
        if (!cfg) {
            NNB_CUDA(cudaFuncSetAttribute(act_quant_tm_kernel<__nv_bfloat16>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
            cfg = true;
        }
        act_quant_tm_kernel<__nv_bfloat16>
            <<<(unsigned)t, 256, smem, e->stream>>>((const __nv_bfloat16*)x, (int)k, q, s, qsum);
    } else {
        NNB_FAIL(NNB_ERR_INVALID, "act_quant_tm: unknown dtype %d", (int)dtype);
    }
    e->launches++;
    NNB_CHECK_LAUNCH("act_quant_tm_kernel");
    return NNB_OK;
}

nnb_status launch_actq_to_plain(nnb_engine* e, const int8_t* q, size_t t, size_t k, int8_t* plain)
{
    NNB_REQUIRE(q && plain && t > 0 && k > 0 && k % 64 == 0, "actq_to_plain: bad arguments");
    actq_to_plain_kernel<<<blocks_for(t * k, 256), 256, 0, e->stream>>>(q, t * k, plain);
    e->launches++;
    NNB_CHECK_LAUNCH("actq_to_plain_kernel");
    return NNB_OK;
}

nnb_status launch_bitlinear_fwd_tm(nnb_engine* e, const uint32_t* wq, size_t wq_stride_words,
                                   const float* tau, const float* bias, const float* residual,
                                   const int8_t* q, const float* s, const int32_t* qsum,
                                   size_t n_mats, size_t t, size_t k, size_t out, void* y,
                                   size_t y_stride_elems, nnb_dtype dtype, int32_t* acc)
{
    NNB_REQUIRE(wq && tau && q && s && qsum && y, "bitlinear_fwd: NULL argument");
    NNB_REQUIRE(t > 0 && out > 0 && n_mats > 0, "bitlinear_fwd: empty shape");
    NNB_REQUIRE(k > 0 && k % 64 == 0, "bitlinear_fwd: k=%zu must be a positive multiple of 64", k);
    NNB_REQUIRE(((uintptr_t)wq & 15) == 0 && ((uintptr_t)q & 15) == 0 && (wq_stride_words % 4) == 0,
                "bitlinear_fwd: weights and activations must be 16-byte aligned");
    NNB_REQUIRE(t <= 0x7fffffff && out <= 0x7fffffff && k <= 0x7fffffff, "bitlinear_fwd: shape too large");
    NNB_REQUIRE(acc == nullptr || n_mats == 1, "bitlinear_fwd: accumulator output needs n_mats == 1");
    NNB_REQUIRE(residual == nullptr || n_mats == 1, "bitlinear_fwd: residual needs n_mats == 1");
    if (dtype == NNB_F32)
        return dispatch_fwd<float>(e, wq, wq_stride_words, tau, bias, residual, q, s, qsum, n_mats, t,
                                   k, out, (float*)y, y_stride_elems, acc);
    if (dtype == NNB_BF16)
        return dispatch_fwd<__nv_bfloat16>(e, wq, wq_stride_words, tau, bias, residual, q, s, qsum,
                                           n_mats, t, k, out, (__nv_bfloat16*)y, y_stride_elems, acc);
    NNB_FAIL(NNB_ERR_INVALID, "bitlinear_fwd: unknown dtype %d", (int)dtype);
}

}  // namespace nnb
