// gemm_tc.cu — the Blackwell tensor-core GEMM of the engine: TMA-fed tcgen05.mma with the
// accumulator in tensor memory, persistent over output tiles.
//
// One kernel template serves the three large GEMMs of a ternary linear
// (include/neuralnet.cpp/compute_layer_bitlinear.hpp:454, 494, 514-534):
//   forward  y[t,o]  = (tau_o*s_t) * sum_k q[t,k]*trit[o,k] (+bias, +residual)   kind::i8, int32 accum
//   dX       dx[t,k] (+)= sum_o dyb[t,o] * trit[o,k]                              kind::f16 (bf16), f32 accum
//   dW       dw[o,k] += sum_t dyb[t,o] * xs[t,k]                                  kind::f16 (bf16), f32 accum
// with dyb = bf16(dy*tau) and xs = bf16(s*q) prepared by small elementwise kernels, and the ternary
// weights expanded once per requantisation to int8 (K permuted like q) and to bf16.
//
// Roles inside a CTA (320 threads): warp 0 issues TMA loads into a shared-memory ring (4 to 8 stages,
// as many as fit), warp 1 issues tcgen05.mma (one thread) and owns the TMEM allocation, warps 2-9 drain
// the accumulator (tcgen05.ld) through the epilogue, two warps per TMEM lane quarter, each taking half of
// the tile's columns.  Two accumulators of BN columns let the epilogue of one tile overlap the main loop
// of the next.  The output tile is 128 x BN with BN in {64, 128, 192, 256}: the large training GEMMs use
// 256, the forward at a few hundred tokens picks the width that fills the SMs best.  Every mbarrier wait is bounded: on expiry the kernel raises
// an error flag and all roles leave their loops, TMEM is released, and the host reports NNB_ERR_TIMEOUT.
#include <cuda.h>

#include <map>
#include <tuple>

#include "common.cuh"
#include "device_math.cuh"

namespace nnb {
namespace tc {

constexpr int BM = 128;
constexpr int STAGE_A = BM * 128;  // bytes: 128 B of K (or 64 k-rows x 128 B) per row
constexpr int MAX_STAGES = 8;
constexpr int THREADS = 320;
constexpr int EPI_WARPS = 8;
template <int BN>
struct Tile {
    static constexpr int STAGE_B = BN * 128;
    static constexpr int STAGE_BYTES = STAGE_A + STAGE_B;
    static constexpr int EPI_STAGING = EPI_WARPS * 32 * 32 * 4;  // one 32 x 32 f32 transposition tile per epilogue warp
    static constexpr int FIT = (227 * 1024 - 1024 - 256 - EPI_STAGING) / STAGE_BYTES;
    static constexpr int STAGES = FIT > MAX_STAGES ? MAX_STAGES : FIT;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + EPI_STAGING;
    static constexpr uint32_t TMEM_COLS = 2 * BN <= 128 ? 128u : (2 * BN <= 256 ? 256u : 512u);
};
constexpr uint32_t SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// bounded wait: false when the limit was reached (the caller then raises the error flag and leaves)
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    const uint32_t addr = smem_u32(bar);
    for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((it & 1023) == 1023 && *abort_flag) return false;
    }
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tm, uint64_t* bar, int c0, int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tm)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// shared-memory matrix descriptor, 128-byte swizzle (layout type 2), descriptor version 1
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

template <int KIND>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    if (KIND == 0) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}\n"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
    }
}

__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

struct Epi {
    // forward: y = (tau[n]*s[m])*acc (+bias[n]) (+residual[m,n]);  dX: c (+)= acc;  dW: c += acc
    float* out;
    const float* tau;
    const float* s;
    const float* bias;
    const float* residual;
    int accumulate;
    // stacked matrices: column c belongs to matrix c / n_mat and lands at out + (c / n_mat) * mat_stride +
    // row * n_mat + c % n_mat (n_mat = N and mat_stride = 0 for a single matrix)
    int n_mat;
    size_t mat_stride;
    // LM head fused with the categorical distribution (EPI 2 and 3): the logits x = (tau*s)*acc + bias never
    // reach memory.  EPI 2 leaves, per (row, half column tile), the partial log-sum-exp triple
    // (max, sum e^(x-max), sum (x-max) e^(x-max)) in part_m / part_s / part_u [(2*tile + half) * M + row] and the
    // action's logit in act_logit[row].  EPI 3 recomputes x and writes d loss / d logits, already multiplied by
    // tau and rounded to bf16 (the operand of the head's backward GEMMs), to dyb (M, N), and the column sums of
    // every 32-row block to db_part[(row / 32) * N + col] (the bias gradient, finished in a fixed order).
    const int32_t* actions;
    float *part_m, *part_s, *part_u, *act_logit;
    const float *lse, *ent, *up_lp, *up_ent;
    __nv_bfloat16* dyb;
    float* db_part;
    // EPI 0: when set, the result is rounded to bf16 and stored here (same indexing) instead of `out`
    __nv_bfloat16* out_b;
    // EPI 1: splits > 1 cuts the contraction into that many slices of k_tiles_per_split stages; slice i is a tile of its
    // own and stores (never accumulates) its product at out + i * split_stride
    int splits;
    int k_tiles_per_split;
    size_t split_stride;
};

// KIND 0: int8 (A, B K-major, 128 k per stage).  KIND 1: bf16 (64 k per stage), A/B K- or MN-major.
// EPI 0: forward, 1: plain store/accumulate.
template <int KIND, bool A_MN, bool B_MN, int EPI, int BN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, Epi ep, int M, int N,
               int KC, int* __restrict__ err)
{
    constexpr int STAGES = Tile<BN>::STAGES, STAGE_BYTES = Tile<BN>::STAGE_BYTES;
    constexpr uint32_t TMEM_COLS = Tile<BN>::TMEM_COLS;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    uint64_t* full = bars;                 // [STAGES] TMA -> MMA
    uint64_t* empty = bars + STAGES;       // [STAGES] MMA -> TMA
    uint64_t* acc_full = bars + 2 * STAGES;      // [2] MMA -> epilogue
    uint64_t* acc_empty = bars + 2 * STAGES + 2; // [2] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = err;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch();  // the next kernel of the stream may take the SM as soon as this CTA leaves it
    constexpr int KE = KIND == 0 ? 128 : 64;  // contraction elements per stage
    const int ktiles_all = (KC + KE - 1) / KE;
    const bool split = EPI == 1 && ep.splits > 1;
    const int kt_per = split ? ep.k_tiles_per_split : ktiles_all;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int mn_tiles = tiles_m * tiles_n;
    const int n_tiles = mn_tiles * (split ? ep.splits : 1);
    // with few row tiles, CTAs that run side by side take the row tiles of one column tile, so a tile of B
    // (the weights, in the forward) comes from DRAM once and from L2 for the others
    const bool m_fast = tiles_m <= 8;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], EPI_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // barriers and TMEM are set up; operands written by the previous kernel of the stream are touched from here on
    pdl_wait();

    if (warp == 0) {
        // ---------------- TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int sp = tile / mn_tiles, t2 = tile - sp * mn_tiles;
                const int tm = m_fast ? t2 % tiles_m : t2 / tiles_n, tn = m_fast ? t2 / tiles_m : t2 % tiles_n;
                const int kt0 = sp * kt_per, kt1 = min(ktiles_all, kt0 + kt_per);
                for (int kt = kt0; kt < kt1 && ok; ++kt, ++it) {
                    const int st = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (it >= STAGES && !mbar_wait(&empty[st], ph ^ 1, abort_flag)) { ok = false; break; }
                    unsigned char* sa = smem + st * STAGE_BYTES;
                    unsigned char* sb = sa + STAGE_A;
                    mbar_expect_tx(&full[st], STAGE_BYTES);
                    if (!A_MN) {
                        tma_load_2d(sa, &tmA, &full[st], kt * KE, tm * BM);
                    } else {
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * 8192, &tmA, &full[st], tm * BM + c * 64, kt * KE);
                    }
                    if (!B_MN) {
                        tma_load_2d(sb, &tmB, &full[st], kt * KE, tn * BN);
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * 8192, &tmB, &full[st], tn * BN + c * 64, kt * KE);
                    }
                }
            }
            if (!ok) atomicExch(err, 1);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = (KIND == 0 ? (2u << 4) | (1u << 7) | (1u << 10) : (1u << 4) | (1u << 7) | (1u << 10)) |
                                       ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(BN >> 3) << 17) |
                                       ((uint32_t)(BM >> 4) << 24);
            uint32_t it = 0, tcount = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tcount) {
                const int acc = tcount & 1;
                if (tcount >= 2 && !mbar_wait(&acc_empty[acc], ((tcount >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t d_tmem = tmem_base + acc * BN;
                const int sp = tile / mn_tiles;
                const int ktiles = min(ktiles_all, (sp + 1) * kt_per) - sp * kt_per;
                for (int kt = 0; kt < ktiles; ++kt, ++it) {
                    const int st = it % STAGES;
                    if (!mbar_wait(&full[st], (it / STAGES) & 1, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t sa = smem_u32(smem + st * STAGE_BYTES), sb = sa + STAGE_A;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        // K-major: 32 bytes of K per instruction inside the 128-byte swizzle row;
                        // MN-major: 16 k-rows of 128 bytes per instruction
                        const uint64_t ad = A_MN ? make_desc(sa + ks * 2048, 8192, 1024) : make_desc(sa + ks * 32, 16, 1024);
                        const uint64_t bd = B_MN ? make_desc(sb + ks * 2048, 8192, 1024) : make_desc(sb + ks * 32, 16, 1024);
                        umma<KIND>(d_tmem, ad, bd, idesc, (kt > 0 || ks > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[st]);
                }
                if (ok) umma_commit(&acc_full[acc]);
            }
            if (!ok) atomicExch(err, 1);
        }
    } else {
        // ---------------- epilogue: warps 2..9, TMEM lane quarter = warp % 4, column half = (warp - 2) / 4.
        // tcgen05.ld hands a thread 32 columns of ONE row; storing that directly would scatter every store
        // instruction over 32 rows.  Each warp therefore transposes its 32 x 32 block through a swizzled
        // 4 KB staging tile: afterwards 8 lanes cover the 32 columns of a row with 16-byte accesses, a store
        // (and the residual / accumulate load) instruction covers 4 full 128-byte rows, and tau / bias are
        // one 16-byte load per chunk.
        const int quarter = warp & 3;
        const int chalf = (warp - 2) >> 2;
        float* stg = reinterpret_cast<float*>(smem + STAGES * STAGE_BYTES + 256) + (warp - 2) * 1024;
        const int lc = (lane & 7) * 4, lr = lane >> 3;
        const bool aligned = (((uintptr_t)ep.out | (uintptr_t)ep.tau | (uintptr_t)ep.bias | (uintptr_t)ep.residual) & 15) == 0 &&
                             ((uintptr_t)ep.out_b & 7) == 0 &&
                             (ep.n_mat & 3) == 0 && (ep.mat_stride & 3) == 0 && (ep.split_stride & 3) == 0;
        uint32_t tcount = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++tcount) {
            const int sp = tile / mn_tiles, t2 = tile - sp * mn_tiles;
            const int tm = m_fast ? t2 % tiles_m : t2 / tiles_n, tn = m_fast ? t2 / tiles_m : t2 % tiles_n;
            float* const outp = split ? ep.out + (size_t)sp * ep.split_stride : ep.out;
            const int acc = tcount & 1;
            const int row0 = tm * BM + quarter * 32;
            const int row = row0 + lane;
            constexpr int NCHUNK = BN / 64;  // 32-column chunks per warp
            if constexpr (EPI == 2 || EPI == 3) {
                // ---- LM head fused with log-softmax: a thread owns one row of the accumulator (what tcgen05.ld hands it)
                const bool valid = row < M;
                const float srow = valid ? ep.s[row] : 0.0f;
                const int act = valid ? ep.actions[row] : -1;
                float m_run = -INFINITY, s_run = 0.0f, u_run = 0.0f, ax = 0.0f;
                bool have_ax = false;
                float lse_r = 0.0f, h_r = 0.0f, ul = 0.0f, ue = 0.0f;
                if (EPI == 3 && valid) {
                    lse_r = ep.lse[row];
                    ul = ep.up_lp[row];
                    if (ep.up_ent) {
                        ue = ep.up_ent[row];
                        h_r = ep.ent[row];
                    }
                }
                const bool vec_ok = (((uintptr_t)ep.tau | (uintptr_t)ep.bias) & 15) == 0;
                if (!mbar_wait(&acc_full[acc], (tcount >> 1) & 1, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
                for (int ci = 0; ci < NCHUNK; ++ci) {
                    const int c0 = chalf * (BN / 2) + ci * 32;
                    const int col0 = tn * BN + c0;
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c0, r);
                    if (col0 >= N) continue;  // warp-uniform
                    const bool full = col0 + 32 <= N;
                    float x[32];
                    if (full && vec_ok) {
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4) {
                            const float4 t4 = *reinterpret_cast<const float4*>(ep.tau + col0 + 4 * j4);
                            const float4 b4 = ep.bias ? *reinterpret_cast<const float4*>(ep.bias + col0 + 4 * j4) : make_float4(0.f, 0.f, 0.f, 0.f);
                            x[4 * j4 + 0] = __fadd_rn(__fmul_rn(__fmul_rn(t4.x, srow), (float)(int)r[4 * j4 + 0]), b4.x);
                            x[4 * j4 + 1] = __fadd_rn(__fmul_rn(__fmul_rn(t4.y, srow), (float)(int)r[4 * j4 + 1]), b4.y);
                            x[4 * j4 + 2] = __fadd_rn(__fmul_rn(__fmul_rn(t4.z, srow), (float)(int)r[4 * j4 + 2]), b4.z);
                            x[4 * j4 + 3] = __fadd_rn(__fmul_rn(__fmul_rn(t4.w, srow), (float)(int)r[4 * j4 + 3]), b4.w);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int col = col0 + j;
                            x[j] = col < N ? __fadd_rn(__fmul_rn(__fmul_rn(ep.tau[col], srow), (float)(int)r[j]), ep.bias ? ep.bias[col] : 0.0f)
                                           : -INFINITY;
                        }
                    }
                    if constexpr (EPI == 2) {
                        float cm = x[0];
#pragma unroll
                        for (int j = 1; j < 32; ++j) cm = fmaxf(cm, x[j]);
                        if (cm > m_run) {
                            if (m_run > -INFINITY) {
                                const float f = __expf(m_run - cm);
                                u_run = f * (u_run + (m_run - cm) * s_run);
                                s_run *= f;
                            }
                            m_run = cm;
                        }
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float d = x[j] - m_run;  // -inf for a column past the vocabulary
                            const float ev = __expf(d);
                            s_run += ev;
                            u_run += ev > 0.0f ? d * ev : 0.0f;
                            if (col0 + j == act) { ax = x[j]; have_ax = true; }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const bool in = full || col0 + j < N;
                            const float lp = x[j] - lse_r;
                            const float pr = in ? __expf(lp) : 0.0f;
                            float dl = ul * ((col0 + j == act ? 1.0f : 0.0f) - pr);
                            if (ue != 0.0f) dl -= ue * pr * (lp + h_r);
                            r[j] = __float_as_uint(in ? dl : 0.0f);
                        }
                        // transpose the 32 x 32 block through the staging tile: afterwards a lane holds 4 columns of 8 rows
#pragma unroll
                        for (int c4 = 0; c4 < 8; ++c4)
                            *reinterpret_cast<uint4*>(stg + lane * 32 + ((c4 ^ (lane & 7)) << 2)) =
                                make_uint4(r[4 * c4], r[4 * c4 + 1], r[4 * c4 + 2], r[4 * c4 + 3]);
                        __syncwarp();
                        float4 cs = make_float4(0.f, 0.f, 0.f, 0.f);
                        float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
                        const int colb = col0 + lc;
                        if (vec_ok && colb + 3 < N) t4 = *reinterpret_cast<const float4*>(ep.tau + colb);
                        else {
                            if (colb + 3 < N) t4.w = ep.tau[colb + 3];
                            if (colb < N) t4.x = ep.tau[colb];
                            if (colb + 1 < N) t4.y = ep.tau[colb + 1];
                            if (colb + 2 < N) t4.z = ep.tau[colb + 2];
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = i * 4 + lr;
                            const float4 a = *reinterpret_cast<const float4*>(stg + rr * 32 + (((lane & 7) ^ (rr & 7)) << 2));
                            cs.x += a.x; cs.y += a.y; cs.z += a.z; cs.w += a.w;
                            if (row0 + rr < M) {
                                __nv_bfloat16* dst = ep.dyb + (size_t)(row0 + rr) * N + colb;
                                if (colb + 3 < N) {
                                    const __nv_bfloat162 p0 = __floats2bfloat162_rn(a.x * t4.x, a.y * t4.y);
                                    const __nv_bfloat162 p1 = __floats2bfloat162_rn(a.z * t4.z, a.w * t4.w);
                                    uint2 o;
                                    o.x = *reinterpret_cast<const uint32_t*>(&p0);
                                    o.y = *reinterpret_cast<const uint32_t*>(&p1);
                                    *reinterpret_cast<uint2*>(dst) = o;
                                } else {
                                    if (colb < N) dst[0] = __float2bfloat16_rn(a.x * t4.x);
                                    if (colb + 1 < N) dst[1] = __float2bfloat16_rn(a.y * t4.y);
                                    if (colb + 2 < N) dst[2] = __float2bfloat16_rn(a.z * t4.z);
                                }
                            }
                        }
                        // column sums over the block's 32 rows: the four lane groups (lr = 0..3) hold 8 rows each
                        cs.x += __shfl_xor_sync(0xffffffffu, cs.x, 8); cs.y += __shfl_xor_sync(0xffffffffu, cs.y, 8);
                        cs.z += __shfl_xor_sync(0xffffffffu, cs.z, 8); cs.w += __shfl_xor_sync(0xffffffffu, cs.w, 8);
                        cs.x += __shfl_xor_sync(0xffffffffu, cs.x, 16); cs.y += __shfl_xor_sync(0xffffffffu, cs.y, 16);
                        cs.z += __shfl_xor_sync(0xffffffffu, cs.z, 16); cs.w += __shfl_xor_sync(0xffffffffu, cs.w, 16);
                        if (lr == 0 && row0 < M) {
                            float* dp = ep.db_part + (size_t)(row0 >> 5) * N + colb;
                            if (colb + 3 < N) *reinterpret_cast<float4*>(dp) = cs;
                            else {
                                if (colb < N) dp[0] = cs.x;
                                if (colb + 1 < N) dp[1] = cs.y;
                                if (colb + 2 < N) dp[2] = cs.z;
                            }
                        }
                        __syncwarp();
                    }
                }
                if constexpr (EPI == 2) {
                    if (valid) {
                        const size_t pi = (size_t)(tn * 2 + chalf) * M + row;
                        ep.part_m[pi] = m_run;
                        ep.part_s[pi] = s_run;
                        ep.part_u[pi] = u_run;
                        if (have_ax) ep.act_logit[row] = ax;
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[acc]);
                continue;
            }
            // what a chunk needs from global memory (tau, bias, and the residual or the values to accumulate
            // into) is fetched one chunk ahead, the first chunk's before the accumulator is even ready, so
            // that DRAM latency stays off the path between tcgen05.ld and the stores
            const float* pre_src = EPI == 0 ? ep.residual : (ep.accumulate ? outp : nullptr);
            float4 pre[2][8], tau4[2], bias4[2];
            auto fetch = [&](int ci, int slot) {
                const int col0 = tn * BN + chalf * (BN / 2) + ci * 32;
                tau4[slot] = bias4[slot] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int i = 0; i < 8; ++i) pre[slot][i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (!(aligned && col0 + 32 <= N)) return;
                if (EPI == 0) {
                    tau4[slot] = *reinterpret_cast<const float4*>(ep.tau + col0 + lc);
                    if (ep.bias) bias4[slot] = *reinterpret_cast<const float4*>(ep.bias + col0 + lc);
                }
                if (!pre_src) return;
                const int mat = col0 / ep.n_mat;
                const size_t off0 = (size_t)mat * ep.mat_stride + (size_t)(col0 - mat * ep.n_mat);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rr = i * 4 + lr;
                    if (row0 + rr < M) pre[slot][i] = *reinterpret_cast<const float4*>(pre_src + off0 + (size_t)(row0 + rr) * ep.n_mat + lc);
                }
            };
            const float srow = (EPI == 0 && row < M) ? ep.s[row] : 0.0f;
            fetch(0, 0);
            if (!mbar_wait(&acc_full[acc], (tcount >> 1) & 1, abort_flag)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
            for (int ci = 0; ci < NCHUNK; ++ci) {
                const int slot = ci & 1;
                const int c0 = chalf * (BN / 2) + ci * 32;
                if (ci + 1 < NCHUNK) fetch(ci + 1, slot ^ 1);
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c0, r);
                const int col0 = tn * BN + c0;
                if (col0 >= N) continue;  // warp-uniform
                const int mat = col0 / ep.n_mat;
                const size_t off0 = (size_t)mat * ep.mat_stride + (size_t)(col0 - mat * ep.n_mat);
                if (aligned && col0 + 32 <= N) {
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4)
                        *reinterpret_cast<uint4*>(stg + lane * 32 + ((c4 ^ (lane & 7)) << 2)) =
                            make_uint4(r[4 * c4], r[4 * c4 + 1], r[4 * c4 + 2], r[4 * c4 + 3]);
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int rr = i * 4 + lr;
                        const float sr = __shfl_sync(0xffffffffu, srow, rr);
                        const uint4 a = *reinterpret_cast<const uint4*>(stg + rr * 32 + (((lane & 7) ^ (rr & 7)) << 2));
                        if (row0 + rr < M) {
                            const size_t off = off0 + (size_t)(row0 + rr) * ep.n_mat + lc;
                            const float4 t4 = tau4[slot], b4 = bias4[slot], p4 = pre[slot][i];
                            float4 o;
                            if (EPI == 0) {
                                o.x = __fmul_rn(__fmul_rn(t4.x, sr), (float)(int)a.x);
                                o.y = __fmul_rn(__fmul_rn(t4.y, sr), (float)(int)a.y);
                                o.z = __fmul_rn(__fmul_rn(t4.z, sr), (float)(int)a.z);
                                o.w = __fmul_rn(__fmul_rn(t4.w, sr), (float)(int)a.w);
                                if (ep.bias) {
                                    o.x = __fadd_rn(o.x, b4.x); o.y = __fadd_rn(o.y, b4.y);
                                    o.z = __fadd_rn(o.z, b4.z); o.w = __fadd_rn(o.w, b4.w);
                                }
                                if (ep.residual) {
                                    o.x = __fadd_rn(p4.x, o.x); o.y = __fadd_rn(p4.y, o.y);
                                    o.z = __fadd_rn(p4.z, o.z); o.w = __fadd_rn(p4.w, o.w);
                                }
                            } else {
                                o = make_float4(__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w));
                                if (ep.accumulate) {
                                    o.x += p4.x; o.y += p4.y; o.z += p4.z; o.w += p4.w;
                                }
                            }
                            if (EPI == 0 && ep.out_b) {
                                const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                                uint2 w2;
                                w2.x = *reinterpret_cast<const uint32_t*>(&lo);
                                w2.y = *reinterpret_cast<const uint32_t*>(&hi);
                                *reinterpret_cast<uint2*>(ep.out_b + off) = w2;
                            } else {
                                *reinterpret_cast<float4*>(outp + off) = o;
                            }
                        }
                    }
                    __syncwarp();
                } else if (row < M) {
                    // ragged right edge or unaligned operands: the row owner writes its own columns
                    const size_t off = off0 + (size_t)row * ep.n_mat;
                    for (int j = 0; j < 32; ++j) {
                        const int col = col0 + j;
                        if (col >= N) break;
                        float x;
                        if (EPI == 0) {
                            x = __fmul_rn(__fmul_rn(ep.tau[col], srow), (float)(int)r[j]);
                            if (ep.bias) x = __fadd_rn(x, ep.bias[col]);
                            if (ep.residual) x = __fadd_rn(ep.residual[off + j], x);
                        } else {
                            x = __uint_as_float(r[j]);
                            if (ep.accumulate) x += outp[off + j];
                        }
                        if (EPI == 0 && ep.out_b) ep.out_b[off + j] = __float2bfloat16_rn(x);
                        else outp[off + j] = x;
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
        }
        if (!ok && lane == 0) atomicExch(err, 1);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 2-D row-major matrix (rows, cols) of `esize`-byte elements; box = (box_cols, box_rows), 128-byte swizzle.
// Encoding a map costs several microseconds of host time, and the same buffers recur step after step,
// so encoded maps are memoised per thread.
static nnb_status make_map(CUtensorMap* tm, const void* base, CUtensorMapDataType dt, size_t esize, size_t rows, size_t cols,
                           uint32_t box_cols, uint32_t box_rows)
{
    typedef std::tuple<const void*, int, size_t, size_t, uint32_t, uint32_t> Key;
    static thread_local std::map<Key, CUtensorMap> cache;
    const Key key(base, (int)dt, rows, cols, box_cols, box_rows);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *tm = it->second;
        return NNB_OK;
    }
    if (cache.size() > 8192) cache.clear();
    EncodeTiledFn fn = encode_fn();
    if (!fn) NNB_FAIL(NNB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    NNB_REQUIRE(((uintptr_t)base & 15) == 0 && (cols * esize) % 16 == 0,
                "tensor-core GEMM operand must be 16-byte aligned with a row pitch that is a multiple of 16 bytes");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * esize};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) NNB_FAIL(NNB_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    cache[key] = *tm;
    return NNB_OK;
}

template <int KIND, bool A_MN, bool B_MN, int EPI, int BN>
static nnb_status launch(nnb_engine* e, const CUtensorMap& ta, const CUtensorMap& tb, const Epi& ep, size_t M, size_t N, size_t KC)
{
    auto kern = gemm_tc_kernel<KIND, A_MN, B_MN, EPI, BN>;
    constexpr int SMEM_BYTES = Tile<BN>::SMEM_BYTES;
    static bool cfg_dev[64] = {}; bool& cfg = cfg_dev[e->device & 63];  // the attribute is per device
    if (!cfg) {
        NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        cfg = true;
    }
    int* flag = e->dev_flags;
    const size_t tiles = ceil_div(M, BM) * ceil_div(N, BN) * (size_t)(EPI == 1 && ep.splits > 1 ? ep.splits : 1);
    const unsigned grid = (unsigned)(tiles < (size_t)e->sm_count ? tiles : (size_t)e->sm_count);
    launch_ex(e, kern, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, ta, tb, ep, (int)M, (int)N, (int)KC, flag);
    e->launches++;
    NNB_CHECK_LAUNCH("gemm_tc_kernel");
    return NNB_OK;
}

}  // namespace tc

// Width of the forward output tile.  A launch runs ceil(tiles / SMs) rounds of tiles; a round costs a fixed
// part (pipeline fill, epilogue of the last tile, barrier turnarounds: about what 230 columns of a K = 2048
// main loop cost) plus a main loop proportional to BN * K.  Measured on 10240 x 2048 x 6144: 5.1 / 6.2 /
// 6.7 / 8.5 us per round for BN = 64 / 128 / 192 / 256.  Wide tiles win whenever they fill the SMs; narrow
// ones only pay off for a few hundred tokens, where they turn a half-empty round into a full one.
static int g_forward_bn_override = 0;
static int choose_forward_bn(size_t t, size_t k, size_t out, int sm_count)
{
    if (g_forward_bn_override) return g_forward_bn_override;
    const int cand[4] = {256, 192, 128, 64};
    int best = 256;
    size_t best_cost = (size_t)-1;
    for (int bn : cand) {
        const size_t tiles = ceil_div(t, (size_t)tc::BM) * ceil_div(out, (size_t)bn);
        const size_t cost = ceil_div(tiles, (size_t)sm_count) * (230 * 2048 + (size_t)bn * k);
        if (cost < best_cost) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

template <int BN>
static nnb_status tc_forward_bn(nnb_engine* e, const int8_t* q, const int8_t* w8, const tc::Epi& ep, size_t t, size_t k, size_t out)
{
    using namespace tc;
    CUtensorMap ta, tb;
    NNB_TRY(make_map(&ta, q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, t, k, 128, BM));
    NNB_TRY(make_map(&tb, w8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, out, k, 128, BN));
    return launch<0, false, false, 0, BN>(e, ta, tb, ep, t, out, k);
}

// forward: q (T,K) permuted int8, w8 (OUT,K) int8 trits in the same K permutation
// n_mats > 1: w8 / tau / bias hold n_mats matrices of `out` rows one after the other and matrix m writes the
// (t, out) block at y + m * y_stride; one launch covers them all when out is a multiple of 32
nnb_status launch_tc_forward(nnb_engine* e, const int8_t* q, const int8_t* w8, const float* tau, const float* s,
                             const float* bias, const float* residual, size_t t, size_t k, size_t out, float* y,
                             size_t n_mats, size_t y_stride, __nv_bfloat16* y_bf16)
{
    NNB_REQUIRE(!y_bf16 || (n_mats == 1 && !residual), "tc_forward: the bf16 output takes one matrix and no residual");
    if (n_mats > 1 && out % 32 != 0) {
        for (size_t m = 0; m < n_mats; ++m)
            NNB_TRY(launch_tc_forward(e, q, w8 + m * out * k, tau + m * out, s, bias ? bias + m * out : nullptr,
                                      residual ? residual + m * y_stride : nullptr, t, k, out, y + m * y_stride, 1, 0));
        return NNB_OK;
    }
    tc::Epi ep{y, tau, s, bias, residual, 0, (int)out, n_mats > 1 ? y_stride : 0};
    ep.out_b = y_bf16;
    out *= n_mats;
    switch (choose_forward_bn(t, k, out, e->sm_count)) {
        case 64: return tc_forward_bn<64>(e, q, w8, ep, t, k, out);
        case 128: return tc_forward_bn<128>(e, q, w8, ep, t, k, out);
        case 192: return tc_forward_bn<192>(e, q, w8, ep, t, k, out);
        default: return tc_forward_bn<256>(e, q, w8, ep, t, k, out);
    }
}

nnb_status tc_set_forward_tile(int bn)
{
    NNB_REQUIRE(bn == 0 || bn == 64 || bn == 128 || bn == 192 || bn == 256, "forward tile width %d: 0 (automatic), 64, 128, 192 or 256", bn);
    g_forward_bn_override = bn;
    return NNB_OK;
}

// ---- LM head fused with CategoricalDistribution (include/neuralnet.cpp/rl_policy.hpp:92-187; the reference's own
// pattern for not re-reading (V, T) logits is the online log-sum-exp fold of its sparse cross-entropy,
// include/neuralnet.cpp/compute_loss.hpp:315-429).
// merge of the per-tile partials: lse = m + log s, logp = x_action - lse, H = log s - u / s
__global__ void __launch_bounds__(256)
lmhead_merge_kernel(const float* __restrict__ pm, const float* __restrict__ ps, const float* __restrict__ pu,
                    const float* __restrict__ act_logit, int n_part, int M, float* __restrict__ lse, float* __restrict__ logp,
                    float* __restrict__ ent)
{
    // 32 rows per CTA (lanes = rows, so that the partial arrays are read along their contiguous axis), 8 warps splitting
    // the partials; the warps' results are merged in a fixed order
    __shared__ float sm_m[8][32], sm_s[8][32], sm_u[8][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * 32 + lane;
    float m = -INFINITY, s = 0.0f, u = 0.0f;
    if (row < M) {
        for (int p = warp; p < n_part; p += 8) {
            const float sp = ps[(size_t)p * M + row];
            if (!(sp > 0.0f)) continue;
            const float mp = pm[(size_t)p * M + row], up = pu[(size_t)p * M + row];
            if (mp > m) {
                if (m > -INFINITY) {
                    const float f = __expf(m - mp);
                    u = f * (u + (m - mp) * s);
                    s *= f;
                }
                m = mp;
            }
            const float dm = mp - m, f = __expf(dm);
            s += sp * f;
            u += (up + dm * sp) * f;
        }
    }
    sm_m[warp][lane] = m;
    sm_s[warp][lane] = s;
    sm_u[warp][lane] = u;
    __syncthreads();
    if (warp != 0 || row >= M) return;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; ++w) mm = fmaxf(mm, sm_m[w][lane]);
    float ss = 0.0f, uu = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const float sw = sm_s[w][lane];
        if (sw > 0.0f) {
            const float dm = sm_m[w][lane] - mm, f = __expf(dm);
            ss += sw * f;
            uu += (sm_u[w][lane] + dm * sw) * f;
        }
    }
    const float ls = __logf(ss);
    lse[row] = mm + ls;
    if (logp) logp[row] = act_logit[row] - (mm + ls);
    if (ent) ent[row] = ls - uu / ss;
}

size_t tc_lmhead_scratch_floats(size_t t, size_t v)
{
    const size_t n_part = 2 * ceil_div(v, (size_t)256);
    const size_t fwd = 3 * n_part * t + t;             // partial triples + the action's logit
    const size_t bwd = ceil_div(t, (size_t)32) * v;    // column sums per 32-row block
    return fwd > bwd ? fwd : bwd;
}

// forward: log-prob of the action, entropy (optional) and log-sum-exp of every row, logits never stored.
// scratch: tc_lmhead_scratch_floats(t, v) floats
nnb_status launch_tc_lmhead_fwd(nnb_engine* e, const int8_t* q, const int8_t* w8, const float* tau, const float* s, const float* bias,
                                const int32_t* actions, size_t t, size_t k, size_t v, float* scratch, float* lse, float* logp, float* ent)
{
    using namespace tc;
    constexpr int BN = 256;
    const size_t n_part = 2 * ceil_div(v, (size_t)BN);
    CUtensorMap ta, tb;
    NNB_TRY(make_map(&ta, q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, t, k, 128, BM));
    NNB_TRY(make_map(&tb, w8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, v, k, 128, BN));
    Epi ep{};
    ep.tau = tau;
    ep.s = s;
    ep.bias = bias;
    ep.n_mat = (int)v;
    ep.actions = actions;
    ep.part_m = scratch;
    ep.part_s = scratch + n_part * t;
    ep.part_u = scratch + 2 * n_part * t;
    ep.act_logit = scratch + 3 * n_part * t;
    NNB_TRY((launch<0, false, false, 2, BN>(e, ta, tb, ep, t, v, k)));
    lmhead_merge_kernel<<<(unsigned)ceil_div(t, 32), 256, 0, e->stream>>>(ep.part_m, ep.part_s, ep.part_u, ep.act_logit, (int)n_part, (int)t,
                                                                          lse, logp, ent);
    e->launches++;
    NNB_CHECK_LAUNCH("lmhead_merge_kernel");
    return NNB_OK;
}

__global__ void __launch_bounds__(256)
colsum_blocks_kernel(const float* __restrict__ part, int n_blocks, int O, float* __restrict__ db)
{
    const int o = blockIdx.x * 256 + threadIdx.x;
    if (o >= O) return;
    float acc = 0.0f;
    for (int c = 0; c < n_blocks; ++c) acc += part[(size_t)c * O + o];
    db[o] += acc;
}

// backward: dyb (t, v) bf16 = bf16(d loss / d logits * tau) with d logits = (onehot - p) * up_lp - p * (log p + H) * up_ent
// recomputed from the same integer GEMM, and db += column sums of d logits.  v % 4 == 0.
nnb_status launch_tc_lmhead_bwd(nnb_engine* e, const int8_t* q, const int8_t* w8, const float* tau, const float* s, const float* bias,
                                const int32_t* actions, const float* lse, const float* ent, const float* up_lp, const float* up_ent,
                                size_t t, size_t k, size_t v, float* scratch, __nv_bfloat16* dyb, float* db)
{
    using namespace tc;
    constexpr int BN = 256;
    NNB_REQUIRE(v % 4 == 0 && (((uintptr_t)dyb | (uintptr_t)scratch) & 15) == 0, "fused LM-head backward: vocabulary %zu must be a multiple of 4", v);
    CUtensorMap ta, tb;
    NNB_TRY(make_map(&ta, q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, t, k, 128, BM));
    NNB_TRY(make_map(&tb, w8, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, v, k, 128, BN));
    Epi ep{};
    ep.tau = tau;
    ep.s = s;
    ep.bias = bias;
    ep.n_mat = (int)v;
    ep.actions = actions;
    ep.lse = lse;
    ep.ent = ent;
    ep.up_lp = up_lp;
    ep.up_ent = up_ent;
    ep.dyb = dyb;
    ep.db_part = scratch;
    NNB_TRY((launch<0, false, false, 3, BN>(e, ta, tb, ep, t, v, k)));
    const size_t n_blocks = ceil_div(t, (size_t)32);
    colsum_blocks_kernel<<<(unsigned)ceil_div(v, 256), 256, 0, e->stream>>>(scratch, (int)n_blocks, (int)v, db);
    e->launches++;
    NNB_CHECK_LAUNCH("colsum_blocks_kernel");
    return NNB_OK;
}

// dX: dyb (T,OUT) bf16, wb (OUT,K) bf16 trits; dx (T,K) f32
nnb_status launch_tc_dx(nnb_engine* e, const __nv_bfloat16* dyb, const __nv_bfloat16* wb, size_t t, size_t k, size_t out,
                        float* dx, bool accumulate)
{
    using namespace tc;
    CUtensorMap ta, tb;
    NNB_TRY(make_map(&ta, dyb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, t, out, 64, BM));
    NNB_TRY(make_map(&tb, wb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, k, 64, 64));
    Epi ep{dx, nullptr, nullptr, nullptr, nullptr, accumulate ? 1 : 0, (int)k, 0};
    return launch<1, false, true, 1, 256>(e, ta, tb, ep, t, k, out);
}

// c (T,N) f32 = a (T,K) bf16 . b (N,K)^T bf16: both operands K-major (the dense head of tied embeddings)
nnb_status launch_tc_nt(nnb_engine* e, const __nv_bfloat16* a, const __nv_bfloat16* b, size_t t, size_t k, size_t n, float* c)
{
    using namespace tc;
    NNB_REQUIRE(k % 8 == 0 && n % 4 == 0 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) == 0,
                "tc_nt: K must be a multiple of 8, N of 4, operands 16-byte aligned");
    CUtensorMap ta, tb;
    NNB_TRY(make_map(&ta, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, t, k, 64, BM));
    NNB_TRY(make_map(&tb, b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, n, k, 64, 256));
    Epi ep{c, nullptr, nullptr, nullptr, nullptr, 0, (int)n, 0};
    return launch<1, false, false, 1, 256>(e, ta, tb, ep, t, n, k);
}

// dW: dyb (T,OUT) bf16, xs (T,K) bf16; dw (OUT,K) f32 +=
// The contraction runs over the tokens, so the tile count is fixed by the weight matrix alone: a 768 x 768 matrix is 18
// tiles of 128 x 256 on 148 SMs, each walking all the tokens (narrower tiles fill the SMs but then every CTA streams
// both operands for all the tokens through L2, which costs as much).  Small matrices therefore split the token axis:
// slice i of every tile is a tile of its own and leaves its product in part[i]; dw_split_reduce_kernel adds the slices
// to dw in order, so the sum does not depend on the schedule.
__global__ void __launch_bounds__(256)
dw_split_reduce_kernel(const float* __restrict__ part, int splits, size_t n4, float* __restrict__ dw)
{
    const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n4) return;
    float4 a = reinterpret_cast<const float4*>(dw)[i];
    for (int s = 0; s < splits; ++s) {
        const float4 v = reinterpret_cast<const float4*>(part)[(size_t)s * n4 + i];
        a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    reinterpret_cast<float4*>(dw)[i] = a;
}

constexpr size_t DW_PART_FLOATS = (size_t)148 * 128 * 256;  // one 128 x 256 slice per SM

nnb_status launch_tc_dw(nnb_engine* e, const __nv_bfloat16* dyb, const __nv_bfloat16* xs, size_t t, size_t k, size_t out,
                        float* dw)
{
    using namespace tc;
    CUtensorMap ta, tb;
    NNB_TRY(make_map(&ta, dyb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, t, out, 64, 64));
    NNB_TRY(make_map(&tb, xs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, t, k, 64, 64));
    Epi ep{dw, nullptr, nullptr, nullptr, nullptr, 1, (int)k, 0};
    const size_t tiles = ceil_div(out, (size_t)BM) * ceil_div(k, (size_t)256), k_tiles = ceil_div(t, (size_t)64);
    // split while the slices fit the SMs, each keeps at least 16 stages, and the partial products fit their buffer
    size_t splits = std::min<size_t>(std::min<size_t>((size_t)e->sm_count / tiles, k_tiles / 16), DW_PART_FLOATS / (out * k));
    if (tiles * 2 <= (size_t)e->sm_count && splits >= 2 && (out * k) % 4 == 0 && ((uintptr_t)dw & 15) == 0) {
        if (!e->dw_part) {
            cudaError_t er = cudaMalloc((void**)&e->dw_part, DW_PART_FLOATS * sizeof(float));
            if (er != cudaSuccess) {
                cudaGetLastError();
                NNB_FAIL(NNB_ERR_OOM, "out of device memory for the weight-gradient partial products");
            }
            e->dw_part_floats = DW_PART_FLOATS;
        }
        const size_t per = ceil_div(k_tiles, splits);
        splits = ceil_div(k_tiles, per);  // no empty slice
        ep.out = e->dw_part;
        ep.accumulate = 0;
        ep.splits = (int)splits;
        ep.k_tiles_per_split = (int)per;
        ep.split_stride = out * k;
        NNB_TRY((launch<1, true, true, 1, 256>(e, ta, tb, ep, out, k, t)));
        const size_t n4 = out * k / 4;
        dw_split_reduce_kernel<<<(unsigned)ceil_div(n4, 256), 256, 0, e->stream>>>(e->dw_part, (int)splits, n4, dw);
        e->launches++;
        NNB_CHECK_LAUNCH("dw_split_reduce_kernel");
        return NNB_OK;
    }
    return launch<1, true, true, 1, 256>(e, ta, tb, ep, out, k, t);
}

// reads (and clears) the device error flag of the tensor-core GEMMs; synchronises the stream
nnb_status tc_check_errors(nnb_engine* e)
{
    int h = 0;
    int* flag = e->dev_flags;
    NNB_CUDA(cudaMemcpyAsync(&h, flag, sizeof(int), cudaMemcpyDeviceToHost, e->stream));
    NNB_CUDA(cudaStreamSynchronize(e->stream));
    if (h) {
        NNB_CUDA(cudaMemsetAsync(flag, 0, sizeof(int), e->stream));
        NNB_FAIL(NNB_ERR_TIMEOUT, "a tensor-core GEMM gave up on a bounded barrier wait");
    }
    return NNB_OK;
}

// ------------------------------------------------------------- operand preparation
// ternary container -> int8 trits with K permuted per 64-block like q, and bf16 trits in natural order
__global__ void expand_weights_kernel(const uint32_t* __restrict__ wq, size_t n_words, int8_t* __restrict__ w8,
                                      __nv_bfloat16* __restrict__ wb)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_words) return;
    const uint32_t w = wq[idx];
    if (w8) {
        // word t of its 64-block: masked register i = trits {i, 4+i, 8+i, 12+i} -> bytes [16i + 4t, +4)
        const size_t blk = idx >> 2;
        const int t = (int)(idx & 3);
        uint32_t* dst = reinterpret_cast<uint32_t*>(w8 + blk * 64);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t codes = (w >> (2 * i)) & 0x03030303u;
            dst[4 * i + t] = __vsub4(codes, 0x02020202u);
        }
    }
    if (wb) {
        uint32_t o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t c0 = (w >> (4 * i)) & 3u, c1 = (w >> (4 * i + 2)) & 3u;
            const uint32_t lo = c0 == 3u ? 0x3F80u : (c0 == 1u ? 0xBF80u : 0u);
            const uint32_t hi = c1 == 3u ? 0x3F80u : (c1 == 1u ? 0xBF80u : 0u);
            o[i] = lo | (hi << 16);
        }
        uint4* d = reinterpret_cast<uint4*>(wb + idx * 16);
        d[0] = make_uint4(o[0], o[1], o[2], o[3]);
        d[1] = make_uint4(o[4], o[5], o[6], o[7]);
    }
}

nnb_status launch_expand_weights(nnb_engine* e, const uint32_t* wq, size_t rows, size_t k, int8_t* w8, __nv_bfloat16* wb)
{
    const size_t n_words = rows * (k / 16);
    expand_weights_kernel<<<(unsigned)ceil_div(n_words, 256), 256, 0, e->stream>>>(wq, n_words, w8, wb);
    e->launches++;
    NNB_CHECK_LAUNCH("expand_weights_kernel");
    return NNB_OK;
}

// dyb[t,o] = bf16(dy[t,o] * tau[o])
__global__ void scale_to_bf16_kernel(const float* __restrict__ dy, const float* __restrict__ tau, size_t n, int O,
                                     __nv_bfloat16* __restrict__ out)
{
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i >= n) return;
    const int o = (int)(i % O);
    const float a = dy[i] * tau[o];
    const float b = (i + 1 < n) ? dy[i + 1] * tau[(o + 1) % O] : 0.0f;
    *reinterpret_cast<__nv_bfloat162*>(out + i) = __floats2bfloat162_rn(a, b);
}

// The two uses of dy in one pass: dyb[t,o] = bf16(dy[t,o] * tau[o]) and db[o] += sum_t dy[t,o].
// grid (ceil(O/256), ceil(T/chunk)), 128 threads, two adjacent columns per thread.  The column sums of a
// token chunk go to part[chunk][o]; colsum_finish_kernel adds the chunks in ascending order, so the bias
// gradient does not depend on the order in which CTAs retire (row_reduce_sum of the reference,
// include/neuralnet.cpp/compute_layer_bitlinear.hpp:538-541, is deterministic too).
__global__ void __launch_bounds__(128)
scale_colsum_kernel(const float* __restrict__ dy, const float* __restrict__ tau, int T, int O, int chunk,
                    __nv_bfloat16* __restrict__ out, size_t ld, float* __restrict__ part)
{
    const int o = (blockIdx.x * 128 + threadIdx.x) * 2;
    if (o >= O) return;
    const int t0 = blockIdx.y * chunk, t1 = min(T, t0 + chunk);
    const float2 tv = *reinterpret_cast<const float2*>(tau + o);
    float sa = 0.0f, sb = 0.0f;
    int t = t0;
    for (; t + 4 <= t1; t += 4) {
        float2 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = *reinterpret_cast<const float2*>(dy + (size_t)(t + u) * O + o);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            sa += v[u].x;
            sb += v[u].y;
            *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(t + u) * ld + o) = __floats2bfloat162_rn(v[u].x * tv.x, v[u].y * tv.y);
        }
    }
    for (; t < t1; ++t) {
        const float2 v = *reinterpret_cast<const float2*>(dy + (size_t)t * O + o);
        sa += v.x;
        sb += v.y;
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)t * ld + o) = __floats2bfloat162_rn(v.x * tv.x, v.y * tv.y);
    }
    *reinterpret_cast<float2*>(part + (size_t)blockIdx.y * O + o) = make_float2(sa, sb);
}

// the same with four adjacent columns per thread (16-byte loads, R rows in flight): out, ld multiples of 4
template <int R>
__global__ void __launch_bounds__(128)
scale_colsum4_kernel(const float* __restrict__ dy, const float* __restrict__ tau, int T, int O, int chunk,
                     __nv_bfloat16* __restrict__ out, size_t ld, float* __restrict__ part)
{
    const int o = (blockIdx.x * 128 + threadIdx.x) * 4;
    if (o >= O) return;
    const int t0 = blockIdx.y * chunk, t1 = min(T, t0 + chunk);
    const float4 tv = *reinterpret_cast<const float4*>(tau + o);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    int t = t0;
    for (; t + R <= t1; t += R) {
        float4 v[R];
#pragma unroll
        for (int u = 0; u < R; ++u) v[u] = *reinterpret_cast<const float4*>(dy + (size_t)(t + u) * O + o);
#pragma unroll
        for (int u = 0; u < R; ++u) {
            acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w;
            const __nv_bfloat162 p0 = __floats2bfloat162_rn(v[u].x * tv.x, v[u].y * tv.y);
            const __nv_bfloat162 p1 = __floats2bfloat162_rn(v[u].z * tv.z, v[u].w * tv.w);
            uint2 w;
            w.x = *reinterpret_cast<const uint32_t*>(&p0);
            w.y = *reinterpret_cast<const uint32_t*>(&p1);
            *reinterpret_cast<uint2*>(out + (size_t)(t + u) * ld + o) = w;
        }
    }
    for (; t < t1; ++t) {
        const float4 v = *reinterpret_cast<const float4*>(dy + (size_t)t * O + o);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        const __nv_bfloat162 p0 = __floats2bfloat162_rn(v.x * tv.x, v.y * tv.y);
        const __nv_bfloat162 p1 = __floats2bfloat162_rn(v.z * tv.z, v.w * tv.w);
        uint2 w;
        w.x = *reinterpret_cast<const uint32_t*>(&p0);
        w.y = *reinterpret_cast<const uint32_t*>(&p1);
        *reinterpret_cast<uint2*>(out + (size_t)t * ld + o) = w;
    }
    *reinterpret_cast<float4*>(part + (size_t)blockIdx.y * O + o) = acc;
}

// db[o] += part[0][o] + part[1][o] + ... in that order
__global__ void __launch_bounds__(256)
colsum_finish_kernel(const float* __restrict__ part, int n_chunks, int O, float* __restrict__ db)
{
    const int o = blockIdx.x * 256 + threadIdx.x;
    if (o >= O) return;
    float acc = 0.0f;
    for (int c = 0; c < n_chunks; ++c) acc += part[(size_t)c * O + o];
    db[o] += acc;
}

// one launch for the bias gradients of many linears: blockIdx.y selects the descriptor
__global__ void __launch_bounds__(256)
colsum_finish_multi_kernel(const ColsumDesc* __restrict__ descs)
{
    const ColsumDesc d = descs[blockIdx.y];
    const int o = blockIdx.x * 256 + threadIdx.x;
    if (o >= d.out) return;
    float acc = 0.0f;
    for (int c = 0; c < d.n_chunks; ++c) acc += d.part[(size_t)c * d.out + o];
    d.db[o] += acc;
}

nnb_status launch_colsum_finish_all(nnb_engine* e, ColsumSink* sink)
{
    if (!sink || sink->descs.empty()) return NNB_OK;
    NNB_REQUIRE(sink->descs.size() <= sink->desc_cap, "colsum sink: %zu descriptors, room for %zu", sink->descs.size(), sink->desc_cap);
    int max_out = 0;
    for (const ColsumDesc& d : sink->descs) max_out = d.out > max_out ? d.out : max_out;
    NNB_CUDA(cudaMemcpyAsync(sink->d_descs, sink->descs.data(), sink->descs.size() * sizeof(ColsumDesc), cudaMemcpyHostToDevice, e->stream));
    dim3 grid((unsigned)ceil_div((size_t)max_out, 256), (unsigned)sink->descs.size());
    colsum_finish_multi_kernel<<<grid, 256, 0, e->stream>>>(sink->d_descs);
    e->launches++;
    NNB_CHECK_LAUNCH("colsum_finish_multi_kernel");
    sink->descs.clear();
    sink->used = 0;
    return NNB_OK;
}

// where a launch puts its partial sums: the sink's buffer (finished later) or the engine's scratch (finished at once)
static nnb_status colsum_part(nnb_engine* e, ColsumSink* sink, size_t n_chunks, size_t out, float* db, float** part)
{
    const size_t need = n_chunks * out;
    if (sink && sink->used + need <= sink->cap && sink->descs.size() < sink->desc_cap) {
        *part = sink->buf + sink->used;
        sink->used += (need + 3) & ~(size_t)3;
        sink->descs.push_back(ColsumDesc{*part, db, (int)n_chunks, (int)out});
        return NNB_OK;
    }
    NNB_TRY(e->ensure_scratch(need * sizeof(float)));
    *part = (float*)e->scratch;
    return 1;  // caller finishes immediately
}

// Activation backward fused with the preparation of the next GEMM's operand: with h (T, F1) the
// pre-activation (F1 = 2F for SwiGLU, gate | up; F for QuickGELU) and da (T, F) the gradient of the
// activation's output, dh = act'(h) o da never reaches memory as f32: dyb[t,c] = bf16(dh[t,c] * tau[c]) and
// db[c] += sum_t dh[t,c].  Same grid as scale_colsum_kernel over the F output features.
template <typename HT>
__device__ __forceinline__ float2 ld_h2(const HT* p);
template <>
__device__ __forceinline__ float2 ld_h2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <>
__device__ __forceinline__ float2 ld_h2<__nv_bfloat16>(const __nv_bfloat16* p)
{
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// HT: type of the saved pre-activation (f32, or bf16 where the forward stored it so)
template <int MODE, typename HT = float>
__global__ void __launch_bounds__(128)
act_bwd_scale_colsum_kernel(const HT* __restrict__ h, const float* __restrict__ da, const float* __restrict__ tau, int T,
                            int F, int chunk, __nv_bfloat16* __restrict__ out, float* __restrict__ part)
{
    const int f = (blockIdx.x * 128 + threadIdx.x) * 2;
    if (f >= F) return;
    const int F1 = MODE >= 2 ? 2 * F : F;
    const int t0 = blockIdx.y * chunk, t1 = min(T, t0 + chunk);
    const float2 tg = *reinterpret_cast<const float2*>(tau + f);
    const float2 tu = MODE >= 2 ? *reinterpret_cast<const float2*>(tau + F + f) : make_float2(0.f, 0.f);
    float sg0 = 0.f, sg1 = 0.f, su0 = 0.f, su1 = 0.f;
    for (int t = t0; t < t1; t += 2) {
        float2 gv[2], uv[2], go[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int tt = min(t + u, t1 - 1);
            gv[u] = ld_h2<HT>(h + (size_t)tt * F1 + f);
            uv[u] = MODE >= 2 ? ld_h2<HT>(h + (size_t)tt * F1 + F + f) : make_float2(0.f, 0.f);
            go[u] = *reinterpret_cast<const float2*>(da + (size_t)tt * F + f);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (t + u >= t1) break;
            float dgx, dgy, dux = 0.f, duy = 0.f;
            if (MODE == 3) {
                const float r0 = fmaxf(gv[u].x, 0.0f), r1 = fmaxf(gv[u].y, 0.0f);
                dgx = go[u].x * uv[u].x * (2.0f * r0);
                dgy = go[u].y * uv[u].y * (2.0f * r1);
                dux = go[u].x * (r0 * r0);
                duy = go[u].y * (r1 * r1);
            } else if (MODE == 2) {
                const float s0 = __fdividef(1.0f, 1.0f + __expf(-gv[u].x)), s1 = __fdividef(1.0f, 1.0f + __expf(-gv[u].y));
                dgx = go[u].x * uv[u].x * (s0 * (1.0f + gv[u].x * (1.0f - s0)));
                dgy = go[u].y * uv[u].y * (s1 * (1.0f + gv[u].y * (1.0f - s1)));
                dux = go[u].x * gv[u].x * s0;
                duy = go[u].y * gv[u].y * s1;
            } else {
                const float b0 = gv[u].x * 1.702f, b1 = gv[u].y * 1.702f;
                const float s0 = __fdividef(1.0f, 1.0f + __expf(-b0)), s1 = __fdividef(1.0f, 1.0f + __expf(-b1));
                dgx = go[u].x * (s0 * (1.0f + b0 * (1.0f - s0)));
                dgy = go[u].y * (s1 * (1.0f + b1 * (1.0f - s1)));
            }
            sg0 += dgx; sg1 += dgy;
            *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(t + u) * F1 + f) = __floats2bfloat162_rn(dgx * tg.x, dgy * tg.y);
            if (MODE >= 2) {
                su0 += dux; su1 += duy;
                *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(t + u) * F1 + F + f) = __floats2bfloat162_rn(dux * tu.x, duy * tu.y);
            }
        }
    }
    float* prow = part + (size_t)blockIdx.y * F1;
    *reinterpret_cast<float2*>(prow + f) = make_float2(sg0, sg1);
    if (MODE >= 2) *reinterpret_cast<float2*>(prow + F + f) = make_float2(su0, su1);
}

// xs[t,k] = bf16(s[t] * q[t, perm(k)]) in natural feature order.  One thread per 64-feature block: it reads
// the block's 64 permuted bytes with four 16-byte loads and writes 128 contiguous bytes of bf16, so that
// both sides of the kernel move 16 bytes per lane.  Source feature j of a block sits at byte
// 16*(j%4) + 4*(j/16) + (j/4)%4 (the layout act_quant writes).
__global__ void __launch_bounds__(256)
dequant_to_bf16_kernel(const int8_t* __restrict__ q, const float* __restrict__ s, size_t T, int K,
                       __nv_bfloat16* __restrict__ out)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // one 64-byte block of q
    const int bpr = K / 64;
    if (idx >= T * (size_t)bpr) return;
    const size_t t = idx / bpr;
    const float sc = s[t];
    const uint4* src = reinterpret_cast<const uint4*>(q) + idx * 4;
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 v = src[i];
        w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
    }
    uint4* dst = reinterpret_cast<uint4*>(out) + idx * 8;
#pragma unroll
    for (int c = 0; c < 8; ++c) {  // output chunk c: features 8c .. 8c+7
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int j = 8 * c + e;
            const int byte = 16 * (j % 4) + 4 * (j / 16) + (j / 4) % 4;
            f[e] = (float)(int8_t)((w[byte >> 2] >> (8 * (byte & 3))) & 0xFFu) * sc;
        }
        uint4 o;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(f[0], f[1]), p1 = __floats2bfloat162_rn(f[2], f[3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(f[4], f[5]), p3 = __floats2bfloat162_rn(f[6], f[7]);
        o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
        o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
        dst[c] = o;
    }
}

nnb_status launch_scale_to_bf16(nnb_engine* e, const float* dy, const float* tau, size_t t, size_t out, __nv_bfloat16* dyb)
{
    NNB_REQUIRE(out % 2 == 0, "scale_to_bf16: out=%zu must be even", out);
    const size_t n = t * out;
    scale_to_bf16_kernel<<<(unsigned)ceil_div(n / 2, 256), 256, 0, e->stream>>>(dy, tau, n, (int)out, dyb);
    e->launches++;
    NNB_CHECK_LAUNCH("scale_to_bf16_kernel");
    return NNB_OK;
}

// mode 1 QuickGELU, 2 SwiGLU, 3 ReLU2GLU; F even
nnb_status launch_act_bwd_scale_colsum(nnb_engine* e, int mode, const float* h, const float* da, const float* tau, size_t t,
                                       size_t F, __nv_bfloat16* dyb, float* db, ColsumSink* sink, bool h_bf16)
{
    NNB_REQUIRE(F % 2 == 0 && mode >= 1 && mode <= 3, "act_bwd_scale_colsum: bad arguments");
    const int chunk = 128;
    dim3 grid((unsigned)ceil_div(F, 256), (unsigned)ceil_div(t, chunk));
    NNB_REQUIRE(grid.y <= 65535, "act_bwd_scale_colsum: too many tokens (%zu)", t);
    const size_t F1 = mode >= 2 ? 2 * F : F;
    float* part = nullptr;
    const nnb_status where = colsum_part(e, sink, grid.y, F1, db, &part);
    if (where < 0) return where;
    if (h_bf16) {
        const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(h);
        if (mode == 2) act_bwd_scale_colsum_kernel<2, __nv_bfloat16><<<grid, 128, 0, e->stream>>>(hb, da, tau, (int)t, (int)F, chunk, dyb, part);
        else if (mode == 3) act_bwd_scale_colsum_kernel<3, __nv_bfloat16><<<grid, 128, 0, e->stream>>>(hb, da, tau, (int)t, (int)F, chunk, dyb, part);
        else act_bwd_scale_colsum_kernel<1, __nv_bfloat16><<<grid, 128, 0, e->stream>>>(hb, da, tau, (int)t, (int)F, chunk, dyb, part);
    } else if (mode == 2) act_bwd_scale_colsum_kernel<2><<<grid, 128, 0, e->stream>>>(h, da, tau, (int)t, (int)F, chunk, dyb, part);
    else if (mode == 3) act_bwd_scale_colsum_kernel<3><<<grid, 128, 0, e->stream>>>(h, da, tau, (int)t, (int)F, chunk, dyb, part);
    else act_bwd_scale_colsum_kernel<1><<<grid, 128, 0, e->stream>>>(h, da, tau, (int)t, (int)F, chunk, dyb, part);
    e->launches++;
    if (where == 1) {
        colsum_finish_kernel<<<(unsigned)ceil_div(F1, 256), 256, 0, e->stream>>>(part, (int)grid.y, (int)F1, db);
        e->launches++;
    }
    NNB_CHECK_LAUNCH("act_bwd_scale_colsum_kernel");
    return NNB_OK;
}

// dyb_ld: row pitch of dyb in elements (0 = out), so that several matrices' gradients can sit side by side
nnb_status launch_scale_colsum(nnb_engine* e, const float* dy, const float* tau, size_t t, size_t out, __nv_bfloat16* dyb,
                               float* db, size_t dyb_ld, ColsumSink* sink)
{
    NNB_REQUIRE(out % 2 == 0 && dyb_ld % 2 == 0, "scale_colsum: out=%zu must be even", out);
    const int chunk = 128;
    dim3 grid((unsigned)ceil_div(out, 256), (unsigned)ceil_div(t, chunk));
    NNB_REQUIRE(grid.y <= 65535, "scale_colsum: too many tokens (%zu)", t);
    float* part = nullptr;
    const nnb_status where = colsum_part(e, sink, grid.y, out, db, &part);
    if (where < 0) return where;
    const size_t ld = dyb_ld ? dyb_ld : out;
    const bool vec4 = out % 4 == 0 && ld % 4 == 0 && (((uintptr_t)dy | (uintptr_t)tau | (uintptr_t)part) & 15) == 0 && ((uintptr_t)dyb & 7) == 0;
    if (vec4) {
        dim3 grid4((unsigned)ceil_div(out, 512), grid.y);
        // rows a thread keeps in flight: 4 (NNB_COLSUM_ROWS=8 for A/B runs, read once per process).  Measured on the 1B
        // training micro-batch: cold-cache 43 us per launch with 4 rows against 59 us with 8; inside the step, where dy
        // is partly L2-resident, 99.4-99.8 against 101.5-102.8 ms per micro-batch (three runs each, alternating)
        static const int rows = [] { const char* ev = getenv("NNB_COLSUM_ROWS"); return ev && ev[0] == '8' ? 8 : 4; }();
        if (rows == 4) scale_colsum4_kernel<4><<<grid4, 128, 0, e->stream>>>(dy, tau, (int)t, (int)out, chunk, dyb, ld, part);
        else scale_colsum4_kernel<8><<<grid4, 128, 0, e->stream>>>(dy, tau, (int)t, (int)out, chunk, dyb, ld, part);
    } else {
        scale_colsum_kernel<<<grid, 128, 0, e->stream>>>(dy, tau, (int)t, (int)out, chunk, dyb, ld, part);
    }
    e->launches++;
    if (where == 1) {
        colsum_finish_kernel<<<(unsigned)ceil_div(out, 256), 256, 0, e->stream>>>(part, (int)grid.y, (int)out, db);
        e->launches++;
    }
    NNB_CHECK_LAUNCH("scale_colsum_kernel");
    return NNB_OK;
}

nnb_status launch_dequant_to_bf16(nnb_engine* e, const int8_t* q, const float* s, size_t t, size_t k, __nv_bfloat16* xs)
{
    NNB_REQUIRE(k % 64 == 0 && (((uintptr_t)q | (uintptr_t)xs) & 15) == 0, "dequant_to_bf16: k=%zu must be a multiple of 64, operands 16-byte aligned", k);
    dequant_to_bf16_kernel<<<(unsigned)ceil_div(t * (k / 64), 256), 256, 0, e->stream>>>(q, s, t, (int)k, xs);
    e->launches++;
    NNB_CHECK_LAUNCH("dequant_to_bf16_kernel");
    return NNB_OK;
}

}  // namespace nnb
