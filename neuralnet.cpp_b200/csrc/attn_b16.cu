// attn_b16.cu — causal self-attention of the teacher-forced pass on tensor cores (bf16 operands, f32
// accumulation, online softmax), used when the policy is not in the exact numeric mode.
//   forward   O = softmax(scale * Q K^T) V                         compute_layer_attention.hpp:698-828
//   backward  P = exp(scale*S - lse); dV = P^T dO; dS = P o (dO V^T - D); dQ = scale * dS K; dK = scale * dS^T Q
//             (the reference recomputes W from Q, K and forms R = rowsum(W o P), X = W o (P - R)) :830-988
// (paths under include/neuralnet.cpp/ of the reference).
//
// Operands are bf16 token-major (n*S, H*dk) matrices made once per layer by rope_pack_kernel from the f32
// projections (RoPE applied to q and k on the way); dO is converted by the kernel that forms
// D = rowsum(dO o O).  All kernels stage tiles with cp.async into padded shared memory and read fragments
// with ldmatrix; the forward double-buffers its K/V tiles, the backward kernels keep one tile in flight and run
// two CTAs per SM.  The backward is two
// kernels, one per output owner (key tiles own dK/dV, query tiles own dQ), so no atomics are needed; the
// inverse rotation of dQ and dK happens in their epilogues, where a thread holds both halves of a pair.
// Head dims 64 and 128.
#include "common.cuh"
#include "device_math.cuh"

namespace nnb {
namespace ab {

typedef __nv_bfloat16 bf16;

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
__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// 16-byte asynchronous copy; with ok == false the destination is zero-filled and nothing is read
__device__ __forceinline__ void cp16(void* smem, const void* gmem, bool ok)
{
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    const int n = ok ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(a), "l"(gmem), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// Where the rows of one sequence live (see SeqMap): positions [0, P) at pre_base + r, positions >= P at
// own_base + (r - P).  For the plain layout both pieces are contiguous.
struct RowAddr {
    size_t pre_base, own_base;
    int P;
    __device__ __forceinline__ size_t at(int r) const { return r < P ? pre_base + r : own_base + (r - P); }
};
__device__ __forceinline__ RowAddr row_addr(const SeqMap& m, int b)
{
    RowAddr ra;
    ra.P = m.P;
    ra.pre_base = map_row(m, b, 0);
    ra.own_base = map_row(m, b, m.P);
    return ra;
}

// stage ROWS rows x DK features of a bf16 matrix with d features per row; rows at or beyond S are zero
template <int DK, int LD, int ROWS, int THREADS>
__device__ __forceinline__ void stage(const bf16* __restrict__ src, const RowAddr& ra, int row0, int S, int d, int col0, bf16* dst)
{
    constexpr int CH = DK / 8;  // 16-byte chunks per row
    for (int i = threadIdx.x; i < ROWS * CH; i += THREADS) {
        const int r = i / CH, c = (i % CH) * 8;
        const bool ok = row0 + r < S;
        const int rr = ok ? row0 + r : S - 1;
        cp16(dst + r * LD + c, src + ra.at(rr) * d + col0 + c, ok);
    }
}

// ------------------------------------------------------------------ RoPE + bf16 pack
// q, k, v: (T, d) f32.  out: three (T, d) bf16 planes T*d apart: q and k
// rotated by the row's position (row_pos[row], or row % S without that table) when rope tables are given,
// v converted.  One CTA per row.
__global__ void __launch_bounds__(256)
rope_pack_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                 const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, const int* __restrict__ row_pos, int S,
                 int H, int dk, size_t T, bf16* __restrict__ out)
{
    const size_t row = blockIdx.x;
    const int pos = row_pos ? row_pos[row] : (int)(row % S);
    const int d = H * dk, half = dk / 2;
    // q, k: groups of four consecutive pair indices j (half % 4 == 0)
    const int groups = H * (half / 4);
    for (int i = threadIdx.x; i < 2 * groups; i += 256) {
        const int pl = i / groups, gi = i % groups;
        const int h = gi / (half / 4), j = (gi % (half / 4)) * 4;
        const float* src = (pl == 0 ? q : k) + row * d + (size_t)h * dk;
        bf16* dst = out + (size_t)pl * T * d + row * d + (size_t)h * dk;
        const float4 a = *reinterpret_cast<const float4*>(src + j);
        const float4 b = *reinterpret_cast<const float4*>(src + j + half);
        float4 c = make_float4(1.f, 1.f, 1.f, 1.f), sn = make_float4(0.f, 0.f, 0.f, 0.f);
        if (rope_cos) {
            c = *reinterpret_cast<const float4*>(rope_cos + (size_t)pos * half + j);
            sn = *reinterpret_cast<const float4*>(rope_sin + (size_t)pos * half + j);
        }
        uint2 lo, hi;
        lo.x = pack2(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y);
        lo.y = pack2(a.z * c.z - b.z * sn.z, a.w * c.w - b.w * sn.w);
        hi.x = pack2(b.x * c.x + a.x * sn.x, b.y * c.y + a.y * sn.y);
        hi.y = pack2(b.z * c.z + a.z * sn.z, b.w * c.w + a.w * sn.w);
        *reinterpret_cast<uint2*>(dst + j) = lo;
        *reinterpret_cast<uint2*>(dst + j + half) = hi;
    }
    const float* vs = v + row * d;
    bf16* vd = out + 2 * T * d + row * d;
    for (int i = threadIdx.x; i < d / 4; i += 256) {
        const float4 a = reinterpret_cast<const float4*>(vs)[i];
        uint2 o;
        o.x = pack2(a.x, a.y);
        o.y = pack2(a.z, a.w);
        reinterpret_cast<uint2*>(vd)[i] = o;
    }
}

// token-major bf16 keys / values (n*S, H*dk) -> decode cache layout (n, H / kv_rep, alloc, dk); one CTA per row.
// kv_rep > 1 (grouped-query attention): the rows hold every KV head kv_rep times, the cache one copy (the first).
__global__ void __launch_bounds__(256)
kv_to_cache_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v, int S, int H, int dk, int alloc, int kv_rep,
                   bf16* __restrict__ kc, bf16* __restrict__ vc)
{
    const size_t row = blockIdx.x;
    const int b = (int)(row / S), pos = (int)(row % S);
    const int d = H * dk, Hkv = H / kv_rep;
    for (int c = threadIdx.x * 8; c < Hkv * dk; c += 256 * 8) {
        const int hk = c / dk, cc = c % dk;
        const size_t dst = (((size_t)b * Hkv + hk) * alloc + pos) * dk + cc;
        const size_t src = row * d + (size_t)hk * kv_rep * dk + cc;
        *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(k + src);
        *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(v + src);
    }
}

// ------------------------------------------------------------------ forward
// grid (n*H, ceil(S/128)), 128 threads: warp w owns query rows 32w..32w+31 of the tile (two m16 blocks);
// key tiles of 64 rows, double-buffered.  Late query tiles (the long ones under the causal mask) are
// scheduled first.
template <int DK>
__global__ void __launch_bounds__(128)
attn_fwd_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v, const SeqMap map,
                size_t rows, int H, float scale, float* __restrict__ out, float* __restrict__ lse)
{
    const int S = map.S;
    constexpr int LD = DK + 8;
    extern __shared__ __align__(16) unsigned char smraw[];
    bf16* Qs = reinterpret_cast<bf16*>(smraw);
    bf16* Ks = Qs + 128 * LD;       // [2][64*LD]
    bf16* Vs = Ks + 2 * 64 * LD;    // [2][64*LD]
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int d = H * DK;
    const int q0 = (gridDim.y - 1 - blockIdx.y) * 128;
    // in a grouped batch the shared prefix rows are computed by the group's first member only
    const int first_row = (map.group > 1 && b % map.group != 0) ? map.P : 0;
    if (q0 + 128 <= first_row) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const RowAddr base = row_addr(map, b);
    const int col0 = h * DK;
    const float sl2 = scale * 1.4426950408889634f;

    const int n_tiles = min(q0 + 127, S - 1) / 64 + 1;
    stage<DK, LD, 128, 128>(q, base, q0, S, d, col0, Qs);
    stage<DK, LD, 64, 128>(k, base, 0, S, d, col0, Ks);
    stage<DK, LD, 64, 128>(v, base, 0, S, d, col0, Vs);
    cp_commit();

    float o[2][DK / 8][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int i = 0; i < DK / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) o[mt][i][j] = 0.0f;
    float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY}, l[4] = {0.f, 0.f, 0.f, 0.f};  // index mt*2 + hh
    const int wrow0 = q0 + warp * 32;

    for (int jt = 0; jt < n_tiles; ++jt) {
        const int j0 = jt * 64;
        if (jt + 1 < n_tiles) {
            const int nb = (jt + 1) & 1;
            stage<DK, LD, 64, 128>(k, base, j0 + 64, S, d, col0, Ks + nb * 64 * LD);
            stage<DK, LD, 64, 128>(v, base, j0 + 64, S, d, col0, Vs + nb * 64 * LD);
            cp_commit();
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        if (j0 <= wrow0 + 31) {
            const bf16* Kb = Ks + (jt & 1) * 64 * LD;
            const bf16* Vb = Vs + (jt & 1) * 64 * LD;
            float s[2][8][4];
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) s[mt][i][j] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < DK / 16; ++ks) {
                uint32_t aq[2][4];
#pragma unroll
                for (int mt = 0; mt < 2; ++mt)
                    ldsm(aq[mt], Qs + (warp * 32 + mt * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + ks * 16 + 8 * (lane >> 4));
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t bk[4];
                    ldsm(bk, Kb + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * LD + ks * 16 + 8 * ((lane >> 3) & 1));
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        mma16816(s[mt][np * 2], aq[mt], bk[0], bk[1]);
                        mma16816(s[mt][np * 2 + 1], aq[mt], bk[2], bk[3]);
                    }
                }
            }
            const bool need_mask = (j0 + 63 > wrow0) || (j0 + 64 > S);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        if (need_mask) {
                            const int key = j0 + nt * 8 + 2 * t4 + (c & 1);
                            const int row = wrow0 + mt * 16 + g + 8 * (c >> 1);
                            if (key > row || key >= S) s[mt][nt][c] = -INFINITY;
                        }
                        mx[c >> 1] = fmaxf(mx[c >> 1], s[mt][nt][c]);
                    }
                }
                float corr[2], msc[2];
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                    const float mnew = fmaxf(m[mt * 2 + r], mx[r]);
                    corr[r] = (mnew == -INFINITY) ? 1.0f : ex2((m[mt * 2 + r] - mnew) * sl2);
                    m[mt * 2 + r] = mnew;
                    msc[r] = (mnew == -INFINITY) ? 0.0f : mnew * sl2;
                    l[mt * 2 + r] *= corr[r];
                }
#pragma unroll
                for (int i = 0; i < DK / 8; ++i) {
                    o[mt][i][0] *= corr[0]; o[mt][i][1] *= corr[0];
                    o[mt][i][2] *= corr[1]; o[mt][i][3] *= corr[1];
                }
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float p = ex2(s[mt][nt][c] * sl2 - msc[c >> 1]);
                        s[mt][nt][c] = p;
                        l[mt * 2 + (c >> 1)] += p;
                    }
                }
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                uint32_t pa[2][4];
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    pa[mt][0] = pack2(s[mt][2 * kk][0], s[mt][2 * kk][1]);
                    pa[mt][1] = pack2(s[mt][2 * kk][2], s[mt][2 * kk][3]);
                    pa[mt][2] = pack2(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
                    pa[mt][3] = pack2(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
                }
#pragma unroll
                for (int np = 0; np < DK / 16; ++np) {
                    uint32_t bv[4];
                    ldsm_t(bv, Vb + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + np * 16 + 8 * (lane >> 4));
#pragma unroll
                    for (int mt = 0; mt < 2; ++mt) {
                        mma16816(o[mt][np * 2], pa[mt], bv[0], bv[1]);
                        mma16816(o[mt][np * 2 + 1], pa[mt], bv[2], bv[3]);
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
        const int row_a = wrow0 + mt * 16 + g, row_b = row_a + 8;
        const bool ok_a = row_a < S && row_a >= first_row, ok_b = row_b < S && row_b >= first_row;
        const float inv_a = 1.0f / l[mt * 2], inv_b = 1.0f / l[mt * 2 + 1];
#pragma unroll
        for (int i = 0; i < DK / 8; ++i) {
            const int c = col0 + i * 8 + 2 * t4;
            if (ok_a) *reinterpret_cast<float2*>(out + base.at(row_a) * d + c) = make_float2(o[mt][i][0] * inv_a, o[mt][i][1] * inv_a);
            if (ok_b) *reinterpret_cast<float2*>(out + base.at(row_b) * d + c) = make_float2(o[mt][i][2] * inv_b, o[mt][i][3] * inv_b);
        }
        if (t4 == 0) {
            if (ok_a) lse[map_vec(map, b, h, row_a, H, rows)] = m[mt * 2] * scale + logf(l[mt * 2]);
            if (ok_b) lse[map_vec(map, b, h, row_b, H, rows)] = m[mt * 2 + 1] * scale + logf(l[mt * 2 + 1]);
        }
    }
}

// ------------------------------------------------------------------ backward
// delta[b,h,i] = sum_c dO[row,h,c] * O[row,h,c], and dO as bf16.  One warp per (row, head), 4 features per lane.
__global__ void __launch_bounds__(256)
delta_pack_kernel(const float* __restrict__ dout, const float* __restrict__ out, int S, int H, int dk, size_t n_rows,
                  int grouped, float* __restrict__ delta, bf16* __restrict__ dob)
{
    const size_t w = (size_t)blockIdx.x * 8 + threadIdx.x / 32;  // (row, h)
    if (w >= n_rows * H) return;
    const size_t row = w / H;
    const int h = (int)(w % H), lane = threadIdx.x & 31;
    const size_t off = row * (size_t)(H * dk) + (size_t)h * dk;
    float a = 0.0f;
    for (int c = lane * 4; c < dk; c += 128) {
        const float4 g = *reinterpret_cast<const float4*>(dout + off + c);
        const float4 o = *reinterpret_cast<const float4*>(out + off + c);
        a = fmaf(g.x, o.x, fmaf(g.y, o.y, fmaf(g.z, o.z, fmaf(g.w, o.w, a))));
        uint2 pk;
        pk.x = pack2(g.x, g.y);
        pk.y = pack2(g.z, g.w);
        *reinterpret_cast<uint2*>(dob + off + c) = pk;
    }
    a = warp_sum(a);
    const size_t b = row / S, i = row % S;
    if (lane == 0) delta[grouped ? (size_t)h * n_rows + row : (b * H + h) * S + i] = a;
}

// S = Q K^T and dP = dO V^T for a 64 x 64 (query, key) block, then P and dS as bf16 into shared memory.
// 8 warps: wr = warp & 3 owns query rows 16wr.., wc = warp >> 2 owns keys 32wc..32wc+31.
template <int DK, bool WANT_P>
__device__ __forceinline__ void score_block(const bf16* Qs, const bf16* Gs, const bf16* Ks, const bf16* Vs, const float* Ls,
                                            const float* Dl, int i0, int k0, int S, float scale, bf16* Ps, bf16* Ds)
{
    constexpr int LD = DK + 8, LP = 64 + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int wr = warp & 3, wc = warp >> 2;
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
            const int rl = wr * 16 + g + 8 * hh;  // row inside the query tile
            const int row = i0 + rl;
            const float lr = Ls[rl], dr = Dl[rl];
            float pv[2], dsv[2];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int key = k0 + wc * 32 + nt * 8 + 2 * t4 + c;
                const bool ok = key <= row && row < S && key < S;
                const float p = ok ? __expf(s[nt][hh * 2 + c] * scale - lr) : 0.0f;
                pv[c] = p;
                dsv[c] = p * (dp[nt][hh * 2 + c] - dr);
            }
            const int cidx = wc * 32 + nt * 8 + 2 * t4;
            if (WANT_P) *reinterpret_cast<uint32_t*>(Ps + rl * LP + cidx) = pack2(pv[0], pv[1]);
            *reinterpret_cast<uint32_t*>(Ds + rl * LP + cidx) = pack2(dsv[0], dsv[1]);
        }
    }
}

// feature offset of the np-th 16-wide chunk owned by column group wc: the first half of a thread's chunks
// lies in [0, DK/2), the second half at the same offsets in [DK/2, DK), so both members of a RoPE pair
// (j, j + DK/2) are accumulated by the same thread
template <int DK>
__device__ __forceinline__ int chunk_base(int wc, int np)
{
    constexpr int NCH = DK / 32;  // chunks per thread (half of the head, 16 features each)
    return (np < NCH / 2 ? 0 : DK / 2) + wc * (DK / 4) + (np % (NCH / 2)) * 16;
}

// store (and optionally un-rotate) a 16-row x DK/2-feature accumulator: acc[np*2 + e][c] is row g (+8 for
// c >= 2), feature chunk_base(wc, np) + e*8 + 2*t4 + (c & 1)
template <int DK>
__device__ __forceinline__ void store_rows(float (&acc)[DK / 16][4], float mul, const float* rope_cos, const float* rope_sin,
                                           int row_a, int first_row, int S, const RowAddr& base, int d, int col0, int wc,
                                           float* dst)
{
    constexpr int NCH = DK / 32, half = DK / 2;
    const int lane = threadIdx.x & 31, t4 = lane & 3;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int row = row_a + 8 * hh;
        if (row >= S || row < first_row) continue;
        float* drow = dst + base.at(row) * d + col0;
#pragma unroll
        for (int np = 0; np < NCH / 2; ++np) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = wc * (DK / 4) + np * 16 + e * 8 + 2 * t4;  // pair index in [0, half)
                float lo[2] = {acc[np * 2 + e][hh * 2] * mul, acc[np * 2 + e][hh * 2 + 1] * mul};
                float hi[2] = {acc[(np + NCH / 2) * 2 + e][hh * 2] * mul, acc[(np + NCH / 2) * 2 + e][hh * 2 + 1] * mul};
                if (rope_cos) {
                    const float2 c = *reinterpret_cast<const float2*>(rope_cos + (size_t)row * half + j);
                    const float2 sn = *reinterpret_cast<const float2*>(rope_sin + (size_t)row * half + j);
                    const float a0 = lo[0], a1 = lo[1], b0 = hi[0], b1 = hi[1];
                    lo[0] = a0 * c.x + b0 * sn.x; lo[1] = a1 * c.y + b1 * sn.y;
                    hi[0] = b0 * c.x - a0 * sn.x; hi[1] = b1 * c.y - a1 * sn.y;
                }
                *reinterpret_cast<float2*>(drow + j) = make_float2(lo[0], lo[1]);
                *reinterpret_cast<float2*>(drow + j + half) = make_float2(hi[0], hi[1]);
            }
        }
    }
}

// dK, dV: grid (n*H, ceil(S/64)) over key tiles (late tiles, the short ones, last), 256 threads.  The key
// tile's K and V stay in shared memory; Q and dO tiles of 64 queries stream through a double buffer.
template <int DK, int NBUF>
__global__ void __launch_bounds__(256, NBUF == 1 ? 2 : 1)
attn_bwd_dkv_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                    const bf16* __restrict__ dob, const float* __restrict__ lse, const float* __restrict__ delta,
                    const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, const SeqMap map, size_t rows, int H,
                    float scale, float* __restrict__ dk, float* __restrict__ dv, float* __restrict__ part)
{
    const int S = map.S;
    constexpr int LD = DK + 8, LP = 64 + 8, NCH = DK / 32;
    extern __shared__ __align__(16) unsigned char smraw[];
    bf16* Ks = reinterpret_cast<bf16*>(smraw);
    bf16* Vs = Ks + 64 * LD;
    bf16* Qs = Vs + 64 * LD;           // [NBUF][64*LD]
    bf16* Gs = Qs + NBUF * 64 * LD;    // [NBUF][64*LD]  dO
    bf16* Ps = Gs + NBUF * 64 * LD;    // [q][key]
    bf16* Ds = Ps + 64 * LP;           // dS [q][key]
    float* Ls = reinterpret_cast<float*>(Ds + 64 * LP);  // [NBUF][64]
    float* Dl = Ls + NBUF * 64;                          // [NBUF][64]
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int d = H * DK;
    const int k0 = blockIdx.y * 64;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2;
    const int wr = warp & 3, wc = warp >> 2;
    const RowAddr base = row_addr(map, b);
    const int col0 = h * DK;
    // Grouped batch, key tile inside the shared prefix (P is a multiple of 64 then): every member adds the
    // share of its own queries (the first member also that of the prefix queries) into its slice of `part`
    // ((2, n_seq, P, d): dK then dV), which prefix_sum_kernel adds up afterwards.
    const bool prefix_tile = map.group > 1 && k0 < map.P;
    const int q_start = (prefix_tile && b % map.group != 0) ? map.P : k0;

    auto load_q = [&](int i0, int buf) {
        stage<DK, LD, 64, 256>(q, base, i0, S, d, col0, Qs + buf * 64 * LD);
        stage<DK, LD, 64, 256>(dob, base, i0, S, d, col0, Gs + buf * 64 * LD);
        if (threadIdx.x < 64) {
            const int qi = i0 + threadIdx.x;
            Ls[buf * 64 + threadIdx.x] = qi < S ? lse[map_vec(map, b, h, qi, H, rows)] : 0.0f;
            Dl[buf * 64 + threadIdx.x] = qi < S ? delta[map_vec(map, b, h, qi, H, rows)] : 0.0f;
        }
    };
    stage<DK, LD, 64, 256>(k, base, k0, S, d, col0, Ks);
    stage<DK, LD, 64, 256>(v, base, k0, S, d, col0, Vs);
    load_q(q_start, 0);
    cp_commit();

    float adk[DK / 16][4], adv[DK / 16][4];
#pragma unroll
    for (int i = 0; i < DK / 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) adk[i][j] = adv[i][j] = 0.0f;

    // NBUF == 2: the next Q / dO tile streams in while this one is used, one CTA per SM.  NBUF == 1: one tile in
    // flight per CTA, two CTAs per SM, each covering the other's load.
    const int n_it = (S - q_start + 63) / 64;
    for (int it = 0; it < n_it; ++it) {
        const int i0 = q_start + it * 64, buf = NBUF == 2 ? (it & 1) : 0;
        if (NBUF == 2 && it + 1 < n_it) {
            load_q(i0 + 64, buf ^ 1);
            cp_commit();
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        const bf16* Qb = Qs + buf * 64 * LD;
        const bf16* Gb = Gs + buf * 64 * LD;
        score_block<DK, true>(Qb, Gb, Ks, Vs, Ls + buf * 64, Dl + buf * 64, i0, k0, S, scale, Ps, Ds);
        __syncthreads();
        // dV[key][f] += P^T dO, dK[key][f] += dS^T Q; key rows 16wr.., feature chunks of column group wc
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {  // contraction over the 64 queries of the tile
            uint32_t ap[4], ad[4];
            const int qr = ks * 16 + (lane & 7) + 8 * (lane >> 4), kc = wr * 16 + 8 * ((lane >> 3) & 1);
            ldsm_t(ap, Ps + qr * LP + kc);
            ldsm_t(ad, Ds + qr * LP + kc);
#pragma unroll
            for (int np = 0; np < NCH; ++np) {
                uint32_t bg[4], bq[4];
                const int rr = ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), cc = chunk_base<DK>(wc, np) + 8 * (lane >> 4);
                ldsm_t(bg, Gb + rr * LD + cc);
                ldsm_t(bq, Qb + rr * LD + cc);
                mma16816(adv[np * 2], ap, bg[0], bg[1]);
                mma16816(adv[np * 2 + 1], ap, bg[2], bg[3]);
                mma16816(adk[np * 2], ad, bq[0], bq[1]);
                mma16816(adk[np * 2 + 1], ad, bq[2], bq[3]);
            }
        }
        __syncthreads();
        if (NBUF == 1 && it + 1 < n_it) {
            load_q(i0 + 64, 0);
            cp_commit();
        }
    }
    const int row_a = k0 + wr * 16 + g;
    if (prefix_tile) {
        RowAddr pa;
        pa.P = map.P;
        pa.pre_base = (size_t)b * map.P;
        pa.own_base = 0;
        const size_t plane = (size_t)gridDim.x / H * map.P * d;  // n_seq * P * d
        store_rows<DK>(adk, scale, rope_cos, rope_sin, row_a, 0, S, pa, d, col0, wc, part);
        store_rows<DK>(adv, 1.0f, nullptr, nullptr, row_a, 0, S, pa, d, col0, wc, part + plane);
    } else {
        store_rows<DK>(adk, scale, rope_cos, rope_sin, row_a, 0, S, base, d, col0, wc, dk);
        store_rows<DK>(adv, 1.0f, nullptr, nullptr, row_a, 0, S, base, d, col0, wc, dv);
    }
}

// prefix rows of a grouped batch: dst[row of (group, r)] = sum over the group's members of part[member][r]
__global__ void prefix_sum_kernel(const float* __restrict__ part, const SeqMap map, int d, float* __restrict__ dst)
{
    const int grp = blockIdx.x / map.P, r = blockIdx.x % map.P;
    const size_t drow = map_row(map, grp * map.group, r);
    for (int c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int mm = 0; mm < map.group; ++mm) {
            const float4 v = *reinterpret_cast<const float4*>(part + ((size_t)(grp * map.group + mm) * map.P + r) * d + c);
            a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
        }
        *reinterpret_cast<float4*>(dst + drow * d + c) = a;
    }
}

// dQ: grid (n*H, ceil(S/64)) over query tiles (late tiles first), 256 threads.  Q and dO of the tile stay
// in shared memory; K and V tiles of 64 keys stream through a double buffer.
template <int DK, int NBUF>
__global__ void __launch_bounds__(256, NBUF == 1 ? 2 : 1)
attn_bwd_dq_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                   const bf16* __restrict__ dob, const float* __restrict__ lse, const float* __restrict__ delta,
                   const float* __restrict__ rope_cos, const float* __restrict__ rope_sin, const SeqMap map, size_t rows, int H,
                   float scale, float* __restrict__ dq)
{
    const int S = map.S;
    constexpr int LD = DK + 8, LP = 64 + 8, NCH = DK / 32;
    extern __shared__ __align__(16) unsigned char smraw[];
    bf16* Qs = reinterpret_cast<bf16*>(smraw);
    bf16* Gs = Qs + 64 * LD;
    bf16* Ks = Gs + 64 * LD;           // [NBUF][64*LD]
    bf16* Vs = Ks + NBUF * 64 * LD;    // [NBUF][64*LD]
    bf16* Ds = Vs + NBUF * 64 * LD;    // dS [q][key]
    float* Ls = reinterpret_cast<float*>(Ds + 64 * LP);
    float* Dl = Ls + 64;
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int d = H * DK;
    const int i0 = (gridDim.y - 1 - blockIdx.y) * 64;
    const int first_row = (map.group > 1 && b % map.group != 0) ? map.P : 0;  // prefix rows belong to the first member
    if (i0 + 64 <= first_row) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2;
    const int wr = warp & 3, wc = warp >> 2;
    const RowAddr base = row_addr(map, b);
    const int col0 = h * DK;

    stage<DK, LD, 64, 256>(q, base, i0, S, d, col0, Qs);
    stage<DK, LD, 64, 256>(dob, base, i0, S, d, col0, Gs);
    stage<DK, LD, 64, 256>(k, base, 0, S, d, col0, Ks);
    stage<DK, LD, 64, 256>(v, base, 0, S, d, col0, Vs);
    cp_commit();
    if (threadIdx.x < 64) {
        const int qi = i0 + threadIdx.x;
        Ls[threadIdx.x] = qi < S ? lse[map_vec(map, b, h, qi, H, rows)] : 0.0f;
        Dl[threadIdx.x] = qi < S ? delta[map_vec(map, b, h, qi, H, rows)] : 0.0f;
    }
    float acc[DK / 16][4];
#pragma unroll
    for (int i = 0; i < DK / 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    const int n_it = min(i0 + 63, S - 1) / 64 + 1;
    for (int it = 0; it < n_it; ++it) {
        const int k0 = it * 64, buf = NBUF == 2 ? (it & 1) : 0;
        if (NBUF == 2 && it + 1 < n_it) {
            stage<DK, LD, 64, 256>(k, base, k0 + 64, S, d, col0, Ks + (buf ^ 1) * 64 * LD);
            stage<DK, LD, 64, 256>(v, base, k0 + 64, S, d, col0, Vs + (buf ^ 1) * 64 * LD);
            cp_commit();
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        const bf16* Kb = Ks + buf * 64 * LD;
        const bf16* Vb = Vs + buf * 64 * LD;
        score_block<DK, false>(Qs, Gs, Kb, Vb, Ls, Dl, i0, k0, S, scale, nullptr, Ds);
        __syncthreads();
        // dQ[q][f] += dS K; query rows 16wr.., feature chunks of column group wc
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {  // contraction over the 64 keys
            uint32_t ads[4];
            const int r = wr * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = ks * 16 + 8 * (lane >> 4);
            ldsm(ads, Ds + r * LP + c);
#pragma unroll
            for (int np = 0; np < NCH; ++np) {
                uint32_t bk[4];
                const int rr = ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), cc = chunk_base<DK>(wc, np) + 8 * (lane >> 4);
                ldsm_t(bk, Kb + rr * LD + cc);
                mma16816(acc[np * 2], ads, bk[0], bk[1]);
                mma16816(acc[np * 2 + 1], ads, bk[2], bk[3]);
            }
        }
        __syncthreads();
        if (NBUF == 1 && it + 1 < n_it) {
            stage<DK, LD, 64, 256>(k, base, k0 + 64, S, d, col0, Ks);
            stage<DK, LD, 64, 256>(v, base, k0 + 64, S, d, col0, Vs);
            cp_commit();
        }
    }
    store_rows<DK>(acc, scale, rope_cos, rope_sin, i0 + wr * 16 + g, first_row, S, base, d, col0, wc, dq);
}

template <typename K>
static nnb_status set_smem(K kern, size_t smem)
{
    NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    return NNB_OK;
}

}  // namespace ab

bool attn_b16_supported(size_t dk, size_t d) { return (dk == 64 || dk == 128) && d % 8 == 0; }

nnb_status launch_rope_pack_b16(nnb_engine* e, const float* q, const float* k, const float* v, const float* rope_cos,
                                const float* rope_sin, size_t T, size_t S, size_t H, size_t dk, __nv_bfloat16* out,
                                const int* row_pos)
{
    NNB_REQUIRE(dk % 8 == 0, "rope_pack: head dim %zu must be a multiple of 8", dk);
    NNB_REQUIRE((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15) == 0, "rope_pack: operands must be 16-byte aligned");
    ab::rope_pack_kernel<<<(unsigned)T, 256, 0, e->stream>>>(q, k, v, rope_cos, rope_sin, row_pos, (int)S, (int)H, (int)dk, T, out);
    e->launches++;
    NNB_CHECK_LAUNCH("rope_pack_kernel");
    return NNB_OK;
}

nnb_status launch_kv_to_cache(nnb_engine* e, const __nv_bfloat16* k, const __nv_bfloat16* v, size_t n_seq, size_t S, size_t H,
                              size_t dk, __nv_bfloat16* kc, __nv_bfloat16* vc, size_t alloc, size_t kv_rep)
{
    NNB_REQUIRE(dk % 8 == 0 && S <= alloc && kv_rep >= 1 && H % kv_rep == 0, "kv_to_cache: bad shape");
    ab::kv_to_cache_kernel<<<(unsigned)(n_seq * S), 256, 0, e->stream>>>(k, v, (int)S, (int)H, (int)dk, (int)alloc, (int)kv_rep, kc, vc);
    e->launches++;
    NNB_CHECK_LAUNCH("kv_to_cache_kernel");
    return NNB_OK;
}

static nnb_status check_map(const SeqMap* map, size_t n_seq, size_t S, SeqMap* out)
{
    if (!map) {
        *out = SeqMap{(int)S, 0, (int)S, 1};
        return NNB_OK;
    }
    *out = *map;
    NNB_REQUIRE((size_t)map->S == S && map->P + map->G == map->S && map->group >= 1, "attention: inconsistent sequence map");
    if (map->group > 1)
        NNB_REQUIRE(map->P % 64 == 0 && n_seq % map->group == 0,
                    "attention: a grouped batch needs a prompt length that is a multiple of 64 and whole groups");
    return NNB_OK;
}

nnb_status launch_attn_fwd_b16(nnb_engine* e, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                               size_t n_seq, size_t S, size_t H, size_t dk, float* out, float* lse, const SeqMap* map)
{
    using namespace ab;
    SeqMap m;
    NNB_TRY(check_map(map, n_seq, S, &m));
    const size_t rows = map_rows_total(m, n_seq);
    const float scale = 1.0f / sqrtf((float)dk);
    dim3 grid((unsigned)(n_seq * H), (unsigned)ceil_div(S, 128));
    const size_t smem = (128 + 4 * 64) * (dk + 8) * 2;
    static bool cfg_dev[64] = {}; bool& cfg = cfg_dev[e->device & 63];  // the attribute is per device
    if (!cfg) {
        NNB_TRY(set_smem(attn_fwd_kernel<128>, (128 + 4 * 64) * 136 * 2));
        NNB_TRY(set_smem(attn_fwd_kernel<64>, (128 + 4 * 64) * 72 * 2));
        cfg = true;
    }
    if (dk == 128) attn_fwd_kernel<128><<<grid, 128, smem, e->stream>>>(q, k, v, m, rows, (int)H, scale, out, lse);
    else attn_fwd_kernel<64><<<grid, 128, smem, e->stream>>>(q, k, v, m, rows, (int)H, scale, out, lse);
    e->launches++;
    NNB_CHECK_LAUNCH("attn_fwd_kernel (bf16)");
    return NNB_OK;
}

// dob: bf16 scratch (rows, H*dk); delta: f32 scratch, one value per (row, head).  With rope tables the
// gradients of q and k are returned with respect to the un-rotated projections.
nnb_status launch_attn_bwd_b16(nnb_engine* e, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                               const float* out, const float* dout, const float* lse, float* delta, __nv_bfloat16* dob,
                               const float* rope_cos, const float* rope_sin, size_t n_seq, size_t S, size_t H, size_t dk,
                               float* dq, float* dkk, float* dvv, const SeqMap* map, float* part)
{
    using namespace ab;
    SeqMap m;
    NNB_TRY(check_map(map, n_seq, S, &m));
    const bool grouped = m.group > 1;
    NNB_REQUIRE(!grouped || part, "attention backward: a grouped batch needs the prefix scratch");
    const size_t rows = map_rows_total(m, n_seq);
    const float scale = 1.0f / sqrtf((float)dk);
    delta_pack_kernel<<<(unsigned)ceil_div(rows * H, 8), 256, 0, e->stream>>>(dout, out, (int)S, (int)H, (int)dk, rows,
                                                                             grouped ? 1 : 0, delta, dob);
    dim3 grid((unsigned)(n_seq * H), (unsigned)ceil_div(S, 64));
    // One buffer per streamed tile and two CTAs per SM, each covering the other's loads: measured 776 us against
    // 1051 us for double-buffered tiles with one CTA per SM (16 x 640 x 16 heads x 128, pack and delta included).
    constexpr int NBUF = 1;
    auto smem_kv_of = [](size_t dkv) { return (2 + 2 * NBUF) * 64 * (dkv + 8) * 2 + 2 * 64 * 72 * 2 + 2 * NBUF * 64 * 4; };
    auto smem_q_of = [](size_t dkv) { return (2 + 2 * NBUF) * 64 * (dkv + 8) * 2 + 64 * 72 * 2 + 128 * 4; };
    const size_t smem_kv = smem_kv_of(dk), smem_q = smem_q_of(dk);
    static bool cfg_dev[64] = {}; bool& cfg = cfg_dev[e->device & 63];  // the attribute is per device
    if (!cfg) {
        NNB_TRY(set_smem(attn_bwd_dkv_kernel<128, NBUF>, smem_kv_of(128)));
        NNB_TRY(set_smem(attn_bwd_dkv_kernel<64, NBUF>, smem_kv_of(64)));
        NNB_TRY(set_smem(attn_bwd_dq_kernel<128, NBUF>, smem_q_of(128)));
        NNB_TRY(set_smem(attn_bwd_dq_kernel<64, NBUF>, smem_q_of(64)));
        cfg = true;
    }
    if (dk == 128) {
        attn_bwd_dkv_kernel<128, NBUF><<<grid, 256, smem_kv, e->stream>>>(q, k, v, dob, lse, delta, rope_cos, rope_sin, m, rows, (int)H,
                                                                          scale, dkk, dvv, part);
        attn_bwd_dq_kernel<128, NBUF><<<grid, 256, smem_q, e->stream>>>(q, k, v, dob, lse, delta, rope_cos, rope_sin, m, rows, (int)H,
                                                                        scale, dq);
    } else {
        attn_bwd_dkv_kernel<64, NBUF><<<grid, 256, smem_kv, e->stream>>>(q, k, v, dob, lse, delta, rope_cos, rope_sin, m, rows, (int)H,
                                                                         scale, dkk, dvv, part);
        attn_bwd_dq_kernel<64, NBUF><<<grid, 256, smem_q, e->stream>>>(q, k, v, dob, lse, delta, rope_cos, rope_sin, m, rows, (int)H,
                                                                       scale, dq);
    }
    e->launches += 3;
    if (grouped) {
        const size_t d = H * dk, plane = n_seq * (size_t)m.P * d;
        const unsigned blocks = (unsigned)((n_seq / m.group) * m.P);
        prefix_sum_kernel<<<blocks, 256, 0, e->stream>>>(part, m, (int)d, dkk);
        prefix_sum_kernel<<<blocks, 256, 0, e->stream>>>(part + plane, m, (int)d, dvv);
        e->launches += 2;
    }
    NNB_CHECK_LAUNCH("attention backward kernels (bf16)");
    return NNB_OK;
}

}  // namespace nnb
