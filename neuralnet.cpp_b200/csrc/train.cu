// train.cu — kernels of the teacher-forced forward and the backward pass of the ternary GPT
// policy (token-major, T = sequences x positions):
//   embedding gather / scatter-add          compute_layer_gpt.hpp:475-489, 620-636
//   RoPE over whole sequences and its inverse   compute_position_encoding.hpp:126-145
//   causal attention, online softmax forward    compute_layer_attention.hpp:698-828
//   attention backward (recompute P from lse)   compute_layer_attention.hpp:830-988
//   RMSNorm backward                            compute_layer_mlp.hpp:716-746
//   QuickGELU / SwiGLU backward                 compute_layer_mlp.hpp:254-270, 332-369
// (paths are under include/neuralnet.cpp/ of the reference).
#include <algorithm>

#include "common.cuh"
#include "device_math.cuh"

namespace nnb {

// ------------------------------------------------------------- embedding
__global__ void embed_fwd_kernel(const float* __restrict__ tok_emb, const float* __restrict__ pos_emb,
                                 const int32_t* __restrict__ tokens, int S, int d, int vocab, float* __restrict__ x)
{
    const size_t row = blockIdx.x;  // b*S + t
    const int t = (int)(row % S);
    int tok = tokens[row];
    tok = min(max(tok, 0), vocab - 1);
    const float* e = tok_emb + (size_t)tok * d;
    const float* p = pos_emb ? pos_emb + (size_t)t * d : nullptr;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = e[i];
        if (p) v = __fadd_rn(v, p[i]);
        x[row * d + i] = v;
    }
}

__global__ void embed_bwd_kernel(const float* __restrict__ g, const int32_t* __restrict__ tokens, int S, int d,
                                 int vocab, float* __restrict__ g_tok, float* __restrict__ g_pos)
{
    const size_t row = blockIdx.x;
    const int t = (int)(row % S);
    int tok = tokens[row];
    tok = min(max(tok, 0), vocab - 1);
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = g[row * d + i];
        atomicAdd(g_tok + (size_t)tok * d + i, v);
        if (g_pos) atomicAdd(g_pos + (size_t)t * d + i, v);
    }
}

// The same two kernels for an explicit row table (token and position of every row), which is how the
// teacher-forced pass lays out its micro-batch (see SeqMap): one thread per (sequence, position) fills the table.
__global__ void build_rows_kernel(const int32_t* __restrict__ tokens, const SeqMap map, size_t n, int32_t* __restrict__ row_tok,
                                  int32_t* __restrict__ row_pos)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int b = (int)(idx / map.S), r = (int)(idx % map.S);
    if (map.group > 1 && r < map.P && b % map.group != 0) return;  // the prompt rows belong to the first member
    const size_t row = map_row(map, b, r);
    row_tok[row] = tokens[idx];
    row_pos[row] = r;
}

__global__ void embed_rows_fwd_kernel(const float* __restrict__ tok_emb, const float* __restrict__ pos_emb,
                                      const int32_t* __restrict__ row_tok, const int32_t* __restrict__ row_pos, int d, int vocab,
                                      float* __restrict__ x)
{
    const size_t row = blockIdx.x;
    const int tok = min(max(row_tok[row], 0), vocab - 1);
    const float* e = tok_emb + (size_t)tok * d;
    const float* p = pos_emb ? pos_emb + (size_t)row_pos[row] * d : nullptr;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = e[i];
        if (p) v = __fadd_rn(v, p[i]);
        x[row * d + i] = v;
    }
}

__global__ void embed_rows_bwd_kernel(const float* __restrict__ g, const int32_t* __restrict__ row_tok,
                                      const int32_t* __restrict__ row_pos, int d, int vocab, float* __restrict__ g_tok,
                                      float* __restrict__ g_pos)
{
    const size_t row = blockIdx.x;
    const int tok = min(max(row_tok[row], 0), vocab - 1);
    const int t = row_pos[row];
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = g[row * d + i];
        atomicAdd(g_tok + (size_t)tok * d + i, v);
        if (g_pos) atomicAdd(g_pos + (size_t)t * d + i, v);
    }
}

// ------------------------------------------------------------------ RoPE
// In place on x (rows, d) viewed as heads of dk; position of a row = row % S.
// sign = +1 forward, -1 backward (the rotation is orthogonal: inverse = opposite angle).
__global__ void rope_kernel(float* __restrict__ x, const float* __restrict__ rope_cos,
                            const float* __restrict__ rope_sin, int S, int H, int dk, float sign)
{
    const size_t row = blockIdx.x;
    const int pos = (int)(row % S);
    const int half = dk / 2;
    float* xr = x + row * (size_t)(H * dk);
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
        const int h = i / half, j = i % half;
        const float c = rope_cos[(size_t)pos * half + j], sn = __fmul_rn(sign, rope_sin[(size_t)pos * half + j]);
        float* v = xr + (size_t)h * dk;
        const float a = v[j], b = v[j + half];
        v[j] = __fadd_rn(__fmul_rn(a, c), __fmul_rn(-b, sn));
        v[j + half] = __fadd_rn(__fmul_rn(b, c), __fmul_rn(a, sn));
    }
}

// ---------------------------------------------------- causal attention, forward
// q, k, v: (n*S, d) token-major (the three slabs of the qkv buffer), post-RoPE.
// One warp per query.  Keys are processed in tiles of 32 held in shared memory: lane j scores
// key j, then the lanes switch to owning output features for the P.V update (online softmax).
constexpr int ATT_WARPS = 8;
// EXACT: scores, softmax sums and the P.V accumulation in f64 (the value then rounds once to
// f32, independent of the tile order), so that the int8 quantisation that follows sees the same
// activations as the high-precision restatement.
template <bool EXACT>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_fwd_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v, int S,
                int H, int dk, float scale, float* __restrict__ out, float* __restrict__ lse)
{
    typedef typename AccT<EXACT>::type acc_t;
    extern __shared__ float sm[];
    const int dkp = dk + 1;
    float* Ks = sm;                       // 32 x dkp
    float* Vs = Ks + 32 * dkp;            // 32 x dkp
    float* Qs = Vs + 32 * dkp;            // ATT_WARPS x dk (scaled)
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int d = H * dk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = blockIdx.y * ATT_WARPS;
    const int qi = q0 + warp;             // query position of this warp
    const bool qvalid = qi < S;
    const size_t base = (size_t)b * S;
    float* qs = Qs + warp * dk;
    if (qvalid)
        for (int i = lane; i < dk; i += 32) qs[i] = __fmul_rn(q[(base + qi) * d + (size_t)h * dk + i], scale);
    acc_t o[4] = {0, 0, 0, 0};
    acc_t m = -INFINITY, l = 0;
    const int last_q = min(S - 1, q0 + ATT_WARPS - 1);
    for (int j0 = 0; j0 <= last_q; j0 += 32) {
        __syncthreads();
        for (int i = threadIdx.x; i < 32 * dk; i += ATT_WARPS * 32) {
            const int r = i / dk, c = i % dk;
            const int j = j0 + r;
            float kv = 0.0f, vv = 0.0f;
            if (j < S) {
                kv = k[(base + j) * d + (size_t)h * dk + c];
                vv = v[(base + j) * d + (size_t)h * dk + c];
            }
            Ks[r * dkp + c] = kv;
            Vs[r * dkp + c] = vv;
        }
        __syncthreads();
        if (!qvalid || j0 > qi) continue;
        const int j = j0 + lane;
        acc_t sc = -INFINITY;
        if (j <= qi) {
            acc_t a = 0;
            const float* kr = Ks + lane * dkp;
            for (int c = 0; c < dk; ++c) a += (acc_t)qs[c] * (acc_t)kr[c];
            sc = a;
        }
        acc_t tmax = sc;
        for (int off = 16; off > 0; off >>= 1) {
            const acc_t other = shfl_xor_t(tmax, off);
            tmax = other > tmax ? other : tmax;
        }
        const acc_t m_new = m > tmax ? m : tmax;
        acc_t p, corr;
        if (EXACT) {
            p = (j <= qi) ? (acc_t)exp((double)(sc - m_new)) : (acc_t)0;
            corr = (acc_t)exp((double)(m - m_new));
        } else {
            p = (j <= qi) ? (acc_t)__expf((float)(sc - m_new)) : (acc_t)0;
            corr = (acc_t)__expf((float)(m - m_new));
        }
        l = l * corr + warp_sum_t(p);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] *= corr;
        for (int jj = 0; jj < 32; ++jj) {
            const acc_t pj = __shfl_sync(0xffffffffu, p, jj);
            if (pj != (acc_t)0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = lane + 32 * i;
                    if (c < dk) o[i] += pj * (acc_t)Vs[jj * dkp + c];
                }
            }
        }
        m = m_new;
    }
    if (qvalid) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = lane + 32 * i;
            if (c < dk) out[(base + qi) * d + (size_t)h * dk + c] = (float)(o[i] / l);
        }
        if (lane == 0) lse[((size_t)b * H + h) * S + qi] = (float)(m + (acc_t)log((double)l));
    }
}

// D[b,h,i] = sum_c dO[i,c] * O[i,c]
__global__ void attn_bwd_delta_kernel(const float* __restrict__ dout, const float* __restrict__ out, int S, int H,
                                      int dk, size_t n_rows, float* __restrict__ delta)
{
    const size_t w = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;  // (row, h)
    if (w >= n_rows * H) return;
    const size_t row = w / H;
    const int h = (int)(w % H), lane = threadIdx.x & 31;
    const int d = H * dk;
    float a = 0.0f;
    for (int c = lane; c < dk; c += 32) a = fmaf(dout[row * d + (size_t)h * dk + c], out[row * d + (size_t)h * dk + c], a);
    a = warp_sum(a);
    const size_t b = row / S, i = row % S;
    if (lane == 0) delta[(b * H + h) * S + i] = a;
}

// dQ: one warp per query, key tiles in shared memory.  dq = scale * sum_j ds_ij k_j,
// ds_ij = p_ij (dO_i . v_j - D_i), p_ij = exp(s_ij - lse_i)
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_bwd_dq_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                   const float* __restrict__ dout, const float* __restrict__ lse, const float* __restrict__ delta,
                   int S, int H, int dk, float scale, float* __restrict__ dq)
{
    extern __shared__ float sm[];
    const int dkp = dk + 1;
    float* Ks = sm;
    float* Vs = Ks + 32 * dkp;
    float* Qs = Vs + 32 * dkp;              // ATT_WARPS x dk scaled q
    float* Gs = Qs + ATT_WARPS * dk;        // ATT_WARPS x dk dO
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int d = H * dk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = blockIdx.y * ATT_WARPS;
    const int qi = q0 + warp;
    const bool qvalid = qi < S;
    const size_t base = (size_t)b * S;
    float* qs = Qs + warp * dk;
    float* gs = Gs + warp * dk;
    float li = 0.0f, di = 0.0f;
    if (qvalid) {
        for (int i = lane; i < dk; i += 32) {
            qs[i] = __fmul_rn(q[(base + qi) * d + (size_t)h * dk + i], scale);
            gs[i] = dout[(base + qi) * d + (size_t)h * dk + i];
        }
        li = lse[((size_t)b * H + h) * S + qi];
        di = delta[((size_t)b * H + h) * S + qi];
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const int last_q = min(S - 1, q0 + ATT_WARPS - 1);
    for (int j0 = 0; j0 <= last_q; j0 += 32) {
        __syncthreads();
        for (int i = threadIdx.x; i < 32 * dk; i += ATT_WARPS * 32) {
            const int r = i / dk, c = i % dk;
            const int j = j0 + r;
            float kv = 0.0f, vv = 0.0f;
            if (j < S) {
                kv = k[(base + j) * d + (size_t)h * dk + c];
                vv = v[(base + j) * d + (size_t)h * dk + c];
            }
            Ks[r * dkp + c] = kv;
            Vs[r * dkp + c] = vv;
        }
        __syncthreads();
        if (!qvalid || j0 > qi) continue;
        const int j = j0 + lane;
        float ds = 0.0f;
        if (j <= qi) {
            float sc = 0.0f, dp = 0.0f;
            const float* kr = Ks + lane * dkp;
            const float* vr = Vs + lane * dkp;
            for (int c = 0; c < dk; ++c) {
                sc = fmaf(qs[c], kr[c], sc);
                dp = fmaf(gs[c], vr[c], dp);
            }
            const float p = __expf(sc - li);
            ds = p * (dp - di);
        }
        for (int jj = 0; jj < 32; ++jj) {
            const float dsj = __shfl_sync(0xffffffffu, ds, jj);
            if (dsj != 0.0f) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = lane + 32 * i;
                    if (c < dk) acc[i] = fmaf(dsj, Ks[jj * dkp + c], acc[i]);
                }
            }
        }
    }
    if (qvalid) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = lane + 32 * i;
            if (c < dk) dq[(base + qi) * d + (size_t)h * dk + c] = acc[i] * scale;
        }
    }
}

// dK, dV: one warp per key, query tiles (scaled q, dO, lse, D) in shared memory.
// dv_j = sum_i p_ij dO_i ; dk_j = sum_i ds_ij (scale q_i)
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_bwd_dkv_kernel(const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                    const float* __restrict__ dout, const float* __restrict__ lse, const float* __restrict__ delta,
                    int S, int H, int dk, float scale, float* __restrict__ dkk, float* __restrict__ dvv)
{
    extern __shared__ float sm[];
    const int dkp = dk + 1;
    float* Qs = sm;                         // 32 x dkp scaled q
    float* Gs = Qs + 32 * dkp;              // 32 x dkp dO
    float* Ks = Gs + 32 * dkp;              // ATT_WARPS x dk
    float* Vs = Ks + ATT_WARPS * dk;        // ATT_WARPS x dk
    float* Ls = Vs + ATT_WARPS * dk;        // 32 lse
    float* Ds = Ls + 32;                    // 32 delta
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int d = H * dk;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k0 = blockIdx.y * ATT_WARPS;
    const int kj = k0 + warp;
    const bool kvalid = kj < S;
    const size_t base = (size_t)b * S;
    float* ks = Ks + warp * dk;
    float* vs = Vs + warp * dk;
    if (kvalid)
        for (int i = lane; i < dk; i += 32) {
            ks[i] = k[(base + kj) * d + (size_t)h * dk + i];
            vs[i] = v[(base + kj) * d + (size_t)h * dk + i];
        }
    float ak[4] = {0.f, 0.f, 0.f, 0.f}, av[4] = {0.f, 0.f, 0.f, 0.f};
    const int first_tile = (k0 / 32) * 32;
    for (int i0 = first_tile; i0 < S; i0 += 32) {
        __syncthreads();
        for (int i = threadIdx.x; i < 32 * dk; i += ATT_WARPS * 32) {
            const int r = i / dk, c = i % dk;
            const int qi = i0 + r;
            float qv = 0.0f, gv = 0.0f;
            if (qi < S) {
                qv = __fmul_rn(q[(base + qi) * d + (size_t)h * dk + c], scale);
                gv = dout[(base + qi) * d + (size_t)h * dk + c];
            }
            Qs[r * dkp + c] = qv;
            Gs[r * dkp + c] = gv;
        }
        if (threadIdx.x < 32) {
            const int qi = i0 + threadIdx.x;
            Ls[threadIdx.x] = qi < S ? lse[((size_t)b * H + h) * S + qi] : 0.0f;
            Ds[threadIdx.x] = qi < S ? delta[((size_t)b * H + h) * S + qi] : 0.0f;
        }
        __syncthreads();
        if (!kvalid || i0 + 31 < kj) continue;
        const int qi = i0 + lane;
        float p = 0.0f, ds = 0.0f;
        if (qi < S && qi >= kj) {
            float sc = 0.0f, dp = 0.0f;
            const float* qr = Qs + lane * dkp;
            const float* gr = Gs + lane * dkp;
            for (int c = 0; c < dk; ++c) {
                sc = fmaf(qr[c], ks[c], sc);
                dp = fmaf(gr[c], vs[c], dp);
            }
            p = __expf(sc - Ls[lane]);
            ds = p * (dp - Ds[lane]);
        }
        for (int ii = 0; ii < 32; ++ii) {
            const float pi = __shfl_sync(0xffffffffu, p, ii);
            const float dsi = __shfl_sync(0xffffffffu, ds, ii);
            if (pi != 0.0f || dsi != 0.0f) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int c = lane + 32 * i;
                    if (c < dk) {
                        av[i] = fmaf(pi, Gs[ii * dkp + c], av[i]);
                        ak[i] = fmaf(dsi, Qs[ii * dkp + c], ak[i]);
                    }
                }
            }
        }
    }
    if (kvalid) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = lane + 32 * i;
            if (c < dk) {
                dkk[(base + kj) * d + (size_t)h * dk + c] = ak[i];
                dvv[(base + kj) * d + (size_t)h * dk + c] = av[i];
            }
        }
    }
}

// ----------------------------------------------------------- RMSNorm backward
// gy = dy*gamma; normed = x*sinv; m = sum(gy*normed)/F; dx = (gy - m*normed)*sinv (+ residual)
// dgamma[f] += sum_t dy[t,f]*normed[t,f].  One warp per token, TOK tokens per CTA; gamma
// gradients are reduced in shared memory and flushed with one atomic per feature per CTA.
constexpr int RN_TOK = 16;
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const float* x /* may be dx: in place */, const float* __restrict__ gamma, const float* __restrict__ dy,
                   const float* __restrict__ residual, size_t T, int F, float* dx,
                   float* __restrict__ dgamma)
{
    extern __shared__ float dg[];  // F
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < F; i += 256) dg[i] = 0.0f;
    __syncthreads();
    const float inv_f = __frcp_rn((float)F);
    for (int tt = warp; tt < RN_TOK; tt += 8) {
        const size_t t = (size_t)blockIdx.x * RN_TOK + tt;
        if (t >= T) break;
        const float* xr = x + t * F;
        const float* gr = dy + t * F;
        float ss = 0.0f;
        for (int i = lane; i < F; i += 32) ss = fmaf(xr[i], xr[i], ss);
        ss = warp_sum(ss);
        const float sinv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fmul_rn(ss, inv_f), 1e-5f)));
        float dot = 0.0f;
        for (int i = lane; i < F; i += 32) dot = fmaf(gr[i] * gamma[i], xr[i] * sinv, dot);
        dot = warp_sum(dot) * inv_f;
        for (int i = lane; i < F; i += 32) {
            const float normed = xr[i] * sinv;
            const float gy = gr[i] * gamma[i];
            float v = (gy - dot * normed) * sinv;
            if (residual) v += residual[t * F + i];
            dx[t * F + i] = v;
            atomicAdd(dg + i, gr[i] * normed);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < F; i += 256)
        if (dg[i] != 0.0f) atomicAdd(dgamma + i, dg[i]);
}

// Same operator for F = 128*NV: a warp keeps a token's x and dy*gamma in registers (NV float4 each per
// lane, all loads of a pass in flight together) and its share of the gamma gradient too; warps walk the
// tokens with a grid-wide stride, so there is one shared-memory reduction and one flush per CTA.
template <int NV>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_vec_kernel(const float* x /* may be dx: in place */, const float* __restrict__ gamma, const float* __restrict__ dy,
                       const float* __restrict__ residual, size_t T, float* dx, float* __restrict__ dgamma)
{
    constexpr int F = 128 * NV;
    __shared__ float dg[F];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < F; i += 256) dg[i] = 0.0f;
    __syncthreads();
    const float inv_f = __frcp_rn((float)F);
    float4 dgr[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) dgr[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (size_t t = (size_t)blockIdx.x * 8 + warp; t < T; t += (size_t)gridDim.x * 8) {
        const float4* xr = reinterpret_cast<const float4*>(x + t * F);
        const float4* gr = reinterpret_cast<const float4*>(dy + t * F);
        float4 xv[NV], gv[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) xv[j] = xr[j * 32 + lane];
#pragma unroll
        for (int j = 0; j < NV; ++j) gv[j] = gr[j * 32 + lane];
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j) ss = fmaf(xv[j].x, xv[j].x, fmaf(xv[j].y, xv[j].y, fmaf(xv[j].z, xv[j].z, fmaf(xv[j].w, xv[j].w, ss))));
        ss = warp_sum(ss);
        const float sinv = __frcp_rn(__fsqrt_rn(__fadd_rn(__fmul_rn(ss, inv_f), 1e-5f)));
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            xv[j].x *= sinv; xv[j].y *= sinv; xv[j].z *= sinv; xv[j].w *= sinv;  // normed
            dgr[j].x = fmaf(gv[j].x, xv[j].x, dgr[j].x); dgr[j].y = fmaf(gv[j].y, xv[j].y, dgr[j].y);
            dgr[j].z = fmaf(gv[j].z, xv[j].z, dgr[j].z); dgr[j].w = fmaf(gv[j].w, xv[j].w, dgr[j].w);
            const float4 gm = __ldg(reinterpret_cast<const float4*>(gamma) + j * 32 + lane);
            gv[j].x *= gm.x; gv[j].y *= gm.y; gv[j].z *= gm.z; gv[j].w *= gm.w;  // gy
            dot = fmaf(gv[j].x, xv[j].x, fmaf(gv[j].y, xv[j].y, fmaf(gv[j].z, xv[j].z, fmaf(gv[j].w, xv[j].w, dot))));
        }
        dot = warp_sum(dot) * inv_f;
        float4* dxr = reinterpret_cast<float4*>(dx + t * F);
        const float4* rr = residual ? reinterpret_cast<const float4*>(residual + t * F) : nullptr;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            float4 o = make_float4((gv[j].x - dot * xv[j].x) * sinv, (gv[j].y - dot * xv[j].y) * sinv,
                                   (gv[j].z - dot * xv[j].z) * sinv, (gv[j].w - dot * xv[j].w) * sinv);
            if (rr) {
                const float4 r = rr[j * 32 + lane];
                o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
            }
            dxr[j * 32 + lane] = o;
        }
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int c = (j * 32 + lane) * 4;
        atomicAdd(dg + c, dgr[j].x); atomicAdd(dg + c + 1, dgr[j].y);
        atomicAdd(dg + c + 2, dgr[j].z); atomicAdd(dg + c + 3, dgr[j].w);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < F; i += 256)
        if (dg[i] != 0.0f) atomicAdd(dgamma + i, dg[i]);
}

// ------------------------------------------------------- activation backward
// MODE 1 QuickGELU: dh = da * s*(1 + bx*(1-s)), s = sigmoid(bx), bx = 1.702 h
// MODE 2 SwiGLU: h = (gate|up): dgate = da*up*s*(1+gate*(1-s)), dup = da*gate*s
// MODE 3 ReLU2GLU: h = (gate|up), r = relu(gate): dgate = da*up*2r, dup = da*r*r (compute_layer_mlp.hpp:425-440)
template <int MODE>
__global__ void act_bwd_kernel(const float* __restrict__ h, const float* __restrict__ da, size_t T, int F,
                               float* __restrict__ dh)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * F) return;
    const size_t t = idx / F;
    const int f = (int)(idx % F);
    if (MODE == 1) {
        const float xv = h[idx];
        const float bx = xv * 1.702f;
        const float sg = 1.0f / (1.0f + nnb_expf(-bx));
        dh[idx] = da[idx] * (sg * (1.0f + bx * (1.0f - sg)));
    } else {
        const float gv = h[t * 2 * F + f], uv = h[t * 2 * F + F + f];
        const float go = da[idx];
        if (MODE == 3) {
            const float rv = fmaxf(gv, 0.0f);
            dh[t * 2 * F + f] = go * uv * (2.0f * rv);
            dh[t * 2 * F + F + f] = go * (rv * rv);
        } else {
            const float sg = 1.0f / (1.0f + nnb_expf(-gv));
            dh[t * 2 * F + f] = go * uv * (sg * (1.0f + gv * (1.0f - sg)));
            dh[t * 2 * F + F + f] = go * gv * sg;
        }
    }
}

// four features per thread (F a multiple of 4), same arithmetic
template <int MODE>
__global__ void __launch_bounds__(256)
act_bwd_vec_kernel(const float* __restrict__ h, const float* __restrict__ da, size_t T, int F, float* __restrict__ dh)
{
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // float4 index into da
    const int F4 = F >> 2;
    if (idx >= T * F4) return;
    const size_t t = idx / F4;
    const int f = (int)(idx % F4);
    const float4 go = reinterpret_cast<const float4*>(da)[idx];
    const float g4[4] = {go.x, go.y, go.z, go.w};
    if (MODE == 1) {
        const float4 xv = reinterpret_cast<const float4*>(h)[idx];
        const float x4[4] = {xv.x, xv.y, xv.z, xv.w};
        float o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float bx = x4[i] * 1.702f;
            const float sg = 1.0f / (1.0f + nnb_expf(-bx));
            o[i] = g4[i] * (sg * (1.0f + bx * (1.0f - sg)));
        }
        reinterpret_cast<float4*>(dh)[idx] = make_float4(o[0], o[1], o[2], o[3]);
    } else {
        const float4 gv = reinterpret_cast<const float4*>(h + t * 2 * F)[f];
        const float4 uv = reinterpret_cast<const float4*>(h + t * 2 * F + F)[f];
        const float ga[4] = {gv.x, gv.y, gv.z, gv.w}, ua[4] = {uv.x, uv.y, uv.z, uv.w};
        float og[4], ou[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (MODE == 3) {
                const float rv = fmaxf(ga[i], 0.0f);
                og[i] = g4[i] * ua[i] * (2.0f * rv);
                ou[i] = g4[i] * (rv * rv);
            } else {
                const float sg = 1.0f / (1.0f + nnb_expf(-ga[i]));
                og[i] = g4[i] * ua[i] * (sg * (1.0f + ga[i] * (1.0f - sg)));
                ou[i] = g4[i] * ga[i] * sg;
            }
        }
        reinterpret_cast<float4*>(dh + t * 2 * F)[f] = make_float4(og[0], og[1], og[2], og[3]);
        reinterpret_cast<float4*>(dh + t * 2 * F + F)[f] = make_float4(ou[0], ou[1], ou[2], ou[3]);
    }
}

// --------------------------------------------------- row gather / scatter / add
// dst[i,:] = src[index(i),:] where decision i = (b, g) maps to row b*S + P-1+g
__global__ void gather_decisions_kernel(const float* __restrict__ src, int S, int P, int G, int d,
                                        float* __restrict__ dst)
{
    const size_t i = blockIdx.x;
    const size_t b = i / G, g = i % G;
    const size_t row = b * S + P - 1 + g;
    for (int c = threadIdx.x; c < d; c += blockDim.x) dst[i * d + c] = src[row * d + c];
}

// dst (n*S, d) = 0 everywhere except decision rows, which get src
__global__ void scatter_decisions_kernel(const float* __restrict__ src, int S, int P, int G, int d,
                                         float* __restrict__ dst)
{
    const size_t row = blockIdx.x;
    const size_t b = row / S;
    const int t = (int)(row % S);
    const int g = t - (P - 1);
    const bool hit = g >= 0 && g < G;
    for (int c = threadIdx.x; c < d; c += blockDim.x)
        dst[row * d + c] = hit ? src[(b * G + g) * d + c] : 0.0f;
}

// grouped layout: decision (b, g) reads the row of position P-1+g of sequence b (g = 0: the shared last
// prompt row of b's group)
__global__ void gather_decisions_map_kernel(const float* __restrict__ src, const SeqMap map, int d, float* __restrict__ dst)
{
    const size_t i = blockIdx.x;
    const int b = (int)(i / map.G), g = (int)(i % map.G);
    const size_t row = map_row(map, b, map.P - 1 + g);
    for (int c = threadIdx.x; c < d; c += blockDim.x) dst[i * d + c] = src[row * d + c];
}

// grouped layout, one CTA per destination row: own rows take their decision's gradient, the last prompt row of
// a group takes the sum of its members' first decisions (in member order), every other row is zero
__global__ void scatter_decisions_map_kernel(const float* __restrict__ src, const SeqMap map, int d, float* __restrict__ dst)
{
    const size_t row = blockIdx.x;
    const size_t rpg = (size_t)map.P + (size_t)map.group * map.G;
    const int grp = (int)(row / rpg);
    const int o = (int)(row % rpg);
    for (int c = threadIdx.x; c < d; c += blockDim.x) {
        float v = 0.0f;
        if (o < map.P) {
            if (o == map.P - 1)
                for (int mm = 0; mm < map.group; ++mm) v += src[((size_t)(grp * map.group + mm) * map.G) * d + c];
        } else {
            const int mm = (o - map.P) / map.G, g = (o - map.P) % map.G + 1;
            if (g < map.G) v = src[((size_t)(grp * map.group + mm) * map.G + g) * d + c];
        }
        dst[row * d + c] = v;
    }
}

// value head: value[i] = w . x[i,:] + b   (Linear(d -> 1) on the final-norm output)
__global__ void value_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                 size_t n, int d, float* __restrict__ value)
{
    const size_t i = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (i >= n) return;
    const int lane = threadIdx.x & 31;
    float a = 0.0f;
    for (int c = lane; c < d; c += 32) a = fmaf(x[i * d + c], w[c], a);
    a = warp_sum(a);
    if (lane == 0) value[i] = a + b[0];
}

// dx[i,:] += dv[i]*w ; dw += sum_i dv[i]*x[i,:] ; db += sum_i dv[i]
// grid (feature blocks of 256, decision chunks): a CTA walks its chunk of decisions and leaves its partial sums of dw
// (d floats) and db (one float) in part[chunk]; value_bwd_finish_kernel adds the chunks up in order, so the result does
// not depend on which CTA ran first
__global__ void __launch_bounds__(256)
value_bwd_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ dv, size_t n, int d,
                 size_t chunk, float* __restrict__ dx, float* __restrict__ part)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const size_t i0 = (size_t)blockIdx.y * chunk, i1 = i0 + chunk < n ? i0 + chunk : n;
    float aw = 0.0f, ab = 0.0f;
    const float wc = c < d ? w[c] : 0.0f;
    for (size_t i = i0; i < i1; ++i) {
        const float g = dv[i];
        if (c < d) {
            dx[i * d + c] += g * wc;
            aw = fmaf(g, x[i * d + c], aw);
        }
        if (c == 0) ab += g;
    }
    float* prow = part + (size_t)blockIdx.y * (d + 1);
    if (c < d) prow[c] = aw;
    if (c == 0) prow[d] = ab;
}

__global__ void __launch_bounds__(256)
value_bwd_finish_kernel(const float* __restrict__ part, int n_chunks, int d, float* __restrict__ dw, float* __restrict__ db)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c > d) return;
    float a = 0.0f;
    for (int k = 0; k < n_chunks; ++k) a += part[(size_t)k * (d + 1) + c];
    if (c < d) dw[c] += a;
    else db[0] += a;
}

__global__ void add_kernel(float* __restrict__ dst, const float* __restrict__ src, size_t n)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] += src[i];
}

// ------------------------------------------------------------------ launchers
nnb_status launch_embed_fwd(nnb_engine* e, const float* tok_emb, const float* pos_emb, const int32_t* tokens,
                            size_t n_rows, size_t S, size_t d, size_t vocab, float* x)
{
    embed_fwd_kernel<<<(unsigned)n_rows, 128, 0, e->stream>>>(tok_emb, pos_emb, tokens, (int)S, (int)d, (int)vocab, x);
    e->launches++;
    NNB_CHECK_LAUNCH("embed_fwd_kernel");
    return NNB_OK;
}

nnb_status launch_embed_bwd(nnb_engine* e, const float* g, const int32_t* tokens, size_t n_rows, size_t S, size_t d,
                            size_t vocab, float* g_tok, float* g_pos)
{
    embed_bwd_kernel<<<(unsigned)n_rows, 128, 0, e->stream>>>(g, tokens, (int)S, (int)d, (int)vocab, g_tok, g_pos);
    e->launches++;
    NNB_CHECK_LAUNCH("embed_bwd_kernel");
    return NNB_OK;
}

nnb_status launch_build_rows(nnb_engine* e, const int32_t* tokens, const SeqMap& map, size_t n_seq, int32_t* row_tok,
                             int32_t* row_pos)
{
    const size_t n = n_seq * map.S;
    build_rows_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, e->stream>>>(tokens, map, n, row_tok, row_pos);
    e->launches++;
    NNB_CHECK_LAUNCH("build_rows_kernel");
    return NNB_OK;
}

nnb_status launch_embed_rows_fwd(nnb_engine* e, const float* tok_emb, const float* pos_emb, const int32_t* row_tok,
                                 const int32_t* row_pos, size_t n_rows, size_t d, size_t vocab, float* x)
{
    embed_rows_fwd_kernel<<<(unsigned)n_rows, 128, 0, e->stream>>>(tok_emb, pos_emb, row_tok, row_pos, (int)d, (int)vocab, x);
    e->launches++;
    NNB_CHECK_LAUNCH("embed_rows_fwd_kernel");
    return NNB_OK;
}

nnb_status launch_embed_rows_bwd(nnb_engine* e, const float* g, const int32_t* row_tok, const int32_t* row_pos, size_t n_rows,
                                 size_t d, size_t vocab, float* g_tok, float* g_pos)
{
    embed_rows_bwd_kernel<<<(unsigned)n_rows, 128, 0, e->stream>>>(g, row_tok, row_pos, (int)d, (int)vocab, g_tok, g_pos);
    e->launches++;
    NNB_CHECK_LAUNCH("embed_rows_bwd_kernel");
    return NNB_OK;
}

nnb_status launch_gather_decisions_map(nnb_engine* e, const float* src, const SeqMap& map, size_t n_seq, size_t d, float* dst)
{
    gather_decisions_map_kernel<<<(unsigned)(n_seq * map.G), 128, 0, e->stream>>>(src, map, (int)d, dst);
    e->launches++;
    NNB_CHECK_LAUNCH("gather_decisions_map_kernel");
    return NNB_OK;
}

nnb_status launch_scatter_decisions_map(nnb_engine* e, const float* src, const SeqMap& map, size_t n_seq, size_t d, float* dst)
{
    scatter_decisions_map_kernel<<<(unsigned)map_rows_total(map, n_seq), 128, 0, e->stream>>>(src, map, (int)d, dst);
    e->launches++;
    NNB_CHECK_LAUNCH("scatter_decisions_map_kernel");
    return NNB_OK;
}

nnb_status launch_rope(nnb_engine* e, float* x, const float* rope_cos, const float* rope_sin, size_t n_rows,
                       size_t S, size_t H, size_t dk, bool backward)
{
    rope_kernel<<<(unsigned)n_rows, 128, 0, e->stream>>>(x, rope_cos, rope_sin, (int)S, (int)H, (int)dk,
                                                         backward ? -1.0f : 1.0f);
    e->launches++;
    NNB_CHECK_LAUNCH("rope_kernel");
    return NNB_OK;
}

nnb_status launch_attn_fwd(nnb_engine* e, bool exact, const float* q, const float* k, const float* v, size_t n_seq,
                           size_t S, size_t H, size_t dk, float* out, float* lse)
{
    NNB_REQUIRE(dk <= 128, "attention: head dim %zu > 128", dk);
    if (!exact && attn_b16_supported(dk, H * dk)) {
        // standalone operator on f32 operands: bf16 copies live in stream-ordered scratch
        const size_t td = n_seq * S * H * dk;
        __nv_bfloat16* tmp = nullptr;
        NNB_CUDA(cudaMallocAsync((void**)&tmp, 3 * td * sizeof(__nv_bfloat16), e->stream));
        nnb_status st = launch_rope_pack_b16(e, q, k, v, nullptr, nullptr, n_seq * S, S, H, dk, tmp);
        if (st == NNB_OK) st = launch_attn_fwd_b16(e, tmp, tmp + td, tmp + 2 * td, n_seq, S, H, dk, out, lse);
        cudaFreeAsync(tmp, e->stream);
        return st;
    }
    const size_t smem = (2 * 32 * (dk + 1) + ATT_WARPS * dk) * sizeof(float);
    static size_t cfg_dev[64] = {}; size_t& cfg = cfg_dev[e->device & 63];
    if (smem > cfg) {
        NNB_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        NNB_CUDA(cudaFuncSetAttribute(attn_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cfg = smem;
    }
    dim3 grid((unsigned)(n_seq * H), (unsigned)ceil_div(S, ATT_WARPS));
    const float scale = 1.0f / sqrtf((float)dk);
    if (exact)
        attn_fwd_kernel<true><<<grid, ATT_WARPS * 32, smem, e->stream>>>(q, k, v, (int)S, (int)H, (int)dk, scale, out, lse);
    else
        attn_fwd_kernel<false><<<grid, ATT_WARPS * 32, smem, e->stream>>>(q, k, v, (int)S, (int)H, (int)dk, scale, out, lse);
    e->launches++;
    NNB_CHECK_LAUNCH("attn_fwd_kernel");
    return NNB_OK;
}

nnb_status launch_attn_bwd(nnb_engine* e, bool exact, const float* q, const float* k, const float* v, const float* out,
                           const float* dout, const float* lse, float* delta, size_t n_seq, size_t S, size_t H,
                           size_t dk, float* dq, float* dkk, float* dvv)
{
    NNB_REQUIRE(dk <= 128, "attention: head dim %zu > 128", dk);
    const float scale = 1.0f / sqrtf((float)dk);
    const size_t rows = n_seq * S;
    if (!exact && attn_b16_supported(dk, H * dk)) {
        const size_t td = rows * H * dk;
        __nv_bfloat16* tmp = nullptr;
        NNB_CUDA(cudaMallocAsync((void**)&tmp, 4 * td * sizeof(__nv_bfloat16), e->stream));
        nnb_status st = launch_rope_pack_b16(e, q, k, v, nullptr, nullptr, rows, S, H, dk, tmp);
        if (st == NNB_OK)
            st = launch_attn_bwd_b16(e, tmp, tmp + td, tmp + 2 * td, out, dout, lse, delta, tmp + 3 * td, nullptr, nullptr, n_seq, S,
                                     H, dk, dq, dkk, dvv);
        cudaFreeAsync(tmp, e->stream);
        return st;
    }
    attn_bwd_delta_kernel<<<(unsigned)ceil_div(rows * H, 8), 256, 0, e->stream>>>(dout, out, (int)S, (int)H, (int)dk,
                                                                                 rows, delta);
    const size_t smem_q = (2 * 32 * (dk + 1) + 2 * ATT_WARPS * dk) * sizeof(float);
    const size_t smem_kv = (2 * 32 * (dk + 1) + 2 * ATT_WARPS * dk + 64) * sizeof(float);
    static size_t cfg_q_dev[64] = {}, cfg_kv_dev[64] = {}; size_t &cfg_q = cfg_q_dev[e->device & 63], &cfg_kv = cfg_kv_dev[e->device & 63];
    if (smem_q > cfg_q) {
        NNB_CUDA(cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q));
        cfg_q = smem_q;
    }
    if (smem_kv > cfg_kv) {
        NNB_CUDA(cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv));
        cfg_kv = smem_kv;
    }
    dim3 grid((unsigned)(n_seq * H), (unsigned)ceil_div(S, ATT_WARPS));
    attn_bwd_dq_kernel<<<grid, ATT_WARPS * 32, smem_q, e->stream>>>(q, k, v, dout, lse, delta, (int)S, (int)H, (int)dk,
                                                                   scale, dq);
    attn_bwd_dkv_kernel<<<grid, ATT_WARPS * 32, smem_kv, e->stream>>>(q, k, v, dout, lse, delta, (int)S, (int)H,
                                                                     (int)dk, scale, dkk, dvv);
    e->launches += 3;
    NNB_CHECK_LAUNCH("attention backward kernels");
    return NNB_OK;
}

nnb_status launch_rmsnorm_bwd(nnb_engine* e, const float* x, const float* gamma, const float* dy,
                              const float* residual, size_t T, size_t F, float* dx, float* dgamma)
{
    const bool al = (((uintptr_t)x | (uintptr_t)gamma | (uintptr_t)dy | (uintptr_t)residual | (uintptr_t)dx) & 15) == 0;
    if (al && (F == 2048 || F == 1024 || F == 512)) {
        const unsigned grid = (unsigned)std::min<size_t>(ceil_div(T, 8), (size_t)e->sm_count);
        if (F == 2048) rmsnorm_bwd_vec_kernel<16><<<grid, 256, 0, e->stream>>>(x, gamma, dy, residual, T, dx, dgamma);
        else if (F == 1024) rmsnorm_bwd_vec_kernel<8><<<grid, 256, 0, e->stream>>>(x, gamma, dy, residual, T, dx, dgamma);
        else rmsnorm_bwd_vec_kernel<4><<<grid, 256, 0, e->stream>>>(x, gamma, dy, residual, T, dx, dgamma);
        e->launches++;
        NNB_CHECK_LAUNCH("rmsnorm_bwd_vec_kernel");
        return NNB_OK;
    }
    const size_t smem = F * sizeof(float);
    static size_t cfg_dev[64] = {}; size_t& cfg = cfg_dev[e->device & 63];
    if (smem > cfg && smem > 48 * 1024) {
        NNB_CUDA(cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cfg = smem;
    }
    rmsnorm_bwd_kernel<<<(unsigned)ceil_div(T, RN_TOK), 256, smem, e->stream>>>(x, gamma, dy, residual, T, (int)F, dx,
                                                                               dgamma);
    e->launches++;
    NNB_CHECK_LAUNCH("rmsnorm_bwd_kernel");
    return NNB_OK;
}

nnb_status launch_act_bwd(nnb_engine* e, int mode, const float* h, const float* da, size_t T, size_t F, float* dh)
{
    if (F % 4 == 0 && (((uintptr_t)h | (uintptr_t)da | (uintptr_t)dh) & 15) == 0) {
        const unsigned g4 = (unsigned)ceil_div(T * (F / 4), 256);
        if (mode == 1) act_bwd_vec_kernel<1><<<g4, 256, 0, e->stream>>>(h, da, T, (int)F, dh);
        else if (mode == 3) act_bwd_vec_kernel<3><<<g4, 256, 0, e->stream>>>(h, da, T, (int)F, dh);
        else act_bwd_vec_kernel<2><<<g4, 256, 0, e->stream>>>(h, da, T, (int)F, dh);
        e->launches++;
        NNB_CHECK_LAUNCH("act_bwd_vec_kernel");
        return NNB_OK;
    }
    const unsigned grid = (unsigned)ceil_div(T * F, 256);
    if (mode == 1) act_bwd_kernel<1><<<grid, 256, 0, e->stream>>>(h, da, T, (int)F, dh);
    else if (mode == 3) act_bwd_kernel<3><<<grid, 256, 0, e->stream>>>(h, da, T, (int)F, dh);
    else act_bwd_kernel<2><<<grid, 256, 0, e->stream>>>(h, da, T, (int)F, dh);
    e->launches++;
    NNB_CHECK_LAUNCH("act_bwd_kernel");
    return NNB_OK;
}

nnb_status launch_gather_decisions(nnb_engine* e, const float* src, size_t n_seq, size_t S, size_t P, size_t G,
                                   size_t d, float* dst)
{
    gather_decisions_kernel<<<(unsigned)(n_seq * G), 128, 0, e->stream>>>(src, (int)S, (int)P, (int)G, (int)d, dst);
    e->launches++;
    NNB_CHECK_LAUNCH("gather_decisions_kernel");
    return NNB_OK;
}

nnb_status launch_scatter_decisions(nnb_engine* e, const float* src, size_t n_seq, size_t S, size_t P, size_t G,
                                    size_t d, float* dst)
{
    scatter_decisions_kernel<<<(unsigned)(n_seq * S), 128, 0, e->stream>>>(src, (int)S, (int)P, (int)G, (int)d, dst);
    e->launches++;
    NNB_CHECK_LAUNCH("scatter_decisions_kernel");
    return NNB_OK;
}

nnb_status launch_value_fwd(nnb_engine* e, const float* x, const float* w, const float* b, size_t n, size_t d,
                            float* value)
{
    value_fwd_kernel<<<(unsigned)ceil_div(n, 8), 256, 0, e->stream>>>(x, w, b, n, (int)d, value);
    e->launches++;
    NNB_CHECK_LAUNCH("value_fwd_kernel");
    return NNB_OK;
}

// scratch: at least (d + 1) floats; the more it holds (up to one row of d + 1 per 64 decisions), the more CTAs share
// the decisions
nnb_status launch_value_bwd(nnb_engine* e, const float* x, const float* w, const float* dv, size_t n, size_t d,
                            float* dx, float* dw, float* db, float* scratch, size_t scratch_floats)
{
    NNB_REQUIRE(scratch && scratch_floats >= d + 1 && n > 0, "value_bwd: scratch of at least d + 1 floats");
    size_t n_chunks = std::min<size_t>(std::min<size_t>(ceil_div(n, 64), scratch_floats / (d + 1)), 4096);
    const size_t chunk = ceil_div(n, n_chunks);
    n_chunks = ceil_div(n, chunk);
    value_bwd_kernel<<<dim3((unsigned)ceil_div(d, 256), (unsigned)n_chunks), 256, 0, e->stream>>>(x, w, dv, n, (int)d, chunk, dx,
                                                                                                    scratch);
    e->launches++;
    NNB_CHECK_LAUNCH("value_bwd_kernel");
    value_bwd_finish_kernel<<<(unsigned)ceil_div(d + 1, 256), 256, 0, e->stream>>>(scratch, (int)n_chunks, (int)d, dw, db);
    e->launches++;
    NNB_CHECK_LAUNCH("value_bwd_finish_kernel");
    return NNB_OK;
}

nnb_status launch_add(nnb_engine* e, float* dst, const float* src, size_t n)
{
    add_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, e->stream>>>(dst, src, n);
    e->launches++;
    NNB_CHECK_LAUNCH("add_kernel");
    return NNB_OK;
}

}  // namespace nnb
