// decode.cu — kernels of one batched decode step of the ternary GPT policy:
// embedding, RMSNorm fused with activation quantisation, RoPE + KV-cache append + attention,
// FFN activation fused with quantisation, and the sampler.
//
// Reference semantics (per sequence; the batch dimension only runs sequences side by side):
//   GPTModel::forward_step           include/neuralnet.cpp/compute_layer_gpt.hpp:693-725
//   AttentionBase::forward_step      include/neuralnet.cpp/compute_layer_attention.hpp:1003-1092
//   RMSNorm::forward                 include/neuralnet.cpp/compute_layer_mlp.hpp:686-707
//   RotaryEmbedding::apply_step      include/neuralnet.cpp/compute_position_encoding.hpp:149-168
//   GeLU / SwiGLU forward            include/neuralnet.cpp/compute_layer_mlp.hpp:243-252,317-330
//   sample_next_token_               include/neuralnet.cpp/compute_layer_base.hpp:1025-1163
//
// Two numeric modes.  EXACT: f32 storage, every float reduction accumulated in f64 and rounded
// once (independent of the reduction tree), exp as a fixed fmaf sequence; this is the mode
// whose greedy rollouts are compared token by token with the CPU restatement.  Fast: bf16 KV
// cache, f32 accumulation.
#include "common.cuh"
#include "device_math.cuh"

namespace nnb {

// ---------------------------------------------------------------- embedding
// x[b,:] = tok_emb[token[b, col],:] (+ pos_emb[pos,:]) with d_pos = {pos, col}: the position inside the context
// window and the column of the token buffer.  They differ only after the window of a long generation has slid.
__global__ void embed_kernel(const float* __restrict__ tok_emb, const float* __restrict__ pos_emb,
                             const int32_t* __restrict__ tokens, int tokens_stride,
                             const int* __restrict__ d_pos, int d, int vocab, float* __restrict__ x)
{
    const int b = blockIdx.x;
    pdl_launch();
    pdl_wait();
    const int pos = d_pos[0];
    int tok = tokens[(size_t)b * tokens_stride + d_pos[1]];
    tok = min(max(tok, 0), vocab - 1);
    const float* e = tok_emb + (size_t)tok * d;
    const float* p = pos_emb ? pos_emb + (size_t)pos * d : nullptr;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = e[i];
        if (p) v = __fadd_rn(v, p[i]);
        x[(size_t)b * d + i] = v;
    }
}

// -------------------------------------------- row transform + quantisation
// One CTA per token.  MODE 0: RMSNorm(x)*gamma.  MODE 1: QuickGELU(h).  MODE 2: SwiGLU(h) with
// h = (gate | up).  MODE 3: identity.  MODE 4: ReLU2GLU(h) = relu(gate)^2 * up (include/neuralnet.cpp/compute_layer_mlp.hpp:384-440).  The transformed row is quantised to the engine's int8
// layout (see ternary.cu) and optionally also written as f32 (`f_out`).
// NORM (MODE 1, 2, 4 only): the activated row goes through RMSNorm(.)*gamma before it is quantised (SubLN of the
// feed-forward, include/neuralnet.cpp/compute_layer_feedforward.hpp:201-206); f_out then receives the activated row
// before the norm, which is what the norm's backward needs.
template <typename InT>
__device__ __forceinline__ float ld_in(const InT* p);
template <>
__device__ __forceinline__ float ld_in<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld_in<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename InT>
__device__ __forceinline__ float4 ld_in4(const InT* p);  // four consecutive elements, p aligned to four of them
template <>
__device__ __forceinline__ float4 ld_in4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 ld_in4<__nv_bfloat16>(const __nv_bfloat16* p)
{
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(t.x << 16), __uint_as_float(t.x & 0xffff0000u), __uint_as_float(t.y << 16),
                       __uint_as_float(t.y & 0xffff0000u));
}

// InT: the input's type; bf16 where the producing GEMM stored its result so (the fc1 output in the fast mode)
template <int MODE, bool EXACT, bool NORM = false, typename InT = float>
__global__ void __launch_bounds__(256)
row_quant_kernel(const InT* __restrict__ in, const float* __restrict__ gamma, int k, int in_stride,
                 int8_t* __restrict__ q, float* __restrict__ s, int32_t* __restrict__ qsum,
                 float* __restrict__ f_out)
{
    extern __shared__ float row[];
    __shared__ double red_d[8];
    __shared__ float red_f[8];
    __shared__ int red_i[8];
    const size_t tok = blockIdx.x;
    const InT* xr = in + tok * (size_t)in_stride;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    float sinv = 0.0f;
    if (MODE == 0) {
        float ssf;
        if (EXACT) {
            double ss = 0.0;
            for (int i = tid; i < k; i += 256) {
                const float v = ld_in<InT>(xr + i);
                ss += (double)__fmul_rn(v, v);
            }
            ss = warp_sum_d(ss);
            if (lane == 0) red_d[warp] = ss;
            __syncthreads();
            ss = 0.0;
#pragma unroll
            for (int w = 0; w < 8; ++w) ss += red_d[w];
            ssf = (float)ss;
        } else {
            float ss = 0.0f;
            for (int i = tid; i < k; i += 256) {
                const float v = ld_in<InT>(xr + i);
                ss = fmaf(v, v, ss);
            }
            ss = warp_sum(ss);
            if (lane == 0) red_f[warp] = ss;
            __syncthreads();
            ss = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) ss += red_f[w];
            ssf = ss;
        }
        const float v = __fadd_rn(__fmul_rn(ssf, __frcp_rn((float)k)), 1e-5f);
        sinv = __frcp_rn(__fsqrt_rn(v));
        __syncthreads();
    }
    float mx = 0.0f;
    double ss_act = 0.0;
    float ssf_act = 0.0f;
    for (int i = tid; i < k; i += 256) {
        float v;
        if (MODE == 0) {
            v = __fmul_rn(__fmul_rn(ld_in<InT>(xr + i), sinv), gamma[i]);
        } else if (MODE == 1) {
            const float xv = ld_in<InT>(xr + i);
            v = __fdiv_rn(xv, __fadd_rn(1.0f, nnb_expf(-__fmul_rn(xv, 1.702f))));
        } else if (MODE == 2) {
            const float gv = ld_in<InT>(xr + i), uv = ld_in<InT>(xr + k + i);
            const float sig = __fdiv_rn(1.0f, __fadd_rn(1.0f, nnb_expf(-gv)));
            v = __fmul_rn(__fmul_rn(gv, sig), uv);
        } else if (MODE == 4) {
            const float rv = fmaxf(ld_in<InT>(xr + i), 0.0f), uv = ld_in<InT>(xr + k + i);
            v = __fmul_rn(__fmul_rn(rv, rv), uv);
        } else {
            v = ld_in<InT>(xr + i);
        }
        row[i] = v;
        if (f_out) f_out[tok * (size_t)k + i] = v;
        if (NORM) {
            if (EXACT) ss_act += (double)__fmul_rn(v, v);
            else ssf_act = fmaf(v, v, ssf_act);
        } else {
            const float a = fabsf(v);
            if (a > mx) mx = a;
        }
    }
    if (NORM) {
        // the same statistics and roundings as MODE 0, on the activated row
        float ssf;
        if (EXACT) {
            ss_act = warp_sum_d(ss_act);
            if (lane == 0) red_d[warp] = ss_act;
            __syncthreads();
            double t = 0.0;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += red_d[w];
            ssf = (float)t;
        } else {
            ssf_act = warp_sum(ssf_act);
            if (lane == 0) red_f[warp] = ssf_act;
            __syncthreads();
            float t = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += red_f[w];
            ssf = t;
        }
        const float vn = __fadd_rn(__fmul_rn(ssf, __frcp_rn((float)k)), 1e-5f);
        const float sinv_a = __frcp_rn(__fsqrt_rn(vn));
        __syncthreads();
        for (int i = tid; i < k; i += 256) {
            const float v = __fmul_rn(__fmul_rn(row[i], sinv_a), gamma[i]);
            row[i] = v;
            const float a = fabsf(v);
            if (a > mx) mx = a;
        }
    }
    mx = warp_max(mx);
    if (lane == 0) red_f[warp] = mx;
    __syncthreads();
    mx = red_f[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red_f[w]);
    const float sc = __fmul_rn(mx, 1.0f / 127.0f);
    uint32_t* qrow = reinterpret_cast<uint32_t*>(q + tok * (size_t)k);
    int local = 0;
    for (int w = tid; w < k / 4; w += 256) {
        const int blk = w >> 4, wd = w & 15;
        const int i = wd >> 2, t = wd & 3;
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

// Fast-mode variant of row_quant_kernel: same layout and outputs, 16-byte loads and stores, hardware
// exp / divide approximations and f32 sums (the exact mode keeps the kernel above, whose every rounding
// step follows the reference).
template <int MODE, bool NORM = false, typename InT = float>
__global__ void __launch_bounds__(256)
row_quant_fast_kernel(const InT* __restrict__ in, const float* __restrict__ gamma, int k, int in_stride,
                      int8_t* __restrict__ q, float* __restrict__ s, int32_t* __restrict__ qsum, float* __restrict__ f_out)
{
    extern __shared__ __align__(16) float row[];
    __shared__ float red_f[8];
    __shared__ int red_i[8];
    const size_t tok = blockIdx.x;
    const InT* xr = in + tok * (size_t)in_stride;
    float4* row4 = reinterpret_cast<float4*>(row);
    float4* f4 = f_out ? reinterpret_cast<float4*>(f_out + tok * (size_t)k) : nullptr;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nv = k >> 2;
    pdl_launch();
    pdl_wait();

    float sinv = 0.0f;
    if (MODE == 0) {
        float ss = 0.0f;
        for (int c = tid; c < nv; c += 256) {
            const float4 v = ld_in4<InT>(xr + 4 * c);
            row4[c] = v;
            ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
        }
        ss = warp_sum(ss);
        if (lane == 0) red_f[warp] = ss;
        __syncthreads();
        ss = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) ss += red_f[w];
        sinv = rsqrtf(ss / (float)k + 1e-5f);
        __syncthreads();
    }
    float mx = 0.0f, ss_act = 0.0f;
    for (int c = tid; c < nv; c += 256) {
        float4 v;
        if (MODE == 0) {
            const float4 x = row4[c];
            const float4 g = reinterpret_cast<const float4*>(gamma)[c];
            v = make_float4(x.x * sinv * g.x, x.y * sinv * g.y, x.z * sinv * g.z, x.w * sinv * g.w);
        } else if (MODE == 1) {
            const float4 x = ld_in4<InT>(xr + 4 * c);
            v = make_float4(__fdividef(x.x, 1.0f + __expf(-1.702f * x.x)), __fdividef(x.y, 1.0f + __expf(-1.702f * x.y)),
                            __fdividef(x.z, 1.0f + __expf(-1.702f * x.z)), __fdividef(x.w, 1.0f + __expf(-1.702f * x.w)));
        } else if (MODE == 2) {
            const float4 g = ld_in4<InT>(xr + 4 * c), u = ld_in4<InT>(xr + 4 * (nv + c));
            v = make_float4(__fdividef(g.x, 1.0f + __expf(-g.x)) * u.x, __fdividef(g.y, 1.0f + __expf(-g.y)) * u.y,
                            __fdividef(g.z, 1.0f + __expf(-g.z)) * u.z, __fdividef(g.w, 1.0f + __expf(-g.w)) * u.w);
        } else if (MODE == 4) {
            const float4 g = ld_in4<InT>(xr + 4 * c), u = ld_in4<InT>(xr + 4 * (nv + c));
            const float4 r = make_float4(fmaxf(g.x, 0.f), fmaxf(g.y, 0.f), fmaxf(g.z, 0.f), fmaxf(g.w, 0.f));
            v = make_float4(__fmul_rn(__fmul_rn(r.x, r.x), u.x), __fmul_rn(__fmul_rn(r.y, r.y), u.y),
                            __fmul_rn(__fmul_rn(r.z, r.z), u.z), __fmul_rn(__fmul_rn(r.w, r.w), u.w));
        } else {
            v = ld_in4<InT>(xr + 4 * c);
        }
        row4[c] = v;
        if (f4) f4[c] = v;
        if (NORM) ss_act = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss_act))));
        else mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    if (NORM) {
        ss_act = warp_sum(ss_act);
        if (lane == 0) red_f[warp] = ss_act;
        __syncthreads();
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red_f[w];
        const float sinv_a = rsqrtf(t / (float)k + 1e-5f);
        __syncthreads();
        for (int c = tid; c < nv; c += 256) {
            const float4 x = row4[c];
            const float4 g = reinterpret_cast<const float4*>(gamma)[c];
            const float4 v = make_float4(x.x * sinv_a * g.x, x.y * sinv_a * g.y, x.z * sinv_a * g.z, x.w * sinv_a * g.w);
            row4[c] = v;
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    }
    mx = warp_max(mx);
    if (lane == 0) red_f[warp] = mx;
    __syncthreads();
    mx = red_f[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red_f[w]);
    const float sc = __fmul_rn(mx, 1.0f / 127.0f);
    const float inv = sc > 0.0f ? 1.0f / sc : 0.0f;
    uint32_t* qrow = reinterpret_cast<uint32_t*>(q + tok * (size_t)k);
    int local = 0;
    for (int w = tid; w < nv; w += 256) {
        const int blk = w >> 4, wd = w & 15;
        const int i = wd >> 2, t = wd & 3;
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            float v = row[blk * 64 + 16 * t + 4 * b + i] * inv;
            v = (v != v) ? 0.0f : fminf(fmaxf(v, -127.0f), 127.0f);
            const int qi = (int)roundf(v);
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

template <int MODE, bool NORM = false, typename InT = float>
static nnb_status launch_row_quant_mode(nnb_engine* e, bool exact, const InT* in,
                                        const float* gamma, size_t t, size_t k, size_t in_stride,
                                        int8_t* q, float* s, int32_t* qsum, float* f_out)
{
    const size_t smem = k * sizeof(float);
    static bool cfg_dev[64] = {}; bool& cfg = cfg_dev[e->device & 63];  // the attribute is per device
    if (!cfg) {
        NNB_CUDA(cudaFuncSetAttribute(row_quant_kernel<MODE, true, NORM, InT>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        NNB_CUDA(cudaFuncSetAttribute(row_quant_kernel<MODE, false, NORM, InT>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        NNB_CUDA(cudaFuncSetAttribute(row_quant_fast_kernel<MODE, NORM, InT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        cfg = true;
    }
    const bool aligned = in_stride % 4 == 0 && ((uintptr_t)in & 15) == 0 && (!f_out || ((uintptr_t)f_out & 15) == 0) &&
                         ((MODE != 0 && !NORM) || ((uintptr_t)gamma & 15) == 0);
    if (exact)
        row_quant_kernel<MODE, true, NORM, InT><<<(unsigned)t, 256, smem, e->stream>>>(in, gamma, (int)k, (int)in_stride, q, s, qsum,
                                                                                        f_out);
    else if (aligned)
        launch_ex(e, row_quant_fast_kernel<MODE, NORM, InT>, dim3((unsigned)t), dim3(256), smem, in, gamma, (int)k, (int)in_stride, q,
                  s, qsum, f_out);
    else
        row_quant_kernel<MODE, false, NORM, InT><<<(unsigned)t, 256, smem, e->stream>>>(in, gamma, (int)k, (int)in_stride, q, s, qsum,
                                                                                         f_out);
    e->launches++;
    NNB_CHECK_LAUNCH("row_quant_kernel");
    return NNB_OK;
}

template <typename InT>
static nnb_status launch_row_quant_act(nnb_engine* e, int mode, bool norm_after, bool exact, const InT* in, const float* gamma,
                                       size_t t, size_t k, size_t in_stride, int8_t* q, float* s, int32_t* qsum, float* f_out)
{
    if (norm_after) switch (mode) {
            case 1: return launch_row_quant_mode<1, true, InT>(e, exact, in, gamma, t, k, in_stride, q, s, qsum, f_out);
            case 2: return launch_row_quant_mode<2, true, InT>(e, exact, in, gamma, t, k, in_stride, q, s, qsum, f_out);
            default: return launch_row_quant_mode<4, true, InT>(e, exact, in, gamma, t, k, in_stride, q, s, qsum, f_out);
        }
    switch (mode) {
        case 1: return launch_row_quant_mode<1, false, InT>(e, exact, in, gamma, t, k, in_stride, q, s, qsum, f_out);
        case 2: return launch_row_quant_mode<2, false, InT>(e, exact, in, gamma, t, k, in_stride, q, s, qsum, f_out);
        default: return launch_row_quant_mode<4, false, InT>(e, exact, in, gamma, t, k, in_stride, q, s, qsum, f_out);
    }
}

// norm_after: modes 1, 2, 4 only; the activated row is RMS-normalised with gamma before it is quantised.
// in_bf16: modes 1, 2, 4 only; `in` points at bf16 elements (in_stride counts elements)
nnb_status launch_row_quant(nnb_engine* e, int mode, bool exact, const float* in, const float* gamma,
                            size_t t, size_t k, size_t in_stride, int8_t* q, float* s,
                            int32_t* qsum, float* f_out, bool norm_after, bool in_bf16)
{
    NNB_REQUIRE(in && q && s && qsum && t > 0, "row_quant: bad arguments");
    NNB_REQUIRE(k > 0 && k % 64 == 0 && k * 4 <= 96 * 1024, "row_quant: k=%zu must be a multiple of 64 (<= 24576)", k);
    const bool act_mode = mode == 1 || mode == 2 || mode == 4;
    NNB_REQUIRE(!norm_after || (gamma && act_mode), "row_quant: the norm after an activation needs gamma");
    NNB_REQUIRE(!in_bf16 || (act_mode && !exact), "row_quant: bf16 input is for the activation modes of the fast mode");
    if (act_mode) {
        if (in_bf16)
            return launch_row_quant_act<__nv_bfloat16>(e, mode, norm_after, exact, reinterpret_cast<const __nv_bfloat16*>(in), gamma, t, k,
                                                       in_stride, q, s, qsum, f_out);
        return launch_row_quant_act<float>(e, mode, norm_after, exact, in, gamma, t, k, in_stride, q, s, qsum, f_out);
    }
    switch (mode) {
        case 0:
            NNB_REQUIRE(gamma, "row_quant: RMSNorm needs gamma");
            return launch_row_quant_mode<0>(e, exact, in, gamma, t, k, in_stride, q, s, qsum, f_out);
        case 3: return launch_row_quant_mode<3>(e, exact, in, gamma, t, k, in_stride, q, s, qsum, f_out);
    }
    NNB_FAIL(NNB_ERR_INVALID, "row_quant: unknown mode %d", mode);
}

// ------------------------------------------------- decode attention (one new token)
template <typename KV>
__device__ __forceinline__ void load4(const KV* p, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&v)[4])
{
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4])
{
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
template <typename KV>
__device__ __forceinline__ KV to_kv(float v);
template <>
__device__ __forceinline__ float to_kv<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 to_kv<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <typename KV>
__device__ __forceinline__ float from_kv(KV v);
template <>
__device__ __forceinline__ float from_kv<float>(float v) { return v; }
template <>
__device__ __forceinline__ float from_kv<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// grid = B*H, block = 128.  qkv is (3, B, d) f32 (the three projections of the new token).
// Two caches per layer, both (sequence, head, position, dk): a prefix cache shared by the `group`
// consecutive sequences that were given the same prompt (positions [0, pre_len), one row block per
// group) and the sequence's own cache (positions pre_len + i).  With group == 1 / pre_len == 0 only the
// own cache is used.
// 1. RoPE on q and k at position pos; k, v appended to the own cache at row pos - pre_len
// 2. scores_j = (q . k_j) * scale for j <= pos; softmax; out = sum_j p_j v_j
template <typename KV, bool EXACT>
__global__ void __launch_bounds__(128)
attn_decode_kernel(const AttnIn in, KV* __restrict__ kcache, KV* __restrict__ vcache, int own_alloc,
                   const KV* __restrict__ kpre, const KV* __restrict__ vpre, int pre_len, int pre_alloc, int group,
                   const float* __restrict__ rope_cos, const float* __restrict__ rope_sin,
                   const int* __restrict__ d_pos, int B, int H, int dk, int ctx_total, float scale,
                   float* __restrict__ out)
{
    typedef typename AccT<EXACT>::type acc_t;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* qs = reinterpret_cast<float*>(smem_raw);        // dk (padded to 128)
    float* sc = qs + 128;                                  // ctx_total
    acc_t* red = reinterpret_cast<acc_t*>(sc + ((ctx_total + 3) & ~3));  // 8 * dk
    __shared__ float bcast[4];
    __shared__ acc_t bsum[4];

    const int b = blockIdx.x / H, h = blockIdx.x % H;
    const int d = H * dk;
    const int pos = *d_pos;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hkv = H / in.kv_rep, hk = h / in.kv_rep;  // grouped-query attention: kv_rep query heads read one KV head
    const size_t head_off = ((size_t)b * Hkv + hk) * (size_t)own_alloc * dk;
    KV* kc = kcache + head_off - (size_t)pre_len * dk;   // indexed by absolute position >= pre_len
    KV* vc = vcache + head_off - (size_t)pre_len * dk;
    const size_t pre_off = ((size_t)(b / group) * Hkv + hk) * (size_t)pre_alloc * dk;
    const KV* kp = kpre ? kpre + pre_off : nullptr;
    const KV* vp = vpre ? vpre + pre_off : nullptr;
    const float* qn = in.q + (size_t)b * in.stride + (size_t)h * dk;
    const float* kn = in.k + (size_t)b * in.stride + (size_t)hk * dk;
    const float* vn = in.v + (size_t)b * in.stride + (size_t)hk * dk;

    // 1. RoPE + append
    if (rope_cos) {
        const int half = dk / 2;
        for (int j = tid; j < half; j += 128) {
            const float c = rope_cos[(size_t)pos * half + j], sn = rope_sin[(size_t)pos * half + j];
            const float qa = qn[j], qb = qn[j + half];
            const float ka = kn[j], kb = kn[j + half];
            qs[j] = __fadd_rn(__fmul_rn(qa, c), __fmul_rn(-qb, sn));
            qs[j + half] = __fadd_rn(__fmul_rn(qb, c), __fmul_rn(qa, sn));
            kc[(size_t)pos * dk + j] = to_kv<KV>(__fadd_rn(__fmul_rn(ka, c), __fmul_rn(-kb, sn)));
            kc[(size_t)pos * dk + j + half] = to_kv<KV>(__fadd_rn(__fmul_rn(kb, c), __fmul_rn(ka, sn)));
        }
    } else {
        for (int j = tid; j < dk; j += 128) {
            qs[j] = qn[j];
            kc[(size_t)pos * dk + j] = to_kv<KV>(kn[j]);
        }
    }
    for (int j = tid; j < dk; j += 128) vc[(size_t)pos * dk + j] = to_kv<KV>(vn[j]);
    __syncthreads();

    // lane mapping: LPK lanes per key, 4 contiguous features per lane
    const int LPK = dk <= 64 ? 16 : 32;
    const int KPW = 32 / LPK;  // keys per warp iteration
    const int sub = lane / LPK, sl = lane % LPK;
    const int e0 = sl * 4;
    const bool act = e0 < dk;
    float qv[4] = {0.f, 0.f, 0.f, 0.f};
    if (act) {
#pragma unroll
        for (int i = 0; i < 4; ++i) qv[i] = qs[e0 + i];
    }
    const int n_keys = pos + 1;
    const int key_stride = 4 * KPW;

    // 2a. scores
    for (int j0 = warp * KPW; j0 < n_keys; j0 += key_stride) {
        const int j = j0 + sub;
        acc_t part = 0;
        if (act && j < n_keys) {
            float kv[4];
            load4<KV>((j < pre_len ? kp : kc) + (size_t)j * dk + e0, kv);
#pragma unroll
            for (int i = 0; i < 4; ++i) part += (acc_t)qv[i] * (acc_t)kv[i];
        }
        for (int o = LPK / 2; o > 0; o >>= 1) part += shfl_xor_t(part, o);
        if (sl == 0 && j < n_keys) sc[j] = __fmul_rn((float)part, scale);
    }
    __syncthreads();
    // 2b. softmax over sc[0..n_keys)
    float mx = -INFINITY;
    for (int j = tid; j < n_keys; j += 128) mx = fmaxf(mx, sc[j]);
    mx = warp_max(mx);
    if (lane == 0) bcast[warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(bcast[0], bcast[1]), fmaxf(bcast[2], bcast[3]));
    acc_t sum = 0;
    for (int j = tid; j < n_keys; j += 128) {
        const float ev = EXACT ? nnb_expf(__fsub_rn(sc[j], mx)) : __expf(sc[j] - mx);
        sc[j] = ev;
        sum += (acc_t)ev;
    }
    sum = warp_sum_t(sum);
    if (lane == 0) bsum[warp] = sum;
    __syncthreads();
    const float sumf = (float)(bsum[0] + bsum[1] + bsum[2] + bsum[3]);
    for (int j = tid; j < n_keys; j += 128) sc[j] = __fdiv_rn(sc[j], sumf);
    __syncthreads();
    // 2c. out = sum_j p_j v_j
    acc_t o4[4] = {0, 0, 0, 0};
    for (int j0 = warp * KPW; j0 < n_keys; j0 += key_stride) {
        const int j = j0 + sub;
        if (act && j < n_keys) {
            float vv[4];
            load4<KV>((j < pre_len ? vp : vc) + (size_t)j * dk + e0, vv);
            const acc_t p = (acc_t)sc[j];
#pragma unroll
            for (int i = 0; i < 4; ++i) o4[i] += p * (acc_t)vv[i];
        }
    }
    const int grp = warp * KPW + sub;  // 0 .. 4*KPW-1
    if (act) {
#pragma unroll
        for (int i = 0; i < 4; ++i) red[(size_t)grp * dk + e0 + i] = o4[i];
    }
    __syncthreads();
    for (int i = tid; i < dk; i += 128) {
        acc_t a = 0;
        for (int gI = 0; gI < 4 * KPW; ++gI) a += red[(size_t)gI * dk + i];
        out[(size_t)b * d + (size_t)h * dk + i] = (float)a;
    }
}

// Fast-mode variant of attn_decode_kernel for a bf16 cache and head dims 64 / 128: same arguments and
// the same two passes, but every lane reads 16 bytes (8 features) of a key, DK/8 lanes share a key, and
// each lane group keeps U keys in flight, so one CTA has 4*U*512 bytes of cache reads outstanding.
__device__ __forceinline__ void bf16x8_to_float(const uint4& t, float (&v)[8])
{
    v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
    v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
    v[4] = __uint_as_float(t.z << 16); v[5] = __uint_as_float(t.z & 0xffff0000u);
    v[6] = __uint_as_float(t.w << 16); v[7] = __uint_as_float(t.w & 0xffff0000u);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// DK is the head size, DKP the row pitch of the caches in elements: DK rounded up to a multiple of 8, so that
// every key starts on a 16-byte boundary (head size 100 -> pitch 104; the pad features are kept at zero).
template <int DK, int DKP>
__global__ void __launch_bounds__(128)
attn_decode_bf16_kernel(const AttnIn in, __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                        int own_alloc, const __nv_bfloat16* __restrict__ kpre, const __nv_bfloat16* __restrict__ vpre,
                        int pre_len, int pre_alloc, int group, const float* __restrict__ rope_cos,
                        const float* __restrict__ rope_sin, const int* __restrict__ d_pos, int B, int H, int ctx_total,
                        float scale, float* __restrict__ out)
{
    static_assert(DKP % 8 == 0 && DKP >= DK && DKP <= 128, "cache pitch: a multiple of 8 elements, at most 128");
    constexpr int LPK = DKP <= 64 ? 8 : 16;  // lanes per key (a power of two; lanes past DKP/8 idle)
    constexpr int KPW = 32 / LPK;            // keys per warp-wide load
    constexpr int G = 4 * KPW;               // lane groups per CTA
    constexpr int U = 4;                     // keys in flight per lane group
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* qs = reinterpret_cast<float*>(smem_raw);  // DKP
    float* red = qs + DKP;                           // G * DKP
    float* sc = red + G * DKP;                       // ctx_total
    __shared__ float bcast[4];
    __shared__ float bsum[4];

    const int b = blockIdx.x / H, h = blockIdx.x % H;
    const int d = H * DK;
    const int pos = *d_pos;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int Hkv = H / in.kv_rep, hk = h / in.kv_rep;  // grouped-query attention: kv_rep query heads read one KV head
    const size_t head_off = ((size_t)b * Hkv + hk) * (size_t)own_alloc * DKP;
    __nv_bfloat16* kc = kcache + head_off - (size_t)pre_len * DKP;  // indexed by absolute position >= pre_len
    __nv_bfloat16* vc = vcache + head_off - (size_t)pre_len * DKP;
    const size_t pre_off = ((size_t)(b / group) * Hkv + hk) * (size_t)pre_alloc * DKP;
    const __nv_bfloat16* kp = kpre ? kpre + pre_off : nullptr;
    const __nv_bfloat16* vp = vpre ? vpre + pre_off : nullptr;
    const float* qn = in.q + (size_t)b * in.stride + (size_t)h * DK;
    const float* kn = in.k + (size_t)b * in.stride + (size_t)hk * DK;
    const float* vn = in.v + (size_t)b * in.stride + (size_t)hk * DK;

    if (rope_cos) {
        constexpr int half = DK / 2;
        for (int j = tid; j < half; j += 128) {
            const float c = rope_cos[(size_t)pos * half + j], sn = rope_sin[(size_t)pos * half + j];
            const float qa = qn[j], qb = qn[j + half];
            const float ka = kn[j], kb = kn[j + half];
            qs[j] = __fadd_rn(__fmul_rn(qa, c), __fmul_rn(-qb, sn));
            qs[j + half] = __fadd_rn(__fmul_rn(qb, c), __fmul_rn(qa, sn));
            kc[(size_t)pos * DKP + j] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(ka, c), __fmul_rn(-kb, sn)));
            kc[(size_t)pos * DKP + j + half] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(kb, c), __fmul_rn(ka, sn)));
        }
    } else {
        for (int j = tid; j < DK; j += 128) {
            qs[j] = qn[j];
            kc[(size_t)pos * DKP + j] = __float2bfloat16_rn(kn[j]);
        }
    }
    for (int j = tid; j < DK; j += 128) vc[(size_t)pos * DKP + j] = __float2bfloat16_rn(vn[j]);
    if (DKP > DK && tid < DKP - DK) {
        qs[DK + tid] = 0.0f;
        kc[(size_t)pos * DKP + DK + tid] = __float2bfloat16_rn(0.0f);
        vc[(size_t)pos * DKP + DK + tid] = __float2bfloat16_rn(0.0f);
    }
    __syncthreads();

    const int sub = lane / LPK, sl = lane % LPK;
    const int g = warp * KPW + sub;
    const int e0 = sl * 8;
    const bool act = e0 < DKP;
    float qv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) qv[i] = act ? qs[e0 + i] : 0.0f;
    const int n_keys = pos + 1;

    // scores
    for (int base = 0; base < n_keys; base += G * U) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = base + u * G + g;
            raw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (act && j < n_keys) raw[u] = *reinterpret_cast<const uint4*>((j < pre_len ? kp : kc) + (size_t)j * DKP + e0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = base + u * G + g;
            float kv[8];
            bf16x8_to_float(raw[u], kv);
            float part = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) part = fmaf(qv[i], kv[i], part);
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            if (sl == 0 && j < n_keys) sc[j] = part * scale;
        }
    }
    __syncthreads();
    float mx = -INFINITY;
    for (int j = tid; j < n_keys; j += 128) mx = fmaxf(mx, sc[j]);
    mx = warp_max(mx);
    if (lane == 0) bcast[warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(bcast[0], bcast[1]), fmaxf(bcast[2], bcast[3]));
    float sum = 0.0f;
    for (int j = tid; j < n_keys; j += 128) {
        const float ev = __expf(sc[j] - mx);
        sc[j] = ev;
        sum += ev;
    }
    sum = warp_sum(sum);
    if (lane == 0) bsum[warp] = sum;
    __syncthreads();
    const float inv = 1.0f / (bsum[0] + bsum[1] + bsum[2] + bsum[3]);

    // out = sum_j p_j v_j
    float o8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int base = 0; base < n_keys; base += G * U) {
        uint4 raw[U];
        float p[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = base + u * G + g;
            raw[u] = make_uint4(0u, 0u, 0u, 0u);
            p[u] = 0.0f;
            if (act && j < n_keys) {
                raw[u] = *reinterpret_cast<const uint4*>((j < pre_len ? vp : vc) + (size_t)j * DKP + e0);
                p[u] = sc[j];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float vv[8];
            bf16x8_to_float(raw[u], vv);
#pragma unroll
            for (int i = 0; i < 8; ++i) o8[i] = fmaf(p[u], vv[i], o8[i]);
        }
    }
    if (act) {
#pragma unroll
        for (int i = 0; i < 8; ++i) red[g * DKP + e0 + i] = o8[i];
    }
    __syncthreads();
    for (int i = tid; i < DK; i += 128) {
        float a = 0.0f;
#pragma unroll
        for (int gi = 0; gi < G; ++gi) a += red[gi * DKP + i];
        out[(size_t)b * d + (size_t)h * DK + i] = a * inv;
    }
}

template <int DK, int DKP = DK>
static nnb_status launch_attn_decode_bf16(nnb_engine* e, const float* qkv, void* kcache, void* vcache, size_t own_alloc,
                                          const void* kpre, const void* vpre, size_t pre_len, size_t pre_alloc, size_t group,
                                          const float* rope_cos, const float* rope_sin, const int* d_pos, size_t B, size_t H,
                                          float* out, const AttnIn& in)
{
    const size_t ctx_total = pre_len + own_alloc;
    constexpr size_t G = 4 * (32 / (DKP <= 64 ? 8 : 16));
    const size_t smem = (DKP + G * DKP + ((ctx_total + 3) & ~(size_t)3)) * sizeof(float);
    NNB_REQUIRE(smem <= 200 * 1024, "attn_decode: context %zu too long for one CTA", ctx_total);
    auto kern = attn_decode_bf16_kernel<DK, DKP>;
    static size_t cfg_dev[64] = {}; size_t& cfg = cfg_dev[e->device & 63];
    if (smem > cfg) {
        NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cfg = smem;
    }
    (void)qkv;
    kern<<<(unsigned)(B * H), 128, smem, e->stream>>>(in, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, (int)own_alloc,
                                                      (const __nv_bfloat16*)kpre, (const __nv_bfloat16*)vpre, (int)pre_len,
                                                      (int)pre_alloc, (int)group, rope_cos, rope_sin, d_pos, (int)B, (int)H,
                                                      (int)ctx_total, 1.0f / sqrtf((float)DK), out);
    e->launches++;
    NNB_CHECK_LAUNCH("attn_decode_bf16_kernel");
    return NNB_OK;
}

// ---- attention of a whole group's new tokens over the group's shared prompt prefix
__device__ __forceinline__ void ldsm_b16(uint32_t (&r)[4], const void* p)
{
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_t_b16(uint32_t (&r)[4], const void* p)
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

// The sequences of a group (at most 16) share their prompt, so their new tokens attend to the same prefix
// keys and values: one warp takes (group, head), holds the group's 16 rotated queries as one m16 tensor-core
// tile and walks the prefix cache once, instead of every sequence reading it for itself.  It leaves, per
// (sequence, head), the partial softmax over the prefix: pre_ml = (max scaled score, sum of exp) and
// pre_o = sum_j exp(s_j - max) v_j (unnormalised), which attn_decode_fused_kernel merges with the
// sequence's own positions.  grid (n_groups, H/4), 128 threads; queries are rounded to bf16 here.
template <int DK>
__global__ void __launch_bounds__(128)
attn_prefix_kernel(const AttnIn in, const __nv_bfloat16* __restrict__ kpre, const __nv_bfloat16* __restrict__ vpre,
                   int pre_len, int pre_alloc, int group, const float* __restrict__ rope_cos, const float* __restrict__ rope_sin,
                   const int* __restrict__ d_pos, int B, int H, float scale, float* __restrict__ pre_o, float* __restrict__ pre_ml)
{
    constexpr int LD = DK + 8, half = DK / 2, KT = 32;  // KT keys per tile
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw) + (size_t)warp * (16 + 2 * KT) * LD;
    __nv_bfloat16* Ks = Qs + 16 * LD;
    __nv_bfloat16* Vs = Ks + KT * LD;
    const int grp = blockIdx.x, h = blockIdx.y * 4 + warp;
    if (h >= H) return;
    const int pos = *d_pos;

    // the group's queries, rotated, as bf16 rows (rows beyond the group stay zero)
    {
        const int r = lane >> 1;               // member of the group
        const int j0 = (lane & 1) * (half / 2);  // first of this lane's half/2 rotation pairs
        const bool ok = r < group;
        const float* qn = in.q + (size_t)(grp * group + (ok ? r : 0)) * in.stride + (size_t)h * DK;
        for (int j = j0; j < j0 + half / 2; j += 4) {
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f), bq = a;
            if (ok) {
                a = *reinterpret_cast<const float4*>(qn + j);
                bq = *reinterpret_cast<const float4*>(qn + j + half);
            }
            float4 c = make_float4(1.f, 1.f, 1.f, 1.f), sn = make_float4(0.f, 0.f, 0.f, 0.f);
            if (rope_cos) {
                c = *reinterpret_cast<const float4*>(rope_cos + (size_t)pos * half + j);
                sn = *reinterpret_cast<const float4*>(rope_sin + (size_t)pos * half + j);
            }
            uint2 lo, hi;
            lo.x = pack_bf16x2(a.x * c.x - bq.x * sn.x, a.y * c.y - bq.y * sn.y);
            lo.y = pack_bf16x2(a.z * c.z - bq.z * sn.z, a.w * c.w - bq.w * sn.w);
            hi.x = pack_bf16x2(bq.x * c.x + a.x * sn.x, bq.y * c.y + a.y * sn.y);
            hi.y = pack_bf16x2(bq.z * c.z + a.z * sn.z, bq.w * c.w + a.w * sn.w);
            *reinterpret_cast<uint2*>(Qs + r * LD + j) = lo;
            *reinterpret_cast<uint2*>(Qs + r * LD + j + half) = hi;
        }
    }
    __syncwarp();
    uint32_t qf[DK / 16][4];
#pragma unroll
    for (int ks = 0; ks < DK / 16; ++ks) ldsm_b16(qf[ks], Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + ks * 16 + 8 * (lane >> 4));

    const size_t pre_off = ((size_t)grp * (H / in.kv_rep) + h / in.kv_rep) * (size_t)pre_alloc * DK;
    const __nv_bfloat16* kp = kpre + pre_off;
    const __nv_bfloat16* vp = vpre + pre_off;
    float o[DK / 8][4];
#pragma unroll
    for (int i = 0; i < DK / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    constexpr int CH = DK / 8;  // 16-byte chunks per row
    for (int j0 = 0; j0 < pre_len; j0 += KT) {
        __syncwarp();
        for (int i = lane; i < KT * CH; i += 32) {
            const int r = i / CH, c = (i % CH) * 8;
            uint4 kv4 = make_uint4(0u, 0u, 0u, 0u), vv4 = kv4;
            if (j0 + r < pre_len) {
                kv4 = *reinterpret_cast<const uint4*>(kp + (size_t)(j0 + r) * DK + c);
                vv4 = *reinterpret_cast<const uint4*>(vp + (size_t)(j0 + r) * DK + c);
            }
            *reinterpret_cast<uint4*>(Ks + r * LD + c) = kv4;
            *reinterpret_cast<uint4*>(Vs + r * LD + c) = vv4;
        }
        __syncwarp();
        float s[KT / 8][4];
#pragma unroll
        for (int i = 0; i < KT / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < DK / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < KT / 16; ++np) {
                uint32_t bk[4];
                ldsm_b16(bk, Ks + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * LD + ks * 16 + 8 * ((lane >> 3) & 1));
                mma_bf16(s[np * 2], qf[ks], bk[0], bk[1]);
                mma_bf16(s[np * 2 + 1], qf[ks], bk[2], bk[3]);
            }
        }
        float mxv[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = j0 + nt * 8 + 2 * t4 + (c & 1);
                s[nt][c] = key < pre_len ? s[nt][c] * scale : -INFINITY;
                mxv[c >> 1] = fmaxf(mxv[c >> 1], s[nt][c]);
            }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mxv[r] = fmaxf(mxv[r], __shfl_xor_sync(0xffffffffu, mxv[r], 1));
            mxv[r] = fmaxf(mxv[r], __shfl_xor_sync(0xffffffffu, mxv[r], 2));
            const float mnew = fmaxf(m[r], mxv[r]);
            corr[r] = __expf(m[r] - mnew);  // m = -inf on the first tile: exp(-inf) = 0, and l, o are 0 anyway
            m[r] = mnew;
            l[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < DK / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float pj = __expf(s[nt][c] - m[c >> 1]);
                s[nt][c] = pj;
                l[c >> 1] += pj;
            }
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < DK / 16; ++np) {
                uint32_t bv[4];
                ldsm_t_b16(bv, Vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + np * 16 + 8 * (lane >> 4));
                mma_bf16(o[np * 2], pa, bv[0], bv[1]);
                mma_bf16(o[np * 2 + 1], pa, bv[2], bv[3]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = g + 8 * hh;
        if (r >= group) continue;
        const size_t bh = (size_t)(grp * group + r) * H + h;
        float* dst = pre_o + bh * DK;
#pragma unroll
        for (int i = 0; i < DK / 8; ++i)
            *reinterpret_cast<float2*>(dst + i * 8 + 2 * t4) = make_float2(o[i][hh * 2], o[i][hh * 2 + 1]);
        if (t4 == 0) {
            pre_ml[bh * 2] = m[hh];
            pre_ml[bh * 2 + 1] = l[hh];
        }
    }
}

__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, bool valid)
{
    const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
    const int sz = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(sa), "l"(gmem), "r"(sz) : "memory");
}

// Grouped-query decode attention on tensor cores: one CTA per (sequence, KV head).  The REP query heads of the group are
// the rows of one m16 tile (rows beyond REP stay zero), so every cached key and value is loaded once and serves the whole
// group through `mma.sync` bf16; the CTA's 4 warps split the key tiles (32 keys each), each keeps an online softmax over
// its tiles, and the four partial results are merged in shared memory.  Appends the new token's key and value first.
// The cache holds the KV heads only.  Queries are rounded to bf16 here, as in attn_prefix_kernel.
// DK: head size; DKP: row pitch of the caches (DK rounded up to 8 elements, pad features zero); DKM: DK rounded up to the
// 16 features of an mma k-step (the tiles' pad columns stay zero in shared memory).  One query head per KV head (plain
// multi-head attention) is the case REP = 1: the kernel then is a tensor-core streamer for head sizes the CUDA-core
// kernels serve badly (100: 13 of 16 lanes busy there).
template <int DK, int DKP = DK, int DKM = DK>
__global__ void __launch_bounds__(128)
attn_decode_mma_kernel(const AttnIn in, __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache, int own_alloc,
                       const __nv_bfloat16* __restrict__ kpre, const __nv_bfloat16* __restrict__ vpre, int pre_len, int pre_alloc,
                       int group, const float* __restrict__ rope_cos, const float* __restrict__ rope_sin,
                       const int* __restrict__ d_pos, int B, int H, float scale, float* __restrict__ out)
{
    static_assert(DKP % 8 == 0 && DKM % 16 == 0 && DK <= DKP && DKP <= DKM && DKM - DKP <= 8, "pitch and mma padding");
    constexpr int LD = DKM + 8, half = DK / 2, KT = 32, CH = DKP / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // 16 x LD, shared by the warps
    __nv_bfloat16* Ks = Qs + 16 * LD + (size_t)warp * 2 * KT * LD;                  // this warp's key tile
    __nv_bfloat16* Vs = Ks + KT * LD;                                               // and value tile
    // after its last tile a warp parks its partial (o, m, l) over its own key tile: 16 rows x (DK + 2) floats fit in it
    constexpr int PW = DKM + 2;
    static_assert(16 * PW * 4 <= KT * LD * 2, "a warp's partial results fit in its key tile");
    float* mo_w = reinterpret_cast<float*>(Ks);
    const int REP = in.kv_rep, Hkv = H / REP;
    const int b = blockIdx.x / Hkv, hk = blockIdx.x % Hkv;
    const int d = H * DK;
    const int pos = *d_pos;
    const size_t head_off = ((size_t)b * Hkv + hk) * (size_t)own_alloc * DKP;
    __nv_bfloat16* kc = kcache + head_off - (size_t)pre_len * DKP;  // indexed by absolute position >= pre_len
    __nv_bfloat16* vc = vcache + head_off - (size_t)pre_len * DKP;
    const size_t pre_off = ((size_t)(b / group) * Hkv + hk) * (size_t)pre_alloc * DKP;
    const __nv_bfloat16* kp = kpre ? kpre + pre_off : nullptr;
    const __nv_bfloat16* vp = vpre ? vpre + pre_off : nullptr;
    const float* qn = in.q + (size_t)b * in.stride + (size_t)hk * REP * DK;  // the group's query heads are adjacent
    const float* kn = in.k + (size_t)b * in.stride + (size_t)hk * DK;
    const float* vn = in.v + (size_t)b * in.stride + (size_t)hk * DK;

    // rows of the query tile beyond the group's heads: zero
    for (int i = tid; i < (16 - REP) * (LD / 8); i += 128)
        reinterpret_cast<uint4*>(Qs + REP * LD)[i] = make_uint4(0u, 0u, 0u, 0u);
    // pad columns: of the query rows, of every warp's key / value tile (cp.async never writes them), of the cache row
    if constexpr (DKM > DK) {
        constexpr int QPAD = DKM - DK;
        for (int i = tid; i < REP * QPAD; i += 128) Qs[(i / QPAD) * LD + DK + i % QPAD] = __float2bfloat16_rn(0.0f);
        if constexpr (DKM > DKP)
            for (int i = tid; i < 4 * 2 * KT; i += 128)
                *reinterpret_cast<uint4*>(Qs + (16 + i) * LD + DKP) = make_uint4(0u, 0u, 0u, 0u);
        if (DKP > DK && tid < DKP - DK) {
            kc[(size_t)pos * DKP + DK + tid] = __float2bfloat16_rn(0.0f);
            vc[(size_t)pos * DKP + DK + tid] = __float2bfloat16_rn(0.0f);
        }
    }
    // the group's rotated queries as bf16 rows of the m16 tile, the new key and value into the cache
    for (int i = tid; i < REP * half; i += 128) {
        const int r = i / half, j = i % half;
        float c = 1.0f, sn = 0.0f;
        if (rope_cos) {
            c = rope_cos[(size_t)pos * half + j];
            sn = rope_sin[(size_t)pos * half + j];
        }
        const float qa = qn[r * DK + j], qb = qn[r * DK + j + half];
        Qs[r * LD + j] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(qa, c), __fmul_rn(-qb, sn)));
        Qs[r * LD + j + half] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(qb, c), __fmul_rn(qa, sn)));
        if (r == 0) {
            const float ka = kn[j], kb = kn[j + half];
            kc[(size_t)pos * DKP + j] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(ka, c), __fmul_rn(-kb, sn)));
            kc[(size_t)pos * DKP + j + half] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(kb, c), __fmul_rn(ka, sn)));
            vc[(size_t)pos * DKP + j] = __float2bfloat16_rn(vn[j]);
            vc[(size_t)pos * DKP + j + half] = __float2bfloat16_rn(vn[j + half]);
        }
    }
    __syncthreads();
    uint32_t qf[DKM / 16][4];
#pragma unroll
    for (int ks = 0; ks < DKM / 16; ++ks) ldsm_b16(qf[ks], Qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + ks * 16 + 8 * (lane >> 4));

    const int n_keys = pos + 1;
    float o[DKM / 8][4];
#pragma unroll
    for (int i = 0; i < DKM / 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.0f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    // Tiles travel global -> shared memory with cp.async, one commit group per key tile and per value tile, in the order
    // K(t), V(t), K(t+1), V(t+1), ...: the next key tile is requested as soon as the scores of the current one are formed
    // (its buffer is free then), the next value tile right after the P.V product, so a warp always has a tile in flight
    // while it computes.  Rows past the last key are zero-filled.
    auto request = [&](int j0, const __nv_bfloat16* pre, __nv_bfloat16* own, __nv_bfloat16* dst) {
        if (j0 < n_keys) {
            for (int i = lane; i < KT * CH; i += 32) {
                const int r = i / CH, c = (i % CH) * 8;
                const int j = j0 + r;
                const bool ok = j < n_keys;
                // (an unread source still has to be an address inside the cache)
                const __nv_bfloat16* src = ok ? (j < pre_len ? pre : own) + (size_t)j * DKP + c : own + (size_t)pre_len * DKP;
                cp_async16_zfill(dst + r * LD + c, src, ok);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    request(warp * KT, kp, kc, Ks);
    request(warp * KT, vp, vc, Vs);
    for (int j0 = warp * KT; j0 < n_keys; j0 += 4 * KT) {
        asm volatile("cp.async.wait_group 1;\n" ::: "memory");  // K(t) has landed (V(t) may still be on its way)
        __syncwarp();
        float s[KT / 8][4];
#pragma unroll
        for (int i = 0; i < KT / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < DKM / 16; ++ks) {
#pragma unroll
            for (int np = 0; np < KT / 16; ++np) {
                uint32_t bk[4];
                ldsm_b16(bk, Ks + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * LD + ks * 16 + 8 * ((lane >> 3) & 1));
                mma_bf16(s[np * 2], qf[ks], bk[0], bk[1]);
                mma_bf16(s[np * 2 + 1], qf[ks], bk[2], bk[3]);
            }
        }
        __syncwarp();
        request(j0 + 4 * KT, kp, kc, Ks);
        float mxv[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = j0 + nt * 8 + 2 * t4 + (c & 1);
                s[nt][c] = key < n_keys ? s[nt][c] * scale : -INFINITY;
                mxv[c >> 1] = fmaxf(mxv[c >> 1], s[nt][c]);
            }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mxv[r] = fmaxf(mxv[r], __shfl_xor_sync(0xffffffffu, mxv[r], 1));
            mxv[r] = fmaxf(mxv[r], __shfl_xor_sync(0xffffffffu, mxv[r], 2));
            const float mnew = fmaxf(m[r], mxv[r]);
            corr[r] = __expf(m[r] - mnew);  // m = -inf on the first tile: exp(-inf) = 0, and l, o are 0 anyway
            m[r] = mnew;
            l[r] *= corr[r];
        }
#pragma unroll
        for (int i = 0; i < DKM / 8; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
#pragma unroll
        for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float pj = __expf(s[nt][c] - m[c >> 1]);
                s[nt][c] = pj;
                l[c >> 1] += pj;
            }
        asm volatile("cp.async.wait_group 1;\n" ::: "memory");  // V(t) has landed (K(t+1) may still be on its way)
        __syncwarp();
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
            uint32_t pa[4];
            pa[0] = pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
            pa[1] = pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
            pa[2] = pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[3] = pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int np = 0; np < DKM / 16; ++np) {
                uint32_t bv[4];
                ldsm_t_b16(bv, Vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LD + np * 16 + 8 * (lane >> 4));
                mma_bf16(o[np * 2], pa, bv[0], bv[1]);
                mma_bf16(o[np * 2 + 1], pa, bv[2], bv[3]);
            }
        }
        __syncwarp();
        request(j0 + 4 * KT, vp, vc, Vs);
    }
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    // park this warp's partial (o, m, l) of the real rows; a warp without any tile leaves m = -inf, l = 0
    __syncwarp();
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = g + 8 * hh;
        if (r >= REP) continue;
        float* dst = mo_w + (size_t)r * PW;
#pragma unroll
        for (int i = 0; i < DKM / 8; ++i) {
            dst[i * 8 + 2 * t4] = o[i][hh * 2];
            dst[i * 8 + 2 * t4 + 1] = o[i][hh * 2 + 1];
        }
        if (t4 == 0) {
            dst[DKM] = m[hh];
            dst[DKM + 1] = l[hh];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < REP * DK; idx += 128) {
        const int r = idx / DK, i = idx % DK;
        // warp w's partials live in its key tile
        const float* mo0 = reinterpret_cast<const float*>(Qs + 16 * LD);
        constexpr size_t WSTRIDE = (size_t)2 * KT * LD / 2;  // floats between two warps' tiles
        float mall = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mall = fmaxf(mall, mo0[w * WSTRIDE + (size_t)r * PW + DKM]);
        float num = 0.0f, den = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* src = mo0 + w * WSTRIDE + (size_t)r * PW;
            const float wgt = __expf(src[DKM] - mall);  // exp(-inf) = 0 for a warp that saw no key
            num = fmaf(wgt, src[i], num);
            den = fmaf(wgt, src[DKM + 1], den);
        }
        out[(size_t)b * d + (size_t)(hk * REP + r) * DK + i] = num / den;
    }
}

template <int DK, int DKP = DK, int DKM = DK>
static nnb_status launch_attn_decode_mma(nnb_engine* e, void* kcache, void* vcache, size_t own_alloc, const void* kpre,
                                         const void* vpre, size_t pre_len, size_t pre_alloc, size_t group, const float* rope_cos,
                                         const float* rope_sin, const int* d_pos, size_t B, size_t H, float* out, const AttnIn& in)
{
    constexpr size_t LD = DKM + 8;
    const size_t smem = (16 * LD + 4 * 2 * 32 * LD) * sizeof(__nv_bfloat16);
    auto kern = attn_decode_mma_kernel<DK, DKP, DKM>;
    static bool cfg_dev[64] = {}; bool& cfg = cfg_dev[e->device & 63];  // the attribute is per device
    if (!cfg) {
        NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        cfg = true;
    }
    kern<<<(unsigned)(B * (H / (size_t)in.kv_rep)), 128, smem, e->stream>>>(in, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache,
                                                                            (int)own_alloc, (const __nv_bfloat16*)kpre,
                                                                            (const __nv_bfloat16*)vpre, (int)pre_len, (int)pre_alloc,
                                                                            (int)group, rope_cos, rope_sin, d_pos, (int)B, (int)H,
                                                                            1.0f / sqrtf((float)DK), out);
    e->launches++;
    NNB_CHECK_LAUNCH("attn_decode_mma_kernel");
    return NNB_OK;
}

// Decode attention of ALL heads of a sequence in one CTA, one warp per head, followed by the int8
// quantisation of the token's attention output (the input of the output projection): what
// attn_decode_bf16_kernel + row_quant_fast_kernel<3> compute, in one launch and without block-wide
// barriers inside the attention part.  grid = B, block = 32*H (H <= 32).  A warp streams its head's keys
// and values with 16-byte loads, U keys in flight per lane group; with ~55 resident warps per SM that
// keeps > 100 KB of cache reads outstanding per SM.  att (B, d) f32 is optional.
template <int DK, int U, int MAXT>
__global__ void __launch_bounds__(MAXT)
attn_decode_fused_kernel(const AttnIn in, __nv_bfloat16* __restrict__ kcache, __nv_bfloat16* __restrict__ vcache,
                         int own_alloc, const __nv_bfloat16* __restrict__ kpre, const __nv_bfloat16* __restrict__ vpre,
                         int pre_len, int pre_alloc, int group, const float* __restrict__ rope_cos,
                         const float* __restrict__ rope_sin, const int* __restrict__ d_pos, int B, int H, int ctx_pad,
                         float scale, float* __restrict__ att, int8_t* __restrict__ q8, float* __restrict__ s_out,
                         int32_t* __restrict__ qsum_out, const float* __restrict__ pre_o, const float* __restrict__ pre_ml)
{
    constexpr int LPK = DK / 8;    // lanes per key
    constexpr int KPW = 32 / LPK;  // keys per warp-wide load
    // U = keys in flight per lane group: 4 when two 512-thread CTAs share an SM (64 registers per thread), 8 for
    // batches of about one CTA per SM, where the loads of a single CTA have to cover the memory latency
    constexpr int half = DK / 2;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* orow = reinterpret_cast<float*>(smem_raw);  // d
    float* sc_all = orow + H * DK;                     // H * ctx_pad
    __shared__ float red_f[32];
    __shared__ int red_i[32];

    const int b = blockIdx.x, h = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int d = H * DK;
    pdl_launch();
    pdl_wait();
    const int pos = *d_pos;
    float* sc = sc_all + (size_t)h * ctx_pad;
    const int Hkv = H / in.kv_rep, hk = h / in.kv_rep;  // the warps of a KV group append the same key and value
    const size_t head_off = ((size_t)b * Hkv + hk) * (size_t)own_alloc * DK;
    __nv_bfloat16* kc = kcache + head_off - (size_t)pre_len * DK;  // indexed by absolute position >= pre_len
    __nv_bfloat16* vc = vcache + head_off - (size_t)pre_len * DK;
    const size_t pre_off = ((size_t)(b / group) * Hkv + hk) * (size_t)pre_alloc * DK;
    const __nv_bfloat16* kp = kpre ? kpre + pre_off : nullptr;
    const __nv_bfloat16* vp = vpre ? vpre + pre_off : nullptr;
    const float* qn = in.q + (size_t)b * in.stride + (size_t)h * DK;
    const float* kn = in.k + (size_t)b * in.stride + (size_t)hk * DK;
    const float* vn = in.v + (size_t)b * in.stride + (size_t)hk * DK;

    const int sub = lane / LPK, sl = lane % LPK;
    const int e0 = sl * 8;
    // this lane's 8 features of q and of the new key, rotated; the partner half comes from global memory too
    float qv[8], kv_new[8];
    {
        const int ep = e0 < half ? e0 + half : e0 - half;
        float qa[8], qb[8], ka[8], kb[8];
        *reinterpret_cast<float4*>(qa) = *reinterpret_cast<const float4*>(qn + e0);
        *reinterpret_cast<float4*>(qa + 4) = *reinterpret_cast<const float4*>(qn + e0 + 4);
        *reinterpret_cast<float4*>(ka) = *reinterpret_cast<const float4*>(kn + e0);
        *reinterpret_cast<float4*>(ka + 4) = *reinterpret_cast<const float4*>(kn + e0 + 4);
        if (rope_cos) {
            *reinterpret_cast<float4*>(qb) = *reinterpret_cast<const float4*>(qn + ep);
            *reinterpret_cast<float4*>(qb + 4) = *reinterpret_cast<const float4*>(qn + ep + 4);
            *reinterpret_cast<float4*>(kb) = *reinterpret_cast<const float4*>(kn + ep);
            *reinterpret_cast<float4*>(kb + 4) = *reinterpret_cast<const float4*>(kn + ep + 4);
            const float sgn = e0 < half ? -1.0f : 1.0f;  // first half: a*c - b*s, second half: b*c + a*s
            const int j0 = e0 % half;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float c = rope_cos[(size_t)pos * half + j0 + i], sn = sgn * rope_sin[(size_t)pos * half + j0 + i];
                qv[i] = qa[i] * c + qb[i] * sn;
                kv_new[i] = ka[i] * c + kb[i] * sn;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) { qv[i] = qa[i]; kv_new[i] = ka[i]; }
        }
    }
    if (sub == 0) {
        float vv[8];
        *reinterpret_cast<float4*>(vv) = *reinterpret_cast<const float4*>(vn + e0);
        *reinterpret_cast<float4*>(vv + 4) = *reinterpret_cast<const float4*>(vn + e0 + 4);
        uint4 pk, pv;
        pk.x = pack_bf16x2(kv_new[0], kv_new[1]); pk.y = pack_bf16x2(kv_new[2], kv_new[3]);
        pk.z = pack_bf16x2(kv_new[4], kv_new[5]); pk.w = pack_bf16x2(kv_new[6], kv_new[7]);
        pv.x = pack_bf16x2(vv[0], vv[1]); pv.y = pack_bf16x2(vv[2], vv[3]);
        pv.z = pack_bf16x2(vv[4], vv[5]); pv.w = pack_bf16x2(vv[6], vv[7]);
        *reinterpret_cast<uint4*>(kc + (size_t)pos * DK + e0) = pk;
        *reinterpret_cast<uint4*>(vc + (size_t)pos * DK + e0) = pv;
    }
    __syncwarp();
    const int n_keys = pos + 1;
    // With pre_o / pre_ml the shared prefix has been attended to already (attn_prefix_kernel, all members of a
    // group at once): this kernel covers the sequence's own positions and merges the two partial softmaxes.
    const int j_first = pre_o ? pre_len : 0;

    // scores
    float mx = -INFINITY;
    for (int base = j_first; base < n_keys; base += KPW * U) {
        uint4 raw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = base + u * KPW + sub;
            raw[u] = make_uint4(0u, 0u, 0u, 0u);
            if (j < n_keys) raw[u] = *reinterpret_cast<const uint4*>((j < pre_len ? kp : kc) + (size_t)j * DK + e0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = base + u * KPW + sub;
            float kf[8];
            bf16x8_to_float(raw[u], kf);
            float part = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) part = fmaf(qv[i], kf[i], part);
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
            part *= scale;
            if (j < n_keys) {
                mx = fmaxf(mx, part);
                if (sl == 0) sc[j] = part;
            }
        }
    }
    mx = warp_max(mx);
    __syncwarp();
    float sum = 0.0f;
    for (int j = j_first + lane; j < n_keys; j += 32) {
        const float ev = __expf(sc[j] - mx);
        sc[j] = ev;
        sum += ev;
    }
    sum = warp_sum(sum);
    float w_own = 1.0f, w_pre = 0.0f;
    if (pre_o) {
        const float m_pre = pre_ml[((size_t)b * H + h) * 2], l_pre = pre_ml[((size_t)b * H + h) * 2 + 1];
        const float m_all = fmaxf(mx, m_pre);
        w_own = __expf(mx - m_all);
        w_pre = __expf(m_pre - m_all);
        sum = w_own * sum + w_pre * l_pre;
    }
    const float inv = 1.0f / sum;
    __syncwarp();

    // out = sum_j p_j v_j
    float o8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int base = j_first; base < n_keys; base += KPW * U) {
        uint4 raw[U];
        float pj[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int j = base + u * KPW + sub;
            raw[u] = make_uint4(0u, 0u, 0u, 0u);
            pj[u] = 0.0f;
            if (j < n_keys) {
                raw[u] = *reinterpret_cast<const uint4*>((j < pre_len ? vp : vc) + (size_t)j * DK + e0);
                pj[u] = sc[j];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float vf[8];
            bf16x8_to_float(raw[u], vf);
#pragma unroll
            for (int i = 0; i < 8; ++i) o8[i] = fmaf(pj[u], vf[i], o8[i]);
        }
    }
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1)
#pragma unroll
        for (int i = 0; i < 8; ++i) o8[i] += __shfl_xor_sync(0xffffffffu, o8[i], o);
    if (sub == 0) {
        if (pre_o) {
            const float* po = pre_o + ((size_t)b * H + h) * DK + e0;
            const float4 p0 = *reinterpret_cast<const float4*>(po), p1 = *reinterpret_cast<const float4*>(po + 4);
            const float pv[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) o8[i] = w_own * o8[i] + w_pre * pv[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) o8[i] *= inv;
        float* dst = orow + h * DK + e0;
        *reinterpret_cast<float4*>(dst) = make_float4(o8[0], o8[1], o8[2], o8[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(o8[4], o8[5], o8[6], o8[7]);
        if (att) {
            float* ga = att + (size_t)b * d + (size_t)h * DK + e0;
            *reinterpret_cast<float4*>(ga) = make_float4(o8[0], o8[1], o8[2], o8[3]);
            *reinterpret_cast<float4*>(ga + 4) = make_float4(o8[4], o8[5], o8[6], o8[7]);
        }
    }
    __syncthreads();
    if (!q8) return;

    // int8 quantisation of the token's row (same rule and layout as row_quant_fast_kernel)
    const int tid = threadIdx.x, nthr = blockDim.x;
    float amx = 0.0f;
    for (int i = tid; i < d; i += nthr) amx = fmaxf(amx, fabsf(orow[i]));
    amx = warp_max(amx);
    if (lane == 0) red_f[h] = amx;
    __syncthreads();
    amx = red_f[0];
    for (int w = 1; w < H; ++w) amx = fmaxf(amx, red_f[w]);
    const float scq = __fmul_rn(amx, 1.0f / 127.0f);
    const float invq = scq > 0.0f ? 1.0f / scq : 0.0f;
    uint32_t* qrow = reinterpret_cast<uint32_t*>(q8 + (size_t)b * d);
    int local = 0;
    for (int w = tid; w < d / 4; w += nthr) {
        const int blk = w >> 4, wd = w & 15;
        const int i = wd >> 2, t = wd & 3;
        uint32_t word = 0;
#pragma unroll
        for (int bb = 0; bb < 4; ++bb) {
            float v = orow[blk * 64 + 16 * t + 4 * bb + i] * invq;
            v = (v != v) ? 0.0f : fminf(fmaxf(v, -127.0f), 127.0f);
            const int qi = (int)roundf(v);
            local += qi;
            word |= (uint32_t)(uint8_t)(int8_t)qi << (8 * bb);
        }
        qrow[w] = word;
    }
    local = warp_sum_i(local);
    if (lane == 0) red_i[h] = local;
    __syncthreads();
    if (tid == 0) {
        int tot = 0;
        for (int w = 0; w < H; ++w) tot += red_i[w];
        qsum_out[b] = tot;
        s_out[b] = scq;
    }
}

bool attn_decode_fused_supported(size_t H, size_t dk) { return (dk == 64 || dk == 128) && H >= 1 && H <= 32; }

// fast mode only (bf16 caches).  att may be NULL; q8 / s / qsum may be NULL together (attention only).
nnb_status launch_attn_decode_fused(nnb_engine* e, const float* qkv, void* kcache, void* vcache, size_t own_alloc,
                                    const void* kpre, const void* vpre, size_t pre_len, size_t pre_alloc, size_t group,
                                    const float* rope_cos, const float* rope_sin, const int* d_pos, size_t B, size_t H,
                                    size_t dk, float* att, int8_t* q8, float* s, int32_t* qsum, float* pre_o, float* pre_ml,
                                    const AttnIn* in_opt)
{
    NNB_REQUIRE(attn_decode_fused_supported(H, dk), "attn_decode_fused: %zu heads of %zu features unsupported", H, dk);
    const AttnIn in = attn_in_or_planes(in_opt, qkv, B, H * dk);
    NNB_REQUIRE(in.kv_rep >= 1 && H % (size_t)in.kv_rep == 0, "attn_decode_fused: %zu heads do not divide into KV groups of %d", H, in.kv_rep);
    NNB_REQUIRE((pre_o == nullptr) == (pre_ml == nullptr), "attn_decode_fused: pre_o and pre_ml go together");
    // a shared prefix read by groups of at most 16 sequences is attended to once per group
    const bool batched_prefix = pre_o && pre_len > 0 && group > 1 && group <= 16 && B % group == 0;
    if (batched_prefix) {
        const size_t smem_p = 4 * (16 + 64) * (dk + 8) * sizeof(__nv_bfloat16);
        const float scale_p = 1.0f / sqrtf((float)dk);
        dim3 grid_p((unsigned)(B / group), (unsigned)ceil_div(H, 4));
        static bool cfg_p_dev[64] = {}; bool& cfg_p = cfg_p_dev[e->device & 63];  // the attribute is per device
        if (!cfg_p) {
            NNB_CUDA(cudaFuncSetAttribute(attn_prefix_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 80 * 136 * 2));
            NNB_CUDA(cudaFuncSetAttribute(attn_prefix_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 80 * 72 * 2));
            cfg_p = true;
        }
        if (dk == 128)
            attn_prefix_kernel<128><<<grid_p, 128, smem_p, e->stream>>>(in, (const __nv_bfloat16*)kpre, (const __nv_bfloat16*)vpre,
                                                                       (int)pre_len, (int)pre_alloc, (int)group, rope_cos, rope_sin,
                                                                       d_pos, (int)B, (int)H, scale_p, pre_o, pre_ml);
        else
            attn_prefix_kernel<64><<<grid_p, 128, smem_p, e->stream>>>(in, (const __nv_bfloat16*)kpre, (const __nv_bfloat16*)vpre,
                                                                      (int)pre_len, (int)pre_alloc, (int)group, rope_cos, rope_sin,
                                                                      d_pos, (int)B, (int)H, scale_p, pre_o, pre_ml);
        e->launches++;
        NNB_CHECK_LAUNCH("attn_prefix_kernel");
    }
    const float* use_o = batched_prefix ? pre_o : nullptr;
    const float* use_ml = batched_prefix ? pre_ml : nullptr;
    NNB_REQUIRE(group >= 1 && (pre_len == 0 || (kpre && vpre)), "attn_decode_fused: bad prefix arguments");
    NNB_REQUIRE((q8 == nullptr) == (s == nullptr) && (q8 == nullptr) == (qsum == nullptr), "attn_decode_fused: q8, s, qsum go together");
    const size_t ctx_pad = (pre_len + own_alloc + 3) & ~(size_t)3;
    const size_t smem = (H * dk + H * ctx_pad) * sizeof(float);
    NNB_REQUIRE(smem <= 200 * 1024, "attn_decode_fused: context %zu too long for one CTA", pre_len + own_alloc);
    const float scale = 1.0f / sqrtf((float)dk);
    // few sequences (about one CTA per SM or less) and at most 16 heads: the variant with more loads in flight
    const bool deep = H <= 16 && B <= (size_t)e->sm_count * 3 / 2;
#define NNB_FUSED(DKV)                                                                                                    \
    if (deep) NNB_FUSED_V(DKV, 8, 512) else NNB_FUSED_V(DKV, 4, 1024)
#define NNB_FUSED_V(DKV, UV, MT)                                                                                          \
    {                                                                                                                     \
        auto kern = attn_decode_fused_kernel<DKV, UV, MT>;                                                                \
        static size_t cfg_dev[64] = {}; size_t& cfg = cfg_dev[e->device & 63];                                                                                            \
        if (smem > cfg) {                                                                                                 \
            NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                 \
            cfg = smem;                                                                                                   \
        }                                                                                                                 \
        launch_ex(e, kern, dim3((unsigned)B), dim3((unsigned)(32 * H)), smem, in, (__nv_bfloat16*)kcache,                 \
                  (__nv_bfloat16*)vcache, (int)own_alloc, (const __nv_bfloat16*)kpre, (const __nv_bfloat16*)vpre, (int)pre_len, \
                  (int)pre_alloc, (int)group, rope_cos, rope_sin, d_pos, (int)B, (int)H, (int)ctx_pad, scale, att, q8, s, qsum, \
                  use_o, use_ml);                                                                                            \
    }
    if (dk == 128) NNB_FUSED(128) else NNB_FUSED(64)
#undef NNB_FUSED
#undef NNB_FUSED_V
    e->launches++;
    NNB_CHECK_LAUNCH("attn_decode_fused_kernel");
    return NNB_OK;
}

// Row pitch, in elements, of the caches launch_attn_decode expects: the head size, except where the fast kernel
// wants every key on a 16-byte boundary (bf16 caches, head size 100 -> 104, pad features zero).
size_t attn_decode_kv_pitch(bool exact, size_t dk) { return (!exact && dk == 100) ? 104 : dk; }

nnb_status launch_attn_decode(nnb_engine* e, bool exact, const float* qkv, void* kcache, void* vcache,
                              size_t own_alloc, const void* kpre, const void* vpre, size_t pre_len, size_t pre_alloc,
                              size_t group, const float* rope_cos, const float* rope_sin, const int* d_pos, size_t B,
                              size_t H, size_t dk, float* out, size_t kv_pitch, const AttnIn* in_opt)
{
    if (kv_pitch == 0) kv_pitch = dk;
    const AttnIn in = attn_in_or_planes(in_opt, qkv, B, H * dk);
    NNB_REQUIRE(in.kv_rep >= 1 && H % (size_t)in.kv_rep == 0, "attn_decode: %zu heads do not divide into KV groups of %d", H, in.kv_rep);
    NNB_REQUIRE(kv_pitch == dk || kv_pitch == attn_decode_kv_pitch(exact, dk), "attn_decode: cache pitch %zu unsupported for head size %zu",
                kv_pitch, dk);
    NNB_REQUIRE(dk % 4 == 0 && dk <= 128 && dk >= 8, "attn_decode: head dim %zu unsupported (multiple of 4, <= 128)", dk);
    NNB_REQUIRE(group >= 1 && (pre_len == 0 || (kpre && vpre)), "attn_decode: bad prefix arguments");
    // Grouped queries on head sizes 64 / 128 (2 to 16 query heads per KV head): the tensor-core kernel that serves a whole
    // group per CTA.  NNB_GQA_KERNEL=0 in the environment keeps one CTA per query head instead (for A/B timing).
    static int gqa_kernel = -1;
    if (gqa_kernel < 0) {
        const char* ev = getenv("NNB_GQA_KERNEL");
        gqa_kernel = (ev && ev[0] == '0') ? 0 : 1;
    }
    // NNB_MMA_MHA=1 / 0: plain multi-head attention always / never on it (for A/B timing against the CUDA-core kernels)
    static int mma_mha = -1, mma_mha_off = 0;
    if (mma_mha < 0) {
        const char* ev = getenv("NNB_MMA_MHA");
        mma_mha = (ev && ev[0] == '1') ? 1 : 0;
        mma_mha_off = (ev && ev[0] == '0') ? 1 : 0;
    }
    // Plain multi-head attention takes this kernel too when the cache is roomy: measured at 128 sequences x 16 heads of
    // 128, it streams the cache a third faster than the CUDA-core kernel (0.0035 against 0.0052 ms per position over 24
    // layers) but its larger CTAs cost 0.3 ms more per step at short contexts; the break-even is near 200 positions.
    const bool roomy = pre_len + own_alloc >= 512 && !mma_mha_off;
    if (!exact && gqa_kernel && (in.kv_rep >= 2 || mma_mha || roomy) && in.kv_rep <= 16 && (dk == 128 || dk == 64)) {
        if (dk == 128)
            return launch_attn_decode_mma<128>(e, kcache, vcache, own_alloc, kpre, vpre, pre_len, pre_alloc, group, rope_cos,
                                               rope_sin, d_pos, B, H, out, in);
        return launch_attn_decode_mma<64>(e, kcache, vcache, own_alloc, kpre, vpre, pre_len, pre_alloc, group, rope_cos, rope_sin,
                                          d_pos, B, H, out, in);
    }
    if (!exact && dk == 128)
        return launch_attn_decode_bf16<128>(e, qkv, kcache, vcache, own_alloc, kpre, vpre, pre_len, pre_alloc, group, rope_cos,
                                            rope_sin, d_pos, B, H, out, in);
    if (!exact && dk == 64)
        return launch_attn_decode_bf16<64>(e, qkv, kcache, vcache, own_alloc, kpre, vpre, pre_len, pre_alloc, group, rope_cos,
                                           rope_sin, d_pos, B, H, out, in);
    // head size 100 (caches of pitch attn_decode_kv_pitch(false, 100) = 104): the tensor-core streamer, multi-head or
    // grouped; NNB_MMA_DK100=0 in the environment keeps the CUDA-core kernel (for A/B timing)
    static int mma100 = -1;
    if (mma100 < 0) {
        const char* ev = getenv("NNB_MMA_DK100");
        mma100 = (ev && ev[0] == '0') ? 0 : 1;
    }
    // (below a few hundred cached positions the CUDA-core kernel's lighter prologue wins: measured crossover at ~150
    // positions for 128 sequences x 32 heads; the choice goes by the cache's capacity, known on the host)
    if (!exact && dk == 100 && kv_pitch == 104 && mma100 && in.kv_rep <= 16 && pre_len + own_alloc >= 512)
        return launch_attn_decode_mma<100, 104, 112>(e, kcache, vcache, own_alloc, kpre, vpre, pre_len, pre_alloc, group, rope_cos,
                                                     rope_sin, d_pos, B, H, out, in);
    if (!exact && dk == 100 && kv_pitch == 104)  // caches of pitch attn_decode_kv_pitch(false, 100)
        return launch_attn_decode_bf16<100, 104>(e, qkv, kcache, vcache, own_alloc, kpre, vpre, pre_len, pre_alloc, group,
                                                 rope_cos, rope_sin, d_pos, B, H, out, in);
    const float scale = 1.0f / sqrtf((float)dk);
    const size_t acc_sz = exact ? 8 : 4;
    const size_t ctx_total = pre_len + own_alloc;
    const size_t smem = 128 * 4 + ((ctx_total + 3) & ~(size_t)3) * 4 + 8 * dk * acc_sz + 16;
    NNB_REQUIRE(smem <= 200 * 1024, "attn_decode: context %zu too long for one CTA", ctx_total);
    const unsigned grid = (unsigned)(B * H);
    if (exact) {
        auto kern = attn_decode_kernel<float, true>;
        static size_t cfg_dev[64] = {}; size_t& cfg = cfg_dev[e->device & 63];
        if (smem > cfg) {
            NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            cfg = smem;
        }
        kern<<<grid, 128, smem, e->stream>>>(in, (float*)kcache, (float*)vcache, (int)own_alloc, (const float*)kpre,
                                             (const float*)vpre, (int)pre_len, (int)pre_alloc, (int)group, rope_cos, rope_sin,
                                             d_pos, (int)B, (int)H, (int)dk, (int)ctx_total, scale, out);
    } else {
        auto kern = attn_decode_kernel<__nv_bfloat16, false>;
        static size_t cfg_dev[64] = {}; size_t& cfg = cfg_dev[e->device & 63];
        if (smem > cfg) {
            NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            cfg = smem;
        }
        kern<<<grid, 128, smem, e->stream>>>(in, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, (int)own_alloc,
                                             (const __nv_bfloat16*)kpre, (const __nv_bfloat16*)vpre, (int)pre_len,
                                             (int)pre_alloc, (int)group, rope_cos, rope_sin, d_pos, (int)B, (int)H, (int)dk,
                                             (int)ctx_total, scale, out);
    }
    e->launches++;
    NNB_CHECK_LAUNCH("attn_decode_kernel");
    return NNB_OK;
}

// ------------------------------------------------------------------ sampler
__device__ __forceinline__ float key_float(uint32_t k)  // inverse of float_key
{
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}
__device__ __forceinline__ uint32_t float_key(float v)
{
    // order-preserving map float -> uint32 (larger float -> larger key)
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One CTA (1024 threads) per sequence.  logits (B, V) f32.  Writes the chosen token at
// tokens[b, pos+1], and log softmax(raw logits)[token] into logp[b, gen_index] where
// gen_index = pos + 1 - prompt_len.
// The row is read from global memory once and kept in shared memory.  Top-k: radix select of the k-th largest
// key (8 bits per pass, one histogram per warp so that only lanes of a warp contend), an ordered compaction by
// a block-wide scan, then the candidates' softmax: exponentials and quotients in parallel, the two running
// sums in ascending index order by one thread, which is the order the reference's sampler adds them in.
constexpr int SAMPLE_NT = 1024, SAMPLE_NW = SAMPLE_NT / 32;

__device__ __forceinline__ void block_scan2(int& a, int& b, int* wa, int* wb, int& tot_a, int& tot_b)
{
    // exclusive scan of (a, b) over the block's threads; wa/wb: SAMPLE_NW ints each
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int ia = a, ib = b;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int ta = __shfl_up_sync(0xffffffffu, ia, o), tb = __shfl_up_sync(0xffffffffu, ib, o);
        if (lane >= o) { ia += ta; ib += tb; }
    }
    if (lane == 31) { wa[warp] = ia; wb[warp] = ib; }
    __syncthreads();
    if (warp == 0) {
        int va = wa[lane], vb = wb[lane];
        int sa = va, sb = vb;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int ta = __shfl_up_sync(0xffffffffu, sa, o), tb = __shfl_up_sync(0xffffffffu, sb, o);
            if (lane >= o) { sa += ta; sb += tb; }
        }
        wa[lane] = sa - va;  // exclusive prefix of the warp totals
        wb[lane] = sb - vb;
        if (lane == 31) { wa[SAMPLE_NW] = sa; wb[SAMPLE_NW] = sb; }
    }
    __syncthreads();
    tot_a = wa[SAMPLE_NW];
    tot_b = wb[SAMPLE_NW];
    a = wa[warp] + ia - a;
    b = wb[warp] + ib - b;
}

// SamplingConfig beyond temperature and top-k, in the reference's order (compute_layer_base.hpp:1025-1163):
// logit bias (the device-side stand-in for the host logits_transform hook) -> repeat penalty over the distinct
// tokens of the history window (the sequence so far, prompt included; positive logits are divided, others
// multiplied) -> temperature -> top-k -> softmax over the candidates -> top-p (smallest prefix, by probability
// descending and index ascending, whose running sum of p reaches top_p; at least one; the kept set is
// renormalised in ascending index order) -> greedy or inverse CDF.  End of sequence: once a sequence has
// sampled `eos` at a generated index >= min_new it is marked done, its length is recorded, and every later
// token of it is `eos` (GPTModel::generate stops there, compute_layer_gpt.hpp:826-828).
template <bool EXACT>
__global__ void __launch_bounds__(SAMPLE_NT)
sample_kernel(const float* __restrict__ logits, int V, SampleOpts o,
              unsigned long long seed, unsigned seq0, const int* __restrict__ d_pos, int prompt_len,
              int32_t* __restrict__ tokens, int tokens_stride, float* __restrict__ logp, int logp_stride,
              float* __restrict__ entropy)
{
    const float temperature = o.temperature;
    const int top_k = o.top_k;
    typedef typename AccT<EXACT>::type acc_t;
    constexpr int NT = SAMPLE_NT, NW = SAMPLE_NW;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // V (raw, then scaled) logits: in shared memory, or in the caller's scratch when a row is too large for it
    const int Vp = (V + 3) & ~3;
    float* lg = o.row_scratch ? o.row_scratch + (size_t)blockIdx.x * Vp : reinterpret_cast<float*>(smem_raw);
    int* cand = reinterpret_cast<int*>(reinterpret_cast<float*>(smem_raw) + (o.row_scratch ? 0 : Vp));  // up to 1024 candidates
    float* cval = reinterpret_cast<float*>(cand + 1024);       // their exponentials, then probabilities
    int* whist = reinterpret_cast<int*>(cval + 1024);          // NW x 256 per-warp histograms
    __shared__ int hist[256];
    __shared__ int scan_a[NW + 1], scan_b[NW + 1];
    __shared__ float red_f[NW];
    __shared__ int red_i[NW];
    __shared__ acc_t red_a[NW];
    __shared__ uint32_t sh_prefix;
    __shared__ int sh_need, sh_tok;

    const int b = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_launch();
    pdl_wait();
    const int pos = d_pos[1];  // the column of the token buffer this step consumed (d_pos[0] is its window position)
    const int gen = pos + 1 - prompt_len;
    const float* row = logits + (size_t)b * V;

    // raw max and log-sum-exp (for the recorded log-prob)
    float mx = -INFINITY;
    for (int i = tid; i < V; i += NT) {
        const float v = row[i];
        lg[i] = v;
        mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    if (lane == 0) red_f[warp] = mx;
    __syncthreads();
    mx = red_f[0];
#pragma unroll
    for (int w = 1; w < NW; ++w) mx = fmaxf(mx, red_f[w]);
    acc_t se = 0, sxe = 0;
    for (int i = tid; i < V; i += NT) {
        const float dlt = lg[i] - mx;
        const float ev = EXACT ? expf(dlt) : __expf(dlt);
        se += (acc_t)ev;
        if (entropy) sxe += (acc_t)ev * (acc_t)dlt;
    }
    se = warp_sum_t(se);
    sxe = warp_sum_t(sxe);
    __syncthreads();
    if (lane == 0) red_a[warp] = se;
    __syncthreads();
    acc_t se_tot = 0;
#pragma unroll
    for (int w = 0; w < NW; ++w) se_tot += red_a[w];
    __syncthreads();
    if (lane == 0) red_a[warp] = sxe;
    __syncthreads();
    acc_t sxe_tot = 0;
#pragma unroll
    for (int w = 0; w < NW; ++w) sxe_tot += red_a[w];
    const float lse = logf((float)se_tot);  // log sum exp(x - mx)
    __syncthreads();

    if (o.logit_bias) {
        for (int i = tid; i < V; i += NT) lg[i] = __fadd_rn(lg[i], o.logit_bias[i]);
        __syncthreads();
    }
    if (o.repeat_penalty > 0.0f && o.repeat_penalty != 1.0f) {
        // one bit per vocabulary entry (the histogram area is free here): whoever sets a token's bit first applies
        // the penalty, so every distinct token of the window is penalised exactly once
        uint32_t* seen = reinterpret_cast<uint32_t*>(whist);
        const int n_words = (V + 31) >> 5;
        for (int i = tid; i < n_words; i += NT) seen[i] = 0u;
        __syncthreads();
        const int hist_len = pos + 1;  // the sequence so far: tokens[b, 0 .. pos]
        const int hbeg = (o.repeat_window > 0 && hist_len > o.repeat_window) ? hist_len - o.repeat_window : 0;
        const int32_t* hist = tokens + (size_t)b * tokens_stride;
        for (int i = hbeg + tid; i < hist_len; i += NT) {
            const int t = hist[i];
            if (t < 0 || t >= V) continue;  // ids outside the vocabulary are looked at, not penalised
            const uint32_t bit = 1u << (t & 31);
            const uint32_t old = atomicOr(&seen[t >> 5], bit);
            if (!(old & bit)) lg[t] = lg[t] > 0.0f ? __fdiv_rn(lg[t], o.repeat_penalty) : __fmul_rn(lg[t], o.repeat_penalty);
        }
        __syncthreads();
    }
    const bool scale_t = temperature > 0.0f && temperature != 1.0f;
    if (scale_t)
        for (int i = tid; i < V; i += NT) lg[i] = __fdiv_rn(lg[i], temperature);
    __syncthreads();

    if (!(temperature > 0.0f)) {
        // greedy: largest value, ties to the smallest index
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = tid; i < V; i += NT) {
            const float v = lg[i];
            if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { red_f[warp] = bv; red_i[warp] = bi; }
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < NW; ++w)
                if (red_f[w] > bv || (red_f[w] == bv && red_i[w] < bi)) { bv = red_f[w]; bi = red_i[w]; }
            sh_tok = bi;
        }
        __syncthreads();
    } else {
        const float r = philox_uniform(seed, seq0 + (unsigned)b, (unsigned)gen);
        const bool trunc = top_k > 0 && top_k < V;
        const bool nucleus = o.top_p < 1.0f;
        if (trunc || (nucleus && V <= 1024)) {
            // radix select of the top_k-th largest key, 8 bits per pass; the row is turned into its keys once
            uint32_t* lgk = reinterpret_cast<uint32_t*>(lg);
            for (int i = tid; i < V; i += NT) lgk[i] = float_key(lg[i]);
            if (tid == 0) { sh_prefix = 0u; sh_need = top_k; }
            if (!trunc) {  // every entry is a candidate (nucleus sampling over a small vocabulary)
                for (int i = tid; i < V; i += NT) cand[i] = i;
                __syncthreads();
            } else {
            int* myhist = whist + warp * 256;
            for (int pass = 3; pass >= 0; --pass) {
                for (int i = lane; i < 256; i += 32) myhist[i] = 0;
                __syncthreads();
                const uint32_t prefix = sh_prefix;
                const uint32_t himask = pass == 3 ? 0u : (0xFFFFFFFFu << (8 * (pass + 1)));
                for (int i0 = 0; i0 < V; i0 += NT) {
                    // lanes of a warp that fall into the same bin add once (in the first pass nearly all of them do)
                    const int i = i0 + tid;
                    int bin = -1;
                    if (i < V) {
                        const uint32_t key = lgk[i];
                        if ((key & himask) == (prefix & himask)) bin = (int)((key >> (8 * pass)) & 0xFF);
                    }
                    if (__ballot_sync(0xffffffffu, bin >= 0) == 0u) continue;  // after the first pass most warps have nothing
                    const unsigned peers = __match_any_sync(0xffffffffu, bin);
                    if (bin >= 0 && lane == __ffs(peers) - 1) atomicAdd(&myhist[bin], __popc(peers));
                }
                __syncthreads();
                if (tid < 256) {
                    int t = 0;
#pragma unroll 8
                    for (int w = 0; w < NW; ++w) t += whist[w * 256 + tid];
                    hist[tid] = t;
                }
                __syncthreads();
                if (tid == 0) {
                    int need = sh_need;
                    int bin = 255;
                    for (; bin > 0; --bin) {
                        if (hist[bin] >= need) break;
                        need -= hist[bin];
                    }
                    sh_prefix = prefix | ((uint32_t)bin << (8 * pass));
                    sh_need = need;
                }
                __syncthreads();
            }
            const uint32_t thr = sh_prefix;  // key of the top_k-th element
            const int need_eq = sh_need;     // how many elements equal to thr are kept (smallest indices)
            // ordered compaction: thread t owns the contiguous index range [t*chunk, (t+1)*chunk)
            // (an odd chunk length keeps the lanes of a warp on different shared-memory banks)
            const int chunk = ((V + NT - 1) / NT) | 1;
            const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);
            int n_gt = 0, n_eq = 0;
            for (int i = lo; i < hi; ++i) {
                const uint32_t key = lgk[i];
                n_gt += key > thr;
                n_eq += key == thr;
            }
            int tot_gt, tot_eq;
            block_scan2(n_gt, n_eq, scan_a, scan_b, tot_gt, tot_eq);  // now exclusive prefixes
            {
                int eq_before = n_eq;
                // selected count before this thread = gt before + min(eq before, need_eq)
                int w = n_gt + min(eq_before, need_eq);
                for (int i = lo; i < hi; ++i) {
                    const uint32_t key = lgk[i];
                    if (key > thr) cand[w++] = i;
                    else if (key == thr) {
                        if (eq_before < need_eq) cand[w++] = i;
                        ++eq_before;
                    }
                }
            }
            __syncthreads();
            }  // trunc
            // softmax over the candidates in ascending index order, f32, then inverse CDF
            const int nc = trunc ? top_k : V;
            float m2 = -INFINITY;
            for (int i = tid; i < nc; i += NT) m2 = fmaxf(m2, key_float(lgk[cand[i]]));
            m2 = warp_max(m2);
            if (lane == 0) red_f[warp] = m2;
            __syncthreads();
            m2 = red_f[0];
#pragma unroll
            for (int w = 1; w < NW; ++w) m2 = fmaxf(m2, red_f[w]);
            for (int i = tid; i < nc; i += NT) cval[i] = nnb_expf(__fsub_rn(key_float(lgk[cand[i]]), m2));
            __syncthreads();
            if (tid == 0) {
                float sum = 0.0f;
                for (int i = 0; i < nc; ++i) sum = __fadd_rn(sum, cval[i]);
                red_f[0] = sum;
            }
            __syncthreads();
            float sum = red_f[0];
            __syncthreads();
            if (nucleus && nc > 1) {
                // candidates ordered by (exponential descending, index ascending): bitonic sort of their slots
                int* ord = whist;          // 1024 slots
                int* keepf = whist + 1024; // 1024 flags
                int n2 = 2;
                while (n2 < nc) n2 <<= 1;
                for (int i = tid; i < n2; i += NT) ord[i] = i < nc ? i : -1;
                auto before = [&](int a, int c) {
                    if (a < 0) return false;
                    if (c < 0) return true;
                    if (cval[a] != cval[c]) return cval[a] > cval[c];
                    return a < c;
                };
                for (int k = 2; k <= n2; k <<= 1)
                    for (int j = k >> 1; j > 0; j >>= 1) {
                        __syncthreads();
                        const int i = tid, ixj = tid ^ j;
                        if (i < n2 && ixj > i) {
                            const int a = ord[i], c = ord[ixj];
                            const bool up = (i & k) == 0;
                            if (up ? before(c, a) : before(a, c)) { ord[i] = c; ord[ixj] = a; }
                        }
                    }
                __syncthreads();
                if (tid == 0) {
                    const float want = o.top_p > 0.0f ? o.top_p : 0.0f;
                    float cum = 0.0f;
                    int keep = 0;
                    for (; keep < nc; ++keep) {
                        cum = __fadd_rn(cum, __fdiv_rn(cval[ord[keep]], sum));
                        if (cum >= want) { ++keep; break; }
                    }
                    if (keep == 0) keep = 1;
                    sh_need = keep;
                }
                for (int i = tid; i < nc; i += NT) keepf[i] = 0;
                __syncthreads();
                const int keep = sh_need;
                for (int i = tid; i < keep; i += NT) keepf[ord[i]] = 1;
                __syncthreads();
                if (tid == 0) {
                    float ks = 0.0f;
                    for (int i = 0; i < nc; ++i)
                        if (keepf[i]) ks = __fadd_rn(ks, cval[i]);
                    red_f[0] = ks;
                }
                __syncthreads();
                sum = red_f[0];
                for (int i = tid; i < nc; i += NT)
                    if (!keepf[i]) cval[i] = -1.0f;  // dropped from the candidate set
                __syncthreads();
            }
            for (int i = tid; i < nc; i += NT)
                if (cval[i] >= 0.0f) cval[i] = __fdiv_rn(cval[i], sum);
            __syncthreads();
            if (tid == 0) {
                float cum = 0.0f;
                int next = -1;
                for (int i = 0; i < nc; ++i) {
                    if (cval[i] < 0.0f) continue;
                    next = cand[i];  // stays the last kept candidate if the draw is never reached
                    cum = __fadd_rn(cum, cval[i]);
                    if (r <= cum) break;
                }
                sh_tok = next;
            }
            __syncthreads();
        } else {
            // full vocabulary: p_i = exp(x_i - max)/sum.  Every thread owns a contiguous chunk of the row: the sum and
            // the CDF are accumulated in f64, chunk by chunk, and joined by a block-wide scan (the reference walks the
            // row in f32, ascending index; the draw lands on the same token except within rounding of a CDF step)
            float m2 = -INFINITY;
            for (int i = tid; i < V; i += NT) m2 = fmaxf(m2, lg[i]);
            m2 = warp_max(m2);
            if (lane == 0) red_f[warp] = m2;
            __syncthreads();
            m2 = red_f[0];
#pragma unroll
            for (int w = 1; w < NW; ++w) m2 = fmaxf(m2, red_f[w]);
            __shared__ double dsum[NW + 1];
            const int chunk = (V + NT - 1) / NT;
            const int lo = min(V, tid * chunk), hi = min(V, lo + chunk);
            double part = 0.0;
            for (int i = lo; i < hi; ++i) {
                const float ev = nnb_expf(__fsub_rn(lg[i], m2));
                lg[i] = ev;
                part += (double)ev;
            }
            part = warp_sum_d(part);
            if (lane == 0) dsum[warp] = part;
            if (tid == 0) sh_tok = V - 1;  // the fallback when the draw is never reached
            __syncthreads();
            double tot = 0.0;
#pragma unroll
            for (int w = 0; w < NW; ++w) tot += dsum[w];
            const float sumf = (float)tot;
            __syncthreads();
            double cpart = 0.0;
            for (int i = lo; i < hi; ++i) cpart += (double)__fdiv_rn(lg[i], sumf);
            // exclusive scan of the chunks' probability mass over the block
            double incl = cpart;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const double up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            if (lane == 31) dsum[warp] = incl;
            __syncthreads();
            double base = 0.0;
            for (int w = 0; w < warp; ++w) base += dsum[w];
            double cum = base + incl - cpart;
            if ((double)r <= base + incl) {  // the first crossing can only lie in a chunk whose end reaches the draw
                for (int i = lo; i < hi; ++i) {
                    cum += (double)__fdiv_rn(lg[i], sumf);
                    if ((double)r <= cum) {
                        atomicMin(&sh_tok, i);
                        break;
                    }
                }
            }
            __syncthreads();
        }
    }
    if (tid == 0) {
        int tok = sh_tok;
        bool finished = false;
        if (o.done) {
            if (o.done[b]) {
                finished = true;
                tok = o.eos;
            } else if (tok == o.eos && gen >= o.min_new) {
                o.done[b] = 1;
                o.gen_len[b] = gen;  // tokens generated before the end-of-sequence token
            }
        }
        tokens[(size_t)b * tokens_stride + pos + 1] = tok;
        if (logp) logp[(size_t)b * logp_stride + gen] = finished ? 0.0f : (row[tok] - mx) - lse;
        if (entropy) entropy[(size_t)b * logp_stride + gen] = finished ? 0.0f : lse - (float)(sxe_tot / se_tot);
    }
}

nnb_status launch_sample(nnb_engine* e, bool exact, const float* logits, size_t B, size_t V,
                         float temperature, int top_k, unsigned long long seed, unsigned seq0,
                         const int* d_pos, int prompt_len, int32_t* tokens, size_t tokens_stride,
                         float* logp, size_t logp_stride, float* entropy)
{
    SampleOpts o;
    o.temperature = temperature;
    o.top_k = top_k;
    return launch_sample_opts(e, exact, logits, B, V, o, seed, seq0, d_pos, prompt_len, tokens, tokens_stride, logp, logp_stride,
                              entropy);
}

bool sample_row_in_smem(size_t V) { return ((V + 3) & ~(size_t)3) * 4 + 2 * 1024 * 4 + SAMPLE_NW * 256 * 4 <= 220 * 1024; }

nnb_status launch_sample_opts(nnb_engine* e, bool exact, const float* logits, size_t B, size_t V, const SampleOpts& o,
                              unsigned long long seed, unsigned seq0, const int* d_pos, int prompt_len, int32_t* tokens,
                              size_t tokens_stride, float* logp, size_t logp_stride, float* entropy)
{
    const int top_k = o.top_k;
    NNB_REQUIRE(logits && tokens && B > 0 && V > 0, "sample: bad arguments");
    NNB_REQUIRE(top_k >= 0 && top_k <= 1024, "sample: top_k=%d out of range (0..1024)", top_k);
    NNB_REQUIRE(V <= 8192 * 32, "sample: vocabulary %zu too large", V);
    if (o.top_p < 1.0f && o.temperature > 0.0f && !((top_k > 0 && (size_t)top_k < V) || V <= 1024))
        NNB_FAIL(NNB_ERR_UNSUPPORTED, "sample: top_p needs at most 1024 candidates (set top_k <= 1024; vocabulary is %zu)", V);
    NNB_REQUIRE((o.done == nullptr) == (o.gen_len == nullptr), "sample: done flags and lengths go together");
    const bool in_smem = sample_row_in_smem(V);
    NNB_REQUIRE(in_smem || o.row_scratch, "sample: a vocabulary of %zu needs the row scratch buffer", V);
    SampleOpts oo = o;
    if (in_smem) oo.row_scratch = nullptr;
    const size_t smem = (in_smem ? ((V + 3) & ~(size_t)3) * 4 : 0) + 2 * 1024 * 4 + SAMPLE_NW * 256 * 4;
    if (exact) {
        auto kern = sample_kernel<true>;
        static size_t cfg_dev[64] = {}; size_t& cfg = cfg_dev[e->device & 63];
        if (smem > cfg) {
            NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            cfg = smem;
        }
        launch_ex(e, kern, dim3((unsigned)B), dim3(SAMPLE_NT), smem, logits, (int)V, oo, seed, seq0, d_pos, prompt_len,
                  tokens, (int)tokens_stride, logp, (int)logp_stride, entropy);
    } else {
        auto kern = sample_kernel<false>;
        static size_t cfg_dev[64] = {}; size_t& cfg = cfg_dev[e->device & 63];
        if (smem > cfg) {
            NNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            cfg = smem;
        }
        launch_ex(e, kern, dim3((unsigned)B), dim3(SAMPLE_NT), smem, logits, (int)V, oo, seed, seq0, d_pos, prompt_len,
                  tokens, (int)tokens_stride, logp, (int)logp_stride, entropy);
    }
    e->launches++;
    NNB_CHECK_LAUNCH("sample_kernel");
    return NNB_OK;
}

__global__ void set_int_kernel(int* p, int v, int v1) { p[0] = v; p[1] = v1; }
__global__ void fill_int_kernel(int* p, int n, int v)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}
nnb_status launch_fill_int(nnb_engine* e, int* p, size_t n, int v)
{
    fill_int_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, e->stream>>>(p, (int)n, v);
    e->launches++;
    NNB_CHECK_LAUNCH("fill_int_kernel");
    return NNB_OK;
}
__global__ void add_int_kernel(int* p, int v)
{
    pdl_wait();
    p[0] += v;
    p[1] += v;
}

// p = {window position, token column}; both move together (launch_add_int) until the window slides
nnb_status launch_set_int(nnb_engine* e, int* p, int v) { return launch_set_int2(e, p, v, v); }
nnb_status launch_set_int2(nnb_engine* e, int* p, int v, int v1)
{
    set_int_kernel<<<1, 1, 0, e->stream>>>(p, v, v1);
    e->launches++;
    NNB_CHECK_LAUNCH("set_int_kernel");
    return NNB_OK;
}
nnb_status launch_add_int(nnb_engine* e, int* p, int v)
{
    launch_ex(e, add_int_kernel, dim3(1), dim3(1), 0, p, v);
    e->launches++;
    NNB_CHECK_LAUNCH("add_int_kernel");
    return NNB_OK;
}

nnb_status launch_embed(nnb_engine* e, const float* tok_emb, const float* pos_emb, const int32_t* tokens,
                        size_t tokens_stride, const int* d_pos, size_t B, size_t d, size_t vocab, float* x)
{
    launch_ex(e, embed_kernel, dim3((unsigned)B), dim3(128), 0, tok_emb, pos_emb, tokens, (int)tokens_stride, d_pos, (int)d,
              (int)vocab, x);
    e->launches++;
    NNB_CHECK_LAUNCH("embed_kernel");
    return NNB_OK;
}

}  // namespace nnb
