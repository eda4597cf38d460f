// rl.cu — advantages, categorical log-prob / entropy, clipped objectives, global-norm clip and
// AdamW as single-pass CUDA kernels.
//
// The reference composes each of these from dozens of elementwise / reduce dispatches with
// host scalar read-backs in between (include/neuralnet.cpp/rl_experience.hpp:273-545,
// rl_policy.hpp:92-187,460-773, compute_optimizer.hpp:134-187,384-436,563-597).  Here each is
// one or two launches and no host round trip: scalars that the reference downloads (units,
// sums, norms) stay in a small device accumulator block.  Sums whose order the reference
// leaves to its engine are accumulated in f64.
#include "common.cuh"
#include "device_math.cuh"

namespace nnb {

// ------------------------------------------------------------------ GAE
// (steps, batch) row = time.  One thread per trajectory walks time backwards; consecutive
// threads read consecutive columns, so every step is one coalesced row access.
__global__ void gae_kernel(const float* __restrict__ rewards, const float* __restrict__ values,
                           const float* __restrict__ done, const float* __restrict__ mask,
                           const float* __restrict__ bootstrap, size_t steps, size_t batch, float gamma,
                           float gl, float* __restrict__ adv_out, float* __restrict__ ret_out)
{
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    float next_adv = 0.0f;
    float next_value = bootstrap ? bootstrap[b] : 0.0f;
    for (size_t ti = steps; ti-- > 0;) {
        const size_t i = ti * batch + b;
        const float r = rewards[i], v = values[i];
        const float cont = done ? __fsub_rn(__fadd_rn(__fmul_rn(r, 0.0f), 1.0f), done[i]) : 1.0f;
        const float delta = __fsub_rn(__fadd_rn(r, __fmul_rn(__fmul_rn(next_value, gamma), cont)), v);
        float adv = __fadd_rn(delta, __fmul_rn(__fmul_rn(next_adv, gl), cont));
        float ret;
        if (mask) {
            const float m = mask[i];
            adv = __fmul_rn(adv, m);
            ret = __fmul_rn(__fadd_rn(adv, v), m);
            next_value = __fmul_rn(v, m);
        } else {
            ret = __fadd_rn(adv, v);
            next_value = v;
        }
        adv_out[i] = adv;
        ret_out[i] = ret;
        next_adv = adv;
    }
}

// MonteCarloReturn::apply (include/neuralnet.cpp/rl_experience.hpp:395-440): ret_t = r_t + gamma * ret_{t+1} * cont,
// cont = 1 - done, the row multiplied by the mask (and the masked row carried to the previous step).
__global__ void mc_return_kernel(const float* __restrict__ rewards, const float* __restrict__ done,
                                 const float* __restrict__ mask, size_t steps, size_t batch, float gamma,
                                 float* __restrict__ out)
{
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    float next = 0.0f;
    for (size_t ti = steps; ti-- > 0;) {
        const size_t i = ti * batch + b;
        const float r = rewards[i];
        const float cont = done ? __fsub_rn(__fadd_rn(__fmul_rn(r, 0.0f), 1.0f), done[i]) : 1.0f;
        float row = __fadd_rn(r, __fmul_rn(__fmul_rn(next, gamma), cont));
        if (mask) row = __fmul_rn(row, mask[i]);
        out[i] = row;
        next = row;
    }
}

// ------------------------------------------------------- group advantages
// One warp per contiguous span of rows: segmented warp reduction of sum, sum of squares and
// count, then (x - mean) * (1/sqrt(var)); zero when the variance is <= eps^2.
__global__ void group_advantage_kernel(const float* __restrict__ returns, const int32_t* __restrict__ first,
                                       const int32_t* __restrict__ count, size_t n_spans, float eps,
                                       float* __restrict__ out)
{
    const size_t span = (size_t)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
    if (span >= n_spans) return;
    const int lane = threadIdx.x & 31;
    const int f = first[span], c = count[span];
    double sw = 0.0, ssq = 0.0;
    for (int i = lane; i < c; i += 32) {
        const float x = returns[f + i];
        sw += (double)x;
        ssq += (double)__fmul_rn(x, x);
    }
    sw = warp_sum_d(sw);
    ssq = warp_sum_d(ssq);
    const float cnt = (float)c;
    const float mean = __fdiv_rn((float)sw, cnt);
    float var = __fsub_rn(__fdiv_rn((float)ssq, cnt), __fmul_rn(mean, mean));
    if (var < 0.0f) var = 0.0f;
    const bool zero = !(var > __fmul_rn(eps, eps));
    const float inv_std = zero ? 0.0f : __frcp_rn(__fsqrt_rn(var));
    for (int i = lane; i < c; i += 32) {
        const float x = returns[f + i];
        out[f + i] = zero ? 0.0f : __fmul_rn(__fsub_rn(x, mean), inv_std);
    }
}

// ------------------------------------------------ masked normaliser (whole vector)
// acc[0..2] = sum(x*m), sum(x*x*m), sum(m)
__global__ void masked_moments_kernel(const float* __restrict__ x, const float* __restrict__ mask, size_t n,
                                      double* __restrict__ acc)
{
    double sw = 0.0, ssq = 0.0, sm = 0.0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float m = mask ? mask[i] : 1.0f;
        const float v = x[i];
        sw += (double)__fmul_rn(v, m);
        ssq += (double)__fmul_rn(__fmul_rn(v, v), m);
        sm += (double)m;
    }
    sw = warp_sum_d(sw);
    ssq = warp_sum_d(ssq);
    sm = warp_sum_d(sm);
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(acc + 0, sw);
        atomicAdd(acc + 1, ssq);
        atomicAdd(acc + 2, sm);
    }
}

__global__ void masked_normalize_apply_kernel(const float* __restrict__ x, const float* __restrict__ mask,
                                              size_t n, float eps, const double* __restrict__ acc,
                                              float* __restrict__ out)
{
    const float count = (float)acc[2];
    bool zero = !(count > 0.0f);
    float mean = 0.0f, inv_std = 0.0f;
    if (!zero) {
        mean = __fdiv_rn((float)acc[0], count);
        float var = __fsub_rn(__fdiv_rn((float)acc[1], count), __fmul_rn(mean, mean));
        if (var < 0.0f) var = 0.0f;
        zero = !(var > __fmul_rn(eps, eps));
        if (!zero) inv_std = __frcp_rn(__fsqrt_rn(var));
    }
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float m = mask ? mask[i] : 1.0f;
        out[i] = zero ? 0.0f : __fmul_rn(__fmul_rn(__fsub_rn(x[i], mean), inv_std), m);
    }
}

// ------------------------------------------- categorical over materialised logits
// One CTA per token, logits (T, V).  logp[t] = log softmax(row)[action]; H[t] = -sum p log p.
__global__ void __launch_bounds__(256)
categorical_fwd_kernel(const float* __restrict__ logits, const int32_t* __restrict__ actions, size_t v,
                       float* __restrict__ logp, float* __restrict__ entropy)
{
    __shared__ float red_f[8];
    __shared__ double red_d[2][8];
    const size_t t = blockIdx.x;
    const float* row = logits + t * v;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float mx = -INFINITY;
    for (size_t j = tid; j < v; j += 256) mx = fmaxf(mx, row[j]);
    mx = warp_max(mx);
    if (lane == 0) red_f[warp] = mx;
    __syncthreads();
    mx = red_f[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red_f[w]);
    double se = 0.0, sxe = 0.0;
    for (size_t j = tid; j < v; j += 256) {
        const double d = (double)row[j] - (double)mx;
        const double ev = exp(d);
        se += ev;
        sxe += ev * d;
    }
    se = warp_sum_d(se);
    sxe = warp_sum_d(sxe);
    if (lane == 0) { red_d[0][warp] = se; red_d[1][warp] = sxe; }
    __syncthreads();
    if (tid == 0) {
        double a = 0.0, b = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) { a += red_d[0][w]; b += red_d[1][w]; }
        const double lse = log(a);
        if (logp) logp[t] = (float)(((double)row[actions[t]] - (double)mx) - lse);
        if (entropy) entropy[t] = (float)(lse - b / a);
    }
}

// dlogits = (onehot - p) * up_lp + (-p * (log p + H)) * up_ent
__global__ void __launch_bounds__(256)
categorical_bwd_kernel(const float* logits /* may be dlogits: in place */, const int32_t* __restrict__ actions,
                       const float* __restrict__ up_lp, const float* __restrict__ up_ent, size_t v,
                       float* dlogits)
{
    __shared__ float red_f[8];
    __shared__ double red_d[2][8];
    __shared__ double sh[2];
    const size_t t = blockIdx.x;
    const float* row = logits + t * v;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float mx = -INFINITY;
    for (size_t j = tid; j < v; j += 256) mx = fmaxf(mx, row[j]);
    mx = warp_max(mx);
    if (lane == 0) red_f[warp] = mx;
    __syncthreads();
    mx = red_f[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red_f[w]);
    double se = 0.0, sxe = 0.0;
    for (size_t j = tid; j < v; j += 256) {
        const double d = (double)row[j] - (double)mx;
        const double ev = exp(d);
        se += ev;
        sxe += ev * d;
    }
    se = warp_sum_d(se);
    sxe = warp_sum_d(sxe);
    if (lane == 0) { red_d[0][warp] = se; red_d[1][warp] = sxe; }
    __syncthreads();
    if (tid == 0) {
        double a = 0.0, b = 0.0;
#pragma unroll
        for (int w = 0; w < 8; ++w) { a += red_d[0][w]; b += red_d[1][w]; }
        sh[0] = log(a);
        sh[1] = log(a) - b / a;  // entropy
    }
    __syncthreads();
    const double lse = sh[0], h = sh[1];
    const double ul = up_lp ? (double)up_lp[t] : 0.0, ue = up_ent ? (double)up_ent[t] : 0.0;
    const int act = actions[t];
    for (size_t j = tid; j < v; j += 256) {
        const double lp = ((double)row[j] - (double)mx) - lse;
        const double p = exp(lp);
        double g = (((int)j == act ? 1.0 : 0.0) - p) * ul;
        g += -p * (lp + h) * ue;
        dlogits[t * v + j] = (float)g;
    }
}

// ------------------------------------------------------ per-token objectives
__global__ void sum_kernel(const float* __restrict__ x, size_t n, double* __restrict__ acc)
{
    double s = 0.0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        s += (double)x[i];
    s = warp_sum_d(s);
    if ((threadIdx.x & 31) == 0) atomicAdd(acc, s);
}

// The fused token objective: clipped policy surrogate + sampled KL against a reference policy +
// entropy bonus.  acc[0] holds units (sum of mask, or the caller's global count).
// Writes d loss / d logp and d loss / d entropy per token and accumulates
//   acc[1] sum surr*m   acc[2] sum ratio*m   acc[3] sum diff^2*m   acc[4] sum outside*m
//   acc[5] sum (logp-ref)*m   acc[6] sum H*m
__global__ void token_objective_kernel(const float* __restrict__ logp, const float* __restrict__ entropy,
                                       const float* __restrict__ old_logp, const float* __restrict__ ref_logp,
                                       const float* __restrict__ adv, const float* __restrict__ mask, size_t n,
                                       float clip_eps, float kl_coef, float ent_coef,
                                       float* __restrict__ up_lp, float* __restrict__ up_ent,
                                       double* __restrict__ acc)
{
    const float units = (float)acc[0];
    const bool live = units > 0.0f;
    const float lower = __fsub_rn(1.0f, clip_eps), upper = __fadd_rn(1.0f, clip_eps);
    const float neg_inv_units = live ? __fdiv_rn(-1.0f, units) : 0.0f;
    const float kl_scale = live ? __fdiv_rn(kl_coef, units) : 0.0f;
    const float ent_scale = live ? __fdiv_rn(-ent_coef, units) : 0.0f;
    double s[6] = {0, 0, 0, 0, 0, 0};
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float m = mask[i];
        float u = 0.0f;
        if (old_logp && adv) {
            const float diff = __fsub_rn(logp[i], old_logp[i]);
            const float ratio = expf(diff);
            const float clipped = ratio < lower ? lower : (ratio > upper ? upper : ratio);
            const float a = adv[i];
            const float obj = __fmul_rn(ratio, a), cobj = __fmul_rn(clipped, a);
            const float surr = fminf(obj, cobj);
            const float positive = ratio > upper ? 0.0f : obj;
            const float negative = ratio < lower ? 0.0f : obj;
            const float factor = a > 0.0f ? positive : negative;
            u = __fmul_rn(__fmul_rn(factor, m), neg_inv_units);
            s[0] += (double)__fmul_rn(__fmul_rn(surr, m), m);
            s[1] += (double)__fmul_rn(__fmul_rn(ratio, m), m);
            s[2] += (double)__fmul_rn(__fmul_rn(__fmul_rn(diff, diff), m), m);
            s[3] += (double)__fmul_rn(__fmul_rn((ratio < lower || ratio > upper) ? 1.0f : 0.0f, m), m);
        }
        if (ref_logp && kl_coef != 0.0f) {
            u = __fadd_rn(u, __fmul_rn(m, kl_scale));
            s[4] += (double)__fmul_rn(__fsub_rn(logp[i], ref_logp[i]), m);
        }
        if (up_lp) up_lp[i] = u;
        if (entropy) {
            s[5] += (double)__fmul_rn(entropy[i], m);
            if (up_ent) up_ent[i] = __fmul_rn(m, ent_scale);
        } else if (up_ent) {
            up_ent[i] = 0.0f;
        }
    }
#pragma unroll
    for (int k = 0; k < 6; ++k) {
        s[k] = warp_sum_d(s[k]);
        if ((threadIdx.x & 31) == 0 && s[k] != 0.0) atomicAdd(acc + 1 + k, s[k]);
    }
}

// report[0..7] = policy_loss, ratio_mean, approx_kl, clip_fraction, kl_loss, entropy_loss,
//                mean entropy, units
__global__ void token_objective_finalize_kernel(const double* __restrict__ acc, float kl_coef, float ent_coef,
                                                float* __restrict__ report)
{
    const float units = (float)acc[0];
    if (!(units > 0.0f)) {
        for (int i = 0; i < 7; ++i) report[i] = 0.0f;
        report[7] = units;
        return;
    }
    report[0] = __fdiv_rn(-(float)acc[1], units);
    report[1] = __fdiv_rn((float)acc[2], units);
    report[2] = __fdiv_rn(__fmul_rn(0.5f, (float)acc[3]), units);
    report[3] = __fdiv_rn((float)acc[4], units);
    report[4] = __fdiv_rn(__fmul_rn(kl_coef, (float)acc[5]), units);
    report[5] = __fdiv_rn(__fmul_rn(-ent_coef, (float)acc[6]), units);
    report[6] = __fdiv_rn((float)acc[6], units);
    report[7] = units;
}

// ClippedValueObjective; acc[0] = units, acc[1] sum max(..)*m, acc[2] sum outside*m
__global__ void clipped_value_kernel(const float* __restrict__ value, const float* __restrict__ returns,
                                     const float* __restrict__ old_value, const float* __restrict__ mask,
                                     size_t n, float clip_eps, float coef, float* __restrict__ grad,
                                     double* __restrict__ acc)
{
    const float units = (float)acc[0];
    const bool live = units > 0.0f;
    const float scale = live ? __fdiv_rn(coef, units) : 0.0f;
    double s0 = 0.0, s1 = 0.0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float m = mask[i], v = value[i];
        const float lo = __fsub_rn(old_value[i], clip_eps), hi = __fadd_rn(old_value[i], clip_eps);
        const float clipped = v < lo ? lo : (v > hi ? hi : v);
        const float diff = __fsub_rn(v, returns[i]), cdiff = __fsub_rn(clipped, returns[i]);
        const float dsq = __fmul_rn(diff, diff), csq = __fmul_rn(cdiff, cdiff);
        const float outside = (v < lo || v > hi) ? 1.0f : 0.0f;
        const float ug = __fmul_rn(diff, 2.0f);
        const float cg = outside > 0.0f ? 0.0f : ug;
        grad[i] = __fmul_rn(__fmul_rn(csq > dsq ? cg : ug, m), scale);
        s0 += (double)__fmul_rn(__fmul_rn(fmaxf(dsq, csq), m), m);
        s1 += (double)__fmul_rn(__fmul_rn(outside, m), m);
    }
    s0 = warp_sum_d(s0);
    s1 = warp_sum_d(s1);
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(acc + 1, s0);
        atomicAdd(acc + 2, s1);
    }
}

// ValueRegressionObjective (include/neuralnet.cpp/rl_policy.hpp:393-439): loss = coef * sum (v-R)^2 m / units,
// grad = (v-R) * m * (2*coef/units); acc[0] = units, acc[1] = sum (v-R)^2 m
__global__ void value_regression_kernel(const float* __restrict__ value, const float* __restrict__ returns,
                                        const float* __restrict__ mask, size_t n, float coef, float* __restrict__ grad,
                                        double* __restrict__ acc)
{
    const float units = (float)acc[0];
    const bool live = units > 0.0f;
    const float scale = live ? __fdiv_rn(__fmul_rn(2.0f, coef), units) : 0.0f;
    double s0 = 0.0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float m = mask[i];
        const float diff = __fsub_rn(value[i], returns[i]);
        grad[i] = __fmul_rn(__fmul_rn(diff, m), scale);
        s0 += (double)__fmul_rn(__fmul_rn(diff, diff), m);
    }
    s0 = warp_sum_d(s0);
    if ((threadIdx.x & 31) == 0) atomicAdd(acc + 1, s0);
}

__global__ void value_regression_finalize_kernel(const double* __restrict__ acc, float coef, float* __restrict__ report)
{
    const float units = (float)acc[0];
    report[0] = units > 0.0f ? __fdiv_rn(__fmul_rn(coef, (float)acc[1]), units) : 0.0f;
    report[1] = units;
}

__global__ void clipped_value_finalize_kernel(const double* __restrict__ acc, float coef, float* __restrict__ report)
{
    const float units = (float)acc[0];
    if (!(units > 0.0f)) { report[0] = report[1] = 0.0f; return; }
    report[0] = __fdiv_rn(__fmul_rn(coef, (float)acc[1]), units);
    report[1] = __fdiv_rn((float)acc[2], units);
}

// ---------------------------------------------------------- optimizer
__global__ void sumsq_kernel(const float* __restrict__ g, size_t n, double* __restrict__ acc)
{
    double s = 0.0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const double v = (double)g[i];
        s += v * v;
    }
    s = warp_sum_d(s);
    if ((threadIdx.x & 31) == 0) atomicAdd(acc, s);
}

// scale gradients by min(1, max_norm/||g||); writes the norm to norm_out
__global__ void clip_scale_kernel(float* __restrict__ g, size_t n, float max_norm, const double* __restrict__ acc,
                                  float* __restrict__ norm_out)
{
    const float norm = __fsqrt_rn((float)acc[0]);
    if (blockIdx.x == 0 && threadIdx.x == 0 && norm_out) *norm_out = norm;
    if (!(max_norm > 0.0f) || !(norm > max_norm)) return;
    const float sc = __fdiv_rn(max_norm, norm);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        g[i] = __fmul_rn(g[i], sc);
}

__global__ void scale_kernel(float* __restrict__ x, size_t n, float sc)
{
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = __fmul_rn(x[i], sc);
}

// AdamW: p *= (1 - lr*wd); m = m*b1 + g*(1-b1); v = v*b2 + g*g*(1-b2);
//        p -= lr * ((m*inv_bc1) / (sqrt(v*inv_bc2) + eps))
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, size_t n, float lr, float beta1, float beta2, float eps,
                             float wd, float inv_bc1, float inv_bc2)
{
    const float decay = __fsub_rn(1.0f, __fmul_rn(lr, wd));
    const float omb1 = __fsub_rn(1.0f, beta1), omb2 = __fsub_rn(1.0f, beta2);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float gi = g[i];
        float pi = p[i];
        if (wd != 0.0f) pi = __fmul_rn(pi, decay);
        const float mi = __fadd_rn(__fmul_rn(m[i], beta1), __fmul_rn(gi, omb1));
        const float vi = __fadd_rn(__fmul_rn(v[i], beta2), __fmul_rn(__fmul_rn(gi, gi), omb2));
        const float up = __fmul_rn(mi, inv_bc1);
        const float den = __fadd_rn(__fsqrt_rn(__fmul_rn(vi, inv_bc2)), eps);
        pi = __fsub_rn(pi, __fmul_rn(lr, __fdiv_rn(up, den)));
        p[i] = pi;
        m[i] = mi;
        v[i] = vi;
    }
}

// ------------------------------------------------------------------ launchers
static inline unsigned grid_for(nnb_engine* e, size_t n, int threads)
{
    size_t g = ceil_div(n, (size_t)threads);
    const size_t cap = (size_t)e->sm_count * 8;
    return (unsigned)(g < cap ? (g ? g : 1) : cap);
}

// 16 f64 accumulators at the start of the engine scratch arena
static nnb_status acc_block(nnb_engine* e, double** acc)
{
    NNB_TRY(e->ensure_scratch(4096));
    *acc = (double*)e->scratch;
    NNB_CUDA(cudaMemsetAsync(*acc, 0, 16 * sizeof(double), e->stream));
    return NNB_OK;
}

__global__ void set_double_kernel(double* p, double v) { *p = v; }

nnb_status launch_gae(nnb_engine* e, const float* rewards, const float* values, const float* done,
                      const float* mask, const float* bootstrap, size_t steps, size_t batch, float gamma,
                      float lambda, float* adv, float* ret)
{
    NNB_REQUIRE(rewards && values && adv && ret, "gae: NULL argument");
    NNB_REQUIRE(steps > 0 && batch > 0, "gae: rewards must not be empty");
    gae_kernel<<<(unsigned)ceil_div(batch, 128), 128, 0, e->stream>>>(rewards, values, done, mask, bootstrap, steps,
                                                                      batch, gamma, gamma * lambda, adv, ret);
    e->launches++;
    NNB_CHECK_LAUNCH("gae_kernel");
    return NNB_OK;
}

nnb_status launch_group_advantage(nnb_engine* e, const float* returns, const int32_t* first, const int32_t* count,
                                  size_t n_spans, float eps, float* out)
{
    NNB_REQUIRE(returns && first && count && out && n_spans > 0, "group_advantage: bad arguments");
    group_advantage_kernel<<<(unsigned)ceil_div(n_spans, 8), 256, 0, e->stream>>>(returns, first, count, n_spans, eps, out);
    e->launches++;
    NNB_CHECK_LAUNCH("group_advantage_kernel");
    return NNB_OK;
}

nnb_status launch_masked_normalize(nnb_engine* e, const float* x, const float* mask, size_t n, float eps, float* out)
{
    NNB_REQUIRE(x && out && n > 0, "masked_normalize: values must not be empty");
    double* acc;
    NNB_TRY(acc_block(e, &acc));
    masked_moments_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(x, mask, n, acc);
    masked_normalize_apply_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(x, mask, n, eps, acc, out);
    e->launches += 2;
    NNB_CHECK_LAUNCH("masked_normalize kernels");
    return NNB_OK;
}

nnb_status launch_categorical_fwd(nnb_engine* e, const float* logits, const int32_t* actions, size_t t, size_t v,
                                  float* logp, float* entropy)
{
    NNB_REQUIRE(logits && actions && (logp || entropy) && t > 0 && v > 0, "categorical: bad arguments");
    categorical_fwd_kernel<<<(unsigned)t, 256, 0, e->stream>>>(logits, actions, v, logp, entropy);
    e->launches++;
    NNB_CHECK_LAUNCH("categorical_fwd_kernel");
    return NNB_OK;
}

nnb_status launch_categorical_bwd(nnb_engine* e, const float* logits, const int32_t* actions, const float* up_lp,
                                  const float* up_ent, size_t t, size_t v, float* dlogits)
{
    NNB_REQUIRE(logits && actions && dlogits && t > 0 && v > 0, "categorical backward: bad arguments");
    categorical_bwd_kernel<<<(unsigned)t, 256, 0, e->stream>>>(logits, actions, up_lp, up_ent, v, dlogits);
    e->launches++;
    NNB_CHECK_LAUNCH("categorical_bwd_kernel");
    return NNB_OK;
}

nnb_status launch_token_objective(nnb_engine* e, const float* logp, const float* entropy, const float* old_logp,
                                  const float* ref_logp, const float* adv, const float* mask, size_t n,
                                  float units_override, float clip_eps, float kl_coef, float ent_coef,
                                  float* up_lp, float* up_ent, float* report)
{
    NNB_REQUIRE(logp && mask && n > 0, "token_objective: bad arguments");
    NNB_REQUIRE((old_logp != nullptr) == (adv != nullptr), "token_objective: old_log_prob and advantage go together");
    double* acc;
    NNB_TRY(acc_block(e, &acc));
    if (units_override > 0.0f) set_double_kernel<<<1, 1, 0, e->stream>>>(acc, (double)units_override);
    else sum_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(mask, n, acc);
    token_objective_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(logp, entropy, old_logp, ref_logp, adv, mask, n,
                                                                       clip_eps, kl_coef, ent_coef, up_lp, up_ent, acc);
    e->launches += 2;
    if (report) {
        token_objective_finalize_kernel<<<1, 1, 0, e->stream>>>(acc, kl_coef, ent_coef, report);
        e->launches++;
    }
    NNB_CHECK_LAUNCH("token_objective kernels");
    return NNB_OK;
}

nnb_status launch_clipped_value(nnb_engine* e, const float* value, const float* returns, const float* old_value,
                                const float* mask, size_t n, float units_override, float clip_eps, float coef,
                                float* grad, float* report)
{
    NNB_REQUIRE(value && returns && old_value && mask && grad && n > 0, "clipped_value: bad arguments");
    double* acc;
    NNB_TRY(acc_block(e, &acc));
    if (units_override > 0.0f) set_double_kernel<<<1, 1, 0, e->stream>>>(acc, (double)units_override);
    else sum_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(mask, n, acc);
    clipped_value_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(value, returns, old_value, mask, n, clip_eps, coef,
                                                                     grad, acc);
    e->launches += 2;
    if (report) {
        clipped_value_finalize_kernel<<<1, 1, 0, e->stream>>>(acc, coef, report);
        e->launches++;
    }
    NNB_CHECK_LAUNCH("clipped_value kernels");
    return NNB_OK;
}

nnb_status launch_value_regression(nnb_engine* e, const float* value, const float* returns, const float* mask, size_t n,
                                   float units_override, float coef, float* grad, float* report)
{
    NNB_REQUIRE(value && returns && mask && grad && n > 0, "value_regression: bad arguments");
    double* acc;
    NNB_TRY(acc_block(e, &acc));
    if (units_override > 0.0f) set_double_kernel<<<1, 1, 0, e->stream>>>(acc, (double)units_override);
    else sum_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(mask, n, acc);
    value_regression_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(value, returns, mask, n, coef, grad, acc);
    e->launches += 2;
    if (report) {
        value_regression_finalize_kernel<<<1, 1, 0, e->stream>>>(acc, coef, report);
        e->launches++;
    }
    NNB_CHECK_LAUNCH("value_regression kernels");
    return NNB_OK;
}

nnb_status launch_mc_return(nnb_engine* e, const float* rewards, const float* done, const float* mask, size_t steps,
                            size_t batch, float gamma, float* out)
{
    NNB_REQUIRE(rewards && out && steps > 0 && batch > 0, "monte_carlo_return: rewards must not be empty");
    mc_return_kernel<<<(unsigned)ceil_div(batch, 128), 128, 0, e->stream>>>(rewards, done, mask, steps, batch, gamma, out);
    e->launches++;
    NNB_CHECK_LAUNCH("mc_return_kernel");
    return NNB_OK;
}

nnb_status launch_clip_grad_norm(nnb_engine* e, float* g, size_t n, float max_norm, float* norm_out)
{
    NNB_REQUIRE(g && n > 0, "clip_grad_norm: bad arguments");
    double* acc;
    NNB_TRY(acc_block(e, &acc));
    sumsq_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(g, n, acc);
    clip_scale_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(g, n, max_norm, acc, norm_out);
    e->launches += 2;
    NNB_CHECK_LAUNCH("clip_grad_norm kernels");
    return NNB_OK;
}

nnb_status launch_scale(nnb_engine* e, float* x, size_t n, float sc)
{
    NNB_REQUIRE(x && n > 0, "scale_inplace: bad arguments");
    scale_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(x, n, sc);
    e->launches++;
    NNB_CHECK_LAUNCH("scale_kernel");
    return NNB_OK;
}

nnb_status launch_adamw(nnb_engine* e, float* p, const float* g, float* m, float* v, size_t n, float lr,
                        float beta1, float beta2, float eps, float wd, int t)
{
    NNB_REQUIRE(p && g && m && v && n > 0 && t >= 1, "adamw: bad arguments");
    const float inv_bc1 = 1.0f / (1.0f - powf(beta1, (float)t));
    const float inv_bc2 = 1.0f / (1.0f - powf(beta2, (float)t));
    adamw_kernel<<<grid_for(e, n, 256), 256, 0, e->stream>>>(p, g, m, v, n, lr, beta1, beta2, eps, wd, inv_bc1, inv_bc2);
    e->launches++;
    NNB_CHECK_LAUNCH("adamw_kernel");
    return NNB_OK;
}

}  // namespace nnb

using namespace nnb;

extern "C" {

nnb_status nnb_gae(nnb_engine* e, const float* d_rewards, const float* d_values, const float* d_done,
                   const float* d_mask, const float* d_bootstrap, size_t steps, size_t batch, float gamma,
                   float lambda, float* d_advantage, float* d_returns)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_gae(e, d_rewards, d_values, d_done, d_mask, d_bootstrap, steps, batch, gamma, lambda, d_advantage,
                      d_returns);
}

nnb_status nnb_group_advantage(nnb_engine* e, const float* d_returns, size_t n, const int32_t* h_first,
                               const int32_t* h_count, size_t n_spans, float eps, float* d_out)
{
    NNB_REQUIRE(e && d_returns && h_first && h_count && d_out, "group_advantage: NULL argument");
    NNB_REQUIRE(n > 0, "group_advantage: returns must not be empty");
    size_t cursor = 0;
    for (size_t s = 0; s < n_spans; ++s) {
        NNB_REQUIRE(h_count[s] > 0, "group_advantage: group row_count must be > 0");
        NNB_REQUIRE((size_t)h_first[s] == cursor, "group_advantage: group spans must be contiguous and non-overlapping");
        cursor += (size_t)h_count[s];
    }
    NNB_REQUIRE(cursor == n, "group_advantage: group spans do not cover all %zu rows", n);
    NNB_TRY(e->ensure_scratch(4096 + 2 * n_spans * sizeof(int32_t)));
    int32_t* d_first = (int32_t*)((char*)e->scratch + 4096);
    int32_t* d_count = d_first + n_spans;
    NNB_CUDA(cudaMemcpyAsync(d_first, h_first, n_spans * 4, cudaMemcpyHostToDevice, e->stream));
    NNB_CUDA(cudaMemcpyAsync(d_count, h_count, n_spans * 4, cudaMemcpyHostToDevice, e->stream));
    return launch_group_advantage(e, d_returns, d_first, d_count, n_spans, eps, d_out);
}

nnb_status nnb_masked_normalize(nnb_engine* e, const float* d_values, const float* d_mask, size_t n, float eps,
                                float* d_out)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_masked_normalize(e, d_values, d_mask, n, eps, d_out);
}

nnb_status nnb_categorical_logp_entropy(nnb_engine* e, const float* d_logits, const int32_t* d_actions, size_t t,
                                        size_t v, float* d_logp, float* d_entropy)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_categorical_fwd(e, d_logits, d_actions, t, v, d_logp, d_entropy);
}

nnb_status nnb_categorical_backward(nnb_engine* e, const float* d_logits, const int32_t* d_actions,
                                    const float* d_up_logp, const float* d_up_entropy, size_t t, size_t v,
                                    float* d_dlogits)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_categorical_bwd(e, d_logits, d_actions, d_up_logp, d_up_entropy, t, v, d_dlogits);
}

nnb_status nnb_token_objective(nnb_engine* e, const float* d_logp, const float* d_entropy, const float* d_old_logp,
                               const float* d_ref_logp, const float* d_advantage, const float* d_mask, size_t n,
                               float units, float clip_eps, float kl_coef, float entropy_coef, float* d_up_logp,
                               float* d_up_entropy, float* d_report)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_token_objective(e, d_logp, d_entropy, d_old_logp, d_ref_logp, d_advantage, d_mask, n, units,
                                  clip_eps, kl_coef, entropy_coef, d_up_logp, d_up_entropy, d_report);
}

nnb_status nnb_clipped_value(nnb_engine* e, const float* d_value, const float* d_returns, const float* d_old_value,
                             const float* d_mask, size_t n, float units, float clip_eps, float coef, float* d_grad,
                             float* d_report)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_clipped_value(e, d_value, d_returns, d_old_value, d_mask, n, units, clip_eps, coef, d_grad,
                                d_report);
}

nnb_status nnb_value_regression(nnb_engine* e, const float* d_value, const float* d_returns, const float* d_mask, size_t n,
                                float units, float coef, float* d_grad, float* d_report)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_value_regression(e, d_value, d_returns, d_mask, n, units, coef, d_grad, d_report);
}

nnb_status nnb_monte_carlo_return(nnb_engine* e, const float* d_rewards, const float* d_done, const float* d_mask,
                                  size_t steps, size_t batch, float gamma, float* d_returns)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_mc_return(e, d_rewards, d_done, d_mask, steps, batch, gamma, d_returns);
}

nnb_status nnb_clip_grad_norm(nnb_engine* e, float* d_grads, size_t n, float max_norm, float* d_norm_out)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_clip_grad_norm(e, d_grads, n, max_norm, d_norm_out);
}

nnb_status nnb_scale_inplace(nnb_engine* e, float* d_x, size_t n, float scale)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_scale(e, d_x, n, scale);
}

nnb_status nnb_adamw_step(nnb_engine* e, float* d_params, const float* d_grads, float* d_m, float* d_v, size_t n,
                          float lr, float beta1, float beta2, float eps, float weight_decay, int t)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_adamw(e, d_params, d_grads, d_m, d_v, n, lr, beta1, beta2, eps, weight_decay, t);
}

}  // extern "C"
