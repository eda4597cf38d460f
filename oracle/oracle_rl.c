/*
 * oracle_rl.c — CPU restatement of the reference's RL arithmetic: advantages, categorical
 * log-prob / entropy, clipped objectives, AdamW.
 *
 * TEST INFRASTRUCTURE ONLY (see oracle.c).  Follows:
 *   GaeAdvantage::apply        include/neuralnet.cpp/rl_experience.hpp:273-380
 *   MaskedNormalizer::apply    include/neuralnet.cpp/rl_experience.hpp:456-498
 *   GroupAdvantage::apply      include/neuralnet.cpp/rl_experience.hpp:516-545
 *   CategoricalDistribution    include/neuralnet.cpp/rl_policy.hpp:92-187
 *   ClippedPolicyObjective     include/neuralnet.cpp/rl_policy.hpp:564-661
 *   EntropyBonusObjective      include/neuralnet.cpp/rl_policy.hpp:460-481
 *   SampledKlObjective         include/neuralnet.cpp/rl_policy.hpp:503-530
 *   ClippedValueObjective      include/neuralnet.cpp/rl_policy.hpp:670-773
 *   Optimizer::clip_grad_norm  include/neuralnet.cpp/compute_optimizer.hpp:134-187
 *   AdamW::step                include/neuralnet.cpp/compute_optimizer.hpp:384-436,563-597
 * Pinned by the known answers of src/rl_experience_test.cpp, src/rl_policy_test.cpp,
 * src/rl_ppo_test.cpp and src/rl_grpo_test.cpp (tests/test_oracle_pins_rl.py).
 * Reductions whose order the reference leaves to its engine are accumulated in double.
 * Vectors are per decision (token); logits are token-major (T, V).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>

#define ORC_API __attribute__((visibility("default")))

/* rewards/values/done/mask (steps, batch) row = time; bootstrap (batch) or NULL */
ORC_API void orc_gae(const float* rewards, const float* values, const float* done, const float* mask,
                     const float* bootstrap, size_t steps, size_t batch, float gamma, float lambda,
                     float* adv_out, float* ret_out)
{
    const float gl = gamma * lambda;
    for (size_t b = 0; b < batch; ++b) {
        float next_adv = 0.0f;
        float next_value = bootstrap ? bootstrap[b] : 0.0f;
        for (size_t ti = steps; ti-- > 0;) {
            const size_t i = ti * batch + b;
            const float r = rewards[i], v = values[i];
            const float cont = done ? (r * 0.0f + 1.0f - done[i]) : 1.0f;
            const float delta = r + next_value * gamma * cont - v;
            float adv = delta + next_adv * gl * cont;
            float ret;
            if (mask) {
                adv = adv * mask[i];
                ret = (adv + v) * mask[i];
            } else {
                ret = adv + v;
            }
            adv_out[i] = adv;
            ret_out[i] = ret;
            next_adv = adv;
            next_value = mask ? v * mask[i] : v;
        }
    }
}

/* MonteCarloReturn::apply (include/neuralnet.cpp/rl_experience.hpp:395-440) */
ORC_API void orc_mc_return(const float* rewards, const float* done, const float* mask, size_t steps, size_t batch,
                           float gamma, float* out)
{
    for (size_t b = 0; b < batch; ++b) {
        float next = 0.0f;
        for (size_t ti = steps; ti-- > 0;) {
            const size_t i = ti * batch + b;
            const float r = rewards[i];
            const float cont = done ? (r * 0.0f + 1.0f - done[i]) : 1.0f;
            float row = r + next * gamma * cont;
            if (mask) row = row * mask[i];
            out[i] = row;
            next = row;
        }
    }
}

/* ValueRegressionObjective (include/neuralnet.cpp/rl_policy.hpp:393-439); returns the loss */
ORC_API float orc_value_regression(const float* value, const float* returns, const float* mask, size_t n, float coef,
                                   float* grad)
{
    double units_d = 0.0;
    for (size_t i = 0; i < n; ++i) units_d += (double)mask[i];
    const float units = (float)units_d;
    if (units <= 0.0f) {
        for (size_t i = 0; i < n; ++i) grad[i] = 0.0f;
        return 0.0f;
    }
    double loss_sum = 0.0;
    const float scale = 2.0f * coef / units;
    for (size_t i = 0; i < n; ++i) {
        const float diff = value[i] - returns[i];
        loss_sum += (double)(diff * diff * mask[i]);
        grad[i] = diff * mask[i] * scale;
    }
    return coef * (float)loss_sum / units;
}

/* population mean / variance over masked entries; zeros when count <= 0 or var <= eps^2;
 * (x - mean) * (1/sqrt(var)) * mask otherwise (no eps in the divisor) */
ORC_API void orc_masked_normalize(const float* values, const float* mask, size_t n, float eps, float* out)
{
    double sw = 0.0, ssq = 0.0, sm = 0.0;
    for (size_t i = 0; i < n; ++i) {
        const float m = mask ? mask[i] : 1.0f;
        sw += (double)(values[i] * m);
        ssq += (double)(values[i] * values[i] * m);
        sm += (double)m;
    }
    const float count = (float)sm;
    if (count <= 0.0f) { for (size_t i = 0; i < n; ++i) out[i] = 0.0f; return; }
    const float mean = (float)sw / count;
    float variance = (float)ssq / count - mean * mean;
    if (variance < 0.0f) variance = 0.0f;
    if (variance <= eps * eps) { for (size_t i = 0; i < n; ++i) out[i] = 0.0f; return; }
    const float inv_std = 1.0f / sqrtf(variance);
    for (size_t i = 0; i < n; ++i) out[i] = (values[i] - mean) * inv_std * (mask ? mask[i] : 1.0f);
}

/* spans: first[i], count[i] contiguous and covering all n rows; returns -1 when they do not */
ORC_API int orc_group_advantage(const float* returns, size_t n, const int32_t* first, const int32_t* count,
                                size_t n_spans, float eps, float* out)
{
    size_t cursor = 0;
    for (size_t s = 0; s < n_spans; ++s) {
        if (count[s] <= 0 || (size_t)first[s] != cursor) return -1;
        cursor += (size_t)count[s];
    }
    if (cursor != n) return -1;
    for (size_t s = 0; s < n_spans; ++s)
        orc_masked_normalize(returns + first[s], NULL, (size_t)count[s], eps, out + first[s]);
    return 0;
}

/* log softmax(logits)[action] and entropy per token; logits (T, V) */
ORC_API void orc_categorical_logp_entropy(const float* logits, const int32_t* actions, size_t t, size_t v,
                                          float* logp, float* entropy)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < t; ++i) {
        const float* row = logits + i * v;
        float mx = row[0];
        for (size_t j = 1; j < v; ++j) if (row[j] > mx) mx = row[j];
        double sum = 0.0;
        for (size_t j = 0; j < v; ++j) sum += exp((double)row[j] - (double)mx);
        const double lse = (double)mx + log(sum);
        if (logp) logp[i] = (float)((double)row[actions[i]] - lse);
        if (entropy) {
            double h = 0.0;
            for (size_t j = 0; j < v; ++j) { const double lp = (double)row[j] - lse; h -= exp(lp) * lp; }
            entropy[i] = (float)h;
        }
    }
}

/* d/dlogits of sum_t up_lp[t]*logp[t] + up_ent[t]*H[t]:
 *   (onehot - p) * up_lp  +  (-p * (logp_all + H)) * up_ent          (rl_policy.hpp:145-187) */
ORC_API void orc_categorical_backward(const float* logits, const int32_t* actions, const float* up_lp,
                                      const float* up_ent, size_t t, size_t v, float* dlogits)
{
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < t; ++i) {
        const float* row = logits + i * v;
        float mx = row[0];
        for (size_t j = 1; j < v; ++j) if (row[j] > mx) mx = row[j];
        double sum = 0.0;
        for (size_t j = 0; j < v; ++j) sum += exp((double)row[j] - (double)mx);
        const double lse = (double)mx + log(sum);
        double h = 0.0;
        if (up_ent) for (size_t j = 0; j < v; ++j) { const double lp = (double)row[j] - lse; h -= exp(lp) * lp; }
        for (size_t j = 0; j < v; ++j) {
            const double lp = (double)row[j] - lse, p = exp(lp);
            double g = 0.0;
            if (up_lp) g += ((j == (size_t)actions[i] ? 1.0 : 0.0) - p) * (double)up_lp[i];
            if (up_ent) g += -p * (lp + h) * (double)up_ent[i];
            dlogits[i * v + j] = (float)g;
        }
    }
}

typedef struct {
    float loss, ratio_mean, approx_kl, clip_fraction;
} orc_policy_metrics;

/* ClippedPolicyObjective on per-token vectors; upstream = d loss / d logp.  units = sum(mask). */
ORC_API void orc_clipped_policy(const float* logp, const float* old_logp, const float* adv, const float* mask,
                                size_t t, float clip_eps, float* upstream, orc_policy_metrics* out)
{
    double units_d = 0.0;
    for (size_t i = 0; i < t; ++i) units_d += (double)mask[i];
    const float units = (float)units_d;
    if (units <= 0.0f) {
        for (size_t i = 0; i < t; ++i) upstream[i] = 0.0f;
        out->loss = out->ratio_mean = out->approx_kl = out->clip_fraction = 0.0f;
        return;
    }
    const float lower = 1.0f - clip_eps, upper = 1.0f + clip_eps;
    double loss_sum = 0.0, ratio_sum = 0.0, kl_sum = 0.0, out_sum = 0.0;
    for (size_t i = 0; i < t; ++i) {
        const float diff = logp[i] - old_logp[i];
        const float ratio = expf(diff);
        const float clipped = ratio < lower ? lower : (ratio > upper ? upper : ratio);
        const float obj = ratio * adv[i], cobj = clipped * adv[i];
        const float surr = obj < cobj ? obj : cobj;
        loss_sum += (double)(surr * mask[i] * mask[i]);
        const float positive = ratio > upper ? 0.0f : ratio * adv[i];
        const float negative = ratio < lower ? 0.0f : ratio * adv[i];
        const float factor = adv[i] > 0.0f ? positive : negative;
        upstream[i] = factor * mask[i] * (-1.0f / units);
        ratio_sum += (double)(ratio * mask[i] * mask[i]);
        kl_sum += (double)(diff * diff * mask[i] * mask[i]);
        out_sum += (double)(((ratio < lower || ratio > upper) ? 1.0f : 0.0f) * mask[i] * mask[i]);
    }
    out->loss = -(float)loss_sum / units;
    out->ratio_mean = (float)ratio_sum / units;
    out->approx_kl = 0.5f * (float)kl_sum / units;
    out->clip_fraction = (float)out_sum / units;
}

/* EntropyBonusObjective: loss = -c * sum(H*mask)/units; upstream_ent = -c*mask/units */
ORC_API float orc_entropy_bonus(const float* entropy, const float* mask, size_t t, float coef, float* upstream_ent)
{
    double units_d = 0.0, s = 0.0;
    for (size_t i = 0; i < t; ++i) units_d += (double)mask[i];
    const float units = (float)units_d;
    if (units <= 0.0f) { for (size_t i = 0; i < t; ++i) upstream_ent[i] = 0.0f; return 0.0f; }
    for (size_t i = 0; i < t; ++i) {
        s += (double)(entropy[i] * mask[i]);
        upstream_ent[i] = mask[i] * (-coef / units);
    }
    return -coef * (float)s / units;
}

/* SampledKlObjective: loss = c * sum((logp - ref)*mask)/units; upstream = mask * c/units */
ORC_API float orc_sampled_kl(const float* logp, const float* ref_logp, const float* mask, size_t t, float coef,
                             float* upstream)
{
    double units_d = 0.0, s = 0.0;
    for (size_t i = 0; i < t; ++i) units_d += (double)mask[i];
    const float units = (float)units_d;
    if (units <= 0.0f) { for (size_t i = 0; i < t; ++i) upstream[i] = 0.0f; return 0.0f; }
    for (size_t i = 0; i < t; ++i) {
        s += (double)((logp[i] - ref_logp[i]) * mask[i]);
        upstream[i] = mask[i] * (coef / units);
    }
    return coef * (float)s / units;
}

/* ClippedValueObjective: loss = c*sum(max((V-R)^2, (clip(V, Vold+-eps)-R)^2)*mask)/units */
ORC_API float orc_clipped_value(const float* value, const float* returns, const float* old_value,
                                const float* mask, size_t n, float clip_eps, float coef, float* grad,
                                float* clip_fraction)
{
    double units_d = 0.0;
    for (size_t i = 0; i < n; ++i) units_d += (double)mask[i];
    const float units = (float)units_d;
    if (units <= 0.0f) {
        for (size_t i = 0; i < n; ++i) grad[i] = 0.0f;
        if (clip_fraction) *clip_fraction = 0.0f;
        return 0.0f;
    }
    double loss_sum = 0.0, clip_sum = 0.0;
    for (size_t i = 0; i < n; ++i) {
        const float lo = old_value[i] - clip_eps, hi = old_value[i] + clip_eps;
        const float v = value[i];
        const float clipped = v < lo ? lo : (v > hi ? hi : v);
        const float diff = v - returns[i], cdiff = clipped - returns[i];
        const float dsq = diff * diff, csq = cdiff * cdiff;
        loss_sum += (double)((dsq > csq ? dsq : csq) * mask[i] * mask[i]);
        const float outside = (v < lo || v > hi) ? 1.0f : 0.0f;
        const float cg = outside > 0.0f ? 0.0f : diff * 2.0f;
        const float ug = diff * 2.0f;
        grad[i] = (csq > dsq ? cg : ug) * mask[i] * (coef / units);
        clip_sum += (double)(outside * mask[i] * mask[i]);
    }
    if (clip_fraction) *clip_fraction = (float)clip_sum / units;
    return coef * (float)loss_sum / units;
}

/* global L2 norm clip: if ||g|| > max_norm, g *= max_norm/||g||.  Returns the norm before clipping. */
ORC_API float orc_clip_grad_norm(float* g, size_t n, float max_norm)
{
    double ss = 0.0;
    for (size_t i = 0; i < n; ++i) ss += (double)g[i] * (double)g[i];
    const float norm = sqrtf((float)ss);
    if (max_norm > 0.0f && norm > max_norm) {
        const float sc = max_norm / norm;
        for (size_t i = 0; i < n; ++i) g[i] *= sc;
    }
    return norm;
}

/* AdamW::step at time t (1-based): decay first, then moments, then the update */
ORC_API void orc_adamw(float* p, const float* g, float* m, float* v, size_t n, float lr, float beta1,
                       float beta2, float eps, float wd, int t)
{
    const float inv_bc1 = 1.0f / (1.0f - powf(beta1, (float)t));
    const float inv_bc2 = 1.0f / (1.0f - powf(beta2, (float)t));
    const float decay = 1.0f - lr * wd;
    for (size_t i = 0; i < n; ++i) {
        float pi = wd != 0.0f ? p[i] * decay : p[i];
        const float mi = m[i] * beta1 + g[i] * (1.0f - beta1);
        const float vi = v[i] * beta2 + g[i] * g[i] * (1.0f - beta2);
        pi = pi - lr * ((mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps));
        p[i] = pi;
        m[i] = mi;
        v[i] = vi;
    }
}
