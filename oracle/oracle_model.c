/*
 * oracle_model.c — CPU restatement of the reference's GPT decode path and sampler.
 *
 * TEST INFRASTRUCTURE ONLY (see oracle.c).  Follows, function by function:
 *   RMSNorm::forward            include/neuralnet.cpp/compute_layer_mlp.hpp:686-707
 *   RotaryEmbedding             include/neuralnet.cpp/compute_position_encoding.hpp:64-80,149-168
 *   AttentionBase::forward_step include/neuralnet.cpp/compute_layer_attention.hpp:1003-1092
 *   GeLU / SwiGLU forward       include/neuralnet.cpp/compute_layer_mlp.hpp:243-252,317-330
 *   GPTBlock/GPTModel step      include/neuralnet.cpp/compute_layer_gpt.hpp:201-218,693-725
 *   GPTModel::generate          include/neuralnet.cpp/compute_layer_gpt.hpp:740-852
 *   sample_next_token_          include/neuralnet.cpp/compute_layer_base.hpp:1025-1163
 *
 * Parity status: the reference's float reduction order (DSL reductions, batched matmul)
 * is engine-defined and not pinned bitwise by any reference test ("parity unpinned" for the
 * float parts; the sampler's rules are pinned by tests/test_oracle_pins_decode.py from
 * src/sampling_test.cpp).  To make "greedy rollouts token-identical" a well-defined gate,
 * every float reduction here accumulates in double and rounds once to f32 (so the result
 * does not depend on summation order), and exp() is a fixed sequence of fmaf steps
 * (orc_expf) rather than libm's.  The reference's per-element arithmetic is otherwise
 * kept rounding by rounding (compiled with -ffp-contract=off).
 *
 * Parameter buffer: one flat f32 array in this order
 *   tok_emb (V,d) | pos_emb (ctx,d) if learned positions |
 *   per layer: ln1_g (d) | wq wk wv (d,d each) | bq bk bv (d each) | wo (d,d) | bo (d) |
 *              ln2_g (d) | w1 (F1,d) | b1 (F1) | w2 (d,F) | b2 (d)      F1 = F (GELU) or 2F (SwiGLU)
 *   lnf_g (d) | head_w (V,d) | head_b (V) | value_w (1,d) | value_b (1) if value head
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* from oracle.c */
uint32_t orc_trit_code_of(float w, float tau);
int8_t orc_i8_quantize(float x, float s);

typedef struct {
    int n_layer, d_model, n_head, d_ff, vocab, ctx;
    int act;        /* 0 = QuickGELU, 1 = SwiGLU */
    int pos;        /* 0 = learned additive, 1 = RoPE */
    int value_head; /* 0 / 1 */
    /* BitNet 2B4T structure switches (docs/internal/22-bitnet-2b4t-architecture.md):
     * sub_ln: an RMSNorm inside each sub-layer, before its output projection (attention output of width d before the
     *   o projection, compute_layer_attention.hpp:482-552,820; activated hidden of width d_ff before fc2,
     *   compute_layer_feedforward.hpp:37-65,201);
     * n_head_kv: grouped-query attention, query head h reads KV head h / (n_head / n_head_kv)
     *   (compute_layer_attention.hpp:444-454); 0 = n_head;
     * tie: the LM head is the token embedding, logits = E x, no head parameters (compute_layer_gpt.hpp:258-264). */
    int sub_ln, n_head_kv, tie;
} orc_gpt_cfg;

static int cfg_hkv(const orc_gpt_cfg* c) { return c->n_head_kv > 0 ? c->n_head_kv : c->n_head; }

typedef struct {
    int in, out;
    const float* w; /* latent (out,in) */
    const float* b; /* (out) */
    float* tau;     /* (out) */
    int8_t* trit;   /* decoded (out,in) */
} orc_lin;

typedef struct {
    const float* ln1_g;
    orc_lin q, k, v, o;
    const float* ln2_g;
    orc_lin fc1, fc2;
    const float* attn_sub_g; /* (d), sub_ln only */
    const float* ffn_sub_g;  /* (d_ff), sub_ln only */
} orc_layer;

typedef struct {
    orc_gpt_cfg cfg;
    const float* tok_emb;
    const float* pos_emb;
    orc_layer* layers;
    const float* lnf_g;
    orc_lin head;
    const float* value_w;
    const float* value_b;
    float* rope_cos; /* (ctx, dk/2) */
    float* rope_sin;
    size_t n_params;
} orc_gpt;

/* ------------------------------------------------------------------ math */
/* exp as a fixed fmaf sequence (Cephes-style range reduction + degree-5 polynomial).
 * x < -86 -> 0, x > 88 -> clamped.  Max error about 1 ulp of libm's expf. */
ORC_API float orc_expf(float x)
{
    if (x < -86.0f) return 0.0f;
    if (x > 88.0f) x = 88.0f;
    const float t = fmaf(x, 1.44269504088896341f, 12582912.0f);
    const float n = t - 12582912.0f;
    float r = fmaf(n, -0.693359375f, x);
    r = fmaf(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    const float r2 = r * r;
    float res = fmaf(p, r2, r) + 1.0f;
    int32_t bits;
    memcpy(&bits, &res, 4);
    bits += ((int32_t)n) << 23;
    memcpy(&res, &bits, 4);
    return res;
}

/* Philox4x32-10 (Salmon et al. 2011): counter (c0..c3), key (k0,k1) */
static void philox4x32_10(uint32_t c[4], uint32_t k0, uint32_t k1)
{
    for (int i = 0; i < 10; ++i) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
        const uint32_t n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
        const uint32_t n3 = (uint32_t)p0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
}

/* uniform in [0,1) with 24 bits, from counter (sequence, step) and a 64-bit seed */
ORC_API float orc_philox_uniform(uint64_t seed, uint32_t sequence, uint32_t step)
{
    uint32_t c[4] = {sequence, step, 0u, 0u};
    philox4x32_10(c, (uint32_t)seed, (uint32_t)(seed >> 32));
    return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}

/* ------------------------------------------------------------- model setup */
static size_t lin_setup(orc_lin* l, const float* base, size_t off_w, size_t off_b, int in, int out)
{
    l->in = in;
    l->out = out;
    l->w = base + off_w;
    l->b = base + off_b;
    l->tau = (float*)malloc(sizeof(float) * (size_t)out);
    l->trit = (int8_t*)malloc((size_t)out * (size_t)in);
    const float inv = 1.0f / (float)in;
    for (int r = 0; r < out; ++r) {
        /* tau = sum |w| * (1/K): f32 terms, double accumulation, one rounding */
        double s = 0.0;
        for (int c = 0; c < in; ++c) s += (double)(fabsf(l->w[(size_t)r * in + c]) * inv);
        l->tau[r] = (float)s;
        for (int c = 0; c < in; ++c)
            l->trit[(size_t)r * in + c] =
                (int8_t)((int)orc_trit_code_of(l->w[(size_t)r * in + c], l->tau[r]) - 2);
    }
    return 0;
}

ORC_API size_t orc_gpt_param_count(const orc_gpt_cfg* c)
{
    const size_t d = c->d_model, F = c->d_ff, V = c->vocab;
    const size_t F1 = c->act >= 1 ? 2 * F : F;
    size_t n = V * d;
    if (c->pos == 0) n += (size_t)c->ctx * d;
    const size_t dkv = (size_t)cfg_hkv(c) * (d / c->n_head);
    n += (size_t)c->n_layer * (d + (d + 2 * dkv) * d + (d + 2 * dkv) + d * d + d + d + F1 * d + F1 + d * F + d);
    if (c->sub_ln) n += (size_t)c->n_layer * (d + F);
    n += d;
    if (!c->tie) n += V * d + V;
    if (c->value_head) n += d + 1;
    return n;
}

ORC_API orc_gpt* orc_gpt_create(const orc_gpt_cfg* c, const float* params)
{
    orc_gpt* m = (orc_gpt*)calloc(1, sizeof(orc_gpt));
    m->cfg = *c;
    const size_t d = c->d_model, F = c->d_ff, V = c->vocab;
    const size_t F1 = c->act >= 1 ? 2 * F : F;
    size_t o = 0;
    m->tok_emb = params + o; o += V * d;
    if (c->pos == 0) { m->pos_emb = params + o; o += (size_t)c->ctx * d; }
    m->layers = (orc_layer*)calloc((size_t)c->n_layer, sizeof(orc_layer));
    for (int l = 0; l < c->n_layer; ++l) {
        orc_layer* L = &m->layers[l];
        L->ln1_g = params + o; o += d;
        const size_t dkv = (size_t)cfg_hkv(c) * (d / c->n_head);
        const size_t wq = o, wk = o + d * d, wv = wk + dkv * d; o += (d + 2 * dkv) * d;
        const size_t bq = o, bk = o + d, bv = bk + dkv; o += d + 2 * dkv;
        lin_setup(&L->q, params, wq, bq, (int)d, (int)d);
        lin_setup(&L->k, params, wk, bk, (int)d, (int)dkv);
        lin_setup(&L->v, params, wv, bv, (int)d, (int)dkv);
        if (c->sub_ln) { L->attn_sub_g = params + o; o += d; }
        const size_t wo = o; o += d * d;
        const size_t bo = o; o += d;
        lin_setup(&L->o, params, wo, bo, (int)d, (int)d);
        L->ln2_g = params + o; o += d;
        const size_t w1 = o; o += F1 * d;
        const size_t b1 = o; o += F1;
        lin_setup(&L->fc1, params, w1, b1, (int)d, (int)F1);
        if (c->sub_ln) { L->ffn_sub_g = params + o; o += F; }
        const size_t w2 = o; o += d * F;
        const size_t b2 = o; o += d;
        lin_setup(&L->fc2, params, w2, b2, (int)F, (int)d);
    }
    m->lnf_g = params + o; o += d;
    if (!c->tie) {
        const size_t hw = o; o += V * d;
        const size_t hb = o; o += V;
        lin_setup(&m->head, params, hw, hb, (int)d, (int)V);
    }
    if (c->value_head) { m->value_w = params + o; o += d; m->value_b = params + o; o += 1; }
    m->n_params = o;
    if (c->pos == 1) {
        /* RotaryEmbedding::fill_pos_column_: theta = pos / 10000^(2j/dk), f32 throughout */
        const int dk = c->d_model / c->n_head, half = dk / 2;
        m->rope_cos = (float*)malloc(sizeof(float) * (size_t)c->ctx * half);
        m->rope_sin = (float*)malloc(sizeof(float) * (size_t)c->ctx * half);
        for (int p = 0; p < c->ctx; ++p)
            for (int j = 0; j < half; ++j) {
                const float theta = (float)p / powf(10000.0f, (float)(2 * j) / (float)dk);
                m->rope_cos[(size_t)p * half + j] = cosf(theta);
                m->rope_sin[(size_t)p * half + j] = sinf(theta);
            }
    }
    return m;
}

static void lin_free(orc_lin* l) { free(l->tau); free(l->trit); }

ORC_API void orc_gpt_destroy(orc_gpt* m)
{
    if (!m) return;
    for (int l = 0; l < m->cfg.n_layer; ++l) {
        orc_layer* L = &m->layers[l];
        lin_free(&L->q); lin_free(&L->k); lin_free(&L->v); lin_free(&L->o);
        lin_free(&L->fc1); lin_free(&L->fc2);
    }
    if (!m->cfg.tie) lin_free(&m->head);
    free(m->layers); free(m->rope_cos); free(m->rope_sin);
    free(m);
}

/* copies of the derived quantisation, for checking the engine's requantisation */
ORC_API void orc_gpt_get_linear(const orc_gpt* m, int layer, int which, float* tau, int8_t* trit)
{
    const orc_lin* l;
    if (layer < 0) l = &m->head;
    else {
        const orc_layer* L = &m->layers[layer];
        const orc_lin* all[6] = {&L->q, &L->k, &L->v, &L->o, &L->fc1, &L->fc2};
        l = all[which];
    }
    if (tau) memcpy(tau, l->tau, sizeof(float) * (size_t)l->out);
    if (trit) memcpy(trit, l->trit, (size_t)l->out * (size_t)l->in);
}

/* --------------------------------------------------------------- operators */
ORC_API void orc_rmsnorm(const float* x, const float* gamma, int f, float eps, float* out)
{
    double ss = 0.0;
    for (int i = 0; i < f; ++i) ss += (double)(x[i] * x[i]);
    const float inv_f = 1.0f / (float)f;
    const float v = (float)ss * inv_f + eps;
    const float sinv = 1.0f / sqrtf(v);
    for (int i = 0; i < f; ++i) {
        const float normed = x[i] * sinv;
        out[i] = normed * gamma[i];
    }
}

/* BitLinear::forward with activation quantisation on one token (compute_layer_bitlinear.hpp:443-455) */
static void quantise_token(const float* x, int k, int8_t* q, float* s_out)
{
    float mx = 0.0f;
    for (int i = 0; i < k; ++i) { const float a = fabsf(x[i]); if (a > mx) mx = a; }
    const float s = mx * (1.0f / 127.0f);
    for (int i = 0; i < k; ++i) q[i] = orc_i8_quantize(x[i], s);
    *s_out = s;
}

static void lin_forward_q(const orc_lin* l, const int8_t* q, float s, float* y)
{
    const int k = l->in;
    for (int r = 0; r < l->out; ++r) {
        const int8_t* w = l->trit + (size_t)r * k;
        int32_t acc = 0;
        for (int i = 0; i < k; ++i) acc += (int32_t)w[i] * (int32_t)q[i];
        const float v = l->tau[r] * s * (float)acc;
        y[r] = v + l->b[r];
    }
}

ORC_API void orc_gpt_linear_forward(const orc_gpt* m, int layer, int which, const float* x, float* y)
{
    const orc_lin* l;
    if (layer < 0) l = &m->head;
    else {
        const orc_layer* L = &m->layers[layer];
        const orc_lin* all[6] = {&L->q, &L->k, &L->v, &L->o, &L->fc1, &L->fc2};
        l = all[which];
    }
    int8_t* q = (int8_t*)malloc((size_t)l->in);
    float s;
    quantise_token(x, l->in, q, &s);
    lin_forward_q(l, q, s, y);
    free(q);
}

static void rope_apply(const orc_gpt* m, float* x /* (H*dk) */, int pos, int H)
{
    const int dk = m->cfg.d_model / m->cfg.n_head, half = dk / 2;
    const float* c = m->rope_cos + (size_t)pos * half;
    const float* s = m->rope_sin + (size_t)pos * half;
    for (int h = 0; h < H; ++h) {
        float* v = x + (size_t)h * dk;
        for (int j = 0; j < half; ++j) {
            const float a = v[j], b = v[j + half];
            /* out = x*cos + rotate_half(x)*sin, rotate_half = (-second half, first half) */
            const float o0 = a * c[j] + (-b) * s[j];
            const float o1 = b * c[j] + a * s[j];
            v[j] = o0;
            v[j + half] = o1;
        }
    }
}

typedef struct {
    float* k; /* (L, ctx, d) post-RoPE keys */
    float* v; /* (L, ctx, d) */
    float *x, *n, *qv, *kv, *vv, *att, *h1, *h2, *sc, *tmp;
    int8_t* q8;
} orc_state;

static orc_state* state_new(const orc_gpt* m)
{
    const orc_gpt_cfg* c = &m->cfg;
    const size_t d = c->d_model, F = c->d_ff, F1 = c->act >= 1 ? 2 * F : F;
    orc_state* s = (orc_state*)calloc(1, sizeof(orc_state));
    s->k = (float*)malloc(sizeof(float) * (size_t)c->n_layer * c->ctx * d);
    s->v = (float*)malloc(sizeof(float) * (size_t)c->n_layer * c->ctx * d);
    s->x = (float*)malloc(sizeof(float) * d);
    s->n = (float*)malloc(sizeof(float) * d);
    s->qv = (float*)malloc(sizeof(float) * d);
    s->kv = (float*)malloc(sizeof(float) * d);
    s->vv = (float*)malloc(sizeof(float) * d);
    s->att = (float*)malloc(sizeof(float) * d);
    s->h1 = (float*)malloc(sizeof(float) * F1);
    s->h2 = (float*)malloc(sizeof(float) * F);
    s->sc = (float*)malloc(sizeof(float) * (size_t)c->ctx);
    s->tmp = (float*)malloc(sizeof(float) * d);
    s->q8 = (int8_t*)malloc(F1 > d ? F1 : d);
    return s;
}

static void state_free(orc_state* s)
{
    free(s->k); free(s->v); free(s->x); free(s->n); free(s->qv); free(s->kv); free(s->vv);
    free(s->att); free(s->h1); free(s->h2); free(s->sc); free(s->tmp); free(s->q8); free(s);
}

/* GPTModel::forward_step for one sequence at position cur_len; logits (V) may be NULL to skip
 * the head (prefill positions whose logits nobody reads). */
static void forward_step(const orc_gpt* m, orc_state* st, int token, int cur_len, float* logits)
{
    const orc_gpt_cfg* c = &m->cfg;
    const int d = c->d_model, H = c->n_head, dk = d / H, F = c->d_ff, Hkv = cfg_hkv(c);
    const float scale = 1.0f / sqrtf((float)dk);
    float s;
    for (int i = 0; i < d; ++i) {
        float v = m->tok_emb[(size_t)token * d + i];
        if (c->pos == 0) v = v + m->pos_emb[(size_t)cur_len * d + i];
        st->x[i] = v;
    }
    for (int l = 0; l < c->n_layer; ++l) {
        const orc_layer* L = &m->layers[l];
        float* kc = st->k + (size_t)l * c->ctx * d;
        float* vc = st->v + (size_t)l * c->ctx * d;
        orc_rmsnorm(st->x, L->ln1_g, d, 1e-5f, st->n);
        quantise_token(st->n, d, st->q8, &s);
        lin_forward_q(&L->q, st->q8, s, st->qv);
        lin_forward_q(&L->k, st->q8, s, st->kv);
        lin_forward_q(&L->v, st->q8, s, st->vv);
        if (c->pos == 1) { rope_apply(m, st->qv, cur_len, H); rope_apply(m, st->kv, cur_len, Hkv); }
        /* the cache holds the n_head_kv heads; query head h reads KV head h / (H / Hkv) */
        memcpy(kc + (size_t)cur_len * d, st->kv, sizeof(float) * (size_t)Hkv * dk);
        memcpy(vc + (size_t)cur_len * d, st->vv, sizeof(float) * (size_t)Hkv * dk);
        const int n_keys = cur_len + 1;
        for (int h = 0; h < H; ++h) {
            const float* qh = st->qv + (size_t)h * dk;
            const int hk = h / (H / Hkv);
            float mx = -INFINITY;
            for (int j = 0; j < n_keys; ++j) {
                const float* kj = kc + (size_t)j * d + (size_t)hk * dk;
                double acc = 0.0;
                for (int i = 0; i < dk; ++i) acc += (double)qh[i] * (double)kj[i];
                const float sc = (float)acc * scale;
                st->sc[j] = sc;
                if (sc > mx) mx = sc;
            }
            double sum = 0.0;
            for (int j = 0; j < n_keys; ++j) { st->sc[j] = orc_expf(st->sc[j] - mx); sum += (double)st->sc[j]; }
            const float sumf = (float)sum;
            for (int j = 0; j < n_keys; ++j) st->sc[j] = st->sc[j] / sumf;
            for (int i = 0; i < dk; ++i) {
                double acc = 0.0;
                for (int j = 0; j < n_keys; ++j)
                    acc += (double)st->sc[j] * (double)vc[(size_t)j * d + (size_t)hk * dk + i];
                st->att[(size_t)h * dk + i] = (float)acc;
            }
        }
        if (c->sub_ln) {  /* SubLN: the heads' output is normalised before the output projection */
            orc_rmsnorm(st->att, L->attn_sub_g, d, 1e-5f, st->n);
            memcpy(st->att, st->n, sizeof(float) * (size_t)d);
        }
        quantise_token(st->att, d, st->q8, &s);
        lin_forward_q(&L->o, st->q8, s, st->tmp);
        for (int i = 0; i < d; ++i) st->x[i] = st->x[i] + st->tmp[i];
        orc_rmsnorm(st->x, L->ln2_g, d, 1e-5f, st->n);
        quantise_token(st->n, d, st->q8, &s);
        lin_forward_q(&L->fc1, st->q8, s, st->h1);
        if (c->act == 0) {
            for (int i = 0; i < F; ++i) {
                const float xv = st->h1[i];
                st->h2[i] = xv / (1.0f + orc_expf(-(xv * 1.702f)));
            }
        } else if (c->act == 2) {
            /* ReLU2GLU (include/neuralnet.cpp/compute_layer_mlp.hpp:384-440): relu(gate)^2 * up */
            for (int i = 0; i < F; ++i) {
                const float gv = st->h1[i], uv = st->h1[F + i];
                const float rv = gv > 0.0f ? gv : 0.0f;
                st->h2[i] = rv * rv * uv;
            }
        } else {
            for (int i = 0; i < F; ++i) {
                const float gv = st->h1[i], uv = st->h1[F + i];
                st->h2[i] = gv * (1.0f / (1.0f + orc_expf(-gv))) * uv;
            }
        }
        if (c->sub_ln) {  /* SubLN: the activated hidden is normalised before fc2 */
            orc_rmsnorm(st->h2, L->ffn_sub_g, F, 1e-5f, st->h1);
            memcpy(st->h2, st->h1, sizeof(float) * (size_t)F);
        }
        quantise_token(st->h2, F, st->q8, &s);
        lin_forward_q(&L->fc2, st->q8, s, st->tmp);
        for (int i = 0; i < d; ++i) st->x[i] = st->x[i] + st->tmp[i];
    }
    if (logits) {
        orc_rmsnorm(st->x, m->lnf_g, d, 1e-5f, st->n);
        if (c->tie) {
            /* tied embeddings: logits = E . ln_f(x), a dense f32 product with the embedding table, no bias */
            for (int v = 0; v < c->vocab; ++v) {
                const float* ev = m->tok_emb + (size_t)v * d;
                double acc = 0.0;
                for (int i = 0; i < d; ++i) acc += (double)ev[i] * (double)st->n[i];
                logits[v] = (float)acc;
            }
        } else {
            quantise_token(st->n, d, st->q8, &s);
            lin_forward_q(&m->head, st->q8, s, logits);
        }
    }
}

/* ------------------------------------------------------------------ sampler */
typedef struct { float v; int i; } cand_t;
static int cand_cmp(const void* a, const void* b)
{
    const cand_t* x = (const cand_t*)a; const cand_t* y = (const cand_t*)b;
    if (x->v != y->v) return x->v > y->v ? -1 : 1;
    return x->i < y->i ? -1 : (x->i > y->i ? 1 : 0);
}
static int int_cmp(const void* a, const void* b) { return *(const int*)a - *(const int*)b; }

/* sample_next_token_ restricted to temperature and top-k (top-p off, no repeat penalty):
 * temperature<=0 -> argmax, ties to the smallest index, r unused; else divide by temperature
 * (when != 1), keep the top_k by (value desc, index asc), softmax over the candidates in
 * ascending index order in f32, inverse CDF with r: first candidate with r <= cumulative,
 * fallback the last candidate.  logits is modified in place like the reference does. */
ORC_API int orc_sample_token(float* logits, int n, float temperature, int top_k, float r)
{
    if (temperature > 0.0f && temperature != 1.0f)
        for (int i = 0; i < n; ++i) logits[i] /= temperature;
    int* cand = (int*)malloc(sizeof(int) * (size_t)n);
    int nc = n;
    if (top_k > 0 && top_k < n) {
        cand_t* order = (cand_t*)malloc(sizeof(cand_t) * (size_t)n);
        for (int i = 0; i < n; ++i) { order[i].v = logits[i]; order[i].i = i; }
        qsort(order, (size_t)n, sizeof(cand_t), cand_cmp);
        nc = top_k;
        for (int i = 0; i < nc; ++i) cand[i] = order[i].i;
        qsort(cand, (size_t)nc, sizeof(int), int_cmp);
        free(order);
    } else {
        for (int i = 0; i < n; ++i) cand[i] = i;
    }
    int next;
    if (temperature > 0.0f) {
        float mx = logits[cand[0]];
        for (int i = 1; i < nc; ++i) if (logits[cand[i]] > mx) mx = logits[cand[i]];
        float sum = 0.0f;
        for (int i = 0; i < nc; ++i) { logits[cand[i]] = orc_expf(logits[cand[i]] - mx); sum += logits[cand[i]]; }
        for (int i = 0; i < nc; ++i) logits[cand[i]] /= sum;
        float cum = 0.0f;
        next = cand[nc - 1];
        for (int i = 0; i < nc; ++i) {
            cum += logits[cand[i]];
            if (r <= cum) { next = cand[i]; break; }
        }
    } else {
        next = cand[0];
        float best = logits[cand[0]];
        for (int i = 1; i < nc; ++i) if (logits[cand[i]] > best) { best = logits[cand[i]]; next = cand[i]; }
    }
    free(cand);
    return next;
}

/* sample_next_token_ with the whole SamplingConfig (include/neuralnet.cpp/compute_layer_base.hpp:1025-1163):
 * bias (stands for the logits_transform hook) -> repeat penalty over the distinct tokens of the history window ->
 * temperature -> top-k -> softmax over the candidates in ascending index order -> top-p -> greedy / inverse CDF.
 * Greedy takes the largest (penalised) logit among the candidates, ties to the smallest index. */
ORC_API int orc_sample_token_cfg(float* logits, int n, float temperature, int top_k, float top_p, float repeat_penalty,
                                 int repeat_window, const float* bias, const int32_t* history, int hist_len, float r)
{
    if (bias)
        for (int i = 0; i < n; ++i) logits[i] += bias[i];
    if (repeat_penalty > 0.0f && repeat_penalty != 1.0f && hist_len > 0) {
        const int begin = (repeat_window > 0 && hist_len > repeat_window) ? hist_len - repeat_window : 0;
        unsigned char* seen = (unsigned char*)calloc((size_t)n, 1);
        for (int i = begin; i < hist_len; ++i) {
            const int t = history[i];
            if (t < 0 || t >= n || seen[t]) continue;
            seen[t] = 1;
            logits[t] = (logits[t] > 0.0f) ? logits[t] / repeat_penalty : logits[t] * repeat_penalty;
        }
        free(seen);
    }
    if (temperature > 0.0f && temperature != 1.0f)
        for (int i = 0; i < n; ++i) logits[i] /= temperature;
    int* cand = (int*)malloc(sizeof(int) * (size_t)n);
    int nc = n;
    if (top_k > 0 && top_k < n) {
        cand_t* order = (cand_t*)malloc(sizeof(cand_t) * (size_t)n);
        for (int i = 0; i < n; ++i) { order[i].v = logits[i]; order[i].i = i; }
        qsort(order, (size_t)n, sizeof(cand_t), cand_cmp);
        nc = top_k;
        for (int i = 0; i < nc; ++i) cand[i] = order[i].i;
        qsort(cand, (size_t)nc, sizeof(int), int_cmp);
        free(order);
    } else {
        for (int i = 0; i < n; ++i) cand[i] = i;
    }
    int next;
    if (!(temperature > 0.0f)) {
        next = cand[0];
        float best = logits[cand[0]];
        for (int i = 1; i < nc; ++i) if (logits[cand[i]] > best) { best = logits[cand[i]]; next = cand[i]; }
        free(cand);
        return next;
    }
    float mx = logits[cand[0]];
    for (int i = 1; i < nc; ++i) if (logits[cand[i]] > mx) mx = logits[cand[i]];
    float sum = 0.0f;
    for (int i = 0; i < nc; ++i) { logits[cand[i]] = orc_expf(logits[cand[i]] - mx); sum += logits[cand[i]]; }
    if (top_p < 1.0f && nc > 1) {
        cand_t* by = (cand_t*)malloc(sizeof(cand_t) * (size_t)nc);
        for (int i = 0; i < nc; ++i) { by[i].v = logits[cand[i]]; by[i].i = cand[i]; }
        qsort(by, (size_t)nc, sizeof(cand_t), cand_cmp);
        const float want = top_p > 0.0f ? top_p : 0.0f;
        float cum = 0.0f;
        int keep = 0;
        for (; keep < nc; ++keep) {
            cum += by[keep].v / sum;
            if (cum >= want) { ++keep; break; }
        }
        if (keep == 0) keep = 1;
        unsigned char* in_keep = (unsigned char*)calloc((size_t)n, 1);
        for (int i = 0; i < keep; ++i) in_keep[by[i].i] = 1;
        float kept_sum = 0.0f;
        int nk = 0;
        for (int i = 0; i < nc; ++i)
            if (in_keep[cand[i]]) { kept_sum += logits[cand[i]]; cand[nk++] = cand[i]; }
        nc = nk;
        sum = kept_sum;
        free(in_keep);
        free(by);
    }
    for (int i = 0; i < nc; ++i) logits[cand[i]] /= sum;
    float cum = 0.0f;
    next = cand[nc - 1];
    for (int i = 0; i < nc; ++i) {
        cum += logits[cand[i]];
        if (r <= cum) { next = cand[i]; break; }
    }
    free(cand);
    return next;
}

/* log softmax(logits)[token] and entropy of the raw (untempered) distribution;
 * CategoricalDistribution::log_prob / entropy, include/neuralnet.cpp/rl_policy.hpp:92-143 */
ORC_API void orc_logprob_entropy(const float* logits, int n, int token, float* logp, float* entropy)
{
    float mx = logits[0];
    for (int i = 1; i < n; ++i) if (logits[i] > mx) mx = logits[i];
    double sum = 0.0;
    for (int i = 0; i < n; ++i) sum += exp((double)logits[i] - (double)mx);
    const double lse = (double)mx + log(sum);
    if (logp) *logp = (float)((double)logits[token] - lse);
    if (entropy) {
        double h = 0.0;
        for (int i = 0; i < n; ++i) {
            const double lp = (double)logits[i] - lse;
            h -= exp(lp) * lp;
        }
        *entropy = (float)h;
    }
}

/* ------------------------------------------------------------------ rollout */
/* GPTModel::generate for a batch of independent sequences: prefill token by token, then
 * sample max_new tokens.  tokens_out (B, P+max_new) int32; logp_out (B, max_new) = log-prob
 * of each sampled token under the raw softmax; logits_out optional (B, max_new, V).
 * The uniform draw of sequence b at generated step t is orc_philox_uniform(seed, seq0+b, t). */
ORC_API int orc_gpt_rollout(const orc_gpt* m, const int32_t* prompts, int B, int P, int max_new,
                            float temperature, int top_k, uint64_t seed, uint32_t seq0,
                            int32_t* tokens_out, float* logp_out, float* logits_out)
{
    const int V = m->cfg.vocab;
    if (P + max_new > m->cfg.ctx || P < 1) return -1;
#pragma omp parallel for schedule(dynamic, 1)
    for (int b = 0; b < B; ++b) {
        orc_state* st = state_new(m);
        float* logits = (float*)malloc(sizeof(float) * (size_t)V);
        float* work = (float*)malloc(sizeof(float) * (size_t)V);
        int32_t* out = tokens_out + (size_t)b * (P + max_new);
        for (int t = 0; t < P; ++t) {
            out[t] = prompts[(size_t)b * P + t];
            forward_step(m, st, out[t], t, t == P - 1 ? logits : NULL);
        }
        for (int t = 0; t < max_new; ++t) {
            if (logits_out) memcpy(logits_out + ((size_t)b * max_new + t) * V, logits, sizeof(float) * (size_t)V);
            memcpy(work, logits, sizeof(float) * (size_t)V);
            const float r = orc_philox_uniform(seed, seq0 + (uint32_t)b, (uint32_t)t);
            const int tok = orc_sample_token(work, V, temperature, top_k, r);
            if (logp_out) orc_logprob_entropy(logits, V, tok, logp_out + (size_t)b * max_new + t, NULL);
            out[P + t] = tok;
            if (t + 1 < max_new) forward_step(m, st, tok, P + t, logits);
        }
        free(logits); free(work);
        state_free(st);
    }
    return 0;
}

/* orc_gpt_rollout with the whole sampling configuration and end-of-sequence handling: after a sequence samples
 * `eos` at a generated index >= min_new it is finished (compute_layer_gpt.hpp:826-828); the rest of its row is
 * filled with eos, log-prob 0, and gen_len_out[b] = tokens generated before it (max_new if never). */
ORC_API int orc_gpt_rollout_cfg(const orc_gpt* m, const int32_t* prompts, int B, int P, int max_new, float temperature,
                                int top_k, float top_p, float repeat_penalty, int repeat_window, const float* bias,
                                int eos, int min_new, uint64_t seed, uint32_t seq0, int32_t* tokens_out, float* logp_out,
                                int32_t* gen_len_out)
{
    const int V = m->cfg.vocab;
    const int ctx = m->cfg.ctx;
    if (P < 1 || (P + max_new > ctx && ctx < 2)) return -1;
#pragma omp parallel for schedule(dynamic, 1)
    for (int b = 0; b < B; ++b) {
        orc_state* st = state_new(m);
        float* logits = (float*)malloc(sizeof(float) * (size_t)V);
        float* work = (float*)malloc(sizeof(float) * (size_t)V);
        int32_t* out = tokens_out + (size_t)b * (P + max_new);
        for (int t = 0; t < P; ++t) out[t] = prompts[(size_t)b * P + t];
        /* GPTModel::generate (include/neuralnet.cpp/compute_layer_gpt.hpp:768-818): a prompt longer than the context
         * is cut to its tail; cur_len counts the tokens in the KV cache */
        int cur_len = 0;
        for (int t = (P > ctx ? P - ctx : 0); t < P; ++t) forward_step(m, st, out[t], cur_len++, logits);
        int done = 0;
        if (gen_len_out) gen_len_out[b] = max_new;
        for (int t = 0; t < max_new; ++t) {
            if (done) {
                out[P + t] = eos;
                if (logp_out) logp_out[(size_t)b * max_new + t] = 0.0f;
                continue;
            }
            if (cur_len >= ctx) {
                /* sliding window: the cache is rebuilt from the last ctx-1 tokens, positions from 0 */
                cur_len = 0;
                const int size = P + t, keep = ctx - 1;
                for (int i = (size > keep ? size - keep : 0); i < size; ++i) forward_step(m, st, out[i], cur_len++, logits);
            }
            memcpy(work, logits, sizeof(float) * (size_t)V);
            const float r = orc_philox_uniform(seed, seq0 + (uint32_t)b, (uint32_t)t);
            const int tok = orc_sample_token_cfg(work, V, temperature, top_k, top_p, repeat_penalty, repeat_window, bias, out,
                                                 P + t, r);
            if (logp_out) orc_logprob_entropy(logits, V, tok, logp_out + (size_t)b * max_new + t, NULL);
            out[P + t] = tok;
            if (eos >= 0 && tok == eos && t >= min_new) {
                done = 1;
                if (gen_len_out) gen_len_out[b] = t;
                continue;
            }
            if (t + 1 < max_new) forward_step(m, st, tok, cur_len++, logits);
        }
        free(logits); free(work);
        state_free(st);
    }
    return 0;
}

/* teacher-forced logits of one sequence through the step path: logits_out (n_tok, V) */
ORC_API int orc_gpt_step_logits(const orc_gpt* m, const int32_t* tokens, int n_tok, float* logits_out)
{
    if (n_tok > m->cfg.ctx) return -1;
    orc_state* st = state_new(m);
    for (int t = 0; t < n_tok; ++t)
        forward_step(m, st, tokens[t], t, logits_out + (size_t)t * m->cfg.vocab);
    state_free(st);
    return 0;
}

/* helpers for the numpy training restatement: the same exp and RoPE tables as the step path */
ORC_API void orc_expf_array(const float* x, size_t n, float* out)
{
    for (size_t i = 0; i < n; ++i) out[i] = orc_expf(x[i]);
}

ORC_API void orc_rope_tables(int dk, int ctx, float* cos_out, float* sin_out)
{
    const int half = dk / 2;
    for (int p = 0; p < ctx; ++p)
        for (int j = 0; j < half; ++j) {
            const float theta = (float)p / powf(10000.0f, (float)(2 * j) / (float)dk);
            cos_out[(size_t)p * half + j] = cosf(theta);
            sin_out[(size_t)p * half + j] = sinf(theta);
        }
}
