// Exercises include/nn_b200.hpp the way the reference's own tests exercise nn::ComputeEngine and BitLinear:
//  - BitLinear forward / backward (W1.58A8) through the call sequence of compute_layer_bitlinear.hpp:417-544 on the
//    reference's test generators (src/ternary_gemm_test.cpp:188-195) and shapes (src/int8_act_test.cpp:475-476),
//    against a host integer reference written like src/int8_act_test.cpp:210-236 (Y bitwise) and the formulas of
//    src/t1_58_test.cpp:254-403 (dX, dW, db);
//  - the write-epoch cache: no re-pack while the latent is untouched, re-pack after a write, and the re-packed words equal
//    a pack from scratch (src/write_epoch_test.cpp:296-297);
//  - the data-movement verbs (docs/usage/03-compute-engine-usage.md:1117-1187);
//  - RLTrainingPipeline::run over a device-side RolloutSource with a GRPO-style update of a tiny ternary GPT policy.
// Exit code 0 = all checks passed, 3 = no usable GPU (the engine's own error is printed), anything else = a failed check.
#include <cmath>
#include <cstdio>
#include <cstring>

#include "nn_b200.hpp"

static int g_fail = 0;
#define CHECK(cond, what)                                   \
    do {                                                    \
        if (!(cond)) {                                      \
            std::fprintf(stderr, "FAILED: %s\n", what);     \
            ++g_fail;                                       \
        }                                                   \
    } while (0)
#define UNWRAP(var, expr)                                                   \
    auto var = (expr);                                                      \
    if (!var) {                                                             \
        std::fprintf(stderr, "%s: %s\n", #expr, var.error().message.c_str()); \
        return 10;                                                          \
    }

using nnb::Tensor;

static int test_bitlinear(std::shared_ptr<nnb::ComputeEngine> eng, std::size_t out, std::size_t in, std::size_t n)
{
    UNWRAP(layer, nnb::BitLinear::create(eng, in, out));
    std::vector<float> W(out * in), X(in * n), B(out), dY(out * n);
    for (std::size_t r = 0; r < out; ++r)
        for (std::size_t c = 0; c < in; ++c) W[r * in + c] = 0.13f * (float)((7 * r + 3 * c) % 11) - 0.6f;
    for (std::size_t k = 0; k < in; ++k)
        for (std::size_t j = 0; j < n; ++j) X[k * n + j] = 0.21f * (float)((k + 2 * j) % 9) - 0.8f;
    for (std::size_t r = 0; r < out; ++r) B[r] = 0.01f * (float)(r % 7) - 0.02f;
    for (std::size_t r = 0; r < out; ++r)
        for (std::size_t j = 0; j < n; ++j) dY[r * n + j] = 0.05f * (float)((3 * r + j) % 13) - 0.3f;
    UNWRAP(u1, eng->upload_span(layer->weight(), W.data(), W.size()));
    UNWRAP(u2, eng->upload_span(layer->bias(), B.data(), B.size()));
    UNWRAP(x, eng->from_vector(in, n, X));
    CHECK(layer->needs_quantize_(), "a fresh layer needs quantising");
    UNWRAP(y, layer->forward(*x));
    CHECK(!layer->needs_quantize_(), "no re-pack while the latent is untouched");
    UNWRAP(hy, eng->download_vector(*y));
    UNWRAP(htau, eng->download_vector(layer->tau()));
    // host reference: tau, strict-threshold trits, per-token absmax/127, half-away rounding, int32 accumulation
    std::vector<int> trit(out * in);
    std::vector<float> tau(out), s(n);
    std::vector<int> q(in * n);
    for (std::size_t r = 0; r < out; ++r) {
        double t = 0;
        for (std::size_t c = 0; c < in; ++c) t += (double)(std::fabs(W[r * in + c]) * (1.0f / (float)in));
        tau[r] = (float)t;
        CHECK(std::fabs(tau[r] - (*htau)[r]) <= 1e-6f, "tau = row_reduce_sum(|W| / K)");
        const float th = (*htau)[r];  // decisions with the engine's tau, as the reference tests do with the layer's
        for (std::size_t c = 0; c < in; ++c) trit[r * in + c] = W[r * in + c] > 0.5f * th ? 1 : (W[r * in + c] < -0.5f * th ? -1 : 0);
    }
    for (std::size_t j = 0; j < n; ++j) {
        float mx = 0;
        for (std::size_t k = 0; k < in; ++k) mx = std::fmax(mx, std::fabs(X[k * n + j]));
        s[j] = mx * (1.0f / 127.0f);
        for (std::size_t k = 0; k < in; ++k) {
            float v = s[j] == 0.0f ? 0.0f : X[k * n + j] / s[j];
            v = std::fmin(std::fmax(v, -127.0f), 127.0f);
            q[k * n + j] = s[j] == 0.0f ? 0 : (int)(v < 0 ? -std::floor(-v + 0.5f) : std::floor(v + 0.5f));
        }
    }
    bool y_bitwise = true;
    for (std::size_t r = 0; r < out; ++r)
        for (std::size_t j = 0; j < n; ++j) {
            int acc = 0;
            for (std::size_t k = 0; k < in; ++k) acc += trit[r * in + k] * q[k * n + j];
            volatile float scale = (*htau)[r] * s[j];
            volatile float prod = scale * (float)acc;
            const float want = prod + B[r];
            if (std::memcmp(&want, &(*hy)[r * n + j], 4) != 0) y_bitwise = false;
        }
    CHECK(y_bitwise, "Y = (tau*s)*float(acc) + b, bitwise");
    // backward
    UNWRAP(dy, eng->from_vector(out, n, dY));
    UNWRAP(dx, layer->backward(*dy));
    UNWRAP(hdx, eng->download_vector(*dx));
    UNWRAP(hgw, eng->download_vector(layer->grad_weight()));
    UNWRAP(hgb, eng->download_vector(layer->grad_bias()));
    double worst = 0;
    for (std::size_t k = 0; k < in; ++k)
        for (std::size_t j = 0; j < n; ++j) {
            double acc = 0;
            for (std::size_t r = 0; r < out; ++r) acc += (double)(*htau)[r] * trit[r * in + k] * (double)dY[r * n + j];
            worst = std::fmax(worst, std::fabs(acc - (*hdx)[k * n + j]));
        }
    CHECK(worst <= 1e-4, "dX = (tau o Wq)^T dY");
    worst = 0;
    for (std::size_t r = 0; r < out; ++r)
        for (std::size_t k = 0; k < in; ++k) {
            double acc = 0;
            for (std::size_t j = 0; j < n; ++j) acc += (double)(dY[r * n + j] * s[j]) * q[k * n + j];
            worst = std::fmax(worst, std::fabs(acc * (*htau)[r] - (*hgw)[r * in + k]) / std::fmax(1.0, std::fabs(acc * (*htau)[r])));
        }
    CHECK(worst <= 1e-5, "dW += ((dY o s) Q^T) o tau");
    worst = 0;
    for (std::size_t r = 0; r < out; ++r) {
        double acc = 0;
        for (std::size_t j = 0; j < n; ++j) acc += dY[r * n + j];
        worst = std::fmax(worst, std::fabs(acc - (*hgb)[r]));
    }
    CHECK(worst <= 1e-5, "db += sum over tokens of dY");
    // write-epoch cache: a write to the latent forces a re-pack whose words equal a pack from scratch
    UNWRAP(before, eng->download_vector(layer->packed()));
    for (auto& w : W) w = -w;
    UNWRAP(u3, eng->upload_span(layer->weight(), W.data(), W.size()));
    CHECK(layer->needs_quantize_(), "a written latent needs re-quantising");
    UNWRAP(y2, layer->forward(*x));
    UNWRAP(repacked, eng->download_vector(layer->packed()));
    UNWRAP(fresh, eng->trit_pack(layer->weight(), layer->tau()));
    UNWRAP(hfresh, eng->download_vector(*fresh));
    CHECK(std::memcmp(repacked->data(), hfresh->data(), hfresh->size() * 4) == 0, "re-packed words equal a pack from scratch");
    CHECK(std::memcmp(repacked->data(), before->data(), before->size() * 4) != 0, "the pack followed the new weights");
    return 0;
}

static int test_data_movement(std::shared_ptr<nnb::ComputeEngine> eng)
{
    std::vector<float> v(6 * 4);
    for (std::size_t i = 0; i < v.size(); ++i) v[i] = (float)i;
    UNWRAP(t, eng->from_vector(6, 4, v));
    const std::uint64_t e0 = t->write_epoch();
    UNWRAP(sl, eng->slice_rows(*t, 2, 3));
    UNWRAP(hs, eng->download_vector(*sl));
    CHECK(hs->size() == 12 && (*hs)[0] == 8.0f && (*hs)[11] == 19.0f, "slice_rows");
    UNWRAP(z, eng->create_tensor(6, 4));
    UNWRAP(ins, eng->insert_rows(*z, 1, *sl));
    UNWRAP(hz, eng->download_vector(*z));
    CHECK((*hz)[0] == 0.0f && (*hz)[4] == 8.0f && (*hz)[15] == 19.0f && (*hz)[16] == 0.0f, "insert_rows");
    UNWRAP(idx, eng->from_vector(3, 1, {5.0f, 0.0f, 9.0f}));
    UNWRAP(g, eng->gather_rows(*t, *idx));
    UNWRAP(hg, eng->download_vector(*g));
    CHECK((*hg)[0] == 20.0f && (*hg)[4] == 0.0f && (*hg)[7] == 3.0f && (*hg)[8] == 0.0f && (*hg)[11] == 0.0f, "gather_rows (out of range -> zero row)");
    UNWRAP(idx2, eng->from_vector(3, 1, {1.0f, 1.0f, 4.0f}));
    UNWRAP(grad, eng->from_vector(3, 4, std::vector<float>(12, 1.5f)));
    UNWRAP(sc, eng->scatter_add_rows(*z, *idx2, *grad));
    UNWRAP(hz2, eng->download_vector(*z));
    CHECK((*hz2)[4] == 11.0f && (*hz2)[16] == 1.5f && (*hz2)[0] == 0.0f, "scatter_add_rows accumulates repeated indices");
    UNWRAP(r, eng->rearrange_3d(*t, 6, 2, 2));  // (6, 2*2) -> (12, 2)
    UNWRAP(hr, eng->download_vector(*r));
    CHECK(r->rows() == 12 && r->cols() == 2 && (*hr)[(1 * 6 + 3) * 2 + 1] == v[3 * 4 + 1 * 2 + 1], "rearrange_3d");
    UNWRAP(back, eng->rearrange_3d(*r, 6, 2, 2, true));
    UNWRAP(hb, eng->download_vector(*back));
    CHECK(*hb == v, "rearrange_3d inverse");
    UNWRAP(tt, eng->transpose(*t));
    UNWRAP(htt, eng->download_vector(*tt));
    CHECK(tt->rows() == 4 && (*htt)[1 * 6 + 2] == v[2 * 4 + 1], "transpose");
    UNWRAP(cm, eng->col_reduce_max(*t));
    UNWRAP(hcm, eng->download_vector(*cm));
    CHECK(hcm->size() == 4 && (*hcm)[0] == 20.0f && (*hcm)[3] == 23.0f, "col_reduce_max");
    UNWRAP(cl, eng->clone(*t));
    UNWRAP(acc, eng->accumulate(*cl, *t));
    UNWRAP(scal, eng->scale_inplace(*cl, 0.5f));
    UNWRAP(hcl, eng->download_vector(*cl));
    CHECK(*hcl == v, "clone + accumulate + scale_inplace");
    CHECK(t->write_epoch() == e0 && cl->write_epoch() > 0, "reads leave the write epoch alone, writes advance it");
    UNWRAP(bad, eng->create_tensor(5, 4));
    CHECK(!eng->accumulate(*bad, *t), "a shape mismatch is an error result, not a crash");
    return 0;
}

static int test_pipeline(std::shared_ptr<nnb::ComputeEngine> eng)
{
    nnb_gpt_config cfg{2, 64, 2, 128, 97, 24, 1, 1, 0, 1};
    UNWRAP(pol, nnb::GptPolicy::create(eng, cfg));
    std::vector<float> flat(pol->param_count());
    std::mt19937 gen(1);
    std::normal_distribution<float> nd(0.0f, 0.05f);
    for (auto& p : flat) p = nd(gen);
    UNWRAP(up, pol->upload_params(flat));
    nnb::GptRolloutSource::Spec spec;
    spec.n_seq = 8;
    spec.prompt_len = 4;
    spec.max_new = 6;
    spec.group_size = 4;
    spec.sampling.top_k = 10;
    std::vector<std::int32_t> prompts(8 * 4);
    for (std::size_t b = 0; b < 8; ++b)
        for (std::size_t t = 0; t < 4; ++t) prompts[b * 4 + t] = (std::int32_t)((b / 4) * 7 + t * 3) % 97;
    auto reward = [](const std::vector<std::int32_t>& tok, std::size_t n, std::size_t S) {
        std::vector<float> r(n);
        for (std::size_t b = 0; b < n; ++b) r[b] = (float)(tok[b * S + S - 1] % 2);
        return r;
    };
    auto source = std::make_unique<nnb::GptRolloutSource>(*pol, spec, prompts, reward);
    nnb::RLPipelineConfig pc;
    pc.batch_size = 1;
    pc.clear_buffer_after_update = true;
    auto sink = std::make_shared<nnb::CollectingMetricSink>();
    UNWRAP(pipe, nnb::RLTrainingPipeline::create(pc, std::move(source), std::make_unique<nnb::UniformBatchSampler>(), sink, 5));
    nnb_policy* ph = pol->handle();
    nnb_engine* e = eng->handle();
    auto update = [&](const std::vector<const nnb::TensorRecord*>& sel, nnb::DeterministicRng&, nnb::MetricSink& metrics) -> nnb::Result<void> {
        const nnb::TensorRecord& rec = *sel[0];
        NNB_TRYR(tok, rec.require("tokens"));
        NNB_TRYR(mask, rec.require("action_mask"));
        NNB_TRYR(adv, rec.require("advantage"));
        NNB_TRYR(old, rec.require("old_log_prob"));
        NNB_TRYR(htok, eng->download_vector(**tok));
        std::vector<std::int32_t> itok(htok->size());
        for (std::size_t i = 0; i < itok.size(); ++i) itok[i] = (std::int32_t)(*htok)[i];
        void* d_tok = nullptr;
        float* d_rep = nullptr;
        if (nnb_alloc(e, itok.size() * 4, &d_tok) != NNB_OK || nnb_alloc(e, 40, (void**)&d_rep) != NNB_OK) return nnb::abi_error("alloc");
        nnb_upload(e, d_tok, itok.data(), itok.size() * 4);
        nnb_objective obj{(*mask)->device_data(), (*old)->device_data(), (*adv)->device_data(), nullptr, nullptr, nullptr, 0.0f, 0.2f, 0.0f, 0.0f, 0.0f, 0.2f};
        nnb_policy_zero_grad(ph);
        nnb_status st = nnb_policy_train_step_grouped(ph, (const std::int32_t*)d_tok, 8, 10, 4, 4, &obj, d_rep);
        if (st == NNB_OK) st = nnb_policy_optimizer_step(ph, 1e-3f, 0.9f, 0.999f, 1e-8f, 0.01f, 1.0f, nullptr);
        float rep[NNB_REPORT_COUNT];
        if (st == NNB_OK) st = nnb_download(e, rep, d_rep, sizeof rep);
        nnb_free(e, d_tok);
        nnb_free(e, d_rep);
        if (st != NNB_OK) return nnb::abi_error("update");
        return metrics.emit({"ratio_mean", rep[NNB_REPORT_RATIO_MEAN]});
    };
    UNWRAP(ran, pipe->run(2, update));
    CHECK(pipe->update_count() == 2 && pipe->rollout_cursor() == 2 && pipe->buffer().empty(), "two rollouts, two updates, buffer cleared");
    CHECK(sink->records().size() == 2 && std::fabs(sink->records()[0].value - 1.0) < 1e-3,
          "the first update sees ratio 1: the teacher-forced log-probs equal the rollout's");
    nnb::DeterministicRng a(7), b(7);
    auto s1 = nnb::UniformBatchSampler(false).sample(10, 10, a);
    std::string st = b.save_state();
    auto s2 = nnb::UniformBatchSampler(false).sample(10, 10, b);
    CHECK(s1 && s2 && *s1 == *s2, "the sampler is deterministic per seed");
    nnb::DeterministicRng c(0);
    CHECK(c.restore_state(st) && *nnb::UniformBatchSampler(false).sample(10, 10, c) == *s1, "rng state round trip");
    CHECK(!nnb::UniformBatchSampler(false).sample(3, 4, a), "sampling more than the buffer holds without replacement is an error");
    return 0;
}

int main()
{
    auto eng = nnb::create_gpu_engine("0");
    if (!eng) {
        std::fprintf(stderr, "engine: %s\n", nnb::last_error());
        return 3;
    }
    const nnb::EngineInfo info = eng->describe();
    CHECK(info.ternary_gemm && info.int8_dot, "describe() reports the ternary and int8 paths");
    int rc = test_bitlinear(eng, 130, 17, 6);
    if (!rc) rc = test_bitlinear(eng, 512, 256, 8);
    if (!rc) rc = test_data_movement(eng);
    if (!rc) rc = test_pipeline(eng);
    if (rc) return rc;
    if (g_fail) {
        std::fprintf(stderr, "%d check(s) failed\n", g_fail);
        return 1;
    }
    std::puts("shim ok");
    return 0;
}
