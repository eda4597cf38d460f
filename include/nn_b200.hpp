// nn_b200.hpp — header-only C++17 host layer over the C-ABI of libnn-b200.so (nn_b200.h), shaped like the
// interfaces the reference's layer / RL code is written against, so that code can be pointed at this engine:
//
//   nnb::ComputeEngine   the verbs BitLinear and the data-movement layers call on nn::ComputeEngine
//                        (docs/internal/12-compute-engine-inventory.md:70-78; obtained like
//                        nn::create_gpu_engine(device) / nn::last_error(),
//                        include/neuralnet.cpp/cli/cli_engine_factory.hpp:51-77)
//   nnb::Tensor          value type over refcounted storage with a write epoch (AGENTS.md:158-164)
//   nnb::Result<T>       the reference returns exstl::Result<T> = std::expected<T, Error{message}> and never throws
//                        (AGENTS.md:240); this is the C++17 stand-in with the same use: if (!r) r.error().message
//   nnb::BitLinear       BitLinear::forward / backward / quantize_weights_ / needs_quantize_ with the call sequence of
//                        include/neuralnet.cpp/compute_layer_bitlinear.hpp:417-544,607-674 (W1.58A8 path)
//   nnb::DeterministicRng, ExperienceBuffer, UniformBatchSampler, MetricSink, RLTrainingPipeline
//                        include/neuralnet.cpp/rl_pipeline.hpp:29-350, same names and preconditions
//   nnb::GptPolicy, GptRolloutSource   the ternary GPT policy object of the library and a device-side RolloutSource
//
// The reference's expression DSL (dsl::compute on arbitrary ExprSpec trees) is not part of this engine: the three
// compositions BitLinear evaluates exist as single verbs (abs, add_row_broadcast, bitlinear_dw_accumulate).
// Nothing here falls back to the CPU: without the library or a B200 every factory returns null / an error.
#ifndef NN_B200_HPP
#define NN_B200_HPP

#include <cstdint>
#include <functional>
#include <memory>
#include <optional>
#include <random>
#include <sstream>
#include <string>
#include <utility>
#include <vector>

#include "nn_b200.h"

namespace nnb {

struct Error {
    std::string message;
};

template <class T>
class Result {
    std::optional<T> value_;
    Error error_;

public:
    Result(T v) : value_(std::move(v)) {}
    Result(Error e) : error_(std::move(e)) {}
    explicit operator bool() const noexcept { return value_.has_value(); }
    bool has_value() const noexcept { return value_.has_value(); }
    T& operator*() { return *value_; }
    const T& operator*() const { return *value_; }
    T* operator->() { return &*value_; }
    const T* operator->() const { return &*value_; }
    const Error& error() const noexcept { return error_; }
};

template <>
class Result<void> {
    bool ok_ = true;
    Error error_;

public:
    Result() = default;
    Result(Error e) : ok_(false), error_(std::move(e)) {}
    explicit operator bool() const noexcept { return ok_; }
    bool has_value() const noexcept { return ok_; }
    const Error& error() const noexcept { return error_; }
};

inline Error fail(const std::string& what) { return Error{what}; }
inline Error abi_error(const char* where)
{
    const char* m = nnb_last_error();
    return Error{std::string(where) + ": " + (m ? m : "?")};
}

// ------------------------------------------------------------------ tensor
class Tensor {
    std::shared_ptr<nnb_tensor> h_;

public:
    Tensor() = default;
    explicit Tensor(nnb_tensor* owned) : h_(owned, [](nnb_tensor* t) { nnb_tensor_destroy(t); }) {}
    bool valid() const noexcept { return h_ != nullptr; }
    std::size_t rows() const noexcept { return nnb_tensor_rows(h_.get()); }
    std::size_t cols() const noexcept { return nnb_tensor_cols(h_.get()); }
    std::uint64_t write_epoch() const noexcept { return nnb_tensor_write_epoch(h_.get()); }
    nnb_tensor* raw() const noexcept { return h_.get(); }
    float* device_data() const noexcept { return nnb_tensor_data(h_.get()); }
};

struct EngineInfo {
    bool ternary_gemm = false, int8_dot = false, int8_dot_accelerated = false;
    std::string description;
    const std::string& text() const { return description; }
};

// ------------------------------------------------------------------ engine
class ComputeEngine : public std::enable_shared_from_this<ComputeEngine> {
    nnb_engine* e_ = nullptr;

    explicit ComputeEngine(nnb_engine* e) : e_(e) {}
    static Result<Tensor> made(nnb_status st, nnb_tensor* t, const char* where)
    {
        if (st != NNB_OK) return abi_error(where);
        return Tensor(t);
    }
    static Result<void> done(nnb_status st, const char* where)
    {
        if (st != NNB_OK) return abi_error(where);
        return {};
    }

public:
    ComputeEngine(const ComputeEngine&) = delete;
    ComputeEngine& operator=(const ComputeEngine&) = delete;
    ~ComputeEngine() { nnb_engine_destroy(e_); }

    static std::shared_ptr<ComputeEngine> create(int device)
    {
        nnb_engine* e = nullptr;
        if (nnb_engine_create(device, &e) != NNB_OK) return nullptr;  // nnb::last_error() says why
        return std::shared_ptr<ComputeEngine>(new ComputeEngine(e));
    }

    nnb_engine* handle() const noexcept { return e_; }
    EngineInfo describe() const
    {
        char buf[512] = "";
        nnb_engine_describe(e_, buf, sizeof(buf));
        EngineInfo i;
        i.description = buf;
        i.ternary_gemm = i.description.find("ternary_gemm=true") != std::string::npos;
        i.int8_dot = i.description.find("int8_dot=true") != std::string::npos;
        i.int8_dot_accelerated = i.description.find("int8_dot_accelerated=true") != std::string::npos;
        return i;
    }
    // begin_batch / end_batch / flush_batch of the reference bracket a recorded command buffer; work here is stream
    // ordered, so the only thing left of them is the synchronisation at the end
    Result<void> begin_batch() { return {}; }
    Result<void> flush_batch() { return done(nnb_engine_sync(e_), "flush_batch"); }
    Result<void> end_batch() { return done(nnb_engine_sync(e_), "end_batch"); }

    Result<Tensor> create_tensor(std::size_t rows, std::size_t cols)
    {
        nnb_tensor* t = nullptr;
        const nnb_status st = nnb_tensor_create(e_, rows, cols, &t);
        return made(st, t, "create_tensor");
    }
    Result<Tensor> try_create_tensor(std::size_t rows, std::size_t cols) { return create_tensor(rows, cols); }
    Result<Tensor> from_vector(std::size_t rows, std::size_t cols, const std::vector<float>& values)
    {
        if (values.size() != rows * cols) return fail("from_vector: value count does not match the shape");
        auto t = create_tensor(rows, cols);
        if (!t) return t;
        if (nnb_tensor_upload(t->raw(), values.data(), values.size()) != NNB_OK) return abi_error("from_vector");
        return t;
    }
    Result<void> upload_span(Tensor& t, const float* src, std::size_t n) { return done(nnb_tensor_upload(t.raw(), src, n), "upload_span"); }
    Result<std::vector<float>> download_vector(const Tensor& t)
    {
        std::vector<float> out(t.rows() * t.cols());
        if (nnb_tensor_download(t.raw(), out.data(), out.size()) != NNB_OK) return abi_error("download_vector");
        return out;
    }
    Result<void> zero(Tensor& t) { return done(nnb_t_zero(t.raw()), "zero"); }
    Result<Tensor> clone(const Tensor& src)
    {
        nnb_tensor* t = nullptr;
        const nnb_status st = nnb_t_clone(src.raw(), &t);
        return made(st, t, "clone");
    }
    Result<void> copy_into(const Tensor& src, Tensor& dst) { return done(nnb_t_copy_into(dst.raw(), src.raw()), "copy_into"); }
    Result<Tensor> transpose(const Tensor& src)
    {
        nnb_tensor* t = nullptr;
        const nnb_status st = nnb_t_transpose(src.raw(), &t);
        return made(st, t, "transpose");
    }
    Result<Tensor> slice_rows(const Tensor& src, std::size_t start_row, std::size_t count)
    {
        nnb_tensor* t = nullptr;
        const nnb_status st = nnb_t_slice_rows(src.raw(), start_row, count, &t);
        return made(st, t, "slice_rows");
    }
    Result<void> insert_rows(Tensor& dst, std::size_t row, const Tensor& src) { return done(nnb_t_insert_rows(dst.raw(), row, src.raw()), "insert_rows"); }
    Result<Tensor> gather_rows(const Tensor& table, const Tensor& indices)
    {
        nnb_tensor* t = nullptr;
        const nnb_status st = nnb_t_gather_rows(table.raw(), indices.raw(), &t);
        return made(st, t, "gather_rows");
    }
    Result<void> scatter_add_rows(Tensor& dst, const Tensor& indices, const Tensor& grad)
    {
        return done(nnb_t_scatter_add_rows(dst.raw(), indices.raw(), grad.raw()), "scatter_add_rows");
    }
    Result<Tensor> rearrange_3d(const Tensor& x, std::size_t M, std::size_t B, std::size_t N, bool inverse = false)
    {
        nnb_tensor* t = nullptr;
        const nnb_status st = nnb_t_rearrange_3d(x.raw(), M, B, N, inverse ? 1 : 0, &t);
        return made(st, t, "rearrange_3d");
    }
    Result<void> scale_inplace(Tensor& t, float s) { return done(nnb_t_scale_inplace(t.raw(), s), "scale_inplace"); }
    Result<void> accumulate(Tensor& dst, const Tensor& src) { return done(nnb_t_accumulate(dst.raw(), src.raw()), "accumulate"); }
    Result<Tensor> col_reduce_max(const Tensor& t)
    {
        nnb_tensor* o = nullptr;
        const nnb_status st = nnb_t_col_reduce_max(t.raw(), &o);
        return made(st, o, "col_reduce_max");
    }
    Result<Tensor> row_reduce_sum(const Tensor& t)
    {
        nnb_tensor* o = nullptr;
        const nnb_status st = nnb_t_row_reduce_sum(t.raw(), &o);
        return made(st, o, "row_reduce_sum");
    }
    // ---- ternary primitives (compute_layer_bitlinear.hpp:443-464,494,516,637-650)
    Result<Tensor> absmean_tau(const Tensor& latent)
    {
        nnb_tensor* o = nullptr;
        const nnb_status st = nnb_t_absmean_tau(latent.raw(), &o);
        return made(st, o, "absmean_tau");
    }
    Result<Tensor> trit_pack(const Tensor& latent, const Tensor& tau)
    {
        nnb_tensor* o = nullptr;
        const nnb_status st = nnb_t_trit_pack(latent.raw(), tau.raw(), &o);
        return made(st, o, "trit_pack");
    }
    Result<void> trit_pack_into(const Tensor& latent, const Tensor& tau, Tensor& dst)
    {
        return done(nnb_t_trit_pack_into(latent.raw(), tau.raw(), dst.raw()), "trit_pack_into");
    }
    Result<Tensor> matmul_q(const Tensor& packed, const Tensor& tau, const Tensor& x)
    {
        nnb_tensor* o = nullptr;
        const nnb_status st = nnb_t_matmul_q(packed.raw(), tau.raw(), x.raw(), &o);
        return made(st, o, "matmul_q");
    }
    Result<Tensor> matmul_q_t(const Tensor& packed, const Tensor& tau, const Tensor& dy, std::size_t m_cols)
    {
        nnb_tensor* o = nullptr;
        const nnb_status st = nnb_t_matmul_q_t(packed.raw(), tau.raw(), dy.raw(), m_cols, &o);
        return made(st, o, "matmul_q_t");
    }
    Result<Tensor> quantize_i8(const Tensor& x, const Tensor& scale, bool col_scale)
    {
        nnb_tensor* o = nullptr;
        const nnb_status st = nnb_t_quantize_i8(x.raw(), scale.raw(), col_scale ? 1 : 0, &o);
        return made(st, o, "quantize_i8");
    }
    Result<Tensor> unpack_i8(const Tensor& packed, std::size_t cols)
    {
        nnb_tensor* o = nullptr;
        const nnb_status st = nnb_t_unpack_i8(packed.raw(), cols, &o);
        return made(st, o, "unpack_i8");
    }
    Result<Tensor> matmul_q_i8(const Tensor& packed, const Tensor& tau, const Tensor& xq, const Tensor& s)
    {
        nnb_tensor* o = nullptr;
        const nnb_status st = nnb_t_matmul_q_i8(packed.raw(), tau.raw(), xq.raw(), s.raw(), &o);
        return made(st, o, "matmul_q_i8");
    }
    // ---- the three DSL compositions of BitLinear as verbs
    Result<Tensor> abs(const Tensor& x)
    {
        nnb_tensor* o = nullptr;
        const nnb_status st = nnb_t_abs(x.raw(), &o);
        return made(st, o, "abs");
    }
    Result<void> add_row_broadcast(Tensor& y, const Tensor& b) { return done(nnb_t_add_row_broadcast(y.raw(), b.raw()), "add_row_broadcast"); }
    Result<void> bitlinear_dw_accumulate(Tensor& grad_w, const Tensor& dy, const Tensor* s, const Tensor& x, const Tensor& tau)
    {
        return done(nnb_t_bitlinear_dw_accumulate(grad_w.raw(), dy.raw(), s ? s->raw() : nullptr, x.raw(), tau.raw()), "bitlinear_dw_accumulate");
    }
};

inline std::shared_ptr<ComputeEngine> create_gpu_engine(const char* device = nullptr)
{
    int index = 0;
    if (device && *device) index = std::atoi(device);
    return ComputeEngine::create(index);
}
inline const char* last_error() { return nnb_last_error(); }

#define NNB_TRYR(var, expr)                  \
    auto var = (expr);                       \
    if (!var) return ::nnb::Error{var.error().message}

// ------------------------------------------------------------------ BitLinear (W1.58A8)
class BitLinear {
    std::shared_ptr<ComputeEngine> engine_;
    std::size_t in_ = 0, out_ = 0;
    Tensor w_, b_, grad_w_, grad_b_, tau_, wq_packed_, input_cache_, act_scale_;
    std::uint64_t quantized_epoch_ = ~0ull;  // write epoch of w_ the packed weights were made from

    BitLinear() = default;

public:
    static Result<BitLinear> create(std::shared_ptr<ComputeEngine> engine, std::size_t in_features, std::size_t out_features)
    {
        BitLinear l;
        l.engine_ = std::move(engine);
        l.in_ = in_features;
        l.out_ = out_features;
        NNB_TRYR(w, l.engine_->create_tensor(out_features, in_features));
        NNB_TRYR(b, l.engine_->create_tensor(out_features, 1));
        NNB_TRYR(gw, l.engine_->create_tensor(out_features, in_features));
        NNB_TRYR(gb, l.engine_->create_tensor(out_features, 1));
        l.w_ = *w;
        l.b_ = *b;
        l.grad_w_ = *gw;
        l.grad_b_ = *gb;
        return l;
    }
    Tensor& weight() { return w_; }
    Tensor& bias() { return b_; }
    Tensor& grad_weight() { return grad_w_; }
    Tensor& grad_bias() { return grad_b_; }
    const Tensor& tau() const { return tau_; }
    const Tensor& packed() const { return wq_packed_; }

    // compute_layer_bitlinear.hpp:607-615: only a latent whose storage was written since the last pack is re-packed
    bool needs_quantize_() const { return !wq_packed_.valid() || quantized_epoch_ != w_.write_epoch(); }
    // :627-674: tau = row_reduce_sum(|W| * (1/K)), then trit_pack[_into]
    Result<void> quantize_weights_()
    {
        NNB_TRYR(tau, engine_->absmean_tau(w_));
        tau_ = *tau;
        if (wq_packed_.valid()) {
            NNB_TRYR(r, engine_->trit_pack_into(w_, tau_, wq_packed_));
        } else {
            NNB_TRYR(p, engine_->trit_pack(w_, tau_));
            wq_packed_ = *p;
        }
        quantized_epoch_ = w_.write_epoch();
        return {};
    }
    // :417-472, the int8-activation branch; input (in_features, tokens)
    Result<Tensor> forward(const Tensor& input)
    {
        if (input.rows() != in_) return fail("bitlinear forward: input shape mismatch");
        if (needs_quantize_()) {
            NNB_TRYR(q, quantize_weights_());
        }
        NNB_TRYR(xabs, engine_->abs(input));
        NNB_TRYR(sraw, engine_->col_reduce_max(*xabs));
        NNB_TRYR(ss, engine_->scale_inplace(*sraw, 1.0f / 127.0f));
        NNB_TRYR(xq, engine_->quantize_i8(input, *sraw, /*col_scale=*/true));
        input_cache_ = *xq;
        act_scale_ = *sraw;
        NNB_TRYR(y, engine_->matmul_q_i8(wq_packed_, tau_, *xq, *sraw));
        NNB_TRYR(yb, engine_->add_row_broadcast(*y, b_));
        return *y;
    }
    // :475-544; grad_output (out_features, tokens); accumulates into grad_weight / grad_bias
    Result<Tensor> backward(const Tensor& grad_output)
    {
        if (grad_output.rows() != out_) return fail("bitlinear backward: grad_output shape mismatch");
        if (!tau_.valid() || !input_cache_.valid() || !act_scale_.valid()) return fail("bitlinear backward: forward must run first");
        NNB_TRYR(gi, engine_->matmul_q_t(wq_packed_, tau_, grad_output, in_));
        NNB_TRYR(xq32, engine_->unpack_i8(input_cache_, grad_output.cols()));
        NNB_TRYR(dw, engine_->bitlinear_dw_accumulate(grad_w_, grad_output, &act_scale_, *xq32, tau_));
        NNB_TRYR(gb, engine_->row_reduce_sum(grad_output));
        NNB_TRYR(acc, engine_->accumulate(grad_b_, *gb));
        return *gi;
    }
};

// ------------------------------------------------------------------ RL pipeline (rl_pipeline.hpp:29-350)
class DeterministicRng {
    std::uint64_t seed_ = 0;
    std::mt19937_64 engine_;

public:
    explicit DeterministicRng(std::uint64_t seed = 0) : seed_(seed), engine_(seed) {}
    std::uint64_t seed() const noexcept { return seed_; }
    std::uint64_t next_u64() { return engine_(); }
    Result<std::size_t> uniform_index(std::size_t upper_exclusive)
    {
        if (upper_exclusive == 0) return fail("DeterministicRng: uniform_index upper bound must be > 0");
        std::uniform_int_distribution<std::size_t> dist(0, upper_exclusive - 1);
        return dist(engine_);
    }
    std::string save_state() const
    {
        std::ostringstream out;
        out << "RNGS1 " << seed_ << ' ' << engine_;
        return out.str();
    }
    Result<void> restore_state(const std::string& state)
    {
        std::istringstream in(state);
        std::string tag;
        std::uint64_t saved = 0;
        in >> tag >> saved;
        if (!in || tag != "RNGS1") return fail("DeterministicRng::restore_state: bad state header");
        in >> engine_;
        if (!in) return fail("DeterministicRng::restore_state: incomplete state");
        seed_ = saved;
        return {};
    }
};

struct NamedTensor {
    std::string name;
    Tensor value;
};

// Named tensors of one rollout (TensorRecord, rl_experience.hpp:32-68); per-decision fields are (n_seq, G) f32
class TensorRecord {
    std::vector<NamedTensor> fields_;

public:
    static Result<TensorRecord> create(std::vector<NamedTensor> fields)
    {
        for (std::size_t i = 0; i < fields.size(); ++i) {
            if (!fields[i].value.valid()) return fail("TensorRecord: field '" + fields[i].name + "' is empty");
            for (std::size_t j = 0; j < i; ++j)
                if (fields[j].name == fields[i].name) return fail("TensorRecord: duplicate field '" + fields[i].name + "'");
        }
        TensorRecord r;
        r.fields_ = std::move(fields);
        return r;
    }
    Result<const Tensor*> require(const std::string& name) const
    {
        for (const auto& f : fields_)
            if (f.name == name) return &f.value;
        return fail("TensorRecord: no field '" + name + "'");
    }
    std::size_t size() const noexcept { return fields_.size(); }
};

class RolloutSource {
public:
    virtual ~RolloutSource() = default;
    virtual Result<TensorRecord> rollout(DeterministicRng& rng) = 0;
};

class ExperienceBuffer {
    std::vector<TensorRecord> records_;
    std::size_t capacity_ = 0;

public:
    explicit ExperienceBuffer(std::size_t capacity = 0) : capacity_(capacity) {}
    Result<void> add(TensorRecord record)
    {
        if (capacity_ > 0 && records_.size() >= capacity_) records_.erase(records_.begin());
        records_.push_back(std::move(record));
        return {};
    }
    std::size_t size() const noexcept { return records_.size(); }
    bool empty() const noexcept { return records_.empty(); }
    std::size_t capacity() const noexcept { return capacity_; }
    void clear() noexcept { records_.clear(); }
    Result<const TensorRecord*> at(std::size_t index) const
    {
        if (index >= records_.size()) return fail("ExperienceBuffer::at: index out of range");
        return &records_[index];
    }
};

class BatchSampler {
public:
    virtual ~BatchSampler() = default;
    virtual Result<std::vector<std::size_t>> sample(std::size_t available, std::size_t batch_size, DeterministicRng& rng) = 0;
};

class UniformBatchSampler final : public BatchSampler {
    bool replacement_ = false;

public:
    explicit UniformBatchSampler(bool replacement = false) : replacement_(replacement) {}
    Result<std::vector<std::size_t>> sample(std::size_t available, std::size_t batch_size, DeterministicRng& rng) override
    {
        if (batch_size == 0) return fail("UniformBatchSampler: batch_size must be > 0");
        if (available == 0) return fail("UniformBatchSampler: buffer is empty");
        if (!replacement_ && batch_size > available) return fail("UniformBatchSampler: batch_size > buffer size without replacement");
        std::vector<std::size_t> out;
        out.reserve(batch_size);
        if (replacement_) {
            for (std::size_t i = 0; i < batch_size; ++i) {
                NNB_TRYR(k, rng.uniform_index(available));
                out.push_back(*k);
            }
            return out;
        }
        std::vector<std::size_t> pool(available);
        for (std::size_t i = 0; i < available; ++i) pool[i] = i;
        for (std::size_t i = 0; i < batch_size; ++i) {
            NNB_TRYR(k, rng.uniform_index(available - i));
            std::swap(pool[i], pool[i + *k]);
            out.push_back(pool[i]);
        }
        return out;
    }
};

struct MetricRecord {
    std::string name;
    double value = 0;
};

class MetricSink {
public:
    virtual ~MetricSink() = default;
    virtual Result<void> emit(const MetricRecord& metric) = 0;
};

class CollectingMetricSink final : public MetricSink {
    std::vector<MetricRecord> records_;

public:
    Result<void> emit(const MetricRecord& metric) override
    {
        records_.push_back(metric);
        return {};
    }
    const std::vector<MetricRecord>& records() const noexcept { return records_; }
};

struct RLPipelineConfig {
    std::size_t batch_size = 1, collect_per_update = 1, buffer_capacity = 0, min_buffer_size = 1;
    bool clear_buffer_after_update = false;
};

class RLTrainingPipeline {
    RLPipelineConfig cfg_;
    std::unique_ptr<RolloutSource> source_;
    std::unique_ptr<BatchSampler> sampler_;
    std::shared_ptr<MetricSink> metrics_;
    ExperienceBuffer buffer_;
    DeterministicRng rng_;
    std::uint64_t update_count_ = 0, rollout_cursor_ = 0;

    RLTrainingPipeline(RLPipelineConfig cfg, std::unique_ptr<RolloutSource> source, std::unique_ptr<BatchSampler> sampler,
                       std::shared_ptr<MetricSink> metrics, std::uint64_t seed)
        : cfg_(cfg), source_(std::move(source)), sampler_(std::move(sampler)), metrics_(std::move(metrics)),
          buffer_(cfg.buffer_capacity), rng_(seed)
    {
    }

public:
    static Result<RLTrainingPipeline> create(RLPipelineConfig cfg, std::unique_ptr<RolloutSource> source, std::unique_ptr<BatchSampler> sampler,
                                             std::shared_ptr<MetricSink> metrics = {}, std::uint64_t seed = 0)
    {
        if (!source || !sampler) return fail("RLTrainingPipeline::create: source and sampler are required");
        if (cfg.batch_size == 0 || cfg.collect_per_update == 0 || cfg.min_buffer_size == 0)
            return fail("RLTrainingPipeline::create: batch / collect / min_buffer must be > 0");
        if (cfg.min_buffer_size < cfg.batch_size) return fail("RLTrainingPipeline::create: min_buffer_size must not be smaller than batch_size");
        if (cfg.buffer_capacity > 0 && cfg.min_buffer_size > cfg.buffer_capacity)
            return fail("RLTrainingPipeline::create: min_buffer_size must not exceed buffer_capacity");
        if (!metrics) metrics = std::make_shared<CollectingMetricSink>();
        return RLTrainingPipeline(cfg, std::move(source), std::move(sampler), std::move(metrics), seed);
    }
    RLTrainingPipeline(RLTrainingPipeline&&) noexcept = default;
    const ExperienceBuffer& buffer() const noexcept { return buffer_; }
    std::uint64_t update_count() const noexcept { return update_count_; }
    std::uint64_t rollout_cursor() const noexcept { return rollout_cursor_; }
    MetricSink& metrics() noexcept { return *metrics_; }

    // update(selected records, rng, metrics) -> Result<void>
    template <class UpdateFn>
    Result<void> run(std::size_t updates, UpdateFn&& update)
    {
        for (std::size_t i = 0; i < updates; ++i) {
            for (std::size_t c = 0; c < cfg_.collect_per_update; ++c) {
                NNB_TRYR(record, source_->rollout(rng_));
                NNB_TRYR(added, buffer_.add(std::move(*record)));
                ++rollout_cursor_;
            }
            if (buffer_.size() < cfg_.min_buffer_size) return fail("RLTrainingPipeline: buffer below min_buffer_size");
            NNB_TRYR(indices, sampler_->sample(buffer_.size(), cfg_.batch_size, rng_));
            if (indices->size() != cfg_.batch_size) return fail("RLTrainingPipeline: sampler returned a wrong batch size");
            std::vector<const TensorRecord*> selected;
            for (std::size_t index : *indices) {
                NNB_TRYR(rec, buffer_.at(index));
                selected.push_back(*rec);
            }
            NNB_TRYR(upd, update(selected, rng_, *metrics_));
            ++update_count_;
            if (cfg_.clear_buffer_after_update) buffer_.clear();
        }
        return {};
    }
};

// ------------------------------------------------------------------ the ternary GPT policy of the library
class GptPolicy {
    std::shared_ptr<ComputeEngine> engine_;
    std::shared_ptr<nnb_policy> p_;
    nnb_gpt_config cfg_{};

public:
    static Result<GptPolicy> create(std::shared_ptr<ComputeEngine> engine, const nnb_gpt_config& cfg)
    {
        nnb_policy* p = nullptr;
        if (nnb_policy_create(engine->handle(), &cfg, &p) != NNB_OK) return abi_error("policy_create");
        GptPolicy g;
        g.engine_ = std::move(engine);
        g.p_ = std::shared_ptr<nnb_policy>(p, [](nnb_policy* q) { nnb_policy_destroy(q); });
        g.cfg_ = cfg;
        return g;
    }
    nnb_policy* handle() const noexcept { return p_.get(); }
    const nnb_gpt_config& config() const noexcept { return cfg_; }
    ComputeEngine& engine() const noexcept { return *engine_; }
    std::size_t param_count() const { return nnb_policy_param_count(p_.get()); }
    Result<void> upload_params(const std::vector<float>& flat)
    {
        if (flat.size() != param_count()) return fail("upload_params: wrong parameter count");
        if (nnb_policy_upload_params(p_.get(), flat.data()) != NNB_OK) return abi_error("upload_params");
        return {};
    }
};

// One call = one batched rollout of `prompts` (n_seq x prompt_len ids, host) with rewards from reward_fn and group
// advantages (GroupAdvantage over `group_size` consecutive sequences), all tensors left on the device.  Record fields:
// tokens (n_seq, P+G), action_mask, advantage, old_log_prob (n_seq, G), reward (n_seq, 1).
class GptRolloutSource final : public RolloutSource {
public:
    struct Spec {
        std::size_t n_seq = 0, prompt_len = 0, max_new = 0, group_size = 1;
        nnb_sampling_config sampling{1.0f, 0, 1.0f, 1.0f, 0, 0, nullptr, -1, 0};
    };
    using RewardFn = std::function<std::vector<float>(const std::vector<std::int32_t>& tokens, std::size_t n_seq, std::size_t seq_len)>;

private:
    GptPolicy policy_;
    Spec spec_;
    std::vector<std::int32_t> prompts_;
    RewardFn reward_;

public:
    GptRolloutSource(GptPolicy policy, Spec spec, std::vector<std::int32_t> prompts, RewardFn reward)
        : policy_(std::move(policy)), spec_(spec), prompts_(std::move(prompts)), reward_(std::move(reward))
    {
    }
    Result<TensorRecord> rollout(DeterministicRng& rng) override
    {
        const std::size_t n = spec_.n_seq, P = spec_.prompt_len, G = spec_.max_new, S = P + G;
        if (prompts_.size() != n * P || n % spec_.group_size != 0) return fail("GptRolloutSource: prompts do not match the spec");
        ComputeEngine& eng = policy_.engine();
        nnb_engine* e = eng.handle();
        void *d_prompts = nullptr, *d_tokens = nullptr;
        if (nnb_alloc(e, n * P * 4, &d_prompts) != NNB_OK || nnb_alloc(e, n * S * 4, &d_tokens) != NNB_OK) return abi_error("rollout alloc");
        auto cleanup = [&]() {
            nnb_free(e, d_prompts);
            nnb_free(e, d_tokens);
        };
        NNB_TRYR(logp, eng.create_tensor(n, G));
        nnb_sampling_config sc = spec_.sampling;
        sc.seed = rng.next_u64();
        nnb_status st = nnb_upload(e, d_prompts, prompts_.data(), n * P * 4);
        if (st == NNB_OK)
            st = nnb_rollout_sampled(policy_.handle(), (const std::int32_t*)d_prompts, n, P, G, spec_.group_size, &sc, 0, (std::int32_t*)d_tokens,
                                     logp->device_data(), nullptr, nullptr);
        std::vector<std::int32_t> h_tokens(n * S);
        if (st == NNB_OK) st = nnb_download(e, h_tokens.data(), d_tokens, n * S * 4);
        cleanup();
        if (st != NNB_OK) return abi_error("rollout");
        nnb_tensor_mark_written(logp->raw());
        std::vector<float> reward = reward_(h_tokens, n, S);
        if (reward.size() != n) return fail("GptRolloutSource: reward_fn must return one value per sequence");
        NNB_TRYR(d_reward, eng.from_vector(n, 1, reward));
        std::vector<std::int32_t> first, count;
        for (std::size_t g = 0; g < n / spec_.group_size; ++g) {
            first.push_back((std::int32_t)(g * spec_.group_size));
            count.push_back((std::int32_t)spec_.group_size);
        }
        NNB_TRYR(adv_seq, eng.create_tensor(n, 1));
        if (nnb_group_advantage(e, d_reward->device_data(), n, first.data(), count.data(), first.size(), 1e-8f, adv_seq->device_data()) != NNB_OK)
            return abi_error("group_advantage");
        auto hadv = eng.download_vector(*adv_seq);
        if (!hadv) return Error{hadv.error().message};
        std::vector<float> adv(n * G), mask(n * G, 1.0f), tok(n * S);
        for (std::size_t b = 0; b < n; ++b)
            for (std::size_t g = 0; g < G; ++g) adv[b * G + g] = (*hadv)[b];
        for (std::size_t i = 0; i < n * S; ++i) tok[i] = (float)h_tokens[i];
        NNB_TRYR(d_adv, eng.from_vector(n, G, adv));
        NNB_TRYR(d_mask, eng.from_vector(n, G, mask));
        NNB_TRYR(d_tok, eng.from_vector(n, S, tok));
        return TensorRecord::create({{"tokens", *d_tok}, {"action_mask", *d_mask}, {"advantage", *d_adv}, {"old_log_prob", *logp}, {"reward", *d_reward}});
    }
};

}  // namespace nnb
#endif  // NN_B200_HPP
