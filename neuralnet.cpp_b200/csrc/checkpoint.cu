// checkpoint.cu — model files for the ternary GPT policy in the reference's two roles
// (include/neuralnet.cpp/model_serialization.hpp:40-89, docs/internal/21-quantized-weights.md:856-881):
//   role Model      (.nnmodel): every BitLinear weight as TernaryPacked3 (base-3, 5 trits per byte, 1.6 bits per
//                   weight) with its per-row tau as aux; everything else Dense f32
//   role Checkpoint (.nnckpt):  every BitLinear weight as TernaryLatent (the f32 master weights); everything else Dense
// Parameter entries follow model_serialization.hpp:581-589 byte for byte:
//   [kind 1B][precision 1B][rows 8B][cols 8B][aux_len 8B][payload_len 8B][aux][payload]
// around them the v8 container: magic "NNNN", version 8, precision tag, role, spec record (length-prefixed),
// training-state length (0), the entries, tokenizer length (0), SHA-256 of everything before it, "NNEND".
// Loading a Model-role file makes it trainable again the way WeightLoadIntent::Trainable does
// (compute_layer_bitlinear.hpp:262-300): the latent becomes the quantiser's fixed point L = trit * (tau * K / n)
// (n = non-zero trits of the row; src/ternary_gemm_test.cpp:658-735) and the file's tau and trits seed the packed
// weights, so the first forward reproduces the saved model bit for bit.
// Two things live in modules that are absent from the reference tree and are therefore this file's own choice
// (parity unpinned): the byte layout of the spec record (a KeyValueRecord there; `key=value` lines here) and the digit
// order of the base-3 code (first trit = least significant digit here).
#include <string.h>

#include <fstream>
#include <sstream>
#include <string>
#include <vector>

#include "common.cuh"
#include "policy.cuh"

namespace nnb {

// ---------------------------------------------------------------- SHA-256 (FIPS 180-4)
struct Sha256 {
    uint32_t h[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au, 0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
    uint8_t buf[64];
    size_t fill = 0;
    uint64_t total = 0;
    static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
    void block(const uint8_t* p)
    {
        static const uint32_t K[64] = {
            0x428a2f98u, 0x71374491u, 0xb5c0fbcfu, 0xe9b5dba5u, 0x3956c25bu, 0x59f111f1u, 0x923f82a4u, 0xab1c5ed5u, 0xd807aa98u, 0x12835b01u,
            0x243185beu, 0x550c7dc3u, 0x72be5d74u, 0x80deb1feu, 0x9bdc06a7u, 0xc19bf174u, 0xe49b69c1u, 0xefbe4786u, 0x0fc19dc6u, 0x240ca1ccu,
            0x2de92c6fu, 0x4a7484aau, 0x5cb0a9dcu, 0x76f988dau, 0x983e5152u, 0xa831c66du, 0xb00327c8u, 0xbf597fc7u, 0xc6e00bf3u, 0xd5a79147u,
            0x06ca6351u, 0x14292967u, 0x27b70a85u, 0x2e1b2138u, 0x4d2c6dfcu, 0x53380d13u, 0x650a7354u, 0x766a0abbu, 0x81c2c92eu, 0x92722c85u,
            0xa2bfe8a1u, 0xa81a664bu, 0xc24b8b70u, 0xc76c51a3u, 0xd192e819u, 0xd6990624u, 0xf40e3585u, 0x106aa070u, 0x19a4c116u, 0x1e376c08u,
            0x2748774cu, 0x34b0bcb5u, 0x391c0cb3u, 0x4ed8aa4au, 0x5b9cca4fu, 0x682e6ff3u, 0x748f82eeu, 0x78a5636fu, 0x84c87814u, 0x8cc70208u,
            0x90befffau, 0xa4506cebu, 0xbef9a3f7u, 0xc67178f2u};
        uint32_t w[64];
        for (int i = 0; i < 16; ++i) w[i] = (uint32_t)p[4 * i] << 24 | (uint32_t)p[4 * i + 1] << 16 | (uint32_t)p[4 * i + 2] << 8 | p[4 * i + 3];
        for (int i = 16; i < 64; ++i) {
            const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
            const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
            w[i] = w[i - 16] + s0 + w[i - 7] + s1;
        }
        uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
        for (int i = 0; i < 64; ++i) {
            const uint32_t t1 = hh + (rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25)) + ((e & f) ^ (~e & g)) + K[i] + w[i];
            const uint32_t t2 = (rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22)) + ((a & b) ^ (a & c) ^ (b & c));
            hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
        }
        h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
    }
    void update(const void* data, size_t n)
    {
        const uint8_t* p = (const uint8_t*)data;
        total += n;
        while (n) {
            const size_t take = n < 64 - fill ? n : 64 - fill;
            memcpy(buf + fill, p, take);
            fill += take; p += take; n -= take;
            if (fill == 64) { block(buf); fill = 0; }
        }
    }
    void finish(uint8_t out[32])
    {
        const uint64_t bits = total * 8;
        uint8_t pad = 0x80;
        update(&pad, 1);
        pad = 0;
        while (fill != 56) update(&pad, 1);
        uint8_t len[8];
        for (int i = 0; i < 8; ++i) len[i] = (uint8_t)(bits >> (56 - 8 * i));
        update(len, 8);
        for (int i = 0; i < 8; ++i) for (int j = 0; j < 4; ++j) out[4 * i + j] = (uint8_t)(h[i] >> (24 - 8 * j));
    }
};

}  // namespace nnb

using namespace nnb;

extern "C" {

// ---------------------------------------------------------------- row codecs (host)
size_t nnb_trit_base3_bytes_per_row(size_t k) { return (k + 4) / 5; }

static inline int trit_at(const uint32_t* words, size_t i) { return (int)((words[i / 16] >> (2 * (i % 16))) & 3u) - 2; }

void nnb_trit_pack_row_base3(const uint32_t* words, size_t k, uint8_t* out)
{
    const size_t nb = nnb_trit_base3_bytes_per_row(k);
    for (size_t b = 0; b < nb; ++b) {
        unsigned v = 0, mul = 1;
        for (size_t j = 0; j < 5; ++j) {
            const size_t i = 5 * b + j;
            const unsigned digit = i < k ? (unsigned)(trit_at(words, i) + 1) : 1u;  // padding = trit 0
            v += digit * mul;
            mul *= 3;
        }
        out[b] = (uint8_t)v;  // <= 242
    }
}

void nnb_trit_unpack_row_base3(const uint8_t* in, size_t k, uint32_t* words)
{
    const size_t wpr = (k + 15) / 16;
    for (size_t w = 0; w < wpr; ++w) words[w] = 0xAAAAAAAAu;  // code 2 = trit 0 everywhere, the tail included
    for (size_t i = 0; i < k; ++i) {
        unsigned v = in[i / 5];
        for (size_t j = 0; j < i % 5; ++j) v /= 3;
        const unsigned code = v % 3 + 1;  // digit 0,1,2 -> trit -1,0,+1 -> code 1,2,3
        words[i / 16] = (words[i / 16] & ~(3u << (2 * (i % 16)))) | (code << (2 * (i % 16)));
    }
}

float nnb_trit_latent_row_scale(const uint32_t* words, size_t k, float tau)
{
    size_t n = 0;
    for (size_t i = 0; i < k; ++i) n += trit_at(words, i) != 0;
    return n == 0 ? 0.0f : tau * (float)k / (float)n;
}

void nnb_trit_dequant_row(const uint32_t* words, size_t k, float tau, float* latent)
{
    const float s = nnb_trit_latent_row_scale(words, k, tau);
    for (size_t i = 0; i < k; ++i) latent[i] = (float)trit_at(words, i) * s;
}

}  // extern "C"

namespace nnb {

struct Writer {
    std::ofstream f;
    Sha256 sha;
    bool ok = true;
    void put(const void* p, size_t n)
    {
        f.write((const char*)p, (std::streamsize)n);
        if (!f) ok = false;
        sha.update(p, n);
    }
    template <class T>
    void pod(T v) { put(&v, sizeof v); }
};

static void write_entry(Writer& w, uint8_t kind, uint64_t rows, uint64_t cols, const void* aux, size_t aux_len, const void* payload,
                        size_t payload_len)
{
    w.pod<uint8_t>(kind);
    w.pod<uint8_t>(0);  // precision tag: f32
    w.pod<uint64_t>(rows);
    w.pod<uint64_t>(cols);
    w.pod<uint64_t>(aux_len);
    w.pod<uint64_t>(payload_len);
    if (aux_len) w.put(aux, aux_len);
    if (payload_len) w.put(payload, payload_len);
}

static const LinW* find_linear(const nnb_policy* p, size_t w_off)
{
    for (const auto& L : p->layers)
        for (const LinW* l : {&L.q, &L.k, &L.v, &L.o, &L.fc1, &L.fc2})
            if (l->w_off == w_off) return l;
    return (p->head.out > 0 && p->head.w_off == w_off) ? &p->head : nullptr;
}

static std::string spec_text(const nnb_policy* p, int role)
{
    const nnb_gpt_config& c = p->cfg;
    std::ostringstream s;
    s << "model=gpt_t1_58\nn_layer=" << c.n_layer << "\nd_model=" << c.d_model << "\nn_head=" << c.n_head << "\nd_ff=" << c.d_ff
      << "\nvocab=" << c.vocab << "\nctx=" << c.ctx << "\nact=" << c.act << "\npos=" << c.pos << "\nvalue_head=" << c.value_head
      << "\nsub_ln=" << c.sub_ln << "\nn_head_kv=" << nnb::cfg_kv_heads(c) << "\ntie_embeddings=" << c.tie_embeddings << "\nrole=" << role << "\nentries=" << p->tensors.size() << "\n";
    return s.str();
}

}  // namespace nnb

extern "C" {

nnb_status nnb_policy_save(nnb_policy* p, const char* path, int role)
{
    NNB_REQUIRE(p && path, "policy_save: NULL argument");
    NNB_REQUIRE(role == 0 || role == 1, "policy_save: role must be 0 (model) or 1 (checkpoint)");
    nnb_engine* e = p->e;
    std::vector<float> flat(p->n_params), tau(p->tau_count);
    std::vector<uint32_t> packed(p->packed_words);
    NNB_CUDA(cudaMemcpyAsync(flat.data(), p->params, flat.size() * 4, cudaMemcpyDeviceToHost, e->stream));
    NNB_CUDA(cudaMemcpyAsync(tau.data(), p->tau, tau.size() * 4, cudaMemcpyDeviceToHost, e->stream));
    NNB_CUDA(cudaMemcpyAsync(packed.data(), p->packed, packed.size() * 4, cudaMemcpyDeviceToHost, e->stream));
    NNB_CUDA(cudaStreamSynchronize(e->stream));
    Writer w;
    w.f.open(path, std::ios::binary | std::ios::trunc);
    if (!w.f) NNB_FAIL(NNB_ERR_INVALID, "policy_save: cannot open '%s' for writing", path);
    w.pod<uint32_t>(0x4E4E4E4Eu);  // "NNNN"
    w.pod<uint32_t>(8u);
    w.pod<uint8_t>(0);             // Scalar = f32
    w.pod<uint8_t>((uint8_t)role);
    const std::string spec = spec_text(p, role);
    w.pod<uint64_t>(spec.size());
    w.put(spec.data(), spec.size());
    w.pod<uint64_t>(0);  // no training-state section
    std::vector<uint8_t> row3;
    for (const TensorInfo& t : p->tensors) {
        const LinW* l = t.name.size() > 7 && t.name.compare(t.name.size() - 7, 7, ".weight") == 0 ? find_linear(p, t.offset) : nullptr;
        if (!l) {
            write_entry(w, 0 /*Dense*/, t.rows, t.cols, nullptr, 0, flat.data() + t.offset, t.rows * t.cols * 4);
        } else if (role == 1) {
            write_entry(w, 1 /*TernaryLatent*/, l->out, l->in, nullptr, 0, flat.data() + l->w_off, l->out * l->in * 4);
        } else {
            const size_t per = nnb_trit_base3_bytes_per_row(l->in), wpr = l->in / 16;
            row3.resize(l->out * per);
            for (size_t r = 0; r < l->out; ++r) nnb_trit_pack_row_base3(packed.data() + l->packed_off + r * wpr, l->in, row3.data() + r * per);
            write_entry(w, 3 /*TernaryPacked3*/, l->out, l->in, tau.data() + l->tau_off, l->out * 4, row3.data(), row3.size());
        }
    }
    w.pod<uint64_t>(0);  // no embedded tokenizer
    uint8_t digest[32];
    Sha256 final_sha = w.sha;
    final_sha.finish(digest);
    w.f.write((const char*)digest, 32);
    w.f.write("NNEND", 5);
    w.f.close();
    if (!w.ok || !w.f) NNB_FAIL(NNB_ERR_INVALID, "policy_save: write error on '%s'", path);
    return NNB_OK;
}

nnb_status nnb_policy_load(nnb_policy* p, const char* path)
{
    NNB_REQUIRE(p && path, "policy_load: NULL argument");
    std::ifstream f(path, std::ios::binary);
    if (!f) NNB_FAIL(NNB_ERR_INVALID, "policy_load: cannot open '%s'", path);
    std::vector<uint8_t> bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    NNB_REQUIRE(bytes.size() >= 18 + 8 + 8 + 37, "policy_load: '%s' is too short to be a model file", path);
    // integrity first: the digest covers everything before it
    NNB_REQUIRE(memcmp(bytes.data() + bytes.size() - 5, "NNEND", 5) == 0, "policy_load: tail marker missing (truncated file?)");
    Sha256 sha;
    sha.update(bytes.data(), bytes.size() - 37);
    uint8_t digest[32];
    sha.finish(digest);
    NNB_REQUIRE(memcmp(digest, bytes.data() + bytes.size() - 37, 32) == 0, "policy_load: checksum mismatch (corrupt file)");
    size_t pos = 0;
    const size_t end = bytes.size() - 37;
    auto need = [&](size_t n) { return pos + n <= end; };
    auto rd = [&](void* dst, size_t n) { memcpy(dst, bytes.data() + pos, n); pos += n; };
    uint32_t magic = 0, version = 0;
    uint8_t prec = 0, role = 0;
    uint64_t spec_len = 0, state_len = 0;
    rd(&magic, 4); rd(&version, 4); rd(&prec, 1); rd(&role, 1); rd(&spec_len, 8);
    NNB_REQUIRE(magic == 0x4E4E4E4Eu, "policy_load: not a model file (bad magic)");
    NNB_REQUIRE(version == 8 && prec == 0 && role <= 1, "policy_load: unsupported version %u / precision %u / role %u", version, prec, role);
    NNB_REQUIRE(need(spec_len + 8), "policy_load: spec record runs past the end of the file");
    const std::string spec((const char*)bytes.data() + pos, (size_t)spec_len);
    pos += spec_len;
    NNB_REQUIRE(spec == spec_text(p, role), "policy_load: the file describes a different model:\n%s", spec.c_str());
    rd(&state_len, 8);
    NNB_REQUIRE(need(state_len), "policy_load: training-state section runs past the end of the file");
    pos += state_len;
    std::vector<float> flat(p->n_params), tau(p->tau_count);
    std::vector<uint32_t> packed(p->packed_words);
    bool seeded = role == 0;
    for (const TensorInfo& t : p->tensors) {
        NNB_REQUIRE(need(34), "policy_load: parameter entry header runs past the end of the file");
        uint8_t kind = 0, ptag = 0;
        uint64_t rows = 0, cols = 0, aux_len = 0, payload_len = 0;
        rd(&kind, 1); rd(&ptag, 1); rd(&rows, 8); rd(&cols, 8); rd(&aux_len, 8); rd(&payload_len, 8);
        NNB_REQUIRE(kind <= 4 && ptag == 0, "policy_load: entry '%s' has kind %u / precision %u", t.name.c_str(), kind, ptag);
        NNB_REQUIRE(aux_len <= end - pos && payload_len <= end - pos - aux_len, "policy_load: entry '%s' runs past the end of the file",
                    t.name.c_str());
        NNB_REQUIRE(rows == t.rows && cols == t.cols, "policy_load: entry '%s' is (%llu, %llu), the model wants (%zu, %zu)", t.name.c_str(),
                    (unsigned long long)rows, (unsigned long long)cols, t.rows, t.cols);
        const uint8_t* aux = bytes.data() + pos;
        const uint8_t* payload = aux + aux_len;
        pos += aux_len + payload_len;
        const LinW* l = t.name.size() > 7 && t.name.compare(t.name.size() - 7, 7, ".weight") == 0 ? find_linear(p, t.offset) : nullptr;
        if (kind == 0 || kind == 1) {
            NNB_REQUIRE(kind == 0 || l != nullptr, "policy_load: entry '%s' is a ternary latent but the parameter is not a ternary weight",
                        t.name.c_str());
            NNB_REQUIRE(payload_len == rows * cols * 4, "policy_load: entry '%s' has %llu payload bytes", t.name.c_str(),
                        (unsigned long long)payload_len);
            memcpy(flat.data() + t.offset, payload, payload_len);
            if (l) seeded = false;  // a latent without tau: the first forward quantises by itself
        } else if (kind == 2 || kind == 3) {
            NNB_REQUIRE(l != nullptr, "policy_load: entry '%s' is packed but the parameter is not a ternary weight", t.name.c_str());
            NNB_REQUIRE(aux_len == rows * 4, "policy_load: packed entry '%s' needs one tau per row", t.name.c_str());
            const size_t wpr = l->in / 16, per = kind == 3 ? nnb_trit_base3_bytes_per_row(l->in) : wpr * 4;
            NNB_REQUIRE(payload_len == rows * per, "policy_load: packed entry '%s' has %llu payload bytes", t.name.c_str(),
                        (unsigned long long)payload_len);
            memcpy(tau.data() + l->tau_off, aux, aux_len);
            for (size_t r = 0; r < l->out; ++r) {
                uint32_t* words = packed.data() + l->packed_off + r * wpr;
                if (kind == 3) nnb_trit_unpack_row_base3(payload + r * per, l->in, words);
                else memcpy(words, payload + r * per, per);
                nnb_trit_dequant_row(words, l->in, tau[l->tau_off + r], flat.data() + l->w_off + r * l->in);
            }
        } else {
            NNB_FAIL(NNB_ERR_UNSUPPORTED, "policy_load: entry '%s' is of the reserved int8 kind", t.name.c_str());
        }
    }
    nnb_engine* e = p->e;
    NNB_CUDA(cudaMemcpyAsync(p->params, flat.data(), flat.size() * 4, cudaMemcpyHostToDevice, e->stream));
    if (seeded) {
        NNB_CUDA(cudaMemcpyAsync(p->tau, tau.data(), tau.size() * 4, cudaMemcpyHostToDevice, e->stream));
        NNB_CUDA(cudaMemcpyAsync(p->packed, packed.data(), packed.size() * 4, cudaMemcpyHostToDevice, e->stream));
    }
    NNB_TRY(policy_requantize(p, seeded));
    NNB_CUDA(cudaStreamSynchronize(e->stream));
    return NNB_OK;
}

}  // extern "C"
