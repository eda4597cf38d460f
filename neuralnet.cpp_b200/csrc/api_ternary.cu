// api_ternary.cu — C-ABI entry points of the ternary linear operators.
#include "common.cuh"

using namespace nnb;

extern "C" {

nnb_status nnb_absmean_tau(nnb_engine* e, const float* d_latent, size_t rows, size_t k, float* d_tau)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_absmean_tau(e, d_latent, rows, k, d_tau);
}

nnb_status nnb_trit_pack(nnb_engine* e, const float* d_latent, const float* d_tau, size_t rows,
                         size_t k, uint32_t* d_packed)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_trit_pack(e, d_latent, d_tau, rows, k, d_packed);
}

nnb_status nnb_col_absmax_scale(nnb_engine* e, const float* d_x, size_t k, size_t n, float* d_s)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_col_absmax_scale(e, d_x, k, n, d_s);
}

nnb_status nnb_quantize_i8(nnb_engine* e, const float* d_x, size_t m, size_t n, const float* d_scale,
                           int col_scale, uint32_t* d_out)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_quantize_i8(e, d_x, m, n, d_scale, col_scale, d_out);
}

nnb_status nnb_unpack_i8(nnb_engine* e, const uint32_t* d_packed, size_t m, size_t n, float* d_out)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_unpack_i8(e, d_packed, m, n, d_out);
}

nnb_status nnb_matmul_q_i8(nnb_engine* e, const uint32_t* d_wq, const float* d_tau,
                           const uint32_t* d_xq, const float* d_s, size_t rows, size_t k, size_t n,
                           float* d_y, int32_t* d_acc)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_matmul_q_i8_ref(e, d_wq, d_tau, d_xq, d_s, rows, k, n, d_y, d_acc);
}

nnb_status nnb_matmul_q(nnb_engine* e, const uint32_t* d_wq, const float* d_tau, const float* d_x,
                        size_t rows, size_t k, size_t n, float* d_c)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_matmul_q_ref(e, d_wq, d_tau, d_x, rows, k, n, d_c);
}

nnb_status nnb_matmul_q_t(nnb_engine* e, const uint32_t* d_wq, const float* d_tau, const float* d_b,
                          size_t rows, size_t mcols, size_t n, float* d_c)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_matmul_q_t_ref(e, d_wq, d_tau, d_b, rows, mcols, n, d_c);
}

size_t nnb_actq_bytes(size_t t, size_t k) { return t * k; }

nnb_status nnb_act_quant_tm(nnb_engine* e, const void* d_x, nnb_dtype dtype, size_t t, size_t k,
                            int8_t* d_q, float* d_s, int32_t* d_qsum)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_act_quant_tm(e, d_x, dtype, t, k, d_q, d_s, d_qsum);
}

nnb_status nnb_actq_to_plain(nnb_engine* e, const int8_t* d_q, size_t t, size_t k, int8_t* d_plain)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_actq_to_plain(e, d_q, t, k, d_plain);
}

nnb_status nnb_bitlinear_fwd_tm(nnb_engine* e, const uint32_t* d_wq, const float* d_tau,
                                const float* d_bias, const int8_t* d_q, const float* d_s,
                                const int32_t* d_qsum, size_t t, size_t k, size_t out, void* d_y,
                                nnb_dtype dtype, int32_t* d_acc)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_bitlinear_fwd_tm(e, d_wq, 0, d_tau, d_bias, nullptr, d_q, d_s, d_qsum, 1, t, k, out,
                                   d_y, 0, dtype, d_acc);
}

nnb_status nnb_bitlinear_fwd_tm_stack(nnb_engine* e, const uint32_t* d_wq, size_t wq_stride_words,
                                      const float* d_tau, const float* d_bias, const int8_t* d_q,
                                      const float* d_s, const int32_t* d_qsum, size_t n_mats,
                                      size_t t, size_t k, size_t out, void* d_y,
                                      size_t y_stride_elems, nnb_dtype dtype)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_bitlinear_fwd_tm(e, d_wq, wq_stride_words, d_tau, d_bias, nullptr, d_q, d_s, d_qsum,
                                   n_mats, t, k, out, d_y, y_stride_elems, dtype, nullptr);
}

nnb_status nnb_bitlinear_dx_tm(nnb_engine* e, const float* d_dy, const uint32_t* d_wq, const float* d_tau, size_t t,
                               size_t k, size_t out, float* d_dx, int accumulate, int exact)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_bitlinear_dx(e, exact != 0, d_dy, d_wq, d_tau, t, k, out, d_dx, accumulate != 0);
}

nnb_status nnb_bitlinear_dw_tm(nnb_engine* e, const float* d_dy, const int8_t* d_q, const float* d_s,
                               const float* d_tau, size_t t, size_t k, size_t out, float* d_dw, int exact)
{
    NNB_REQUIRE(e, "engine is NULL");
    return launch_bitlinear_dw(e, exact != 0, d_dy, d_q, d_s, d_tau, t, k, out, d_dw);
}

nnb_status nnb_expand_weights(nnb_engine* e, const uint32_t* d_wq, size_t rows, size_t k, int8_t* d_w8, void* d_wb)
{
    NNB_REQUIRE(e && d_wq && (d_w8 || d_wb), "expand_weights: NULL argument");
    NNB_REQUIRE(k > 0 && k % 64 == 0, "expand_weights: k=%zu must be a multiple of 64", k);
    return launch_expand_weights(e, d_wq, rows, k, d_w8, (__nv_bfloat16*)d_wb);
}

nnb_status nnb_bitlinear_fwd_tc(nnb_engine* e, const int8_t* d_w8, const float* d_tau, const float* d_bias,
                                const float* d_residual, const int8_t* d_q, const float* d_s, size_t t, size_t k,
                                size_t out, float* d_y)
{
    NNB_REQUIRE(e && d_w8 && d_tau && d_q && d_s && d_y, "bitlinear_fwd_tc: NULL argument");
    NNB_REQUIRE(k > 0 && k % 64 == 0, "bitlinear_fwd_tc: k=%zu must be a multiple of 64", k);
    return launch_tc_forward(e, d_q, d_w8, d_tau, d_s, d_bias, d_residual, t, k, out, d_y);
}

nnb_status nnb_tc_set_forward_tile(int bn) { return tc_set_forward_tile(bn); }

nnb_status nnb_lmhead_logprob_entropy_fwd(nnb_engine* e, const int8_t* d_w8, const float* d_tau, const float* d_bias, const int8_t* d_q,
                                          const float* d_s, const int32_t* d_actions, size_t t, size_t k, size_t v, float* d_logp,
                                          float* d_entropy, float* d_lse)
{
    NNB_REQUIRE(e && d_w8 && d_tau && d_q && d_s && d_actions && d_logp && d_lse, "lmhead_logprob_entropy_fwd: NULL argument");
    NNB_REQUIRE(t > 0 && v > 0 && k > 0 && k % 64 == 0, "lmhead_logprob_entropy_fwd: k=%zu must be a multiple of 64", k);
    NNB_TRY(e->ensure_scratch(tc_lmhead_scratch_floats(t, v) * sizeof(float)));
    return launch_tc_lmhead_fwd(e, d_q, d_w8, d_tau, d_s, d_bias, d_actions, t, k, v, (float*)e->scratch, d_lse, d_logp, d_entropy);
}

nnb_status nnb_lmhead_logprob_entropy_bwd(nnb_engine* e, const int8_t* d_w8, const float* d_tau, const float* d_bias, const int8_t* d_q,
                                          const float* d_s, const int32_t* d_actions, const float* d_lse, const float* d_entropy,
                                          const float* d_up_logp, const float* d_up_entropy, size_t t, size_t k, size_t v, void* d_dyb,
                                          float* d_dbias)
{
    NNB_REQUIRE(e && d_w8 && d_tau && d_q && d_s && d_actions && d_lse && d_up_logp && d_dyb && d_dbias,
                "lmhead_logprob_entropy_bwd: NULL argument");
    NNB_REQUIRE(d_up_entropy == nullptr || d_entropy, "lmhead_logprob_entropy_bwd: the entropy gradient needs the forward's entropy");
    NNB_REQUIRE(t > 0 && v > 0 && v % 4 == 0 && k > 0 && k % 64 == 0, "lmhead_logprob_entropy_bwd: needs k %% 64 == 0 and v %% 4 == 0");
    NNB_TRY(e->ensure_scratch(tc_lmhead_scratch_floats(t, v) * sizeof(float)));
    return launch_tc_lmhead_bwd(e, d_q, d_w8, d_tau, d_s, d_bias, d_actions, d_lse, d_entropy, d_up_logp, d_up_entropy, t, k, v,
                                (float*)e->scratch, (__nv_bfloat16*)d_dyb, d_dbias);
}

nnb_status nnb_bitlinear_bwd_tc(nnb_engine* e, const float* d_dy, const float* d_tau, const void* d_wb,
                                const int8_t* d_q, const float* d_s, size_t t, size_t k, size_t out, void* d_dyb,
                                void* d_xs, float* d_dx, int accumulate_dx, float* d_dw)
{
    NNB_REQUIRE(e && d_dyb && (d_dy == nullptr || d_tau), "bitlinear_bwd_tc: NULL argument");
    NNB_REQUIRE(k % 64 == 0 && out % 8 == 0, "bitlinear_bwd_tc: needs k %% 64 == 0 and out %% 8 == 0 (k=%zu, out=%zu)", k, out);
    // d_dy == NULL: d_dyb (and d_xs) already hold the operands an earlier call prepared; only the GEMMs run
    const bool prepared = d_dy == nullptr;
    if (!prepared) NNB_TRY(launch_scale_to_bf16(e, d_dy, d_tau, t, out, (__nv_bfloat16*)d_dyb));
    if (d_dx) {
        NNB_REQUIRE(d_wb, "bitlinear_bwd_tc: dX needs the bf16 weights");
        NNB_TRY(launch_tc_dx(e, (const __nv_bfloat16*)d_dyb, (const __nv_bfloat16*)d_wb, t, k, out, d_dx, accumulate_dx != 0));
    }
    if (d_dw) {
        NNB_REQUIRE(d_xs && (prepared || (d_q && d_s)), "bitlinear_bwd_tc: dW needs the activation cache and scratch");
        if (!prepared) NNB_TRY(launch_dequant_to_bf16(e, d_q, d_s, t, k, (__nv_bfloat16*)d_xs));
        NNB_TRY(launch_tc_dw(e, (const __nv_bfloat16*)d_dyb, (const __nv_bfloat16*)d_xs, t, k, out, d_dw));
    }
    return NNB_OK;
}

nnb_status nnb_attention_fwd(nnb_engine* e, const float* d_q, const float* d_k, const float* d_v, size_t n_seq,
                             size_t seq_len, size_t n_head, size_t dk, int exact, float* d_out, float* d_lse)
{
    NNB_REQUIRE(e && d_q && d_k && d_v && d_out && d_lse, "attention_fwd: NULL argument");
    NNB_REQUIRE(n_seq > 0 && seq_len > 0 && n_head > 0 && dk > 0 && dk % 4 == 0, "attention_fwd: bad shape");
    return launch_attn_fwd(e, exact != 0, d_q, d_k, d_v, n_seq, seq_len, n_head, dk, d_out, d_lse);
}

nnb_status nnb_attention_bwd(nnb_engine* e, const float* d_q, const float* d_k, const float* d_v, const float* d_out,
                             const float* d_dout, const float* d_lse, size_t n_seq, size_t seq_len, size_t n_head,
                             size_t dk, int exact, float* d_delta, float* d_dq, float* d_dk, float* d_dv)
{
    NNB_REQUIRE(e && d_q && d_k && d_v && d_out && d_dout && d_lse && d_delta && d_dq && d_dk && d_dv,
                "attention_bwd: NULL argument");
    NNB_REQUIRE(n_seq > 0 && seq_len > 0 && n_head > 0 && dk > 0 && dk % 4 == 0, "attention_bwd: bad shape");
    return launch_attn_bwd(e, exact != 0, d_q, d_k, d_v, d_out, d_dout, d_lse, d_delta, n_seq, seq_len, n_head, dk, d_dq,
                           d_dk, d_dv);
}

// Attention with the rotary embedding inside the operator: q and k come un-rotated, the gradients are with
// respect to the un-rotated q and k.  The exact mode composes the rotation kernel with the attention
// kernels on scratch copies; the fast mode uses the fused bf16 path.
nnb_status nnb_attention_rope_fwd(nnb_engine* e, const float* d_q, const float* d_k, const float* d_v,
                                  const float* d_rope_cos, const float* d_rope_sin, size_t n_seq, size_t seq_len,
                                  size_t n_head, size_t dk, int exact, float* d_out, float* d_lse)
{
    NNB_REQUIRE(e && d_q && d_k && d_v && d_rope_cos && d_rope_sin && d_out && d_lse, "attention_rope_fwd: NULL argument");
    NNB_REQUIRE(n_seq > 0 && seq_len > 0 && n_head > 0 && dk > 0 && dk % 4 == 0, "attention_rope_fwd: bad shape");
    const size_t T = n_seq * seq_len, td = T * n_head * dk;
    if (!exact && attn_b16_supported(dk, n_head * dk)) {
        __nv_bfloat16* tmp = nullptr;
        NNB_CUDA(cudaMallocAsync((void**)&tmp, 3 * td * sizeof(__nv_bfloat16), e->stream));
        nnb_status st = launch_rope_pack_b16(e, d_q, d_k, d_v, d_rope_cos, d_rope_sin, T, seq_len, n_head, dk, tmp);
        if (st == NNB_OK) st = launch_attn_fwd_b16(e, tmp, tmp + td, tmp + 2 * td, n_seq, seq_len, n_head, dk, d_out, d_lse);
        cudaFreeAsync(tmp, e->stream);
        return st;
    }
    float* tmp = nullptr;
    NNB_CUDA(cudaMallocAsync((void**)&tmp, 2 * td * sizeof(float), e->stream));
    nnb_status st = NNB_OK;
    if (cudaMemcpyAsync(tmp, d_q, td * 4, cudaMemcpyDeviceToDevice, e->stream) != cudaSuccess ||
        cudaMemcpyAsync(tmp + td, d_k, td * 4, cudaMemcpyDeviceToDevice, e->stream) != cudaSuccess)
        st = NNB_ERR_CUDA;
    if (st == NNB_OK) st = launch_rope(e, tmp, d_rope_cos, d_rope_sin, T, seq_len, n_head, dk, false);
    if (st == NNB_OK) st = launch_rope(e, tmp + td, d_rope_cos, d_rope_sin, T, seq_len, n_head, dk, false);
    if (st == NNB_OK) st = launch_attn_fwd(e, exact != 0, tmp, tmp + td, d_v, n_seq, seq_len, n_head, dk, d_out, d_lse);
    cudaFreeAsync(tmp, e->stream);
    return st;
}

nnb_status nnb_attention_rope_bwd(nnb_engine* e, const float* d_q, const float* d_k, const float* d_v,
                                  const float* d_rope_cos, const float* d_rope_sin, const float* d_out, const float* d_dout,
                                  const float* d_lse, size_t n_seq, size_t seq_len, size_t n_head, size_t dk, int exact,
                                  float* d_delta, float* d_dq, float* d_dk, float* d_dv)
{
    NNB_REQUIRE(e && d_q && d_k && d_v && d_rope_cos && d_rope_sin && d_out && d_dout && d_lse && d_delta && d_dq && d_dk && d_dv,
                "attention_rope_bwd: NULL argument");
    NNB_REQUIRE(n_seq > 0 && seq_len > 0 && n_head > 0 && dk > 0 && dk % 4 == 0, "attention_rope_bwd: bad shape");
    const size_t T = n_seq * seq_len, td = T * n_head * dk;
    if (!exact && attn_b16_supported(dk, n_head * dk)) {
        __nv_bfloat16* tmp = nullptr;
        NNB_CUDA(cudaMallocAsync((void**)&tmp, 4 * td * sizeof(__nv_bfloat16), e->stream));
        nnb_status st = launch_rope_pack_b16(e, d_q, d_k, d_v, d_rope_cos, d_rope_sin, T, seq_len, n_head, dk, tmp);
        if (st == NNB_OK)
            st = launch_attn_bwd_b16(e, tmp, tmp + td, tmp + 2 * td, d_out, d_dout, d_lse, d_delta, tmp + 3 * td, d_rope_cos,
                                     d_rope_sin, n_seq, seq_len, n_head, dk, d_dq, d_dk, d_dv);
        cudaFreeAsync(tmp, e->stream);
        return st;
    }
    float* tmp = nullptr;
    NNB_CUDA(cudaMallocAsync((void**)&tmp, 2 * td * sizeof(float), e->stream));
    nnb_status st = NNB_OK;
    if (cudaMemcpyAsync(tmp, d_q, td * 4, cudaMemcpyDeviceToDevice, e->stream) != cudaSuccess ||
        cudaMemcpyAsync(tmp + td, d_k, td * 4, cudaMemcpyDeviceToDevice, e->stream) != cudaSuccess)
        st = NNB_ERR_CUDA;
    if (st == NNB_OK) st = launch_rope(e, tmp, d_rope_cos, d_rope_sin, T, seq_len, n_head, dk, false);
    if (st == NNB_OK) st = launch_rope(e, tmp + td, d_rope_cos, d_rope_sin, T, seq_len, n_head, dk, false);
    if (st == NNB_OK)
        st = launch_attn_bwd(e, exact != 0, tmp, tmp + td, d_v, d_out, d_dout, d_lse, d_delta, n_seq, seq_len, n_head, dk, d_dq,
                             d_dk, d_dv);
    if (st == NNB_OK) st = launch_rope(e, d_dq, d_rope_cos, d_rope_sin, T, seq_len, n_head, dk, true);
    if (st == NNB_OK) st = launch_rope(e, d_dk, d_rope_cos, d_rope_sin, T, seq_len, n_head, dk, true);
    cudaFreeAsync(tmp, e->stream);
    return st;
}

nnb_status nnb_attention_decode(nnb_engine* e, const float* d_qkv, void* d_kcache, void* d_vcache, size_t ctx_alloc,
                                const void* d_kpre, const void* d_vpre, size_t pre_len, size_t pre_alloc, size_t group,
                                const float* d_rope_cos, const float* d_rope_sin, const int* d_pos, size_t n_seq,
                                size_t n_head, size_t dk, int exact, float* d_out, int8_t* d_q8, float* d_s, int32_t* d_qsum)
{
    NNB_REQUIRE(e && d_qkv && d_kcache && d_vcache && d_pos, "attention_decode: NULL argument");
    NNB_REQUIRE(n_seq > 0 && n_head > 0 && dk > 0 && ctx_alloc > 0, "attention_decode: bad shape");
    NNB_REQUIRE((d_rope_cos == nullptr) == (d_rope_sin == nullptr), "attention_decode: rope tables go together");
    if (d_q8) {
        NNB_REQUIRE(!exact && d_s && d_qsum && attn_decode_fused_supported(n_head, dk) && (n_head * dk) % 64 == 0,
                    "attention_decode: the fused int8 output needs the fast mode, head dim 64 or 128, at most 32 heads");
        // the batched treatment of a shared prefix needs scratch for its partial softmax: stream-ordered here
        float* tmp = nullptr;
        const bool pre = pre_len > 0 && group > 1 && group <= 16;
        const size_t n_o = n_seq * n_head * dk, n_ml = n_seq * n_head * 2;
        if (pre) NNB_CUDA(cudaMallocAsync((void**)&tmp, (n_o + n_ml) * sizeof(float), e->stream));
        const nnb_status st = launch_attn_decode_fused(e, d_qkv, d_kcache, d_vcache, ctx_alloc, d_kpre, d_vpre, pre_len, pre_alloc,
                                                       group, d_rope_cos, d_rope_sin, d_pos, n_seq, n_head, dk, d_out, d_q8, d_s,
                                                       d_qsum, tmp, tmp ? tmp + n_o : nullptr);
        if (tmp) cudaFreeAsync(tmp, e->stream);
        return st;
    }
    NNB_REQUIRE(d_out, "attention_decode: no output requested");
    return launch_attn_decode(e, exact != 0, d_qkv, d_kcache, d_vcache, ctx_alloc, d_kpre, d_vpre, pre_len, pre_alloc, group,
                              d_rope_cos, d_rope_sin, d_pos, n_seq, n_head, dk, d_out);
}

nnb_status nnb_engine_check(nnb_engine* e)
{
    NNB_REQUIRE(e, "engine is NULL");
    return tc_check_errors(e);
}

nnb_status nnb_bitlinear_fwd_host(nnb_engine* e, const uint32_t* d_wq, const float* d_tau,
                                  const float* d_bias, const float* h_x, size_t t, size_t k,
                                  size_t out, float* h_y)
{
    NNB_REQUIRE(e && h_x && h_y, "bitlinear_fwd_host: NULL argument");
    NNB_REQUIRE(t > 0 && k > 0 && k % 64 == 0 && out > 0, "bitlinear_fwd_host: bad shape");
    auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
    const size_t x_b = al(t * k * 4), q_b = al(t * k), s_b = al(t * 4), y_b = al(t * out * 4);
    NNB_TRY(e->ensure_scratch(x_b + q_b + 2 * s_b + y_b));
    unsigned char* base = (unsigned char*)e->scratch;
    float* d_x = (float*)base;
    int8_t* d_q = (int8_t*)(base + x_b);
    float* d_s = (float*)(base + x_b + q_b);
    int32_t* d_qsum = (int32_t*)(base + x_b + q_b + s_b);
    float* d_y = (float*)(base + x_b + q_b + 2 * s_b);
    NNB_CUDA(cudaMemcpyAsync(d_x, h_x, t * k * 4, cudaMemcpyHostToDevice, e->stream));
    NNB_TRY(launch_act_quant_tm(e, d_x, NNB_F32, t, k, d_q, d_s, d_qsum));
    NNB_TRY(launch_bitlinear_fwd_tm(e, d_wq, 0, d_tau, d_bias, nullptr, d_q, d_s, d_qsum, 1, t, k, out,
                                    d_y, 0, NNB_F32, nullptr));
    NNB_CUDA(cudaMemcpyAsync(h_y, d_y, t * out * 4, cudaMemcpyDeviceToHost, e->stream));
    NNB_CUDA(cudaStreamSynchronize(e->stream));
    return NNB_OK;
}

}  // extern "C"
