// tensor.cu — tensor handles and the engine primitives the reference's layers call directly, in the
// reference's own layout (row-major (rows, cols) f32; activations (features, tokens)).
//
// The reference's Tensor is a value type over refcounted storage that carries a write epoch, bumped by
// every engine entry that writes it (AGENTS.md:158-164); BitLinear re-quantises its weights only when the
// latent's epoch moved (include/neuralnet.cpp/compute_layer_bitlinear.hpp:607-615).  nnb_tensor is that
// storage behind a C handle.  The primitives are the data-movement and reduction verbs of
// docs/usage/03-compute-engine-usage.md:1080-1187 (clone, transpose, slice_rows, insert_rows, gather_rows,
// scatter_add_rows, rearrange_3d, scale_inplace, accumulate, col_reduce_max, row_reduce_sum) and the ternary
// primitives of BitLinear on tensors, plus the three expression-DSL compositions BitLinear evaluates
// (abs, + row_broadcast(b), grad_w + ((dY o s) Q^T) o tau), each as one kernel.  These are plain CUDA-core
// kernels for any shape: they exist so that the reference's layer code runs on this engine unchanged;
// the fast path of the RL step is the token-major / policy level of the library.
#include <math.h>

#include "common.cuh"

struct nnb_tensor {
    nnb_engine* e = nullptr;
    size_t rows = 0, cols = 0;
    float* data = nullptr;
    unsigned long long epoch = 0;
};

namespace nnb {

static nnb_status tensor_new(nnb_engine* e, size_t rows, size_t cols, bool zero, nnb_tensor** out)
{
    NNB_REQUIRE(e && out, "tensor_create: NULL argument");
    *out = nullptr;
    NNB_REQUIRE(rows > 0 && cols > 0, "tensor_create: empty shape (%zu, %zu)", rows, cols);
    nnb_tensor* t = new nnb_tensor();
    t->e = e;
    t->rows = rows;
    t->cols = cols;
    cudaError_t er = cudaMalloc((void**)&t->data, rows * cols * sizeof(float));
    if (er != cudaSuccess) {
        cudaGetLastError();
        delete t;
        NNB_FAIL(NNB_ERR_OOM, "tensor_create: cudaMalloc of (%zu, %zu) failed: %s", rows, cols, cudaGetErrorString(er));
    }
    if (zero) cudaMemsetAsync(t->data, 0, rows * cols * sizeof(float), e->stream);
    *out = t;
    return NNB_OK;
}

static inline void wrote(nnb_tensor* t) { t->epoch += 1; }

static inline unsigned grid1(size_t n) { return (unsigned)ceil_div(n, 256); }

__global__ void t_transpose_kernel(const float* __restrict__ in, size_t rows, size_t cols, float* __restrict__ out)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * cols) return;
    const size_t r = i / cols, c = i % cols;
    out[c * rows + r] = in[i];
}

__global__ void t_gather_rows_kernel(const float* __restrict__ table, size_t vocab, size_t d, const float* __restrict__ idx,
                                     size_t num, float* __restrict__ out)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num * d) return;
    const size_t r = i / d, c = i % d;
    const float fi = idx[r];
    const long long id = (long long)fi;
    out[i] = (fi >= 0.0f && (size_t)id < vocab) ? table[(size_t)id * d + c] : 0.0f;  // out-of-range index: zero row
}

__global__ void t_scatter_add_rows_kernel(float* __restrict__ dst, size_t vocab, size_t d, const float* __restrict__ idx,
                                          size_t num, const float* __restrict__ grad)
{
    // one thread per (destination column, table row): the rows that hit it are added in index order, so the
    // result does not depend on thread scheduling
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= vocab * d) return;
    const size_t v = i / d, c = i % d;
    float acc = 0.0f;
    bool any = false;
    for (size_t r = 0; r < num; ++r) {
        const float fi = idx[r];
        if (fi >= 0.0f && (size_t)(long long)fi == v) {
            acc += grad[r * d + c];
            any = true;
        }
    }
    if (any) dst[i] += acc;
}

// inverse = 0: in (M, B*N) -> out (B*M, N), out[b*M + m, n] = in[m, b*N + n]; inverse = 1 the other way
__global__ void t_rearrange_kernel(const float* __restrict__ in, size_t M, size_t B, size_t N, int inverse, float* __restrict__ out)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= M * B * N) return;
    const size_t m = i / (B * N), rem = i % (B * N), b = rem / N, n = rem % N;  // i indexes the (M, B*N) side
    const size_t j = (b * M + m) * N + n;                                       // the (B*M, N) side
    if (inverse) out[i] = in[j];
    else out[j] = in[i];
}

__global__ void t_axpy_kernel(float* __restrict__ dst, const float* __restrict__ src, size_t n, float a, float b)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = __fadd_rn(__fmul_rn(a, dst[i]), __fmul_rn(b, src ? src[i] : 0.0f));
}

__global__ void t_abs_kernel(const float* __restrict__ in, size_t n, float* __restrict__ out)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = fabsf(in[i]);
}

__global__ void t_col_max_kernel(const float* __restrict__ in, size_t rows, size_t cols, float* __restrict__ out)
{
    const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float m = in[c];
    for (size_t r = 1; r < rows; ++r) m = fmaxf(m, in[r * cols + c]);
    out[c] = m;
}

__global__ void t_row_sum_kernel(const float* __restrict__ in, size_t rows, size_t cols, float* __restrict__ out)
{
    const size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    double s = 0.0;
    for (size_t c = 0; c < cols; ++c) s += (double)in[r * cols + c];
    out[r] = (float)s;
}

__global__ void t_add_row_broadcast_kernel(float* __restrict__ y, const float* __restrict__ b, size_t rows, size_t cols)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows * cols) y[i] = __fadd_rn(y[i], b[i / cols]);
}

// grad_w (out, in) += ((dy (out, N) o s (N)) . x (in, N)^T) o tau (out); s may be NULL (no activation quantisation)
__global__ void t_dw_accumulate_kernel(float* __restrict__ gw, const float* __restrict__ dy, const float* __restrict__ s,
                                       const float* __restrict__ x, const float* __restrict__ tau, size_t out, size_t in, size_t n)
{
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= out * in) return;
    const size_t o = i / in, k = i % in;
    double acc = 0.0;
    for (size_t t = 0; t < n; ++t) {
        const float d = s ? __fmul_rn(dy[o * n + t], s[t]) : dy[o * n + t];
        acc += (double)d * (double)x[k * n + t];
    }
    gw[i] = __fadd_rn(gw[i], __fmul_rn((float)acc, tau[o]));
}

}  // namespace nnb

using namespace nnb;

#define T_REQ_SAME_ENGINE(a, b) NNB_REQUIRE((a)->e == (b)->e, "operands belong to different engines")

extern "C" {

nnb_status nnb_tensor_create(nnb_engine* e, size_t rows, size_t cols, nnb_tensor** out) { return tensor_new(e, rows, cols, true, out); }

void nnb_tensor_destroy(nnb_tensor* t)
{
    if (!t) return;
    cudaStreamSynchronize(t->e->stream);
    if (t->data) cudaFree(t->data);
    delete t;
}

size_t nnb_tensor_rows(const nnb_tensor* t) { return t ? t->rows : 0; }
size_t nnb_tensor_cols(const nnb_tensor* t) { return t ? t->cols : 0; }
float* nnb_tensor_data(nnb_tensor* t) { return t ? t->data : nullptr; }
unsigned long long nnb_tensor_write_epoch(const nnb_tensor* t) { return t ? t->epoch : 0ull; }

nnb_status nnb_tensor_mark_written(nnb_tensor* t)
{
    NNB_REQUIRE(t, "tensor is NULL");
    wrote(t);
    return NNB_OK;
}

nnb_status nnb_tensor_upload(nnb_tensor* t, const float* h_src, size_t count)
{
    NNB_REQUIRE(t && h_src, "tensor_upload: NULL argument");
    NNB_REQUIRE(count == t->rows * t->cols, "tensor_upload: %zu values for a (%zu, %zu) tensor", count, t->rows, t->cols);
    NNB_CUDA(cudaMemcpyAsync(t->data, h_src, count * sizeof(float), cudaMemcpyHostToDevice, t->e->stream));
    NNB_CUDA(cudaStreamSynchronize(t->e->stream));
    wrote(t);
    return NNB_OK;
}

nnb_status nnb_tensor_download(const nnb_tensor* t, float* h_dst, size_t count)
{
    NNB_REQUIRE(t && h_dst, "tensor_download: NULL argument");
    NNB_REQUIRE(count == t->rows * t->cols, "tensor_download: %zu values for a (%zu, %zu) tensor", count, t->rows, t->cols);
    NNB_CUDA(cudaMemcpyAsync(h_dst, t->data, count * sizeof(float), cudaMemcpyDeviceToHost, t->e->stream));
    NNB_CUDA(cudaStreamSynchronize(t->e->stream));
    return NNB_OK;
}

nnb_status nnb_t_zero(nnb_tensor* t)
{
    NNB_REQUIRE(t, "zero: tensor is NULL");
    NNB_CUDA(cudaMemsetAsync(t->data, 0, t->rows * t->cols * sizeof(float), t->e->stream));
    wrote(t);
    return NNB_OK;
}

nnb_status nnb_t_clone(const nnb_tensor* src, nnb_tensor** out)
{
    NNB_REQUIRE(src && out, "clone: NULL argument");
    NNB_TRY(tensor_new(src->e, src->rows, src->cols, false, out));
    NNB_CUDA(cudaMemcpyAsync((*out)->data, src->data, src->rows * src->cols * sizeof(float), cudaMemcpyDeviceToDevice, src->e->stream));
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_copy_into(nnb_tensor* dst, const nnb_tensor* src)
{
    NNB_REQUIRE(dst && src, "copy_into: NULL argument");
    T_REQ_SAME_ENGINE(dst, src);
    NNB_REQUIRE(dst->rows == src->rows && dst->cols == src->cols, "copy_into: shape mismatch");
    NNB_CUDA(cudaMemcpyAsync(dst->data, src->data, src->rows * src->cols * sizeof(float), cudaMemcpyDeviceToDevice, src->e->stream));
    wrote(dst);
    return NNB_OK;
}

nnb_status nnb_t_transpose(const nnb_tensor* src, nnb_tensor** out)
{
    NNB_REQUIRE(src && out, "transpose: NULL argument");
    NNB_TRY(tensor_new(src->e, src->cols, src->rows, false, out));
    const size_t n = src->rows * src->cols;
    t_transpose_kernel<<<grid1(n), 256, 0, src->e->stream>>>(src->data, src->rows, src->cols, (*out)->data);
    src->e->launches++;
    NNB_CHECK_LAUNCH("t_transpose_kernel");
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_slice_rows(const nnb_tensor* src, size_t start_row, size_t count, nnb_tensor** out)
{
    NNB_REQUIRE(src && out, "slice_rows: NULL argument");
    NNB_REQUIRE(count > 0 && start_row + count <= src->rows, "slice_rows: rows [%zu, %zu) outside a tensor of %zu rows", start_row,
                start_row + count, src->rows);
    NNB_TRY(tensor_new(src->e, count, src->cols, false, out));
    NNB_CUDA(cudaMemcpyAsync((*out)->data, src->data + start_row * src->cols, count * src->cols * sizeof(float),
                             cudaMemcpyDeviceToDevice, src->e->stream));
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_insert_rows(nnb_tensor* dst, size_t dst_start_row, const nnb_tensor* src)
{
    NNB_REQUIRE(dst && src, "insert_rows: NULL argument");
    T_REQ_SAME_ENGINE(dst, src);
    NNB_REQUIRE(dst->cols == src->cols && dst_start_row + src->rows <= dst->rows, "insert_rows: (%zu, %zu) does not fit at row %zu of (%zu, %zu)",
                src->rows, src->cols, dst_start_row, dst->rows, dst->cols);
    NNB_CUDA(cudaMemcpyAsync(dst->data + dst_start_row * dst->cols, src->data, src->rows * src->cols * sizeof(float),
                             cudaMemcpyDeviceToDevice, src->e->stream));
    wrote(dst);
    return NNB_OK;
}

nnb_status nnb_t_gather_rows(const nnb_tensor* table, const nnb_tensor* indices, nnb_tensor** out)
{
    NNB_REQUIRE(table && indices && out, "gather_rows: NULL argument");
    T_REQ_SAME_ENGINE(table, indices);
    const size_t num = indices->rows * indices->cols;
    NNB_TRY(tensor_new(table->e, num, table->cols, false, out));
    t_gather_rows_kernel<<<grid1(num * table->cols), 256, 0, table->e->stream>>>(table->data, table->rows, table->cols, indices->data, num,
                                                                                 (*out)->data);
    table->e->launches++;
    NNB_CHECK_LAUNCH("t_gather_rows_kernel");
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_scatter_add_rows(nnb_tensor* dst, const nnb_tensor* indices, const nnb_tensor* grad)
{
    NNB_REQUIRE(dst && indices && grad, "scatter_add_rows: NULL argument");
    T_REQ_SAME_ENGINE(dst, indices);
    T_REQ_SAME_ENGINE(dst, grad);
    const size_t num = indices->rows * indices->cols;
    NNB_REQUIRE(grad->rows == num && grad->cols == dst->cols, "scatter_add_rows: gradient (%zu, %zu) does not match %zu indices of width %zu",
                grad->rows, grad->cols, num, dst->cols);
    t_scatter_add_rows_kernel<<<grid1(dst->rows * dst->cols), 256, 0, dst->e->stream>>>(dst->data, dst->rows, dst->cols, indices->data, num,
                                                                                        grad->data);
    dst->e->launches++;
    NNB_CHECK_LAUNCH("t_scatter_add_rows_kernel");
    wrote(dst);
    return NNB_OK;
}

nnb_status nnb_t_rearrange_3d(const nnb_tensor* x, size_t M, size_t B, size_t N, int inverse, nnb_tensor** out)
{
    NNB_REQUIRE(x && out, "rearrange_3d: NULL argument");
    NNB_REQUIRE(M > 0 && B > 0 && N > 0, "rearrange_3d: empty dimension");
    if (!inverse) NNB_REQUIRE(x->rows == M && x->cols == B * N, "rearrange_3d: input must be (M, B*N) = (%zu, %zu)", M, B * N);
    else NNB_REQUIRE(x->rows == B * M && x->cols == N, "rearrange_3d: input must be (B*M, N) = (%zu, %zu)", B * M, N);
    NNB_TRY(tensor_new(x->e, inverse ? M : B * M, inverse ? B * N : N, false, out));
    t_rearrange_kernel<<<grid1(M * B * N), 256, 0, x->e->stream>>>(x->data, M, B, N, inverse, (*out)->data);
    x->e->launches++;
    NNB_CHECK_LAUNCH("t_rearrange_kernel");
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_scale_inplace(nnb_tensor* t, float s)
{
    NNB_REQUIRE(t, "scale_inplace: tensor is NULL");
    const size_t n = t->rows * t->cols;
    t_axpy_kernel<<<grid1(n), 256, 0, t->e->stream>>>(t->data, nullptr, n, s, 0.0f);
    t->e->launches++;
    NNB_CHECK_LAUNCH("t_axpy_kernel");
    wrote(t);
    return NNB_OK;
}

nnb_status nnb_t_accumulate(nnb_tensor* dst, const nnb_tensor* src)
{
    NNB_REQUIRE(dst && src, "accumulate: NULL argument");
    T_REQ_SAME_ENGINE(dst, src);
    NNB_REQUIRE(dst->rows == src->rows && dst->cols == src->cols, "accumulate: shape mismatch (%zu, %zu) vs (%zu, %zu)", dst->rows,
                dst->cols, src->rows, src->cols);
    const size_t n = dst->rows * dst->cols;
    t_axpy_kernel<<<grid1(n), 256, 0, dst->e->stream>>>(dst->data, src->data, n, 1.0f, 1.0f);
    dst->e->launches++;
    NNB_CHECK_LAUNCH("t_axpy_kernel");
    wrote(dst);
    return NNB_OK;
}

nnb_status nnb_t_abs(const nnb_tensor* src, nnb_tensor** out)
{
    NNB_REQUIRE(src && out, "abs: NULL argument");
    NNB_TRY(tensor_new(src->e, src->rows, src->cols, false, out));
    const size_t n = src->rows * src->cols;
    t_abs_kernel<<<grid1(n), 256, 0, src->e->stream>>>(src->data, n, (*out)->data);
    src->e->launches++;
    NNB_CHECK_LAUNCH("t_abs_kernel");
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_col_reduce_max(const nnb_tensor* t, nnb_tensor** out)
{
    NNB_REQUIRE(t && out, "col_reduce_max: NULL argument");
    NNB_TRY(tensor_new(t->e, 1, t->cols, false, out));
    t_col_max_kernel<<<grid1(t->cols), 256, 0, t->e->stream>>>(t->data, t->rows, t->cols, (*out)->data);
    t->e->launches++;
    NNB_CHECK_LAUNCH("t_col_max_kernel");
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_row_reduce_sum(const nnb_tensor* t, nnb_tensor** out)
{
    NNB_REQUIRE(t && out, "row_reduce_sum: NULL argument");
    NNB_TRY(tensor_new(t->e, t->rows, 1, false, out));
    t_row_sum_kernel<<<grid1(t->rows), 256, 0, t->e->stream>>>(t->data, t->rows, t->cols, (*out)->data);
    t->e->launches++;
    NNB_CHECK_LAUNCH("t_row_sum_kernel");
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_add_row_broadcast(nnb_tensor* y, const nnb_tensor* b)
{
    NNB_REQUIRE(y && b, "add_row_broadcast: NULL argument");
    T_REQ_SAME_ENGINE(y, b);
    NNB_REQUIRE(b->rows * b->cols == y->rows, "add_row_broadcast: %zu values for %zu rows", b->rows * b->cols, y->rows);
    t_add_row_broadcast_kernel<<<grid1(y->rows * y->cols), 256, 0, y->e->stream>>>(y->data, b->data, y->rows, y->cols);
    y->e->launches++;
    NNB_CHECK_LAUNCH("t_add_row_broadcast_kernel");
    wrote(y);
    return NNB_OK;
}

/* ---- the ternary primitives of BitLinear on tensors (containers are uint32 words bit-cast into f32 tensors, as in
 *      the reference: compute_layer_bitlinear.hpp:60) */
nnb_status nnb_t_absmean_tau(const nnb_tensor* latent, nnb_tensor** tau)
{
    NNB_REQUIRE(latent && tau, "absmean_tau: NULL argument");
    NNB_TRY(tensor_new(latent->e, latent->rows, 1, false, tau));
    NNB_TRY(launch_absmean_tau(latent->e, latent->data, latent->rows, latent->cols, (*tau)->data));
    wrote(*tau);
    return NNB_OK;
}

nnb_status nnb_t_trit_pack_into(const nnb_tensor* latent, const nnb_tensor* tau, nnb_tensor* packed)
{
    NNB_REQUIRE(latent && tau && packed, "trit_pack_into: NULL argument");
    T_REQ_SAME_ENGINE(latent, tau);
    T_REQ_SAME_ENGINE(latent, packed);
    NNB_REQUIRE(tau->rows * tau->cols == latent->rows, "trit_pack: tau must have one value per row");
    NNB_REQUIRE(packed->rows == latent->rows && packed->cols == (latent->cols + 15) / 16, "trit_pack_into: container must be (%zu, %zu)",
                latent->rows, (latent->cols + 15) / 16);
    NNB_TRY(launch_trit_pack(latent->e, latent->data, tau->data, latent->rows, latent->cols, (uint32_t*)packed->data));
    wrote(packed);
    return NNB_OK;
}

nnb_status nnb_t_trit_pack(const nnb_tensor* latent, const nnb_tensor* tau, nnb_tensor** packed)
{
    NNB_REQUIRE(latent && tau && packed, "trit_pack: NULL argument");
    NNB_TRY(tensor_new(latent->e, latent->rows, (latent->cols + 15) / 16, false, packed));
    const nnb_status st = nnb_t_trit_pack_into(latent, tau, *packed);
    if (st != NNB_OK) {
        nnb_tensor_destroy(*packed);
        *packed = nullptr;
    }
    return st;
}

nnb_status nnb_t_matmul_q(const nnb_tensor* packed, const nnb_tensor* tau, const nnb_tensor* x, nnb_tensor** out)
{
    NNB_REQUIRE(packed && tau && x && out, "matmul_q: NULL argument");
    T_REQ_SAME_ENGINE(packed, x);
    NNB_REQUIRE(packed->cols == (x->rows + 15) / 16 && tau->rows * tau->cols == packed->rows, "matmul_q: shape mismatch");
    NNB_TRY(tensor_new(x->e, packed->rows, x->cols, false, out));
    NNB_TRY(launch_matmul_q_ref(x->e, (const uint32_t*)packed->data, tau->data, x->data, packed->rows, x->rows, x->cols, (*out)->data));
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_matmul_q_t(const nnb_tensor* packed, const nnb_tensor* tau, const nnb_tensor* b, size_t m_cols, nnb_tensor** out)
{
    NNB_REQUIRE(packed && tau && b && out, "matmul_q_t: NULL argument");
    T_REQ_SAME_ENGINE(packed, b);
    NNB_REQUIRE(packed->rows == b->rows && packed->cols == (m_cols + 15) / 16 && tau->rows * tau->cols == packed->rows,
                "matmul_q_t: shape mismatch");
    NNB_TRY(tensor_new(b->e, m_cols, b->cols, false, out));
    NNB_TRY(launch_matmul_q_t_ref(b->e, (const uint32_t*)packed->data, tau->data, b->data, packed->rows, m_cols, b->cols, (*out)->data));
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_quantize_i8(const nnb_tensor* x, const nnb_tensor* scale, int col_scale, nnb_tensor** out)
{
    NNB_REQUIRE(x && scale && out, "quantize_i8: NULL argument");
    T_REQ_SAME_ENGINE(x, scale);
    NNB_REQUIRE(scale->rows * scale->cols == (col_scale ? x->cols : x->rows), "quantize_i8: scale has the wrong length");
    NNB_TRY(tensor_new(x->e, x->rows, (x->cols + 3) / 4, false, out));
    NNB_TRY(launch_quantize_i8(x->e, x->data, x->rows, x->cols, scale->data, col_scale, (uint32_t*)(*out)->data));
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_unpack_i8(const nnb_tensor* packed, size_t cols, nnb_tensor** out)
{
    NNB_REQUIRE(packed && out, "unpack_i8: NULL argument");
    NNB_REQUIRE(packed->cols == (cols + 3) / 4, "unpack_i8: container has %zu words per row, %zu columns need %zu", packed->cols, cols,
                (cols + 3) / 4);
    NNB_TRY(tensor_new(packed->e, packed->rows, cols, false, out));
    NNB_TRY(launch_unpack_i8(packed->e, (const uint32_t*)packed->data, packed->rows, cols, (*out)->data));
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_matmul_q_i8(const nnb_tensor* packed, const nnb_tensor* tau, const nnb_tensor* xq, const nnb_tensor* s, nnb_tensor** out)
{
    NNB_REQUIRE(packed && tau && xq && s && out, "matmul_q_i8: NULL argument");
    T_REQ_SAME_ENGINE(packed, xq);
    const size_t n = s->rows * s->cols, k = xq->rows;
    NNB_REQUIRE(packed->cols == (k + 15) / 16 && xq->cols == (n + 3) / 4 && tau->rows * tau->cols == packed->rows,
                "matmul_q_i8: shape mismatch");
    NNB_TRY(tensor_new(xq->e, packed->rows, n, false, out));
    NNB_TRY(launch_matmul_q_i8_ref(xq->e, (const uint32_t*)packed->data, tau->data, (const uint32_t*)xq->data, s->data, packed->rows, k, n,
                                   (*out)->data, nullptr));
    wrote(*out);
    return NNB_OK;
}

nnb_status nnb_t_bitlinear_dw_accumulate(nnb_tensor* grad_w, const nnb_tensor* dy, const nnb_tensor* s, const nnb_tensor* x,
                                         const nnb_tensor* tau)
{
    NNB_REQUIRE(grad_w && dy && x && tau, "bitlinear_dw_accumulate: NULL argument");
    T_REQ_SAME_ENGINE(grad_w, dy);
    T_REQ_SAME_ENGINE(grad_w, x);
    NNB_REQUIRE(grad_w->rows == dy->rows && grad_w->cols == x->rows && dy->cols == x->cols && tau->rows * tau->cols == dy->rows &&
                    (!s || s->rows * s->cols == dy->cols),
                "bitlinear_dw_accumulate: shape mismatch");
    t_dw_accumulate_kernel<<<grid1(grad_w->rows * grad_w->cols), 256, 0, dy->e->stream>>>(grad_w->data, dy->data, s ? s->data : nullptr,
                                                                                          x->data, tau->data, dy->rows, x->rows, dy->cols);
    dy->e->launches++;
    NNB_CHECK_LAUNCH("t_dw_accumulate_kernel");
    wrote(grad_w);
    return NNB_OK;
}

/* ---- standalone RMSNorm and rotary embedding, token-major (rows = tokens) */
nnb_status nnb_rmsnorm_fwd(nnb_engine* e, const float* d_x, const float* d_gamma, size_t t, size_t f, float* d_y)
{
    NNB_REQUIRE(e && d_x && d_gamma && d_y && t > 0 && f > 0, "rmsnorm_fwd: bad arguments");
    NNB_REQUIRE(f % 64 == 0, "rmsnorm_fwd: feature count %zu must be a multiple of 64", f);
    // the model's own kernel (RMSNorm fused with the int8 quantiser of the next linear): the quantised row goes to scratch
    auto al = [](size_t v) { return (v + 255) & ~(size_t)255; };
    NNB_TRY(e->ensure_scratch(al(t * f) + 2 * al(t * 4)));
    int8_t* q = (int8_t*)e->scratch;
    float* s = (float*)((char*)e->scratch + al(t * f));
    int32_t* qs = (int32_t*)((char*)s + al(t * 4));
    return launch_row_quant(e, 0, true, d_x, d_gamma, t, f, f, q, s, qs, d_y);
}

nnb_status nnb_rmsnorm_bwd(nnb_engine* e, const float* d_x, const float* d_gamma, const float* d_dy, size_t t, size_t f, float* d_dx,
                           float* d_dgamma)
{
    NNB_REQUIRE(e && d_x && d_gamma && d_dy && d_dx && d_dgamma && t > 0 && f > 0, "rmsnorm_bwd: bad arguments");
    return launch_rmsnorm_bwd(e, d_x, d_gamma, d_dy, nullptr, t, f, d_dx, d_dgamma);
}

nnb_status nnb_rope_tables(nnb_engine* e, size_t dk, size_t ctx, float* d_cos, float* d_sin)
{
    NNB_REQUIRE(e && d_cos && d_sin && dk >= 2 && dk % 2 == 0 && ctx > 0, "rope_tables: bad arguments");
    const size_t half = dk / 2;
    NNB_TRY(e->ensure_pinned(2 * ctx * half * sizeof(float)));
    float* cs = (float*)e->pinned;
    float* sn = cs + ctx * half;
    for (size_t pos = 0; pos < ctx; ++pos)
        for (size_t j = 0; j < half; ++j) {
            const float theta = (float)pos / powf(10000.0f, (float)(2 * j) / (float)dk);
            cs[pos * half + j] = cosf(theta);
            sn[pos * half + j] = sinf(theta);
        }
    NNB_CUDA(cudaMemcpyAsync(d_cos, cs, ctx * half * sizeof(float), cudaMemcpyHostToDevice, e->stream));
    NNB_CUDA(cudaMemcpyAsync(d_sin, sn, ctx * half * sizeof(float), cudaMemcpyHostToDevice, e->stream));
    NNB_CUDA(cudaStreamSynchronize(e->stream));
    return NNB_OK;
}

nnb_status nnb_rope_apply(nnb_engine* e, float* d_x, const float* d_cos, const float* d_sin, size_t n_rows, size_t seq_len, size_t n_head,
                          size_t dk, int backward)
{
    NNB_REQUIRE(e && d_x && d_cos && d_sin && n_rows > 0 && seq_len > 0 && dk % 2 == 0, "rope_apply: bad arguments");
    return launch_rope(e, d_x, d_cos, d_sin, n_rows, seq_len, n_head, dk, backward != 0);
}

nnb_status nnb_rope_step(nnb_engine* e, float* d_x, const float* d_cos, const float* d_sin, size_t n_seq, size_t pos, size_t n_head, size_t dk)
{
    NNB_REQUIRE(e && d_x && d_cos && d_sin && n_seq > 0 && dk % 2 == 0, "rope_step: bad arguments");
    const size_t half = dk / 2;  // every row is at position `pos`: a one-row table starting there
    return launch_rope(e, d_x, d_cos + pos * half, d_sin + pos * half, n_seq, 1, n_head, dk, false);
}

}  // extern "C"
