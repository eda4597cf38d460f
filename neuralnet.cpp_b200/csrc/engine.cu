// engine.cu — engine lifetime, device memory and the error channel of the C-ABI.
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace nnb {

static thread_local char g_error[1024] = "";

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

const char* get_error() { return g_error; }

}  // namespace nnb

nnb_status nnb_engine::ensure_scratch(size_t bytes)
{
    if (bytes <= scratch_bytes) return NNB_OK;
    // growing means the old arena may still be in use by enqueued work
    NNB_CUDA(cudaStreamSynchronize(stream));
    if (scratch) NNB_CUDA(cudaFree(scratch));
    scratch = nullptr;
    scratch_bytes = 0;
    size_t want = bytes + bytes / 4 + (1u << 20);
    cudaError_t err = cudaMalloc(&scratch, want);
    if (err != cudaSuccess) {
        cudaGetLastError();
        NNB_FAIL(NNB_ERR_OOM, "scratch allocation of %zu bytes failed: %s", want,
                 cudaGetErrorString(err));
    }
    scratch_bytes = want;
    return NNB_OK;
}

nnb_status nnb_engine::ensure_pinned(size_t bytes)
{
    if (bytes <= pinned_bytes) return NNB_OK;
    NNB_CUDA(cudaStreamSynchronize(stream));
    if (pinned) NNB_CUDA(cudaFreeHost(pinned));
    pinned = nullptr;
    pinned_bytes = 0;
    size_t want = bytes + bytes / 4 + (1u << 16);
    NNB_CUDA(cudaMallocHost(&pinned, want));
    pinned_bytes = want;
    return NNB_OK;
}

extern "C" {

const char* nnb_last_error(void) { return nnb::get_error(); }

nnb_status nnb_engine_create(int device, nnb_engine** out)
{
    NNB_REQUIRE(out != nullptr, "nnb_engine_create: out is NULL");
    *out = nullptr;
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess || count == 0) {
        cudaGetLastError();
        NNB_FAIL(NNB_ERR_CUDA, "no CUDA device available (%s); this engine has no CPU fallback",
                 err != cudaSuccess ? cudaGetErrorString(err) : "device count is 0");
    }
    NNB_REQUIRE(device >= 0 && device < count, "device %d out of range (0..%d)", device, count - 1);
    NNB_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    NNB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        NNB_FAIL(NNB_ERR_UNSUPPORTED,
                 "device %d is sm_%d%d; this engine is built for sm_100a (B200) only", device,
                 prop.major, prop.minor);
    nnb_engine* e = new nnb_engine();
    e->device = device;
    e->sm_count = prop.multiProcessorCount;
    err = cudaStreamCreateWithFlags(&e->own_stream, cudaStreamNonBlocking);
    if (err != cudaSuccess) {
        delete e;
        NNB_FAIL(NNB_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(err));
    }
    e->stream = e->own_stream;
    if (cudaMalloc((void**)&e->dev_flags, 256) != cudaSuccess || cudaMemset(e->dev_flags, 0, 256) != cudaSuccess) {
        cudaGetLastError();
        cudaStreamDestroy(e->own_stream);
        delete e;
        NNB_FAIL(NNB_ERR_OOM, "out of device memory for the engine's flag block");
    }
    char buf[512];
    snprintf(buf, sizeof(buf),
             "nn-b200 engine on %s (sm_%d%d, %d SMs, %.1f GB): ternary_gemm=true int8_dot=true "
             "int8_dot_accelerated=true",
             prop.name, prop.major, prop.minor, prop.multiProcessorCount,
             (double)prop.totalGlobalMem / 1e9);
    e->describe_text = buf;
    // the no-allocation entry point's scratch address is looked up now, so that its calls never touch the
    // module loader; a failure here only surfaces if that entry point is used
    if (nnb::noalloc_prepare(device) != NNB_OK) nnb::set_error("%s", "");
    *out = e;
    return NNB_OK;
}

void nnb_engine_destroy(nnb_engine* e)
{
    if (!e) return;
    cudaSetDevice(e->device);
    cudaStreamSynchronize(e->stream);
    if (e->scratch) cudaFree(e->scratch);
    if (e->dev_flags) cudaFree(e->dev_flags);
    if (e->dw_part) cudaFree(e->dw_part);
    if (e->pinned) cudaFreeHost(e->pinned);
    if (e->own_stream) cudaStreamDestroy(e->own_stream);
    delete e;
}

nnb_status nnb_engine_describe(nnb_engine* e, char* buf, size_t buf_len)
{
    NNB_REQUIRE(e && buf && buf_len > 0, "nnb_engine_describe: bad arguments");
    snprintf(buf, buf_len, "%s", e->describe_text.c_str());
    return NNB_OK;
}

nnb_status nnb_engine_sync(nnb_engine* e)
{
    NNB_REQUIRE(e, "engine is NULL");
    NNB_CUDA(cudaStreamSynchronize(e->stream));
    return NNB_OK;
}

nnb_status nnb_engine_set_stream(nnb_engine* e, void* cuda_stream)
{
    NNB_REQUIRE(e, "engine is NULL");
    NNB_CUDA(cudaStreamSynchronize(e->stream));
    e->stream = (cuda_stream == NNB_STREAM_OWN) ? e->own_stream : (cudaStream_t)cuda_stream;
    return NNB_OK;
}

void* nnb_engine_stream(nnb_engine* e) { return e ? (void*)e->stream : nullptr; }

unsigned long long nnb_engine_launch_count(nnb_engine* e) { return e ? e->launches : 0ull; }

nnb_status nnb_alloc(nnb_engine* e, size_t bytes, void** d_out)
{
    NNB_REQUIRE(e && d_out, "nnb_alloc: bad arguments");
    *d_out = nullptr;
    if (bytes == 0) return NNB_OK;
    NNB_CUDA(cudaSetDevice(e->device));
    cudaError_t err = cudaMalloc(d_out, bytes);
    if (err != cudaSuccess) {
        cudaGetLastError();
        NNB_FAIL(NNB_ERR_OOM, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(err));
    }
    return NNB_OK;
}

nnb_status nnb_free(nnb_engine* e, void* d_ptr)
{
    NNB_REQUIRE(e, "engine is NULL");
    if (!d_ptr) return NNB_OK;
    NNB_CUDA(cudaStreamSynchronize(e->stream));
    NNB_CUDA(cudaFree(d_ptr));
    return NNB_OK;
}

nnb_status nnb_upload(nnb_engine* e, void* d_dst, const void* h_src, size_t bytes)
{
    NNB_REQUIRE(e && (bytes == 0 || (d_dst && h_src)), "nnb_upload: bad arguments");
    if (bytes == 0) return NNB_OK;
    NNB_CUDA(cudaMemcpyAsync(d_dst, h_src, bytes, cudaMemcpyHostToDevice, e->stream));
    NNB_CUDA(cudaStreamSynchronize(e->stream));
    return NNB_OK;
}

nnb_status nnb_download(nnb_engine* e, void* h_dst, const void* d_src, size_t bytes)
{
    NNB_REQUIRE(e && (bytes == 0 || (h_dst && d_src)), "nnb_download: bad arguments");
    if (bytes == 0) return NNB_OK;
    NNB_CUDA(cudaMemcpyAsync(h_dst, d_src, bytes, cudaMemcpyDeviceToHost, e->stream));
    NNB_CUDA(cudaStreamSynchronize(e->stream));
    return NNB_OK;
}

nnb_status nnb_zero(nnb_engine* e, void* d_ptr, size_t bytes)
{
    NNB_REQUIRE(e && (bytes == 0 || d_ptr), "nnb_zero: bad arguments");
    if (bytes == 0) return NNB_OK;
    NNB_CUDA(cudaMemsetAsync(d_ptr, 0, bytes, e->stream));
    return NNB_OK;
}

}  // extern "C"
