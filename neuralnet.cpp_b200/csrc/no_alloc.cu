// no_alloc.cu — group advantages for callers that must not allocate device memory.
//
// Who needs this: a host that has handed all of the GPU's memory to its own pool, a step function
// running inside a region where the CUDA allocator may not be entered (for example while another
// thread holds a capture open, or in a latency-critical loop that forbids driver allocations), or a
// process whose memory budget was fixed at start-up.  nnb_group_advantage keeps its span table in the
// engine's grow-on-demand scratch arena, which calls cudaMalloc the first time and whenever it grows.
// The entry point below does the same computation with the span table in a fixed array that is part
// of the loaded library image, so the call performs no cudaMalloc, cudaFree or any other allocation.
#include "common.cuh"

namespace {

// Scratch of the no-allocation entry point: first rows and row counts of up to NNB_NOALLOC_MAX_GROUPS
// groups (2 x 16384 x 4 bytes = 128 KiB).  Every GPU that loads the library holds this array until the
// process exits.  In host code the name below is only a stand-in for the symbol, not a device
// address; the address is looked up once per device with cudaGetSymbolAddress.
constexpr size_t kMaxGroups = 16384;
static __device__ __align__(256) int32_t g_span_scratch[2 * kMaxGroups];

constexpr int kMaxDevices = 64;
int32_t* g_span_ptr[kMaxDevices] = {nullptr};

}  // namespace

// One-time set-up per device: resolve the device address of the array with `device` current, and put the
// caller's current device back afterwards.  nnb_engine_create calls this, so that the lookup (which may make
// the CUDA runtime load this module's image onto the device) is over before the first operator call.
nnb_status nnb::noalloc_prepare(int device)
{
    NNB_REQUIRE(device >= 0 && device < kMaxDevices, "group_advantage_noalloc: device index %d out of range", device);
    if (g_span_ptr[device]) return NNB_OK;
    int prev = -1;
    NNB_CUDA(cudaGetDevice(&prev));
    if (prev != device) NNB_CUDA(cudaSetDevice(device));
    int32_t* ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress((void**)&ptr, g_span_scratch);
    if (prev != device) cudaSetDevice(prev);
    if (err != cudaSuccess) {
        cudaGetLastError();
        NNB_FAIL(NNB_ERR_CUDA, "cudaGetSymbolAddress of the fixed span scratch failed on device %d: %s", device,
                 cudaGetErrorString(err));
    }
    g_span_ptr[device] = ptr;
    return NNB_OK;
}

extern "C" nnb_status nnb_group_advantage_noalloc(nnb_engine* e, const float* d_returns, size_t n, const int32_t* h_first,
                                                  const int32_t* h_count, size_t n_spans, float eps, float* d_out)
{
    using namespace nnb;
    NNB_REQUIRE(e && d_returns && h_first && h_count && d_out, "group_advantage_noalloc: NULL argument");
    NNB_REQUIRE(n > 0 && n_spans > 0, "group_advantage_noalloc: returns and spans must not be empty");
    NNB_REQUIRE(n_spans <= kMaxGroups,
                "group_advantage_noalloc: %zu groups exceed the fixed scratch of %zu groups; use nnb_group_advantage",
                n_spans, kMaxGroups);
    size_t cursor = 0;
    for (size_t s = 0; s < n_spans; ++s) {
        NNB_REQUIRE(h_count[s] > 0, "group_advantage_noalloc: group row_count must be > 0");
        NNB_REQUIRE((size_t)h_first[s] == cursor, "group_advantage_noalloc: group spans must be contiguous and non-overlapping");
        cursor += (size_t)h_count[s];
    }
    NNB_REQUIRE(cursor == n, "group_advantage_noalloc: group spans do not cover all %zu rows", n);
    // normally resolved by nnb_engine_create; an engine made before this library version's set-up ran gets it here
    NNB_TRY(noalloc_prepare(e->device));
    int32_t* d_first = g_span_ptr[e->device];
    int32_t* d_count = d_first + kMaxGroups;
    // Nothing in the array has to start at zero: the kernel reads only the first n_spans entries of each
    // half, and both are overwritten here, on the same stream, before the kernel runs.
    NNB_CUDA(cudaMemcpyAsync(d_first, h_first, n_spans * sizeof(int32_t), cudaMemcpyHostToDevice, e->stream));
    NNB_CUDA(cudaMemcpyAsync(d_count, h_count, n_spans * sizeof(int32_t), cudaMemcpyHostToDevice, e->stream));
    return launch_group_advantage(e, d_returns, d_first, d_count, n_spans, eps, d_out);
}
