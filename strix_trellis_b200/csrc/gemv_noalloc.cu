// strix_b200_gemv_noalloc: the fused decode GEMV for callers that cannot supply or
// obtain scratch memory.  The split-K scratch (the partial planes of one launch) lives in a
// fixed array inside the library image instead of a caller workspace.
#include <mutex>

#include "api_internal.h"

using namespace sapi;

namespace {

// The whole array is partial planes, starting at offset 0: one plane of 128 floats per
// persistent CTA and activation row (the one-row kernel keeps two half planes per CTA).  A
// launch runs at most one CTA per SM, so 1 MiB covers eight rows on a device of up to 256 SMs
// (a B200 has 148).  Every GPU that loads the library carries this array until exit.
constexpr size_t kScratchBytes = STRIX_B200_NOALLOC_SCRATCH_BYTES;
static_assert(kScratchBytes == 256 * 8 * 128 * sizeof(float), "header out of date");

static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

// In host code `g_scratch` is only a handle for the runtime, not an address a kernel
// could use; the device address is looked up once per device and cached here.
constexpr int kMaxDevices = 64;
void* g_device_address[kMaxDevices] = {};
std::mutex g_setup_lock;

cudaError_t scratch_address(int device, void** out) {
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (!g_device_address[device]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_scratch);  // the calling thread's current device
        if (e != cudaSuccess) return e;
        g_device_address[device] = p;
    }
    *out = g_device_address[device];
    return cudaSuccess;
}

}  // namespace

extern "C" strix_status strix_b200_gemv_noalloc(strix_context c, const strix_matmul_desc* d,
                                                const strix_stream* stream) {
    strix_status s = context_check(c);  // the context's device is the current device
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    View v{};
    s = view_check(c, d, true, v);
    if (s != STRIX_SUCCESS) return s;
    if (v.rows > 8) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    if (d->workspace || d->workspace_bytes) return STRIX_ERROR_INVALID_ARGUMENT;
    s = storage_check(c, *d, v, 0, nullptr, 0);
    if (s != STRIX_SUCCESS || !v.rows) return s;
    const st::DeviceWeights& w = d->weights->device;
    const st::GemvPlan plan = st::plan_gemv(w, v.rows, c->sm_count);
    // Beyond the built-in scratch (more CTAs x rows than the array has planes for): refuse, never
    // fall back to an allocation.
    if (c->device >= kMaxDevices || plan.counter_bytes + plan.partial_bytes > kScratchBytes)
        return STRIX_ERROR_INSUFFICIENT_BUFFER;
    void* scratch = nullptr;
    cudaError_t e = scratch_address(c->device, &scratch);
    if (e != cudaSuccess) return cuda_status(e);
    // The array keeps whatever the previous call left: a completed launch leaves every plane
    // word empty, an aborted one may not, so the planes are marked empty before every call.
    e = st::reset_gemv_scratch(scratch, plan, cs);
    if (e != cudaSuccess) return cuda_status(e);
    // launch_gemv places the planes at the start of the array
    return cuda_status(st::launch_gemv(make_call(c, *d, v), plan, scratch, c->programmatic_launch, cs));
}
