// strix_b200_gemv_noalloc: the fused decode GEMV for callers that cannot supply or
// obtain scratch memory.  The split-K scratch (partial planes)
// lives in a fixed array inside the library image instead of a caller workspace.
#include <mutex>

#include "api_internal.h"

using namespace sapi;

namespace {

// Layout: [reserved: kMaxColumnBlocks x u32][partial planes: kMaxCtas x 2 x 8 rows
// x 128 floats].  Every GPU that loads the library carries this array until exit.
constexpr size_t kMaxColumnBlocks = STRIX_B200_NOALLOC_MAX_OUTPUTS / 128;
constexpr size_t kMaxCtas = 192;  // persistent CTAs (one per SM); B200 has 148
constexpr size_t kCounterBytes = kMaxColumnBlocks * sizeof(unsigned int);
constexpr size_t kPlaneBytes = kMaxCtas * 2 * 8 * 128 * sizeof(float);
static_assert(kCounterBytes % 256 == 0, "planes must stay 256-byte aligned");
static_assert(kCounterBytes + kPlaneBytes == STRIX_B200_NOALLOC_SCRATCH_BYTES, "header out of date");

static __device__ __align__(256) unsigned char g_scratch[kCounterBytes + kPlaneBytes];

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
    // Beyond the built-in scratch: refuse, never fall back to an allocation.
    if (c->device >= kMaxDevices || plan.counter_bytes > kCounterBytes || plan.partial_bytes > kPlaneBytes ||
        (uint64_t)w.outputs > STRIX_B200_NOALLOC_MAX_OUTPUTS)
        return STRIX_ERROR_INSUFFICIENT_BUFFER;
    void* scratch = nullptr;
    cudaError_t e = scratch_address(c->device, &scratch);
    if (e != cudaSuccess) return cuda_status(e);
    // The array keeps whatever the previous call left: a completed launch leaves every plane
    // word empty, an aborted one may not, so the planes are marked empty before every call.
    e = st::reset_gemv_scratch(scratch, plan, cs);
    if (e != cudaSuccess) return cuda_status(e);
    // launch_gemv places the planes right after plan.counter_bytes, inside the array
    return cuda_status(st::launch_gemv(make_call(c, *d, v), plan, scratch, c->programmatic_launch, cs));
}
