// Implementation of the counting CUDA runtime declared in fake/cuda_runtime.h and of the
// kernel-launch layer (st::plan_* / st::launch_*) as recorders.  Linked with the real host
// API sources into the contract test program.
#include <cstdlib>
#include <cstring>

#include "backend.h"
#include "grouped.h"
#include "mock_backend.h"

namespace fake {
State& state() { static State s; return s; }
void reset() { state() = State{}; }
static const std::pair<const uintptr_t, Block>* find_block(const void* p) {
    auto& blocks = state().blocks;
    const uintptr_t at = reinterpret_cast<uintptr_t>(p);
    auto it = blocks.upper_bound(at);
    if (it == blocks.begin()) return nullptr;
    --it;
    return at - it->first < it->second.bytes || (it->second.bytes == 0 && at == it->first) ? &*it : nullptr;
}
}  // namespace fake
using fake::state;

cudaError_t cudaGetDevice(int* device) { ++state().device_queries; *device = state().current_device; return cudaSuccess; }
cudaError_t cudaGetLastError() { return cudaSuccess; }
cudaError_t cudaDeviceGetAttribute(int* value, cudaDeviceAttr attr, int device) {
    if (device < 0 || device >= state().device_count) return cudaErrorInvalidDevice;
    *value = attr == cudaDevAttrComputeCapabilityMajor ? state().capability_major : state().sm_count;
    return cudaSuccess;
}
cudaError_t cudaMalloc(void** out, size_t bytes) {
    const int number = state().allocs++;
    if (number == state().alloc_failure_at) { *out = nullptr; return cudaErrorMemoryAllocation; }
    void* p = std::aligned_alloc(256, (bytes + 255) / 256 * 256 + 256);
    if (!p) return cudaErrorMemoryAllocation;
    state().blocks[reinterpret_cast<uintptr_t>(p)] = fake::Block{bytes, state().current_device};
    *out = p;
    return cudaSuccess;
}
cudaError_t cudaFree(void* p) {
    if (!p) return cudaSuccess;
    auto it = state().blocks.find(reinterpret_cast<uintptr_t>(p));
    if (it == state().blocks.end()) return cudaErrorInvalidValue;
    state().blocks.erase(it);
    ++state().frees;
    std::free(p);
    return cudaSuccess;
}
static cudaError_t copy(void* dst, const void* src, size_t bytes) {
    const int number = state().copies++;
    state().copy_sources.push_back(src);
    if (number == state().copy_failure_at) return cudaErrorLaunchFailure;
    std::memcpy(dst, src, bytes);
    return cudaSuccess;
}
cudaError_t cudaMemcpy(void* dst, const void* src, size_t bytes, cudaMemcpyKind) { return copy(dst, src, bytes); }
cudaError_t cudaMemcpyAsync(void* dst, const void* src, size_t bytes, cudaMemcpyKind, cudaStream_t) { return copy(dst, src, bytes); }
cudaError_t cudaMemset(void* dst, int value, size_t bytes) { ++state().memsets; std::memset(dst, value, bytes); return cudaSuccess; }
cudaError_t cudaMemsetAsync(void* dst, int value, size_t bytes, cudaStream_t) { return cudaMemset(dst, value, bytes); }
cudaError_t cudaStreamSynchronize(cudaStream_t) { ++state().syncs; return state().fail_sync ? cudaErrorLaunchFailure : cudaSuccess; }
cudaError_t cudaDeviceSynchronize() { ++state().syncs; return state().fail_sync ? cudaErrorLaunchFailure : cudaSuccess; }
cudaError_t cudaStreamGetDevice(cudaStream_t s, int* device) {
    ++state().stream_queries;
    auto it = state().streams.find(s);
    if (it == state().streams.end()) return cudaErrorInvalidValue;
    *device = it->second;
    return cudaSuccess;
}
cudaError_t cudaStreamGetFlags(cudaStream_t s, unsigned int* flags) {
    ++state().stream_queries;
    if (!state().streams.count(s)) return cudaErrorInvalidValue;
    *flags = 0;
    return cudaSuccess;
}
cudaError_t cudaStreamIsCapturing(cudaStream_t, cudaStreamCaptureStatus* status) {
    *status = state().capturing ? cudaStreamCaptureStatusActive : cudaStreamCaptureStatusNone;
    return cudaSuccess;
}
cudaError_t cudaPointerGetAttributes(cudaPointerAttributes* out, const void* p) {
    ++state().pointer_queries;
    *out = cudaPointerAttributes{};
    if (const auto* block = fake::find_block(p)) {
        out->type = cudaMemoryTypeDevice;
        out->device = block->second.device;
    }
    return cudaSuccess;
}
static int address_range(unsigned long long* base, size_t* size, unsigned long long p) {
    ++state().range_queries;
    const auto* block = fake::find_block(reinterpret_cast<const void*>(static_cast<uintptr_t>(p)));
    if (!block) return 1;
    *base = block->first;
    *size = block->second.bytes;
    return 0;
}
cudaError_t cudaGetDriverEntryPoint(const char*, void** fn, unsigned long long, cudaDriverEntryPointQueryResult* result) {
    *fn = reinterpret_cast<void*>(&address_range);
    *result = cudaDriverEntryPointSuccess;
    return cudaSuccess;
}

// ---- the launch layer as a recorder ---------------------------------------------------
namespace mock {
Record& record() { static Record r; return r; }
static cudaError_t launched() {
    if (record().fail_launch) return cudaErrorLaunchFailure;
    ++record().launches;
    return cudaSuccess;
}
}  // namespace mock
using mock::record;

namespace st {
cudaError_t configure_device() { record().configured_devices.push_back(fake::state().current_device); return cudaSuccess; }
cudaError_t launch_regroup(const uint32_t* src, uint32_t* dst, int inputs, int outputs, int bits, cudaStream_t) {
    std::memcpy(dst, src, (size_t)inputs * outputs / 8 * bits);  // identity stands in for the regrouping
    return mock::launched();
}
cudaError_t launch_dequantize(const DeviceWeights&, uint16_t*, cudaStream_t) { return mock::launched(); }
cudaError_t launch_input_stages(const DeviceWeights&, const float*, long long, int, uint16_t*, float*, uint16_t*, cudaStream_t) { return mock::launched(); }
cudaError_t launch_output_stages(const DeviceWeights&, const float*, int, int, float*, long long, float, float, cudaStream_t) { return mock::launched(); }
cudaError_t launch_core_exact(const DeviceWeights&, const uint16_t*, int, float*, cudaStream_t) { return mock::launched(); }
cudaError_t launch_decode_rate(const DeviceWeights&, int, int, int, float*, long long*, cudaStream_t) { return mock::launched(); }
GemvPlan plan_gemv(const DeviceWeights& w, int rows, int) {
    GemvPlan p{};
    p.grid = 4; p.splits = 2; p.stages = 2; p.act_blocks = 1;
    p.partial_bytes = align_up((size_t)p.grid * rows * 128 * sizeof(float));
    (void)w;
    return p;
}
cudaError_t reset_gemv_scratch(void* workspace, const GemvPlan& plan, cudaStream_t) {
    ++record().scratch_resets;
    if (plan.counter_bytes + plan.partial_bytes) std::memset(workspace, 0xFF, plan.counter_bytes + plan.partial_bytes);
    return cudaSuccess;
}
cudaError_t launch_gemv(const LinearCall& call, const GemvPlan&, void* workspace, bool, cudaStream_t stream) {
    record().last = call; record().last_workspace = workspace; record().last_stream = stream; record().last_was_gemm = false;
    return mock::launched();
}
GemmPlan plan_gemm(const DeviceWeights& w, int rows, int) {
    GemmPlan p{};
    p.act_bytes = align_up((size_t)rows * w.inputs * 2);
    p.workspace_bytes = p.act_bytes;
    return p;
}
cudaError_t launch_gemm(const LinearCall& call, const GemmPlan&, void* workspace, bool, cudaStream_t stream) {
    record().last = call; record().last_workspace = workspace; record().last_stream = stream; record().last_was_gemm = true;
    return mock::launched();
}
GroupedPlan replan_grouped(const GroupedPlan& sized, int, int, int, int, int) { return sized; }
GroupedPlan plan_grouped(int, int outputs, int, int, int, int) {
    GroupedPlan p{};
    p.splits = 2; p.scratch_splits = 2; p.stages = 2; p.ctas_per_problem = 2;
    p.counter_bytes_per_problem = align_up((size_t)outputs / 128 * 4);
    p.partial_bytes_per_problem = align_up((size_t)outputs * 2 * kGroupRows * 4);
    return p;
}
cudaError_t launch_grouped(const GroupedProblem*, int, int, int, int, const GroupedPlan&, unsigned int*, bool, cudaStream_t) { return mock::launched(); }
cudaError_t launch_swiglu(const float*, const float*, float*, int, int, long long, bool, cudaStream_t) { return mock::launched(); }
cudaError_t launch_moe_route(const unsigned int*, const float*, int, int, const MoeBankEntry*, int, MoeWindow, GroupedProblem*, GroupedProblem*, int*, bool, cudaStream_t) { return mock::launched(); }
cudaError_t launch_moe_combine(const float*, const float*, const int*, int, int, int, float*, long long, float, float, bool, cudaStream_t, const unsigned int*, int, int) { return mock::launched(); }
}  // namespace st
