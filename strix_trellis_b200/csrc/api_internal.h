// Private definitions shared by the host API translation units.
#pragma once
#include <climits>
#include <cmath>
#include <cstring>
#include <new>
#include <vector>

#include "backend.h"
#include "strix_trellis.h"
#include "strix_trellis_b200.h"

struct strix_context_impl {
    int device = 0;
    int sm_count = 148;
    size_t weights_count = 0;
    unsigned int* status = nullptr;  // device word: bounded-wait failures of any kernel
    bool programmatic_launch = true;
};

struct strix_weights_impl {
    strix_context owner = nullptr;
    st::DeviceWeights device{};
    void* allocation = nullptr;
    size_t allocation_bytes = 0;
    size_t plan_refs = 0;
    // Scratch that plans created on these weights own (partial
    // planes).  A captured graph may replay after its plan is destroyed but not after
    // the weights are, so the scratch lives until the weights are destroyed
    // (the reference keeps its completion counters the same way, src/api.hip:24-27).
    std::vector<void*> plan_scratch;
};

namespace sapi {

constexpr uint64_t kAlign = STRIX_TRELLIS_WORKSPACE_ALIGNMENT;

template <class E> inline uint32_t enum_bits(const E& value) {
    static_assert(sizeof(E) == sizeof(uint32_t), "enum ABI");
    uint32_t raw;
    std::memcpy(&raw, &value, sizeof raw);  // never load an out-of-range C enum
    return raw;
}
template <class T> inline strix_status header(const T* d) {
    if (!d) return STRIX_ERROR_INVALID_ARGUMENT;
    if (d->struct_size != sizeof(T) || d->abi_version != STRIX_TRELLIS_ABI_VERSION)
        return STRIX_ERROR_ABI_MISMATCH;
    for (uint64_t v : d->reserved)
        if (v) return STRIX_ERROR_INVALID_ARGUMENT;
    return STRIX_SUCCESS;
}
inline strix_status cuda_status(cudaError_t e) {
    if (e == cudaSuccess) return STRIX_SUCCESS;
    return e == cudaErrorMemoryAllocation ? STRIX_ERROR_OUT_OF_MEMORY : STRIX_ERROR_BACKEND;
}
inline bool mul_ok(uint64_t a, uint64_t b, uint64_t& out) {
    if (b && a > UINT64_MAX / b) return false;
    out = a * b;
    return true;
}
inline bool range_ok(const void* p, uint64_t bytes) {
    return bytes <= SIZE_MAX && bytes <= UINTPTR_MAX - reinterpret_cast<uintptr_t>(p);
}
inline bool overlap(const void* a, uint64_t an, const void* b, uint64_t bn) {
    if (!an || !bn) return false;
    const uintptr_t x = reinterpret_cast<uintptr_t>(a), y = reinterpret_cast<uintptr_t>(b);
    return x < y + bn && y < x + an;
}

strix_status context_check(strix_context c);
strix_status stream_check(strix_context c, const strix_stream* s, cudaStream_t& out);
// A non-empty buffer must be plain device memory of the context's device and lie
// inside one allocation.
strix_status device_buffer(strix_context c, const void* p, uint64_t bytes, uint64_t align);

// A validated dense call: row views (strides in elements), spans in bytes.
struct View {
    int rows = 0;
    uint64_t x_stride = 0, y_stride = 0;
    uint64_t x_bytes = 0, y_bytes = 0;  // accessed span, row gaps included
};
// contiguous = the strix_gemv / strix_gemm tensor rules; otherwise TP row views.
strix_status view_check(strix_context c, const strix_matmul_desc* d, bool contiguous, View& v);
st::LinearCall make_call(strix_context c, const strix_matmul_desc& d, const View& v);

// Scratch requirement of one linear with `rows` rows through the public entry points.
uint64_t linear_workspace(strix_context c, const st::DeviceWeights& w, int rows);
// Enqueue a validated linear.  `zero_counters`: mark the fold scratch empty first (needed
// when the workspace content is unknown, i.e. outside prepared plans).
cudaError_t enqueue_linear(strix_context c, const st::LinearCall& call, void* workspace,
                           bool zero_counters, cudaStream_t stream);

// Caller-declared workspace: size, alignment, aliasing, then device provenance of all
// three buffers (skipped for an empty call).
strix_status storage_check(strix_context c, const strix_matmul_desc& d, const View& v, uint64_t needed,
                           void* workspace, uint64_t bytes);
strix_status submit(strix_context c, const strix_matmul_desc* d, const strix_stream* stream, bool gemv);

}  // namespace sapi
