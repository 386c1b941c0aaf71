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

// ---- small vocabulary of the validation code ---------------------------------------------
// An enum field of a descriptor is whatever 32 bits the caller stored there; it is compared as
// a word and never loaded as the enum type.
template <class E> inline uint32_t enum_bits(const E& field) {
    static_assert(sizeof(E) == 4, "descriptor enums are 32-bit words");
    uint32_t word = 0;
    std::memcpy(&word, &field, 4);
    return word;
}

// Every versioned descriptor starts with {struct_size, abi_version} and ends with a `reserved`
// array.  Order of the verdicts: missing -> invalid argument, wrong size or version -> ABI
// mismatch, non-zero reserved word -> invalid argument.
template <class D> inline strix_status header(const D* desc) {
    if (desc == nullptr) return STRIX_ERROR_INVALID_ARGUMENT;
    const bool same_abi = desc->struct_size == sizeof(D) && desc->abi_version == STRIX_TRELLIS_ABI_VERSION;
    if (!same_abi) return STRIX_ERROR_ABI_MISMATCH;
    uint64_t any = 0;
    for (const uint64_t word : desc->reserved) any |= word;
    return any ? STRIX_ERROR_INVALID_ARGUMENT : STRIX_SUCCESS;
}

inline strix_status cuda_status(cudaError_t e) {
    switch (e) {
    case cudaSuccess: return STRIX_SUCCESS;
    case cudaErrorMemoryAllocation: return STRIX_ERROR_OUT_OF_MEMORY;
    default: return STRIX_ERROR_BACKEND;
    }
}

// a * b without wrap-around
inline bool mul_ok(uint64_t a, uint64_t b, uint64_t& product) {
    return !__builtin_mul_overflow(a, b, &product);
}

// A byte span of the caller's address space.  `fits()` says that begin + bytes neither wraps
// the address space nor exceeds size_t; two spans `touch()` when both are non-empty and share
// at least one byte.
struct Span {
    uintptr_t begin;
    uint64_t bytes;
    Span(const void* p, uint64_t n) : begin(reinterpret_cast<uintptr_t>(p)), bytes(n) {}
    bool fits() const { return bytes <= SIZE_MAX && bytes <= UINTPTR_MAX - begin; }
    bool touch(const Span& o) const {
        if (bytes == 0 || o.bytes == 0) return false;
        return begin < o.begin ? o.begin - begin < bytes : begin - o.begin < o.bytes;
    }
};
inline bool range_ok(const void* p, uint64_t bytes) { return Span(p, bytes).fits(); }
inline bool overlap(const void* a, uint64_t an, const void* b, uint64_t bn) { return Span(a, an).touch(Span(b, bn)); }

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
    int x_dtype = st::DT_F32, y_dtype = st::DT_F32;  // element types (st::DT_*)
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
