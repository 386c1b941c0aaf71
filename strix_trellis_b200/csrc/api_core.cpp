// Host side of the C ABI: contexts, weight preparation, validation, gemv/gemm, frozen
// plans, pre-routed grouped experts.  It mirrors the contract of the reference's
// src/api.hip (status precedence, "validate everything before the first allocation or
// enqueue", non-transactional grouped submission) against the CUDA runtime.
#include "api_internal.h"

namespace sapi {

// Every device call is made with the context's device current; the library never switches.
strix_status context_check(strix_context c) {
    if (c == nullptr) return STRIX_ERROR_INVALID_ARGUMENT;
    int current = -1;
    const cudaError_t e = cudaGetDevice(&current);
    if (e != cudaSuccess) return cuda_status(e);
    return current == c->device ? STRIX_SUCCESS : STRIX_ERROR_INVALID_ARGUMENT;
}

// The stream travels in the descriptor's pointer field.  The null stream needs no look-up;
// any other handle must be a live stream of the context's device.
strix_status stream_check(strix_context c, const strix_stream* s, cudaStream_t& out) {
    const strix_status verdict = header(s);
    if (verdict != STRIX_SUCCESS) return verdict;
    out = static_cast<cudaStream_t>(s->hip_stream);
    if (out == nullptr) return STRIX_SUCCESS;
    int home = -1;
    unsigned int flags = 0;
    const bool alive = cudaStreamGetDevice(out, &home) == cudaSuccess && cudaStreamGetFlags(out, &flags) == cudaSuccess;
    if (!alive) (void)cudaGetLastError();
    return alive && home == c->device ? STRIX_SUCCESS : STRIX_ERROR_INVALID_ARGUMENT;
}

// The allocation that holds an address, from the driver (cuMemGetAddressRange), reached
// through the runtime's entry-point table so that the library has no link-time dependency on
// the driver library.
namespace {
struct Allocation { uintptr_t base; size_t bytes; };
bool containing_allocation(const void* p, Allocation& found) {
    using Query = int (*)(unsigned long long*, size_t*, unsigned long long);
    static const Query query = [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult how;
        const bool ok = cudaGetDriverEntryPoint("cuMemGetAddressRange", &entry, cudaEnableDefault, &how) == cudaSuccess &&
                        how == cudaDriverEntryPointSuccess;
        if (!ok) (void)cudaGetLastError();
        return ok ? reinterpret_cast<Query>(entry) : static_cast<Query>(nullptr);
    }();
    unsigned long long base = 0;
    size_t bytes = 0;
    if (!query || query(&base, &bytes, static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(p))) != 0) return false;
    found = Allocation{static_cast<uintptr_t>(base), bytes};
    return true;
}
}  // namespace

strix_status device_buffer(strix_context c, const void* p, uint64_t bytes, uint64_t align) {
    if (bytes == 0) return STRIX_SUCCESS;  // an empty buffer is never looked at
    const uintptr_t at = reinterpret_cast<uintptr_t>(p);
    if (p == nullptr || at % align != 0 || !range_ok(p, bytes)) return STRIX_ERROR_INVALID_ARGUMENT;
    cudaPointerAttributes kind{};
    if (cudaPointerGetAttributes(&kind, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return STRIX_ERROR_INVALID_ARGUMENT;
    }
    // plain device memory of this device only: no host, pinned-host or managed memory
    if (kind.type != cudaMemoryTypeDevice || kind.device != c->device) return STRIX_ERROR_INVALID_ARGUMENT;
    Allocation owner{};
    if (!containing_allocation(p, owner)) return STRIX_ERROR_INVALID_ARGUMENT;
    const bool inside = at >= owner.base && at - owner.base <= owner.bytes && bytes <= owner.bytes - (at - owner.base);
    return inside ? STRIX_SUCCESS : STRIX_ERROR_INSUFFICIENT_BUFFER;
}

// ---- tensors ----------------------------------------------------------------------
// The reference reserves STRIX_DTYPE_F16 / BF16 and refuses them (include/strix_trellis.h:39-40,
// 62-63); here activations of either type are widened exactly on load and outputs rounded to
// nearest even on store, with the float32 contract in between.
static strix_status tensor_check(const strix_tensor_desc& t, uint64_t width, uint32_t rank,
                                 uint64_t rows, bool contiguous, uint64_t& stride, uint64_t& bytes, int& dtype) {
    const strix_status s = header(&t);
    if (s != STRIX_SUCCESS) return s;
    switch (enum_bits(t.dtype)) {
    case STRIX_DTYPE_F32: dtype = st::DT_F32; break;
    case STRIX_DTYPE_F16: dtype = st::DT_F16; break;
    case STRIX_DTYPE_BF16: dtype = st::DT_BF16; break;
    default: return STRIX_ERROR_UNSUPPORTED_FORMAT;
    }
    if (t.rank != rank) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const uint64_t element = st::dtype_bytes(dtype);
    if (rank == 1) {
        if (t.shape[0] != width || t.shape[1] || t.strides[0] != 1 || t.strides[1])
            return STRIX_ERROR_UNSUPPORTED_FORMAT;
        stride = width;
    } else {
        if (t.shape[0] != rows || t.shape[1] != width || t.strides[1] != 1)
            return STRIX_ERROR_UNSUPPORTED_FORMAT;
        if (contiguous ? t.strides[0] != width : t.strides[0] < width)
            return STRIX_ERROR_UNSUPPORTED_FORMAT;
        stride = t.strides[0];
    }
    // accessed span: (rows-1)*stride + width elements
    uint64_t elements = 0;
    if (rows) {
        if (!mul_ok(rows - 1, stride, elements) || elements > UINT64_MAX - width)
            return STRIX_ERROR_INVALID_ARGUMENT;
        elements += width;
    }
    if (!mul_ok(elements, element, bytes) || !range_ok(t.data, bytes))
        return STRIX_ERROR_INVALID_ARGUMENT;
    if (bytes > t.buffer_bytes) return STRIX_ERROR_INSUFFICIENT_BUFFER;
    if (bytes && (!t.data || reinterpret_cast<uintptr_t>(t.data) % element))
        return STRIX_ERROR_INVALID_ARGUMENT;
    return STRIX_SUCCESS;
}

strix_status view_check(strix_context c, const strix_matmul_desc* d, bool contiguous, View& v) {
    strix_status s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (!d->weights || d->weights->owner != c || !std::isfinite(d->alpha) || !std::isfinite(d->beta))
        return STRIX_ERROR_INVALID_ARGUMENT;
    const st::DeviceWeights& w = d->weights->device;
    const uint32_t rank = d->input.rank;
    if (rank != 1 && rank != 2) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const uint64_t rows = rank == 1 ? 1 : d->input.shape[0];
    if (rows > INT_MAX) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    v.rows = static_cast<int>(rows);
    s = tensor_check(d->input, (uint64_t)w.inputs, rank, rows, contiguous, v.x_stride, v.x_bytes, v.x_dtype);
    if (s != STRIX_SUCCESS) return s;
    s = tensor_check(d->output, (uint64_t)w.outputs, rank, rows, contiguous, v.y_stride, v.y_bytes, v.y_dtype);
    if (s != STRIX_SUCCESS) return s;
    const strix_weights_impl* wi = d->weights;
    if (overlap(d->input.data, v.x_bytes, d->output.data, v.y_bytes) ||
        overlap(d->input.data, v.x_bytes, wi->allocation, wi->allocation_bytes) ||
        overlap(d->output.data, v.y_bytes, wi->allocation, wi->allocation_bytes))
        return STRIX_ERROR_INVALID_ARGUMENT;
    return STRIX_SUCCESS;
}

st::LinearCall make_call(strix_context c, const strix_matmul_desc& d, const View& v) {
    st::LinearCall call{};
    call.w = d.weights->device;
    call.x = static_cast<const float*>(d.input.data);
    call.y = static_cast<float*>(d.output.data);
    call.x_dtype = v.x_dtype;
    call.y_dtype = v.y_dtype;
    call.rows = v.rows;
    call.x_stride = (long long)v.x_stride;
    call.y_stride = (long long)v.y_stride;
    call.alpha = d.alpha;
    call.beta = d.beta;
    call.status = c->status;
    return call;
}

uint64_t linear_workspace(strix_context c, const st::DeviceWeights& w, int rows) {
    if (rows <= 0) return 0;
    if (rows <= 8) {
        const st::GemvPlan p = st::plan_gemv(w, rows, c->sm_count);
        return p.counter_bytes + p.partial_bytes;
    }
    return st::plan_gemm(w, rows, c->sm_count).workspace_bytes;
}

cudaError_t enqueue_linear(strix_context c, const st::LinearCall& call, void* workspace,
                           bool zero_counters, cudaStream_t stream) {
    if (call.rows <= 8) {
        const st::GemvPlan p = st::plan_gemv(call.w, call.rows, c->sm_count);
        if (zero_counters) {  // scratch of unknown content
            const cudaError_t e = st::reset_gemv_scratch(workspace, p, stream);
            if (e != cudaSuccess) return e;
        }
        return st::launch_gemv(call, p, workspace, c->programmatic_launch, stream);
    }
    return st::launch_gemm(call, st::plan_gemm(call.w, call.rows, c->sm_count), workspace, c->programmatic_launch,
                           stream);
}

// workspace declared by the caller: size, alignment, aliasing, then device provenance
strix_status storage_check(strix_context c, const strix_matmul_desc& d, const View& v,
                                  uint64_t needed, void* workspace, uint64_t bytes) {
    if (bytes < needed) return STRIX_ERROR_INSUFFICIENT_BUFFER;
    if (!range_ok(workspace, bytes) ||
        (bytes && (!workspace || reinterpret_cast<uintptr_t>(workspace) % kAlign)))
        return STRIX_ERROR_INVALID_ARGUMENT;
    const strix_weights_impl* wi = d.weights;
    if (overlap(workspace, bytes, d.input.data, v.x_bytes) ||
        overlap(workspace, bytes, d.output.data, v.y_bytes) ||
        overlap(workspace, bytes, wi->allocation, wi->allocation_bytes))
        return STRIX_ERROR_INVALID_ARGUMENT;
    if (!v.rows) return STRIX_SUCCESS;  // empty call: no device inspection at all
    strix_status s = device_buffer(c, d.input.data, v.x_bytes, st::dtype_bytes(v.x_dtype));
    if (s != STRIX_SUCCESS) return s;
    s = device_buffer(c, d.output.data, v.y_bytes, st::dtype_bytes(v.y_dtype));
    if (s != STRIX_SUCCESS) return s;
    return device_buffer(c, workspace, bytes, kAlign);
}

strix_status submit(strix_context c, const strix_matmul_desc* d, const strix_stream* stream,
                           bool gemv) {
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    View v{};
    s = view_check(c, d, true, v);
    if (s != STRIX_SUCCESS) return s;
    if ((gemv && v.rows > 8) || (!gemv && d->input.rank != 2)) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const uint64_t needed = linear_workspace(c, d->weights->device, v.rows);
    s = storage_check(c, *d, v, needed, d->workspace, d->workspace_bytes);
    if (s != STRIX_SUCCESS || !v.rows) return s;
    return cuda_status(enqueue_linear(c, make_call(c, *d, v), d->workspace, true, cs));
}

}  // namespace sapi
