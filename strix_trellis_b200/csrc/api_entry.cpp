// extern "C" entry points of the core surface (contexts, weights, gemv/gemm, plans,
// pre-routed grouped experts).  Reference counterpart: src/api.hip:376-607.
#include "api_internal.h"

using namespace sapi;

struct strix_linear_plan_impl {
    strix_context owner;
    strix_matmul_desc desc;
    st::LinearCall call;
    cudaStream_t stream;
    int rows;
};

namespace {

struct Region { uint64_t offset, bytes; };

strix_status metadata_check(const strix_exl3_metadata_v1& m, uint64_t rows, uint64_t columns) {
    if (m.struct_size != sizeof(m) || m.transport_version != STRIX_TRELLIS_TRANSPORT_VERSION)
        return STRIX_ERROR_ABI_MISMATCH;
    for (uint64_t v : m.reserved)
        if (v) return STRIX_ERROR_INVALID_ARGUMENT;
    if (m.flags) return STRIX_ERROR_INVALID_ARGUMENT;
    if (m.rows != rows || m.columns != columns || !m.rows || !m.columns || m.rows > INT_MAX ||
        m.columns > INT_MAX || m.rows % 128 || m.columns % 128)
        return STRIX_ERROR_UNSUPPORTED_FORMAT;
    if (m.bits_x2 < 2 || m.bits_x2 > 16 || m.bits_x2 % 2) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    uint32_t marker;
    switch (enum_bits(m.codebook)) {
    case STRIX_CODEBOOK_3INST: marker = STRIX_EXL3_MARKER_3INST; break;
    case STRIX_CODEBOOK_MCG: marker = STRIX_EXL3_MARKER_MCG; break;
    case STRIX_CODEBOOK_MUL1: marker = STRIX_EXL3_MARKER_MUL1; break;
    default: return STRIX_ERROR_UNSUPPORTED_FORMAT;
    }
    if (marker != m.marker) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const uint16_t probe = 1;
    if (*reinterpret_cast<const unsigned char*>(&probe) != 1) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    uint64_t packed = 0;
    if (!mul_ok(m.rows, m.columns, packed) || !mul_ok(packed / 8, m.bits_x2 / 2, packed))
        return STRIX_ERROR_UNSUPPORTED_FORMAT;
    if (m.trellis_bytes != packed || m.suh_bytes != m.columns * 2 || m.svh_bytes != m.rows * 2 ||
        (m.bias_bytes && m.bias_bytes != m.rows * 4) || (!m.bias_bytes && m.bias_offset))
        return STRIX_ERROR_UNSUPPORTED_FORMAT;
    return STRIX_SUCCESS;
}

strix_status transport_check(const strix_exl3_transport_desc* d, strix_exl3_metadata_v1& m) {
    strix_status s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (enum_bits(d->format) != STRIX_TRANSPORT_EXL3_CANONICAL ||
        d->transport_version != STRIX_TRELLIS_TRANSPORT_VERSION)
        return STRIX_ERROR_UNSUPPORTED_FORMAT;
    if (!d->metadata || d->metadata_bytes != sizeof(m)) return STRIX_ERROR_INVALID_ARGUMENT;
    std::memcpy(&m, d->metadata, sizeof(m));
    s = metadata_check(m, d->rows, d->columns);
    if (s != STRIX_SUCCESS) return s;
    if (!d->data || !range_ok(d->data, d->data_bytes)) return STRIX_ERROR_INVALID_ARGUMENT;
    const Region r[4] = {{m.trellis_offset, m.trellis_bytes}, {m.suh_offset, m.suh_bytes},
                         {m.svh_offset, m.svh_bytes}, {m.bias_offset, m.bias_bytes}};
    for (int i = 0; i < 4; ++i) {
        if (r[i].offset > d->data_bytes || r[i].bytes > d->data_bytes - r[i].offset)
            return STRIX_ERROR_INSUFFICIENT_BUFFER;
        const uint64_t align = (i == 1 || i == 2) ? 2 : 4;
        if (r[i].bytes && r[i].offset % align) return STRIX_ERROR_UNSUPPORTED_FORMAT;
        for (int j = 0; j < i; ++j)
            if (r[i].bytes && r[j].bytes && r[i].offset < r[j].offset + r[j].bytes &&
                r[j].offset < r[i].offset + r[i].bytes)
                return STRIX_ERROR_INVALID_ARGUMENT;
    }
    return STRIX_SUCCESS;
}

strix_status parts_check(const strix_exl3_parts_desc* d, strix_exl3_metadata_v1& m) {
    strix_status s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (d->transport_version != STRIX_TRELLIS_TRANSPORT_VERSION) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const strix_host_region r[4] = {d->trellis, d->suh, d->svh, d->bias};
    for (int i = 0; i < 4; ++i) {
        if (!r[i].bytes) {
            if (r[i].data || i != 3) return STRIX_ERROR_INVALID_ARGUMENT;
            continue;
        }
        if (!r[i].data || !range_ok(r[i].data, r[i].bytes)) return STRIX_ERROR_INVALID_ARGUMENT;
        for (int j = 0; j < i; ++j)
            if (overlap(r[i].data, r[i].bytes, r[j].data, r[j].bytes)) return STRIX_ERROR_INVALID_ARGUMENT;
    }
    m = {};
    m.struct_size = sizeof(m);
    m.transport_version = d->transport_version;
    m.rows = d->rows;
    m.columns = d->columns;
    m.bits_x2 = d->bits_x2;
    std::memcpy(&m.codebook, &d->codebook, sizeof(m.codebook));
    m.marker = d->marker;
    m.trellis_bytes = d->trellis.bytes;
    m.suh_bytes = d->suh.bytes;
    m.svh_bytes = d->svh.bytes;
    m.bias_bytes = d->bias.bytes;
    // offsets are meaningless for separate regions; give the blob-equivalent layout
    uint64_t at = 0;
    uint64_t* offs[4] = {&m.trellis_offset, &m.suh_offset, &m.svh_offset, &m.bias_offset};
    for (int i = 0; i < 4; ++i) {
        if (!r[i].bytes) continue;
        at = (at + 3) & ~UINT64_C(3);
        *offs[i] = at;
        if (r[i].bytes > UINT64_MAX - at) return STRIX_ERROR_UNSUPPORTED_FORMAT;
        at += r[i].bytes;
    }
    return metadata_check(m, d->rows, d->columns);
}

// One device allocation: [regrouped trellis | suh | svh | bias], 256-byte aligned
// slices.  The transport-order trellis is staged in a temporary device buffer and
// regrouped by a kernel; the stream is drained before host ownership returns.
strix_status prepare_regions(strix_context c, const strix_exl3_metadata_v1& m,
                             const strix_host_region* regions, cudaStream_t cs, strix_weights* out) {
    strix_weights_impl* w = new (std::nothrow) strix_weights_impl;
    if (!w) return STRIX_ERROR_OUT_OF_MEMORY;
    w->owner = c;
    w->device.inputs = static_cast<int>(m.columns);
    w->device.outputs = static_cast<int>(m.rows);
    w->device.bits = static_cast<int>(m.bits_x2 / 2);
    w->device.codebook = static_cast<int>(enum_bits(m.codebook));
    size_t offsets[4];
    uint64_t total = 0;
    for (int i = 0; i < 4; ++i) {
        total = (total + kAlign - 1) & ~(kAlign - 1);
        offsets[i] = static_cast<size_t>(total);
        if (regions[i].bytes > SIZE_MAX - total - kAlign) { delete w; return STRIX_ERROR_OUT_OF_MEMORY; }
        total += regions[i].bytes;
    }
    w->allocation_bytes = static_cast<size_t>(total);
    void* staging = nullptr;
    cudaError_t e = cudaMalloc(&w->allocation, w->allocation_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&staging, static_cast<size_t>(regions[0].bytes));
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        if (w->allocation) (void)cudaFree(w->allocation);
        delete w;
        return cuda_status(e);
    }
    unsigned char* base = static_cast<unsigned char*>(w->allocation);
    w->device.packed = reinterpret_cast<const uint32_t*>(base + offsets[0]);
    w->device.suh = reinterpret_cast<const uint16_t*>(base + offsets[1]);
    w->device.svh = reinterpret_cast<const uint16_t*>(base + offsets[2]);
    w->device.bias = m.bias_bytes ? reinterpret_cast<const float*>(base + offsets[3]) : nullptr;
    for (int i = 0; i < 4 && e == cudaSuccess; ++i) {
        if (!regions[i].bytes) continue;
        void* dst = i == 0 ? staging : static_cast<void*>(base + offsets[i]);
        e = cudaMemcpyAsync(dst, regions[i].data, static_cast<size_t>(regions[i].bytes),
                            cudaMemcpyHostToDevice, cs);
    }
    if (e == cudaSuccess)
        e = st::launch_regroup(static_cast<const uint32_t*>(staging),
                               reinterpret_cast<uint32_t*>(base + offsets[0]), w->device.inputs,
                               w->device.outputs, w->device.bits, cs);
    const cudaError_t done = cudaStreamSynchronize(cs);  // also drains earlier uploads on failure
    (void)cudaFree(staging);
    if (e != cudaSuccess || done != cudaSuccess) {
        (void)cudaFree(w->allocation);
        delete w;
        return cuda_status(e != cudaSuccess ? e : done);
    }
    ++c->weights_count;
    *out = w;
    return STRIX_SUCCESS;
}

strix_status grouped_check(strix_context c, const strix_grouped_moe_desc* d, uint64_t& maximum) {
    strix_status s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (d->group_count > SIZE_MAX / sizeof(strix_matmul_desc) || (d->group_count && !d->groups) ||
        !range_ok(d->groups, d->group_count * sizeof(strix_matmul_desc)))
        return STRIX_ERROR_INVALID_ARGUMENT;
    maximum = 0;
    std::vector<View> views(static_cast<size_t>(d->group_count));
    for (uint64_t i = 0; i < d->group_count; ++i) {
        const strix_matmul_desc& g = d->groups[i];
        if (g.workspace || g.workspace_bytes) return STRIX_ERROR_INVALID_ARGUMENT;
        View& a = views[i];
        s = view_check(c, &g, true, a);
        if (s != STRIX_SUCCESS) return s;
        const uint64_t need = linear_workspace(c, g.weights->device, a.rows);
        if (need > maximum) maximum = need;
        for (uint64_t j = 0; j < i; ++j) {  // no slice may be shared, read/write included
            const strix_matmul_desc& h = d->groups[j];
            const View& b = views[j];
            if (overlap(g.input.data, a.x_bytes, h.input.data, b.x_bytes) ||
                overlap(g.input.data, a.x_bytes, h.output.data, b.y_bytes) ||
                overlap(g.output.data, a.y_bytes, h.input.data, b.x_bytes) ||
                overlap(g.output.data, a.y_bytes, h.output.data, b.y_bytes) ||
                overlap(g.input.data, a.x_bytes, h.weights->allocation, h.weights->allocation_bytes) ||
                overlap(h.input.data, b.x_bytes, g.weights->allocation, g.weights->allocation_bytes) ||
                overlap(g.output.data, a.y_bytes, h.weights->allocation, h.weights->allocation_bytes) ||
                overlap(h.output.data, b.y_bytes, g.weights->allocation, g.weights->allocation_bytes))
                return STRIX_ERROR_INVALID_ARGUMENT;
        }
    }
    return STRIX_SUCCESS;
}

}  // namespace

extern "C" {

uint32_t strix_get_abi_version(void) { return STRIX_TRELLIS_ABI_VERSION; }

const char* strix_status_string(strix_status s) {
    switch (s) {
    case STRIX_SUCCESS: return "success";
    case STRIX_ERROR_INVALID_ARGUMENT: return "invalid argument";
    case STRIX_ERROR_ABI_MISMATCH: return "ABI mismatch";
    case STRIX_ERROR_UNSUPPORTED_FORMAT: return "unsupported format";
    case STRIX_ERROR_UNSUPPORTED_DEVICE: return "unsupported device";
    case STRIX_ERROR_INSUFFICIENT_BUFFER: return "insufficient buffer";
    case STRIX_ERROR_OUT_OF_MEMORY: return "out of memory";
    case STRIX_ERROR_BACKEND: return "CUDA/backend error";
    case STRIX_ERROR_NOT_IMPLEMENTED: return "not implemented";
    default: return "unknown status";
    }
}

void strix_matmul_desc_init(strix_matmul_desc* d) {
    if (!d) return;
    *d = {};
    d->struct_size = sizeof(*d);
    d->abi_version = STRIX_TRELLIS_ABI_VERSION;
    d->alpha = 1.0f;
    d->input.struct_size = d->output.struct_size = sizeof(strix_tensor_desc);
    d->input.abi_version = d->output.abi_version = STRIX_TRELLIS_ABI_VERSION;
    d->input.dtype = d->output.dtype = STRIX_DTYPE_F32;
}

strix_status strix_context_create(const strix_context_desc* d, strix_context* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    strix_status s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (d->flags || d->device_ordinal < 0) return STRIX_ERROR_INVALID_ARGUMENT;
    int major = 0, sms = 0;
    cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, d->device_ordinal);
    if (e == cudaErrorInvalidDevice) { (void)cudaGetLastError(); return STRIX_ERROR_UNSUPPORTED_DEVICE; }
    if (e != cudaSuccess) return cuda_status(e);
    if (major != 10) return STRIX_ERROR_UNSUPPORTED_DEVICE;  // sm_100a kernels only
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d->device_ordinal);
    if (e != cudaSuccess) return cuda_status(e);
    int active = -1;
    e = cudaGetDevice(&active);
    if (e != cudaSuccess) return cuda_status(e);
    if (active != d->device_ordinal) return STRIX_ERROR_INVALID_ARGUMENT;  // never switches devices
    e = st::configure_device();  // function attributes of this device; the active device is the context's
    if (e != cudaSuccess) return cuda_status(e);
    strix_context_impl* c = new (std::nothrow) strix_context_impl;
    if (!c) return STRIX_ERROR_OUT_OF_MEMORY;
    c->device = d->device_ordinal;
    c->sm_count = sms;
    e = cudaMalloc(reinterpret_cast<void**>(&c->status), kAlign);
    if (e == cudaSuccess) e = cudaMemset(c->status, 0, kAlign);
    if (e != cudaSuccess) {
        if (c->status) (void)cudaFree(c->status);
        delete c;
        return cuda_status(e);
    }
    *out = c;
    return STRIX_SUCCESS;
}

strix_status strix_context_destroy(strix_context c) {
    if (!c || c->weights_count) return STRIX_ERROR_INVALID_ARGUMENT;
    (void)cudaFree(c->status);
    delete c;
    return STRIX_SUCCESS;
}

strix_status strix_weights_prepare(strix_context c, const strix_exl3_transport_desc* d,
                                   const strix_stream* stream, strix_weights* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    strix_exl3_metadata_v1 m{};
    s = transport_check(d, m);
    if (s != STRIX_SUCCESS) return s;
    const unsigned char* base = static_cast<const unsigned char*>(d->data);
    const strix_host_region r[4] = {{base + m.trellis_offset, m.trellis_bytes},
                                    {base + m.suh_offset, m.suh_bytes},
                                    {base + m.svh_offset, m.svh_bytes},
                                    {m.bias_bytes ? base + m.bias_offset : nullptr, m.bias_bytes}};
    return prepare_regions(c, m, r, cs, out);
}

strix_status strix_weights_prepare_parts(strix_context c, const strix_exl3_parts_desc* d,
                                         const strix_stream* stream, strix_weights* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    strix_exl3_metadata_v1 m{};
    s = parts_check(d, m);
    if (s != STRIX_SUCCESS) return s;
    const strix_host_region r[4] = {d->trellis, d->suh, d->svh, d->bias};
    return prepare_regions(c, m, r, cs, out);
}

strix_status strix_weights_destroy(strix_weights w) {
    if (!w || w->plan_refs) return STRIX_ERROR_INVALID_ARGUMENT;
    const strix_status s = context_check(w->owner);
    if (s != STRIX_SUCCESS) return s;
    while (!w->plan_scratch.empty()) {
        const cudaError_t e = cudaFree(w->plan_scratch.back());
        if (e != cudaSuccess) return cuda_status(e);
        w->plan_scratch.pop_back();
    }
    const cudaError_t e = cudaFree(w->allocation);
    if (e != cudaSuccess) return cuda_status(e);
    --w->owner->weights_count;
    delete w;
    return STRIX_SUCCESS;
}

strix_status strix_weights_device_span(strix_weights w, const void** data, uint64_t* bytes) {
    if (data) *data = nullptr;
    if (bytes) *bytes = 0;
    if (!w || !data || !bytes) return STRIX_ERROR_INVALID_ARGUMENT;
    *data = w->allocation;
    *bytes = w->allocation_bytes;
    return STRIX_SUCCESS;
}

strix_status strix_matmul_workspace_bytes(strix_context c, const strix_matmul_desc* d, uint64_t* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = 0;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    View v{};
    s = view_check(c, d, true, v);
    if (s == STRIX_SUCCESS) *out = linear_workspace(c, d->weights->device, v.rows);
    return s;
}

strix_status strix_gemv(strix_context c, const strix_matmul_desc* d, const strix_stream* stream) {
    return submit(c, d, stream, true);
}
strix_status strix_gemm(strix_context c, const strix_matmul_desc* d, const strix_stream* stream) {
    return submit(c, d, stream, false);
}

strix_status strix_linear_plan_create(strix_context c, const strix_matmul_desc* d,
                                      const strix_stream* stream, uint32_t operation,
                                      strix_linear_plan* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    if (operation != STRIX_OPERATION_GEMV && operation != STRIX_OPERATION_GEMM)
        return STRIX_ERROR_INVALID_ARGUMENT;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    View v{};
    s = view_check(c, d, true, v);
    if (s != STRIX_SUCCESS) return s;
    const bool gemm = operation == STRIX_OPERATION_GEMM;
    if ((!gemm && v.rows > 8) || (gemm && d->input.rank != 2)) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const uint64_t needed = linear_workspace(c, d->weights->device, v.rows);
    s = storage_check(c, *d, v, needed, d->workspace, d->workspace_bytes);
    if (s != STRIX_SUCCESS) return s;
    if (d->weights->plan_refs == SIZE_MAX) return STRIX_ERROR_OUT_OF_MEMORY;
    strix_linear_plan_impl* p = new (std::nothrow) strix_linear_plan_impl{c, *d, make_call(c, *d, v), cs, v.rows};
    if (!p) return STRIX_ERROR_OUT_OF_MEMORY;
    if (v.rows && v.rows <= 8) {
        // The fold scratch starts empty and every launch leaves it empty, so submit is a
        // single kernel.  Mark it now and drain, so replays on any stream find it empty.
        const st::GemvPlan gp = st::plan_gemv(p->call.w, v.rows, c->sm_count);
        cudaError_t e = st::reset_gemv_scratch(d->workspace, gp, cs);
        if (e == cudaSuccess) e = cudaStreamSynchronize(cs);
        if (e != cudaSuccess) { delete p; return cuda_status(e); }
    }
    ++d->weights->plan_refs;
    *out = p;
    return STRIX_SUCCESS;
}

strix_status strix_linear_plan_submit(strix_linear_plan p) {
    if (!p) return STRIX_ERROR_INVALID_ARGUMENT;
    const strix_status s = context_check(p->owner);
    if (s != STRIX_SUCCESS || !p->rows) return s;
    return cuda_status(enqueue_linear(p->owner, p->call, p->desc.workspace, false, p->stream));
}

strix_status strix_linear_plan_destroy(strix_linear_plan p) {
    if (!p) return STRIX_ERROR_INVALID_ARGUMENT;
    --p->desc.weights->plan_refs;
    delete p;
    return STRIX_SUCCESS;
}

strix_status strix_grouped_moe_workspace_bytes(strix_context c, const strix_grouped_moe_desc* d,
                                               uint64_t* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = 0;
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    uint64_t maximum = 0;
    s = grouped_check(c, d, maximum);
    if (s == STRIX_SUCCESS) *out = maximum;
    return s;
}

strix_status strix_grouped_moe(strix_context c, const strix_grouped_moe_desc* d,
                               const strix_stream* stream) {
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    cudaStream_t cs{};
    s = stream_check(c, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    uint64_t maximum = 0;
    s = grouped_check(c, d, maximum);
    if (s != STRIX_SUCCESS) return s;
    if (d->workspace_bytes < maximum) return STRIX_ERROR_INSUFFICIENT_BUFFER;
    if (!range_ok(d->workspace, d->workspace_bytes) ||
        (d->workspace_bytes && (!d->workspace || reinterpret_cast<uintptr_t>(d->workspace) % kAlign)))
        return STRIX_ERROR_INVALID_ARGUMENT;
    std::vector<View> views(static_cast<size_t>(d->group_count));
    for (uint64_t i = 0; i < d->group_count; ++i) {  // all groups, before the first enqueue
        s = view_check(c, &d->groups[i], true, views[i]);
        if (s != STRIX_SUCCESS) return s;
        s = storage_check(c, d->groups[i], views[i], 0, d->workspace, d->workspace_bytes);
        if (s != STRIX_SUCCESS) return s;
    }
    for (uint64_t i = 0; i < d->group_count; ++i) {
        if (!views[i].rows) continue;
        s = cuda_status(enqueue_linear(c, make_call(c, d->groups[i], views[i]), d->workspace, true, cs));
        if (s != STRIX_SUCCESS) return s;  // earlier groups stay enqueued
    }
    return STRIX_SUCCESS;
}

}  // extern "C"
