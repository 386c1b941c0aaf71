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

// ---- what a layer consists of ------------------------------------------------------------
// Four regions in transport order.  Their sizes follow from the geometry; each starts on a
// multiple of its element size inside a blob; only the bias may be absent.
enum : int { kTiles = 0, kInputScales, kOutputScales, kBias, kRegionCount };
struct RegionRule {
    uint64_t element_bytes;
    bool optional;
};
constexpr RegionRule kRegionRules[kRegionCount] = {{4, false}, {2, false}, {2, false}, {4, true}};

struct LayerGeometry {
    uint64_t outputs = 0, inputs = 0;
    uint32_t bits = 0, codebook = 0;
    bool has_bias = false;
};

uint32_t marker_of(uint32_t codebook, bool& known) {
    known = true;
    switch (codebook) {
    case STRIX_CODEBOOK_3INST: return STRIX_EXL3_MARKER_3INST;
    case STRIX_CODEBOOK_MCG: return STRIX_EXL3_MARKER_MCG;
    case STRIX_CODEBOOK_MUL1: return STRIX_EXL3_MARKER_MUL1;
    default: known = false; return 0;
    }
}

// Geometry, rate, codebook and the byte count of every region; anything off is an
// unsupported format.  `given[i]` are the byte counts the caller declared.
strix_status geometry_check(uint64_t outputs, uint64_t inputs, uint32_t bits_x2, uint32_t codebook,
                            uint32_t marker, const uint64_t (&given)[kRegionCount], LayerGeometry& g) {
    const auto dimension_ok = [](uint64_t n) { return n >= 128 && n <= INT_MAX && n % 128 == 0; };
    if (!dimension_ok(outputs) || !dimension_ok(inputs)) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    // integer rates 1..8 (bits_x2 even) for every codebook; 1.5 / 2.5 / 3.5 (bits_x2 3, 5, 7) for mul1
    // only -- the reference defines them (python/strix_trellis/codec.py:12-20) but keeps them off its
    // GPU transport (python/strix_trellis/container.py:152-153); here the device decodes them too.
    const int rate = st::rate_code(bits_x2);
    if (rate == 0) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    bool known = false;
    if (marker_of(codebook, known) != marker || !known) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    if (st::rate_is_half(rate) && codebook != STRIX_CODEBOOK_MUL1) return STRIX_ERROR_UNSUPPORTED_FORMAT;
#if defined(__BYTE_ORDER__) && __BYTE_ORDER__ != __ORDER_LITTLE_ENDIAN__
    return STRIX_ERROR_UNSUPPORTED_FORMAT;  // transport words are little-endian and uploaded as they are
#endif
    uint64_t weights = 0, tile_bytes = 0;
    if (!mul_ok(outputs, inputs, weights) || !mul_ok(weights / 16, bits_x2, tile_bytes))
        return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const uint64_t expected[kRegionCount] = {tile_bytes, inputs * 2, outputs * 2, outputs * 4};
    for (int i = 0; i < kRegionCount; ++i) {
        const bool absent = kRegionRules[i].optional && given[i] == 0;
        if (!absent && given[i] != expected[i]) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    }
    g.outputs = outputs;
    g.inputs = inputs;
    g.bits = (uint32_t)rate;  // rate code
    g.codebook = codebook;
    g.has_bias = given[kBias] != 0;
    return STRIX_SUCCESS;
}

// Single-blob transport: descriptor, then the metadata record, then where the regions lie.
strix_status blob_check(const strix_exl3_transport_desc* d, LayerGeometry& g, strix_host_region (&regions)[kRegionCount]) {
    strix_status s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (enum_bits(d->format) != STRIX_TRANSPORT_EXL3_CANONICAL || d->transport_version != STRIX_TRELLIS_TRANSPORT_VERSION)
        return STRIX_ERROR_UNSUPPORTED_FORMAT;
    strix_exl3_metadata_v1 m;
    if (d->metadata == nullptr || d->metadata_bytes != sizeof m) return STRIX_ERROR_INVALID_ARGUMENT;
    std::memcpy(&m, d->metadata, sizeof m);  // the caller's record may be unaligned
    if (m.struct_size != sizeof m || m.transport_version != STRIX_TRELLIS_TRANSPORT_VERSION) return STRIX_ERROR_ABI_MISMATCH;
    uint64_t spare = m.flags;
    for (const uint64_t word : m.reserved) spare |= word;
    if (spare) return STRIX_ERROR_INVALID_ARGUMENT;
    if (m.rows != d->rows || m.columns != d->columns) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const uint64_t offsets[kRegionCount] = {m.trellis_offset, m.suh_offset, m.svh_offset, m.bias_offset};
    const uint64_t sizes[kRegionCount] = {m.trellis_bytes, m.suh_bytes, m.svh_bytes, m.bias_bytes};
    s = geometry_check(m.rows, m.columns, m.bits_x2, enum_bits(m.codebook), m.marker, sizes, g);
    if (s != STRIX_SUCCESS) return s;
    if (!g.has_bias && m.bias_offset != 0) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    if (d->data == nullptr || !range_ok(d->data, d->data_bytes)) return STRIX_ERROR_INVALID_ARGUMENT;
    const unsigned char* base = static_cast<const unsigned char*>(d->data);
    for (int i = 0; i < kRegionCount; ++i) {
        if (offsets[i] > d->data_bytes || sizes[i] > d->data_bytes - offsets[i]) return STRIX_ERROR_INSUFFICIENT_BUFFER;
        if (sizes[i] != 0 && offsets[i] % kRegionRules[i].element_bytes != 0) return STRIX_ERROR_UNSUPPORTED_FORMAT;
        regions[i].data = sizes[i] != 0 ? base + offsets[i] : nullptr;
        regions[i].bytes = sizes[i];
        for (int earlier = 0; earlier < i; ++earlier)
            if (overlap(regions[i].data, regions[i].bytes, regions[earlier].data, regions[earlier].bytes))
                return STRIX_ERROR_INVALID_ARGUMENT;
    }
    return STRIX_SUCCESS;
}

// Separate regions: any host alignment is fine (they are copied byte-wise), pointers and
// sizes must agree, nothing may wrap the address space, no two regions may share bytes.
strix_status parts_check(const strix_exl3_parts_desc* d, LayerGeometry& g, strix_host_region (&regions)[kRegionCount]) {
    const strix_status s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (d->transport_version != STRIX_TRELLIS_TRANSPORT_VERSION) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    const strix_host_region given[kRegionCount] = {d->trellis, d->suh, d->svh, d->bias};
    uint64_t sizes[kRegionCount];
    for (int i = 0; i < kRegionCount; ++i) {
        regions[i] = given[i];
        sizes[i] = given[i].bytes;
        if (given[i].bytes == 0) {
            if (given[i].data != nullptr || !kRegionRules[i].optional) return STRIX_ERROR_INVALID_ARGUMENT;
            continue;
        }
        if (given[i].data == nullptr || !range_ok(given[i].data, given[i].bytes)) return STRIX_ERROR_INVALID_ARGUMENT;
        for (int earlier = 0; earlier < i; ++earlier)
            if (overlap(given[i].data, given[i].bytes, given[earlier].data, given[earlier].bytes))
                return STRIX_ERROR_INVALID_ARGUMENT;
    }
    return geometry_check(d->rows, d->columns, d->bits_x2, enum_bits(d->codebook), d->marker, sizes, g);
}

// Device memory that is given back unless it is kept.
struct DeviceBlock {
    void* p = nullptr;
    cudaError_t reserve(size_t bytes) { return cudaMalloc(&p, bytes); }
    void* keep() { void* out = p; p = nullptr; return out; }
    ~DeviceBlock() { if (p) (void)cudaFree(p); }
};

// Upload: ONE device allocation [regrouped tiles | suh | svh | bias] with every slice on a
// 256-byte boundary.  The tiles arrive in transport order in a temporary device buffer and
// a kernel regroups them; the stream is drained before the call returns, whatever happened,
// because copies already enqueued still read the caller's host memory.
strix_status upload_layer(strix_context c, const LayerGeometry& g, const strix_host_region (&regions)[kRegionCount],
                          cudaStream_t cs, strix_weights* out) {
    size_t slice[kRegionCount];
    uint64_t total = 0;
    for (int i = 0; i < kRegionCount; ++i) {
        slice[i] = static_cast<size_t>(total);
        if (regions[i].bytes > SIZE_MAX - total - 2 * kAlign) return STRIX_ERROR_OUT_OF_MEMORY;
        total = (total + regions[i].bytes + kAlign - 1) / kAlign * kAlign;
    }
    strix_weights_impl* w = new (std::nothrow) strix_weights_impl;
    if (!w) return STRIX_ERROR_OUT_OF_MEMORY;
    DeviceBlock home, staging;
    cudaError_t e = home.reserve(static_cast<size_t>(total));
    if (e == cudaSuccess) e = staging.reserve(static_cast<size_t>(regions[kTiles].bytes));
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        delete w;
        return cuda_status(e);
    }
    unsigned char* base = static_cast<unsigned char*>(home.p);
    for (int i = 0; i < kRegionCount && e == cudaSuccess; ++i) {
        if (regions[i].bytes == 0) continue;
        void* target = i == kTiles ? staging.p : base + slice[i];
        e = cudaMemcpyAsync(target, regions[i].data, static_cast<size_t>(regions[i].bytes), cudaMemcpyHostToDevice, cs);
    }
    if (e == cudaSuccess)
        e = st::launch_regroup(static_cast<const uint32_t*>(staging.p), reinterpret_cast<uint32_t*>(base + slice[kTiles]),
                               static_cast<int>(g.inputs), static_cast<int>(g.outputs), static_cast<int>(g.bits), cs);
    const cudaError_t drained = cudaStreamSynchronize(cs);
    if (e != cudaSuccess || drained != cudaSuccess) {
        delete w;
        return cuda_status(e != cudaSuccess ? e : drained);
    }
    w->owner = c;
    w->device.packed = reinterpret_cast<const uint32_t*>(base + slice[kTiles]);
    w->device.suh = reinterpret_cast<const uint16_t*>(base + slice[kInputScales]);
    w->device.svh = reinterpret_cast<const uint16_t*>(base + slice[kOutputScales]);
    w->device.bias = g.has_bias ? reinterpret_cast<const float*>(base + slice[kBias]) : nullptr;
    w->device.inputs = static_cast<int>(g.inputs);
    w->device.outputs = static_cast<int>(g.outputs);
    w->device.bits = static_cast<int>(g.bits);
    w->device.codebook = static_cast<int>(g.codebook);
    w->allocation = home.keep();
    w->allocation_bytes = static_cast<size_t>(total);
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

// Common head of the two preparation entry points: clear the handle, then context and stream.
static strix_status prepare_begin(strix_context c, const strix_stream* stream, strix_weights* out, cudaStream_t& cs) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = nullptr;
    const strix_status s = context_check(c);
    return s != STRIX_SUCCESS ? s : stream_check(c, stream, cs);
}

strix_status strix_weights_prepare(strix_context c, const strix_exl3_transport_desc* d,
                                   const strix_stream* stream, strix_weights* out) {
    cudaStream_t cs{};
    strix_status s = prepare_begin(c, stream, out, cs);
    if (s != STRIX_SUCCESS) return s;
    LayerGeometry g;
    strix_host_region regions[kRegionCount];
    s = blob_check(d, g, regions);
    return s != STRIX_SUCCESS ? s : upload_layer(c, g, regions, cs, out);
}

strix_status strix_weights_prepare_parts(strix_context c, const strix_exl3_parts_desc* d,
                                         const strix_stream* stream, strix_weights* out) {
    cudaStream_t cs{};
    strix_status s = prepare_begin(c, stream, out, cs);
    if (s != STRIX_SUCCESS) return s;
    LayerGeometry g;
    strix_host_region regions[kRegionCount];
    s = parts_check(d, g, regions);
    return s != STRIX_SUCCESS ? s : upload_layer(c, g, regions, cs, out);
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
