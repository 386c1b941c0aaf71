// Host-side contract of the C ABI, checked without a GPU: the real api_*.cpp sources run
// against a CUDA runtime made of counters (fake/cuda_runtime.h) and a launch layer that only
// records (fake_runtime.cpp).  What is asserted is the public behaviour the reference pins for
// its own host layer (tests/test_api_contract.cpp:198-229, 414-449, 471-499, 527-558):
// status precedence, rejection before any allocation / copy / synchronisation, out-handles
// cleared on failure, leak-free failure of every step of weight preparation, plans that
// freeze their descriptor and submit with no query of any kind, lifetime rules, and the
// per-device kernel set-up at context creation.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <vector>

#include "api_internal.h"
#include "mock_backend.h"

static int g_checks = 0;
#define CHECK(cond)                                                                         \
    do {                                                                                    \
        ++g_checks;                                                                         \
        if (!(cond)) {                                                                      \
            std::fprintf(stderr, "contract violated at %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            std::exit(1);                                                                   \
        }                                                                                   \
    } while (0)

using fake::state;
using mock::record;

namespace {

template <class T> T blank() {
    T d{};
    d.struct_size = sizeof(T);
    d.abi_version = STRIX_TRELLIS_ABI_VERSION;
    return d;
}

struct Counts {
    int allocs, frees, copies, memsets, syncs, pointer, range, stream, launches;
    size_t blocks;
    static Counts now() {
        const auto& s = state();
        return {s.allocs, s.frees, s.copies, s.memsets, s.syncs, s.pointer_queries, s.range_queries,
                s.stream_queries, record().launches, s.blocks.size()};
    }
    bool same_traffic(const Counts& o) const {  // nothing allocated, moved or waited for
        return allocs == o.allocs && frees == o.frees && copies == o.copies && memsets == o.memsets &&
               syncs == o.syncs && blocks == o.blocks;
    }
    bool same_queries(const Counts& o) const { return pointer == o.pointer && range == o.range && stream == o.stream; }
};

// A 128-input, 256-output, 3-bit layer on the host.
struct HostLayer {
    std::vector<uint16_t> trellis = std::vector<uint16_t>(128 * 256 * 3 / 16, 0x1234);
    std::vector<uint16_t> suh = std::vector<uint16_t>(128, 0x3C00), svh = std::vector<uint16_t>(256, 0x3C00);
    std::vector<float> bias = std::vector<float>(256, 0.5f);
    strix_exl3_parts_desc parts() {
        auto d = blank<strix_exl3_parts_desc>();
        d.transport_version = 1;
        d.rows = 256; d.columns = 128; d.bits_x2 = 6;
        d.codebook = STRIX_CODEBOOK_MUL1; d.marker = STRIX_EXL3_MARKER_MUL1;
        d.trellis = {trellis.data(), trellis.size() * 2};
        d.suh = {suh.data(), suh.size() * 2};
        d.svh = {svh.data(), svh.size() * 2};
        d.bias = {bias.data(), bias.size() * 4};
        return d;
    }
};

void context_rules() {
    fake::reset();
    record() = mock::Record{};
    auto cd = blank<strix_context_desc>();
    strix_context c = reinterpret_cast<strix_context>(uintptr_t(1));
    cd.device_ordinal = 1;  // not the calling thread's device: the library never switches devices
    CHECK(strix_context_create(&cd, &c) == STRIX_ERROR_INVALID_ARGUMENT && !c);
    cd.device_ordinal = 7;
    CHECK(strix_context_create(&cd, &c) == STRIX_ERROR_UNSUPPORTED_DEVICE && !c);
    cd.device_ordinal = 0;
    state().capability_major = 9;
    CHECK(strix_context_create(&cd, &c) == STRIX_ERROR_UNSUPPORTED_DEVICE && !c);
    state().capability_major = 10;
    cd.struct_size -= 1;
    CHECK(strix_context_create(&cd, &c) == STRIX_ERROR_ABI_MISMATCH && !c);
    cd.struct_size += 1;
    cd.reserved[1] = 1;
    CHECK(strix_context_create(&cd, &c) == STRIX_ERROR_INVALID_ARGUMENT && !c);
    cd.reserved[1] = 0;
    CHECK(record().configured_devices.empty() && state().blocks.empty());
    // a failed status-word allocation leaves nothing behind
    state().alloc_failure_at = state().allocs;
    CHECK(strix_context_create(&cd, &c) == STRIX_ERROR_OUT_OF_MEMORY && !c && state().blocks.empty());
    state().alloc_failure_at = -1;

    // one process, two devices: each context sets up the kernels of ITS device
    strix_context c0 = nullptr, c1 = nullptr;
    record().configured_devices.clear();
    CHECK(strix_context_create(&cd, &c0) == STRIX_SUCCESS && c0);
    state().current_device = 1;
    cd.device_ordinal = 1;
    CHECK(strix_context_create(&cd, &c1) == STRIX_SUCCESS && c1);
    CHECK(record().configured_devices == (std::vector<int>{0, 1}));
    CHECK(c0->device == 0 && c1->device == 1);
    // a context is only usable while its device is current
    HostLayer layer;
    auto parts = layer.parts();
    auto stream = blank<strix_stream>();
    strix_weights w = nullptr;
    CHECK(strix_weights_prepare_parts(c0, &parts, &stream, &w) == STRIX_ERROR_INVALID_ARGUMENT && !w);
    CHECK(strix_weights_prepare_parts(c1, &parts, &stream, &w) == STRIX_SUCCESS && w);
    CHECK(strix_context_destroy(c1) == STRIX_ERROR_INVALID_ARGUMENT);  // weights still alive
    CHECK(strix_weights_destroy(w) == STRIX_SUCCESS);
    CHECK(strix_context_destroy(c1) == STRIX_SUCCESS);
    state().current_device = 0;
    CHECK(strix_context_destroy(c0) == STRIX_SUCCESS);
    CHECK(strix_context_destroy(nullptr) == STRIX_ERROR_INVALID_ARGUMENT);
    CHECK(state().blocks.empty());
}

void prepare_rules(strix_context c) {
    HostLayer layer;
    auto stream = blank<strix_stream>();
    const auto good = layer.parts();
    auto parts = good;
    strix_weights w = nullptr;

    Counts before = Counts::now();
    CHECK(strix_weights_prepare_parts(c, &parts, &stream, &w) == STRIX_SUCCESS && w);
    Counts after = Counts::now();
    CHECK(after.copies == before.copies + 4);          // one copy per region, no staging through the host
    CHECK(after.syncs == before.syncs + 1);            // host bytes may be released when the call returns
    CHECK(after.blocks == before.blocks + 1);          // ONE device allocation survives
    const void* span = nullptr;
    uint64_t span_bytes = 0;
    CHECK(strix_weights_device_span(w, &span, &span_bytes) == STRIX_SUCCESS && span && span_bytes >= 128 * 256 * 3 / 8);
    CHECK(strix_weights_device_span(nullptr, &span, &span_bytes) == STRIX_ERROR_INVALID_ARGUMENT && !span && !span_bytes);
    CHECK(w->device.inputs == 128 && w->device.outputs == 256 && w->device.bits == 3 && w->device.bias);
    CHECK(strix_weights_destroy(w) == STRIX_SUCCESS);
    CHECK(Counts::now().blocks == before.blocks);

    auto refuse = [&](strix_status expected) {
        const Counts b = Counts::now();
        w = reinterpret_cast<strix_weights>(uintptr_t(1));
        CHECK(strix_weights_prepare_parts(c, &parts, &stream, &w) == expected);
        CHECK(!w);                              // the out-handle never keeps garbage
        CHECK(Counts::now().same_traffic(b));   // refused before any allocation, copy or sync
        parts = good;
    };
    parts.struct_size--; refuse(STRIX_ERROR_ABI_MISMATCH);
    parts.abi_version++; refuse(STRIX_ERROR_ABI_MISMATCH);
    parts.reserved[2] = 1; refuse(STRIX_ERROR_INVALID_ARGUMENT);
    parts.transport_version = 2; refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);
    parts.trellis.bytes--; refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);
    parts.columns = UINT64_MAX; refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);
    parts.rows = 200; refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);
    parts.bits_x2 = 5; refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);
    parts.bits_x2 = 18; refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);
    parts.marker ^= 1; refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);
    parts.suh.data = parts.trellis.data; refuse(STRIX_ERROR_INVALID_ARGUMENT);      // regions overlap
    parts.suh.data = nullptr; refuse(STRIX_ERROR_INVALID_ARGUMENT);
    parts.suh.data = reinterpret_cast<void*>(UINTPTR_MAX - 1); refuse(STRIX_ERROR_INVALID_ARGUMENT);  // wraps
    parts.bias.bytes = 0; refuse(STRIX_ERROR_INVALID_ARGUMENT);                   // pointer without bytes
    parts.svh = {nullptr, 0}; refuse(STRIX_ERROR_INVALID_ARGUMENT);               // only the bias is optional
    for (uint32_t raw : {UINT32_MAX, 0x10002u}) {  // enum fields are read as raw 32-bit words
        std::memcpy(&parts.codebook, &raw, sizeof raw);
        refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);
    }
    {   // no handle to write to, no stream descriptor
        const Counts b = Counts::now();
        CHECK(strix_weights_prepare_parts(c, &parts, &stream, nullptr) == STRIX_ERROR_INVALID_ARGUMENT);
        CHECK(strix_weights_prepare_parts(c, &parts, nullptr, &w) == STRIX_ERROR_INVALID_ARGUMENT && !w);
        CHECK(strix_weights_prepare_parts(nullptr, &parts, &stream, &w) == STRIX_ERROR_INVALID_ARGUMENT && !w);
        CHECK(Counts::now().same_traffic(b));
    }
    parts.bias = {nullptr, 0};  // a layer without bias
    CHECK(strix_weights_prepare_parts(c, &parts, &stream, &w) == STRIX_SUCCESS && !w->device.bias);
    CHECK(strix_weights_destroy(w) == STRIX_SUCCESS);
    parts = good;

    // every step of the upload can fail; none may leak device memory or skip the drain
    const size_t held = state().blocks.size();
    for (int step = 0; step < 2; ++step) {
        state().alloc_failure_at = state().allocs + step;
        CHECK(strix_weights_prepare_parts(c, &parts, &stream, &w) == STRIX_ERROR_OUT_OF_MEMORY && !w);
        CHECK(state().blocks.size() == held);
    }
    state().alloc_failure_at = -1;
    for (int step = 0; step < 4; ++step) {
        const int syncs = state().syncs;
        state().copy_failure_at = state().copies + step;
        CHECK(strix_weights_prepare_parts(c, &parts, &stream, &w) == STRIX_ERROR_BACKEND && !w);
        CHECK(state().blocks.size() == held);
        CHECK(state().syncs == syncs + 1);  // copies already enqueued read host memory: drained before return
    }
    state().copy_failure_at = -1;
    record().fail_launch = true;  // the regrouping kernel
    CHECK(strix_weights_prepare_parts(c, &parts, &stream, &w) == STRIX_ERROR_BACKEND && !w && state().blocks.size() == held);
    record().fail_launch = false;
    state().fail_sync = true;
    CHECK(strix_weights_prepare_parts(c, &parts, &stream, &w) == STRIX_ERROR_BACKEND && !w && state().blocks.size() == held);
    state().fail_sync = false;

    // the single-blob form: same rules, plus the region table of the metadata
    std::vector<unsigned char> blob;
    auto meta = strix_exl3_metadata_v1{};
    meta.struct_size = sizeof meta;
    meta.transport_version = 1;
    meta.rows = 256; meta.columns = 128; meta.bits_x2 = 6;
    meta.codebook = STRIX_CODEBOOK_MUL1; meta.marker = STRIX_EXL3_MARKER_MUL1;
    auto put = [&](const void* p, size_t n, uint64_t& off, uint64_t& bytes) {
        while (blob.size() % 4) blob.push_back(0);
        off = blob.size(); bytes = n;
        blob.insert(blob.end(), static_cast<const unsigned char*>(p), static_cast<const unsigned char*>(p) + n);
    };
    put(layer.trellis.data(), layer.trellis.size() * 2, meta.trellis_offset, meta.trellis_bytes);
    put(layer.suh.data(), 256, meta.suh_offset, meta.suh_bytes);
    put(layer.svh.data(), 512, meta.svh_offset, meta.svh_bytes);
    put(layer.bias.data(), 1024, meta.bias_offset, meta.bias_bytes);
    auto td = blank<strix_exl3_transport_desc>();
    td.format = STRIX_TRANSPORT_EXL3_CANONICAL; td.transport_version = 1;
    td.data = blob.data(); td.data_bytes = blob.size();
    td.metadata = &meta; td.metadata_bytes = sizeof meta;
    td.rows = 256; td.columns = 128;
    CHECK(strix_weights_prepare(c, &td, &stream, &w) == STRIX_SUCCESS && w);
    CHECK(strix_weights_destroy(w) == STRIX_SUCCESS);
    const auto good_meta = meta;
    const auto good_td = td;
    auto refuse_blob = [&](strix_status expected) {
        const Counts b = Counts::now();
        w = reinterpret_cast<strix_weights>(uintptr_t(1));
        CHECK(strix_weights_prepare(c, &td, &stream, &w) == expected && !w);
        CHECK(Counts::now().same_traffic(b));
        meta = good_meta; td = good_td;
    };
    td.data_bytes -= 8; refuse_blob(STRIX_ERROR_INSUFFICIENT_BUFFER);        // last region leaves the blob
    meta.suh_offset += 1; refuse_blob(STRIX_ERROR_UNSUPPORTED_FORMAT);       // binary16 region on an odd byte
    meta.svh_offset = meta.suh_offset; refuse_blob(STRIX_ERROR_INVALID_ARGUMENT);  // two regions share bytes
    meta.flags = 1; refuse_blob(STRIX_ERROR_INVALID_ARGUMENT);
    meta.struct_size = 8; refuse_blob(STRIX_ERROR_ABI_MISMATCH);
    td.metadata_bytes -= 1; refuse_blob(STRIX_ERROR_INVALID_ARGUMENT);
    td.rows = 128; refuse_blob(STRIX_ERROR_UNSUPPORTED_FORMAT);              // descriptor and metadata disagree
    td.format = static_cast<strix_transport_format>(7); refuse_blob(STRIX_ERROR_UNSUPPORTED_FORMAT);
    td.data = nullptr; refuse_blob(STRIX_ERROR_INVALID_ARGUMENT);
    meta.bias_bytes = 0; refuse_blob(STRIX_ERROR_UNSUPPORTED_FORMAT);        // offset of an absent bias must be zero
}

void call_and_plan_rules(strix_context c) {
    HostLayer layer;
    auto stream = blank<strix_stream>();
    auto parts = layer.parts();
    strix_weights w = nullptr;
    CHECK(strix_weights_prepare_parts(c, &parts, &stream, &w) == STRIX_SUCCESS);

    void *x = nullptr, *y = nullptr, *ws = nullptr;
    CHECK(cudaMalloc(&x, 16384) == cudaSuccess && cudaMalloc(&y, 16384) == cudaSuccess && cudaMalloc(&ws, 32768) == cudaSuccess);
    strix_matmul_desc d;
    strix_matmul_desc_init(&d);
    CHECK(d.alpha == 1.0f && d.beta == 0.0f && d.struct_size == sizeof d);
    d.weights = w; d.input.data = x; d.output.data = y;
    d.input.rank = d.output.rank = 2;
    d.input.shape[0] = d.output.shape[0] = 2;
    d.input.shape[1] = 128; d.output.shape[1] = 256;
    d.input.strides[0] = 128; d.output.strides[0] = 256;
    d.input.strides[1] = d.output.strides[1] = 1;
    d.input.buffer_bytes = d.output.buffer_bytes = 16384;
    uint64_t need = 0;
    CHECK(strix_matmul_workspace_bytes(c, &d, &need) == STRIX_SUCCESS && need > 0 && need % 256 == 0);
    CHECK(strix_gemv(c, &d, &stream) == STRIX_ERROR_INSUFFICIENT_BUFFER);  // no workspace given
    d.workspace = ws; d.workspace_bytes = need;
    d.alpha = 0.25f; d.beta = -0.5f;
    Counts b = Counts::now();
    CHECK(strix_gemv(c, &d, &stream) == STRIX_SUCCESS && !record().last_was_gemm);
    CHECK(record().last.alpha == 0.25f && record().last.beta == -0.5f && record().last.rows == 2);
    CHECK(record().last.x == x && record().last.y == y && record().last_workspace == ws);
    CHECK(strix_gemm(c, &d, &stream) == STRIX_SUCCESS && !record().last_was_gemm);  // up to 8 rows are vector work
    CHECK(Counts::now().same_traffic(b) && record().launches == b.launches + 2);
    const strix_matmul_desc good = d;
    {   // more than eight rows take the prefill route
        d.input.shape[0] = d.output.shape[0] = 16;
        CHECK(strix_matmul_workspace_bytes(c, &d, &need) == STRIX_SUCCESS && need <= 32768);
        d.workspace_bytes = need;
        CHECK(strix_gemm(c, &d, &stream) == STRIX_SUCCESS && record().last_was_gemm && record().last.rows == 16);
        CHECK(strix_gemv(c, &d, &stream) == STRIX_ERROR_UNSUPPORTED_FORMAT);
        d = good;
    }

    auto refuse = [&](strix_status expected) {
        const Counts k = Counts::now();
        CHECK(strix_gemv(c, &d, &stream) == expected);
        CHECK(strix_gemm(c, &d, &stream) == expected);
        strix_linear_plan p = reinterpret_cast<strix_linear_plan>(uintptr_t(1));
        CHECK(strix_linear_plan_create(c, &d, &stream, STRIX_OPERATION_GEMV, &p) == expected && !p);
        CHECK(Counts::now().same_traffic(k) && record().launches == k.launches);
        d = good;
    };
    const uint32_t bad_enums[] = {UINT32_MAX, 0x10003u};
    for (int side = 0; side < 2; ++side)
        for (uint32_t raw : bad_enums) {
            std::memcpy(side ? &d.output.dtype : &d.input.dtype, &raw, sizeof raw);
            refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);
        }
    d.input.dtype = STRIX_DTYPE_INVALID; refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);
    {   // binary16 / bfloat16 tensors: two bytes per element in the span and alignment rules
        d.input.dtype = STRIX_DTYPE_BF16;
        d.output.dtype = STRIX_DTYPE_F16;
        d.input.buffer_bytes = 2 * 128 * 2;   // exactly two rows of 128 elements
        d.output.buffer_bytes = 2 * 256 * 2;
        CHECK(strix_gemv(c, &d, &stream) == STRIX_SUCCESS);
        CHECK(record().last.x_dtype == st::DT_BF16 && record().last.y_dtype == st::DT_F16);
        d.input.buffer_bytes -= 1;
        CHECK(strix_gemv(c, &d, &stream) == STRIX_ERROR_INSUFFICIENT_BUFFER);
        d.input.buffer_bytes += 1;
        d.output.data = static_cast<char*>(y) + 2;  // two-byte alignment suffices
        CHECK(strix_gemv(c, &d, &stream) == STRIX_SUCCESS);
        d.output.data = static_cast<char*>(y) + 1;
        CHECK(strix_gemv(c, &d, &stream) == STRIX_ERROR_INVALID_ARGUMENT);
        d = good;
    }
    const float bad_scalars[] = {std::numeric_limits<float>::infinity(), -std::numeric_limits<float>::infinity(),
                                 std::numeric_limits<float>::quiet_NaN()};
    for (float v : bad_scalars) {
        d.alpha = v; refuse(STRIX_ERROR_INVALID_ARGUMENT);
        d.beta = v; refuse(STRIX_ERROR_INVALID_ARGUMENT);
    }
    d.output.data = x; refuse(STRIX_ERROR_INVALID_ARGUMENT);                                  // output aliases input
    d.workspace = y; refuse(STRIX_ERROR_INVALID_ARGUMENT);                                    // workspace aliases output
    d.workspace = static_cast<char*>(ws) + 4; refuse(STRIX_ERROR_INVALID_ARGUMENT);           // 256-byte alignment
    d.input.data = const_cast<uint32_t*>(w->device.packed); refuse(STRIX_ERROR_INVALID_ARGUMENT);  // input inside the weights
    d.output.reserved[3] = 1; refuse(STRIX_ERROR_INVALID_ARGUMENT);
    d.input.strides[1] = 2; refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);
    d.input.strides[0] = 256; refuse(STRIX_ERROR_UNSUPPORTED_FORMAT);                         // gemv/gemm want dense rows
    d.input.buffer_bytes = 1; refuse(STRIX_ERROR_INSUFFICIENT_BUFFER);
    d.input.data = static_cast<char*>(x) + 16380; refuse(STRIX_ERROR_INSUFFICIENT_BUFFER);    // runs off its allocation
    std::vector<float> host_rows(256);
    d.input.data = host_rows.data(); refuse(STRIX_ERROR_INVALID_ARGUMENT);                    // host memory
    d.weights = nullptr; refuse(STRIX_ERROR_INVALID_ARGUMENT);
    d.struct_size--; refuse(STRIX_ERROR_ABI_MISMATCH);
    {   // a stream the runtime does not know, and a foreign current device
        auto other = stream;
        other.hip_stream = reinterpret_cast<void*>(uintptr_t(0x20));
        const Counts k = Counts::now();
        CHECK(strix_gemm(c, &d, &other) == STRIX_ERROR_INVALID_ARGUMENT);
        state().current_device = 1;
        CHECK(strix_gemm(c, &d, &stream) == STRIX_ERROR_INVALID_ARGUMENT);
        state().current_device = 0;
        CHECK(record().launches == k.launches);
    }
    d.input.shape[0] = d.output.shape[0] = 9;   // nine rows: a GEMM, not a GEMV
    d.input.buffer_bytes = d.output.buffer_bytes = 16384;
    CHECK(strix_gemv(c, &d, &stream) == STRIX_ERROR_UNSUPPORTED_FORMAT);
    d = good;
    {   // zero rows: validated, nothing inspected on the device, nothing launched, no workspace
        d.input.shape[0] = d.output.shape[0] = 0;
        d.input.data = d.output.data = nullptr; d.input.buffer_bytes = d.output.buffer_bytes = 0;
        d.workspace = nullptr; d.workspace_bytes = 0;
        const Counts k = Counts::now();
        uint64_t none = 1;
        CHECK(strix_matmul_workspace_bytes(c, &d, &none) == STRIX_SUCCESS && none == 0);
        CHECK(strix_gemv(c, &d, &stream) == STRIX_SUCCESS && strix_gemm(c, &d, &stream) == STRIX_SUCCESS);
        CHECK(record().launches == k.launches && Counts::now().same_queries(k));
        d = good;
    }

    // ---- plans ------------------------------------------------------------------------
    state().streams[reinterpret_cast<void*>(uintptr_t(0x10))] = 0;
    stream.hip_stream = reinterpret_cast<void*>(uintptr_t(0x10));
    strix_linear_plan gemv_plan = nullptr, gemm_plan = nullptr;
    CHECK(strix_linear_plan_create(c, &d, &stream, STRIX_OPERATION_GEMV, &gemv_plan) == STRIX_SUCCESS && gemv_plan);
    CHECK(strix_linear_plan_create(c, &d, &stream, STRIX_OPERATION_GEMM, &gemm_plan) == STRIX_SUCCESS && gemm_plan);
    strix_linear_plan unknown_operation = reinterpret_cast<strix_linear_plan>(uintptr_t(1));
    CHECK(strix_linear_plan_create(c, &d, &stream, 77u, &unknown_operation) == STRIX_ERROR_INVALID_ARGUMENT && !unknown_operation);
    CHECK(w->plan_refs == 2);
    CHECK(strix_weights_destroy(w) == STRIX_ERROR_INVALID_ARGUMENT);  // plans hold the weights
    // the caller's descriptor and stream object are dead to the plan from here on
    d.alpha = 99.0f; d.input.data = nullptr; d.output.data = nullptr; d.workspace = nullptr;
    stream.hip_stream = reinterpret_cast<void*>(uintptr_t(0x30));
    b = Counts::now();
    const int device_queries = state().device_queries;
    for (int i = 0; i < 8; ++i) {
        CHECK(strix_linear_plan_submit(gemv_plan) == STRIX_SUCCESS && !record().last_was_gemm);
        CHECK(record().last.alpha == good.alpha && record().last.beta == good.beta && record().last.rows == 2);
        CHECK(record().last.x == good.input.data && record().last.y == good.output.data);
        CHECK(record().last_workspace == good.workspace);
        CHECK(record().last_stream == reinterpret_cast<cudaStream_t>(uintptr_t(0x10)));
    }
    CHECK(strix_linear_plan_submit(gemm_plan) == STRIX_SUCCESS);
    Counts a = Counts::now();
    CHECK(a.same_traffic(b));   // submit: no allocation, copy, memset or synchronisation
    CHECK(a.same_queries(b));   // ... and no pointer, address-range or stream query
    CHECK(a.launches == b.launches + 9);
    CHECK(state().device_queries == device_queries + 9);  // only "is my device current"
    state().current_device = 1;
    CHECK(strix_linear_plan_submit(gemv_plan) == STRIX_ERROR_INVALID_ARGUMENT && record().launches == a.launches);
    state().current_device = 0;
    record().fail_launch = true;
    CHECK(strix_linear_plan_submit(gemv_plan) == STRIX_ERROR_BACKEND);
    record().fail_launch = false;
    CHECK(strix_linear_plan_submit(nullptr) == STRIX_ERROR_INVALID_ARGUMENT);
    CHECK(strix_linear_plan_destroy(nullptr) == STRIX_ERROR_INVALID_ARGUMENT);
    CHECK(strix_linear_plan_destroy(gemv_plan) == STRIX_SUCCESS && w->plan_refs == 1);
    CHECK(strix_weights_destroy(w) == STRIX_ERROR_INVALID_ARGUMENT);
    CHECK(strix_linear_plan_destroy(gemm_plan) == STRIX_SUCCESS);

    // ---- tensor-parallel dense plan on row-strided views --------------------------------
    d = good;
    stream.hip_stream = reinterpret_cast<void*>(uintptr_t(0x10));
    d.workspace = nullptr; d.workspace_bytes = 0;
    d.input.strides[0] = 512; d.output.strides[0] = 1024;   // rows of wider activations
    strix_tp_dense_plan tp = nullptr;
    CHECK(strix_tp_dense_plan_create(c, &d, &stream, &tp) == STRIX_SUCCESS && tp);
    b = Counts::now();
    for (int i = 0; i < 4; ++i) CHECK(strix_tp_dense_plan_submit(tp) == STRIX_SUCCESS);
    a = Counts::now();
    CHECK(a.same_traffic(b) && a.same_queries(b) && a.launches == b.launches + 4);
    CHECK(record().last.x_stride == 512 && record().last.y_stride == 1024);
    CHECK(strix_weights_destroy(w) == STRIX_ERROR_INVALID_ARGUMENT);
    CHECK(strix_tp_dense_plan_destroy(tp) == STRIX_SUCCESS);
    d.input.strides[0] = 64;  // rows overlap
    CHECK(strix_tp_dense_plan_create(c, &d, &stream, &tp) == STRIX_ERROR_UNSUPPORTED_FORMAT && !tp);

    CHECK(w->plan_refs == 0);
    CHECK(strix_weights_destroy(w) == STRIX_SUCCESS);
    CHECK(cudaFree(x) == cudaSuccess && cudaFree(y) == cudaSuccess && cudaFree(ws) == cudaSuccess);
}

}  // namespace

int main() {
    CHECK(strix_get_abi_version() == STRIX_TRELLIS_ABI_VERSION);
    CHECK(std::strcmp(strix_status_string(STRIX_ERROR_OUT_OF_MEMORY), "out of memory") == 0);
    context_rules();

    fake::reset();
    record() = mock::Record{};
    auto cd = blank<strix_context_desc>();
    strix_context c = nullptr;
    CHECK(strix_context_create(&cd, &c) == STRIX_SUCCESS);
    prepare_rules(c);
    call_and_plan_rules(c);
    CHECK(strix_context_destroy(c) == STRIX_SUCCESS);
    CHECK(state().blocks.empty());  // everything the library allocated was returned
    std::printf("contract ok: %d checks\n", g_checks);
    return 0;
}
