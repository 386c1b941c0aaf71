// Entry points declared in strix_trellis_b200.h: stage probes and runtime switches.
#include "api_internal.h"
#include "gemv_partition.h"
#include "grouped.h"

using namespace sapi;

namespace {
strix_status begin(strix_context c, strix_weights w, const strix_stream* stream, cudaStream_t& cs) {
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    if (!w || w->owner != c) return STRIX_ERROR_INVALID_ARGUMENT;
    return stream_check(c, stream, cs);
}
}  // namespace

extern "C" {

strix_status strix_b200_dequantize(strix_context c, strix_weights w, void* out_f16, uint64_t out_bytes,
                                   const strix_stream* stream) {
    cudaStream_t cs{};
    strix_status s = begin(c, w, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    const uint64_t need = (uint64_t)w->device.inputs * w->device.outputs * 2;
    if (out_bytes < need) return STRIX_ERROR_INSUFFICIENT_BUFFER;
    s = device_buffer(c, out_f16, need, 2);
    if (s != STRIX_SUCCESS) return s;
    return cuda_status(st::launch_dequantize(w->device, static_cast<uint16_t*>(out_f16), cs));
}

strix_status strix_b200_input_stages(strix_context c, strix_weights w, const float* x, uint32_t rows,
                                     void* scaled_f16, float* hadamard_f32, void* core_f16,
                                     const strix_stream* stream) {
    cudaStream_t cs{};
    strix_status s = begin(c, w, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    if (!rows) return STRIX_SUCCESS;
    const uint64_t n = (uint64_t)rows * w->device.inputs;
    s = device_buffer(c, x, n * 4, 4);
    if (s == STRIX_SUCCESS && scaled_f16) s = device_buffer(c, scaled_f16, n * 2, 2);
    if (s == STRIX_SUCCESS && hadamard_f32) s = device_buffer(c, hadamard_f32, n * 4, 4);
    if (s == STRIX_SUCCESS && core_f16) s = device_buffer(c, core_f16, n * 2, 2);
    if (s != STRIX_SUCCESS) return s;
    return cuda_status(st::launch_input_stages(w->device, x, w->device.inputs, (int)rows,
                                               static_cast<uint16_t*>(scaled_f16), hadamard_f32,
                                               static_cast<uint16_t*>(core_f16), cs));
}

strix_status strix_b200_output_stages(strix_context c, strix_weights w, const float* core,
                                      uint32_t splits, uint32_t rows, float alpha, float beta, float* y,
                                      const strix_stream* stream) {
    cudaStream_t cs{};
    strix_status s = begin(c, w, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    if (!std::isfinite(alpha) || !std::isfinite(beta) || !splits) return STRIX_ERROR_INVALID_ARGUMENT;
    if (!rows) return STRIX_SUCCESS;
    const uint64_t n = (uint64_t)rows * w->device.outputs;
    s = device_buffer(c, core, n * 4 * splits, 4);
    if (s == STRIX_SUCCESS) s = device_buffer(c, y, n * 4, 4);
    if (s != STRIX_SUCCESS) return s;
    return cuda_status(st::launch_output_stages(w->device, core, (int)splits, (int)rows, y,
                                                w->device.outputs, alpha, beta, cs));
}

strix_status strix_b200_core_exact(strix_context c, strix_weights w, const void* core_f16, uint32_t rows,
                                   float* core_out, const strix_stream* stream) {
    cudaStream_t cs{};
    strix_status s = begin(c, w, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    if (rows < 1 || rows > 64) return STRIX_ERROR_UNSUPPORTED_FORMAT;
    s = device_buffer(c, core_f16, (uint64_t)rows * w->device.inputs * 2, 2);
    if (s == STRIX_SUCCESS) s = device_buffer(c, core_out, (uint64_t)rows * w->device.outputs * 4, 4);
    if (s != STRIX_SUCCESS) return s;
    return cuda_status(st::launch_core_exact(w->device, static_cast<const uint16_t*>(core_f16), (int)rows,
                                             core_out, cs));
}

// Synchronous diagnostic: allocates its two small buffers, runs the probe, waits and averages.
strix_status strix_b200_decode_rate(strix_context c, strix_weights w, uint32_t iterations, uint32_t warps_per_sm,
                                    double* clocks_per_tile, const strix_stream* stream) {
    if (clocks_per_tile) *clocks_per_tile = 0.0;
    if (!clocks_per_tile || iterations < 1 || iterations > (1u << 20) || warps_per_sm < 4 || warps_per_sm > 32 ||
        warps_per_sm % 4)
        return STRIX_ERROR_INVALID_ARGUMENT;
    cudaStream_t cs{};
    strix_status s = begin(c, w, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    const int grid = c->sm_count;
    float* sink = nullptr;
    long long* clocks = nullptr;
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&sink), (size_t)grid * warps_per_sm * 32 * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&clocks), (size_t)grid * sizeof(long long));
    std::vector<long long> host(grid);
    for (int pass = 0; pass < 2 && e == cudaSuccess; ++pass)  // the second pass is the measured one
        e = st::launch_decode_rate(w->device, (int)iterations, (int)warps_per_sm, grid, sink, clocks, cs);
    if (e == cudaSuccess) e = cudaStreamSynchronize(cs);
    if (e == cudaSuccess) e = cudaMemcpy(host.data(), clocks, (size_t)grid * sizeof(long long), cudaMemcpyDeviceToHost);
    if (sink) (void)cudaFree(sink);
    if (clocks) (void)cudaFree(clocks);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return cuda_status(e); }
    double total = 0.0;
    for (long long v : host) total += (double)v;
    // every CTA decodes iterations x 8 tiles per warp, and a quarter of its warps share an SM sub-partition
    *clocks_per_tile = total / grid / ((double)iterations * 8.0 * (double)warps_per_sm / 4.0);
    return STRIX_SUCCESS;
}

strix_status strix_b200_gemv_splits(strix_context c, strix_weights w, uint32_t rows, uint32_t* out) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = 0;
    if (!c || !w || w->owner != c || rows < 1 || rows > 8) return STRIX_ERROR_INVALID_ARGUMENT;
    *out = (uint32_t)st::plan_gemv(w->device, (int)rows, c->sm_count).splits;
    return STRIX_SUCCESS;
}

strix_status strix_b200_moe_combine_rows(strix_context c, const float* rows, const float* scores,
                                         const int32_t* row_valid, uint32_t tokens, uint32_t top_k, uint32_t width,
                                         float* y, uint64_t y_stride, float alpha, float beta,
                                         const strix_stream* stream) {
    strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    // Stream and pointer provenance are inspected with runtime / driver queries, which a
    // capturing stream does not tolerate: while `stream` is being captured into a graph only
    // the arithmetic checks apply.
    cudaStream_t cs = stream ? reinterpret_cast<cudaStream_t>(stream->hip_stream) : nullptr;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cs && cudaStreamIsCapturing(cs, &capturing) != cudaSuccess) {
        (void)cudaGetLastError();
        return STRIX_ERROR_INVALID_ARGUMENT;
    }
    if (capturing == cudaStreamCaptureStatusNone) {
        s = stream_check(c, stream, cs);
        if (s != STRIX_SUCCESS) return s;
    } else if (stream->struct_size != sizeof(strix_stream) || stream->abi_version != STRIX_TRELLIS_ABI_VERSION) {
        return STRIX_ERROR_ABI_MISMATCH;
    }
    if (!std::isfinite(alpha) || !std::isfinite(beta) || top_k < 1 || top_k > STRIX_B200_MOE_MAX_TOP_K ||
        width < 1 || tokens > STRIX_B200_MOE_MAX_ROWS || y_stride < width)
        return STRIX_ERROR_INVALID_ARGUMENT;
    if (!tokens) return STRIX_SUCCESS;
    const uint64_t n_rows = (uint64_t)tokens * top_k * width * 4, n_scores = (uint64_t)tokens * top_k * 4;
    const uint64_t n_y = ((uint64_t)(tokens - 1) * y_stride + width) * 4;
    if (overlap(rows, n_rows, y, n_y) || overlap(scores, n_scores, y, n_y)) return STRIX_ERROR_INVALID_ARGUMENT;
    if (capturing == cudaStreamCaptureStatusNone) {
        s = device_buffer(c, rows, n_rows, 4);
        if (s == STRIX_SUCCESS) s = device_buffer(c, scores, n_scores, 4);
        if (s == STRIX_SUCCESS) s = device_buffer(c, y, n_y, 4);
        if (s == STRIX_SUCCESS && row_valid) s = device_buffer(c, row_valid, (uint64_t)tokens * 4, 4);
        if (s != STRIX_SUCCESS) return s;
    } else if (!rows || !scores || !y) {
        return STRIX_ERROR_INVALID_ARGUMENT;
    }
    return cuda_status(st::launch_moe_combine(rows, scores, row_valid, (int)tokens, (int)top_k, (int)width, y,
                                              (long long)y_stride, alpha, beta, c->programmatic_launch, cs));
}

strix_status strix_b200_moe_combine(strix_context c, const float* rows, const float* scores, uint32_t tokens,
                                    uint32_t top_k, uint32_t width, float* y, uint64_t y_stride, float alpha,
                                    float beta, const strix_stream* stream) {
    return strix_b200_moe_combine_rows(c, rows, scores, nullptr, tokens, top_k, width, y, y_stride, alpha, beta, stream);
}

// Pure host arithmetic: no context, no device.
strix_status strix_b200_gemv_partition(uint64_t inputs, uint64_t outputs, uint32_t grid, uint32_t cta,
                                       uint64_t column_block, uint64_t out[4]) {
    if (!out) return STRIX_ERROR_INVALID_ARGUMENT;
    out[0] = out[1] = out[2] = out[3] = 0;
    if (!inputs || !outputs || inputs % 128 || outputs % 128 || !grid || cta >= grid ||
        inputs > (1ull << 31) || outputs > (1ull << 31))
        return STRIX_ERROR_INVALID_ARGUMENT;
    const long long hblocks = (long long)(inputs / 128), nblocks = (long long)(outputs / 128);
    if (column_block >= (uint64_t)nblocks || (uint64_t)grid > (uint64_t)(hblocks * nblocks))
        return STRIX_ERROR_INVALID_ARGUMENT;
    const long long units = hblocks * nblocks;
    if (units > 0x7FFFFFFF) return STRIX_ERROR_INVALID_ARGUMENT;
    const st::Split split = st::make_split((int)units, (int)grid);
    const st::Range r = st::cta_range(split, (int)cta);
    int first = 0, last = 0;
    st::contributors(split, (int)(column_block * hblocks), (int)((column_block + 1) * hblocks), first, last);
    out[0] = (uint64_t)r.begin;
    out[1] = (uint64_t)r.end;
    out[2] = (uint64_t)first;
    out[3] = (uint64_t)last;
    return STRIX_SUCCESS;
}

strix_status strix_b200_device_status(strix_context c, uint32_t* out_bits) {
    if (!out_bits) return STRIX_ERROR_INVALID_ARGUMENT;
    *out_bits = 0;
    const strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(out_bits, c->status, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemset(c->status, 0, sizeof(uint32_t));
    return cuda_status(e);
}

strix_status strix_b200_set_programmatic_launch(strix_context c, uint32_t enabled) {
    if (!c) return STRIX_ERROR_INVALID_ARGUMENT;
    c->programmatic_launch = enabled != 0;
    return STRIX_SUCCESS;
}

}  // extern "C"
