// Interface between the host API layer (api.cpp) and the CUDA kernels (*.cu).
// Everything here is plain data and plain functions: no allocation, transfer or
// synchronisation happens behind a launch_* call.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "rates.h"

namespace st {

// Prepared weights on the device.  `packed` holds the tiles regrouped per 128 output
// columns: [N/128][I/16][8 column tiles][tile_words(rate) uint32 words]; a column block is one
// contiguous stream of I/128 units of unit_bytes(rate) bytes.
struct DeviceWeights {
    const uint32_t* packed;
    const uint16_t* suh;  // binary16 bits [inputs]
    const uint16_t* svh;  // binary16 bits [outputs]
    const float* bias;    // [outputs] or nullptr
    int inputs;
    int outputs;
    int bits;      // rate code (rates.h): 1..8 integer rates, 9..11 for 1.5 / 2.5 / 3.5
    int codebook;
};

// Element types of activation and output tensors.  F16 and BF16 inputs are widened to float32
// when they are read (exact), outputs are rounded to nearest even when they are stored; the
// arithmetic in between is the float32 contract.
enum : int { DT_F32 = 0, DT_F16 = 1, DT_BF16 = 2 };
inline size_t dtype_bytes(int dtype) { return dtype == DT_F32 ? 4 : 2; }

// Row views: element (r, c) of x is element r * x_stride + c of the buffer at `x` (of type
// x_dtype, so `x` is a float pointer only when x_dtype is DT_F32); likewise y.
struct LinearCall {
    DeviceWeights w;
    const float* x;
    float* y;
    int x_dtype = DT_F32;
    int y_dtype = DT_F32;
    int rows;
    long long x_stride;
    long long y_stride;
    float alpha;
    float beta;
    unsigned int* status;  // device word that collects bounded-wait failures (may be null)
};

// Per-device set-up of every kernel in the library (the opt-in to more than 48 KB of dynamic
// shared memory is a function attribute of ONE device).  Runs when a context is created, with
// the context's device current; launches never set attributes.
cudaError_t configure_device();
int device_sm_count();
// Grid of a grid-stride streaming kernel that wants `ctas` CTAs: at most `deep` per SM.
inline int streaming_grid(long long ctas, int deep = 8) {
    const long long cap = (long long)device_sm_count() * deep;
    return (int)(ctas < cap ? (ctas < 1 ? 1 : ctas) : cap);
}

constexpr size_t kAlign = 256;
inline size_t align_up(size_t v, size_t a = kAlign) { return (v + a - 1) / a * a; }

// ---- one-time regrouping of the transport tile order -----------------------------
// src: [I/16][N/16][8*bits] words (transport order), dst: the prepared order above.
cudaError_t launch_regroup(const uint32_t* src, uint32_t* dst, int inputs, int outputs, int bits,
                           cudaStream_t stream);

// ---- stage probes (parity instruments, same device functions as production) -------
cudaError_t launch_dequantize(const DeviceWeights& w, uint16_t* q_out /*[I][N] f16 bits*/,
                              cudaStream_t stream);
cudaError_t launch_input_stages(const DeviceWeights& w, const float* x, long long x_stride, int rows,
                                uint16_t* scaled16, float* hadamard32, uint16_t* core16,
                                cudaStream_t stream);
cudaError_t launch_output_stages(const DeviceWeights& w, const float* core /*[splits][rows][N]*/,
                                 int splits, int rows, float* y, long long y_stride, float alpha,
                                 float beta, cudaStream_t stream);
// Sequential ascending-i fused multiply-add core, one thread per output: reproduces
// the CPU contract's accumulation order bit for bit (products of two binary16 values
// are exact in float32, so fma(a,q,acc) == RN32(acc + RN32(a*q))).
cudaError_t launch_core_exact(const DeviceWeights& w, const uint16_t* core16 /*[rows][I]*/, int rows,
                              float* core_out /*[rows][N]*/, cudaStream_t stream);

// Decode-rate probe: the GEMV's inner loop (decode + mma) on tiles resident in shared memory,
// `iters` passes over two units on `grid` CTAs of 16 warps; clocks[b] = SM clocks of CTA b.
cudaError_t launch_decode_rate(const DeviceWeights& w, int iters, int warps, int grid, float* sink, long long* clocks,
                               cudaStream_t stream);

// ---- decode GEMV, rows 1..8, everything fused ---------------------------------------
struct GemvPlan {
    int grid;            // persistent CTAs (one per SM, fewer for tiny layers)
    int splits;          // typical number of CTAs that share one column block
    int stages;          // shared-memory ring depth
    int act_blocks;      // H128 blocks of core input staged at a time
    size_t smem_bytes;
    size_t counter_bytes;   // reserved area at the start of the workspace (0: the fold needs no counters)
    size_t partial_bytes;   // float [grid][2][rows][128] after the counters
};
GemvPlan plan_gemv(const DeviceWeights& w, int rows, int sm_count);
// `workspace` must be 256-byte aligned and hold counter_bytes + partial_bytes.  The
// counters must be zero when the kernel starts; it leaves them zero.
// Marks every partial-plane word of a GEMV scratch area "empty".  A completed launch leaves
// the area empty again, so this is needed once per scratch area (plans) or before a launch
// on scratch of unknown content (direct calls).
cudaError_t reset_gemv_scratch(void* workspace, const GemvPlan& plan, cudaStream_t stream);
cudaError_t launch_gemv(const LinearCall& call, const GemvPlan& plan, void* workspace,
                        bool programmatic_launch, cudaStream_t stream);

// ---- prefill GEMM (rows > 8): input stage kernel + tcgen05 core with fused epilogue ---
struct GemmPlan {
    size_t act_bytes;       // binary16 [rows_padded][I] core input
    size_t workspace_bytes;
    int tile_m, tile_n;
    int sm_count;
    int k_splits;           // K partitions per output tile (> 1: raw partial accumulators in the workspace)
    bool tensor_core;       // tcgen05 prefill kernel selected (else 8-row GEMV chunks)
};
GemmPlan plan_gemm(const DeviceWeights& w, int rows, int sm_count);
cudaError_t launch_gemm(const LinearCall& call, const GemmPlan& plan, void* workspace,
                        bool programmatic_launch, cudaStream_t stream);

}  // namespace st
