// Regrouping of the transport tile order, and the stage probes: dequantise, input
// stages, output stages and the exact-order core.  The probes run the SAME device
// functions as the fused kernels, so a bit-exact probe pins the production decoder
// and transforms (the approach of the reference harness, docs/GPU_TESTS.md:97-109).
#include "backend.h"
#include "hadamard.cuh"
#include "sync_primitives.cuh"
#include "trellis_decode.cuh"

namespace st {

// ---- regroup: [I/16][N/16][W] -> [N/128][I/16][8][W], W = 8*bits words ------------
__global__ void regroup_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst,
                               int ktiles, int ntiles, int words) {
    // One thread per word; consecutive threads walk consecutive destination words.
    const long long total = (long long)ktiles * ntiles * words;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int word = (int)(i % words);
        long long t = i / words;
        const int sub = (int)(t % 8); t /= 8;
        const int kt = (int)(t % ktiles);
        const int nb = (int)(t / ktiles);
        dst[i] = src[((long long)kt * ntiles + nb * 8 + sub) * words + word];
    }
}

cudaError_t launch_regroup(const uint32_t* src, uint32_t* dst, int inputs, int outputs, int bits,
                           cudaStream_t stream) {
    const int ktiles = inputs / 16, ntiles = outputs / 16, words = tile_words(bits);
    const long long total = (long long)ktiles * ntiles * words;
    const int block = 256;
    const long long want = (total + block - 1) / block;
    const int grid = streaming_grid(want, 16);
    regroup_kernel<<<grid, block, 0, stream>>>(src, dst, ktiles, ntiles, words);
    return cudaGetLastError();
}

__device__ __forceinline__ const uint32_t* tile_ptr(const DeviceWeights& w, int kt, int nt) {
    const int words = tile_words(w.bits), ktiles = w.inputs / 16;
    return w.packed + (((long long)(nt >> 3) * ktiles + kt) * 8 + (nt & 7)) * words;
}

// ---- dequantise: one warp per tile, through decode_tile_frag ------------------------
template <int K, int CB>
__global__ void dequantize_kernel(DeviceWeights w, uint16_t* __restrict__ q) {
    const int lane = threadIdx.x & 31;
    const int ktiles = w.inputs / 16, ntiles = w.outputs / 16;
    const long long tiles = (long long)ktiles * ntiles;
    for (long long t = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); t < tiles;
         t += (long long)gridDim.x * (blockDim.x >> 5)) {
        const int kt = (int)(t / ntiles), nt = (int)(t % ntiles);
        uint32_t frag[4];
        decode_tile_frag<K, CB>(tile_ptr(w, kt, nt), lane, frag);
        // frag order -> stream positions: frag[0]=(0,1) frag[2]=(2,3) frag[1]=(4,5) frag[3]=(6,7)
        const uint32_t by_pos[4] = {frag[0], frag[2], frag[1], frag[3]};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint16_t v = (uint16_t)(by_pos[j >> 1] >> (16 * (j & 1)));
            const int row = kt * 16 + frag_row(lane, j), col = nt * 16 + frag_col(lane, j);
            q[(long long)row * w.outputs + col] = v;
        }
    }
}

template <int CB>
static cudaError_t dequantize_bits(const DeviceWeights& w, uint16_t* q, int grid, cudaStream_t s) {
    switch (w.bits) {
    case 1: dequantize_kernel<1, CB><<<grid, 256, 0, s>>>(w, q); break;
    case 2: dequantize_kernel<2, CB><<<grid, 256, 0, s>>>(w, q); break;
    case 3: dequantize_kernel<3, CB><<<grid, 256, 0, s>>>(w, q); break;
    case 4: dequantize_kernel<4, CB><<<grid, 256, 0, s>>>(w, q); break;
    case 5: dequantize_kernel<5, CB><<<grid, 256, 0, s>>>(w, q); break;
    case 6: dequantize_kernel<6, CB><<<grid, 256, 0, s>>>(w, q); break;
    case 7: dequantize_kernel<7, CB><<<grid, 256, 0, s>>>(w, q); break;
    case 8: dequantize_kernel<8, CB><<<grid, 256, 0, s>>>(w, q); break;
    case 9: case 10: case 11:  // 1.5 / 2.5 / 3.5 bits per weight exist for mul1 only
        if constexpr (CB == CB_MUL1) {
            if (w.bits == 9) dequantize_kernel<9, CB><<<grid, 256, 0, s>>>(w, q);
            else if (w.bits == 10) dequantize_kernel<10, CB><<<grid, 256, 0, s>>>(w, q);
            else dequantize_kernel<11, CB><<<grid, 256, 0, s>>>(w, q);
            break;
        }
        return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_dequantize(const DeviceWeights& w, uint16_t* q, cudaStream_t stream) {
    const long long tiles = (long long)(w.inputs / 16) * (w.outputs / 16);
    const long long want = (tiles + 7) / 8;
    const int grid = streaming_grid(want);
    switch (w.codebook) {
    case CB_3INST: return dequantize_bits<CB_3INST>(w, q, grid, stream);
    case CB_MCG: return dequantize_bits<CB_MCG>(w, q, grid, stream);
    case CB_MUL1: return dequantize_bits<CB_MUL1>(w, q, grid, stream);
    default: return cudaErrorInvalidValue;
    }
}

// ---- input stages: one warp per (row, 128-block) -------------------------------------
__global__ void input_stages_kernel(const float* __restrict__ x, long long x_stride,
                                    const uint16_t* __restrict__ suh, int inputs, int rows,
                                    uint16_t* scaled16, float* had32, uint16_t* core16) {
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = inputs / 128;
    const long long groups = (long long)rows * blocks_per_row;
    for (long long g = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); g < groups;
         g += (long long)gridDim.x * (blockDim.x >> 5)) {
        const int row = (int)(g / blocks_per_row), begin = (int)(g % blocks_per_row) * 128;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = begin + lane + 32 * j;
            const __half h = scale_input(x[(long long)row * x_stride + c], suh[c]);
            if (scaled16) scaled16[(long long)row * inputs + c] = __half_as_ushort(h);
            v[j] = __half2float(h);
        }
        hadamard128_warp(v, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const long long idx = (long long)row * inputs + begin + lane + 32 * j;
            if (had32) had32[idx] = v[j];
            if (core16) core16[idx] = __half_as_ushort(__float2half_rn(v[j]));
        }
    }
}

cudaError_t launch_input_stages(const DeviceWeights& w, const float* x, long long x_stride, int rows,
                                uint16_t* scaled16, float* had32, uint16_t* core16,
                                cudaStream_t stream) {
    const long long groups = (long long)rows * (w.inputs / 128);
    const long long want = (groups + 7) / 8;
    const int grid = streaming_grid(want);
    input_stages_kernel<<<grid, 256, 0, stream>>>(x, x_stride, w.suh, w.inputs, rows, scaled16, had32,
                                                  core16);
    return cudaGetLastError();
}

// ---- output stages: fold split planes ascending from +0, H128, svh, bias, alpha/beta ---
__global__ void output_stages_kernel(const float* __restrict__ core, int splits, int rows,
                                     const uint16_t* __restrict__ svh, const float* __restrict__ bias,
                                     int outputs, float* y, long long y_stride, float alpha, float beta) {
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = outputs / 128;
    const long long groups = (long long)rows * blocks_per_row;
    for (long long g = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); g < groups;
         g += (long long)gridDim.x * (blockDim.x >> 5)) {
        const int row = (int)(g / blocks_per_row), begin = (int)(g % blocks_per_row) * 128;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < splits; ++s)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                v[j] = __fadd_rn(v[j], core[((long long)s * rows + row) * outputs + begin + lane + 32 * j]);
        hadamard128_warp(v, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = begin + lane + 32 * j;
            float* out = y + (long long)row * y_stride + c;
            *out = finish_output(v[j], svh[c], bias, c, alpha, beta, out);
        }
    }
}

cudaError_t launch_output_stages(const DeviceWeights& w, const float* core, int splits, int rows,
                                 float* y, long long y_stride, float alpha, float beta,
                                 cudaStream_t stream) {
    const long long groups = (long long)rows * (w.outputs / 128);
    const long long want = (groups + 7) / 8;
    const int grid = streaming_grid(want);
    output_stages_kernel<<<grid, 256, 0, stream>>>(core, splits, rows, w.svh, w.bias, w.outputs, y,
                                                   y_stride, alpha, beta);
    return cudaGetLastError();
}

// ---- exact-order core: a warp owns a 16-column tile band and walks K ascending ---------
// Lane t accumulates output column (t%16) for rows (t/16), (t/16)+2, ...; each k-tile is
// decoded once by the warp, transposed through shared memory, then consumed in ascending
// input order with one fma per (row, input).
template <int K, int CB>
__global__ void core_exact_kernel(DeviceWeights w, const uint16_t* __restrict__ a16, int rows,
                                  float* __restrict__ core) {
    __shared__ uint16_t tile[8][16][16];  // [warp][input row][output col]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nt = blockIdx.x * 8 + warp;
    if (nt >= w.outputs / 16) return;
    const int col = lane & 15, row0 = lane >> 4;
    float acc[32];  // rows row0, row0+2, ... (up to 64 rows)
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = 0.f;
    for (int kt = 0; kt < w.inputs / 16; ++kt) {
        uint32_t frag[4];
        decode_tile_frag<K, CB>(tile_ptr(w, kt, nt), lane, frag);
        const uint32_t by_pos[4] = {frag[0], frag[2], frag[1], frag[3]};
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
            tile[warp][frag_row(lane, j)][frag_col(lane, j)] = (uint16_t)(by_pos[j >> 1] >> (16 * (j & 1)));
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const int r = row0 + 2 * i;
            if (r < rows) {
                for (int k = 0; k < 16; ++k) {
                    const float a = half_bits_to_float(a16[(long long)r * w.inputs + kt * 16 + k]);
                    acc[i] = __fmaf_rn(a, half_bits_to_float(tile[warp][k][col]), acc[i]);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const int r = row0 + 2 * i;
        if (r < rows) core[(long long)r * w.outputs + nt * 16 + col] = acc[i];
    }
}

template <int CB>
static cudaError_t core_exact_bits(const DeviceWeights& w, const uint16_t* a, int rows, float* c,
                                   cudaStream_t s) {
    const int grid = (w.outputs / 16 + 7) / 8;
    switch (w.bits) {
    case 1: core_exact_kernel<1, CB><<<grid, 256, 0, s>>>(w, a, rows, c); break;
    case 2: core_exact_kernel<2, CB><<<grid, 256, 0, s>>>(w, a, rows, c); break;
    case 3: core_exact_kernel<3, CB><<<grid, 256, 0, s>>>(w, a, rows, c); break;
    case 4: core_exact_kernel<4, CB><<<grid, 256, 0, s>>>(w, a, rows, c); break;
    case 5: core_exact_kernel<5, CB><<<grid, 256, 0, s>>>(w, a, rows, c); break;
    case 6: core_exact_kernel<6, CB><<<grid, 256, 0, s>>>(w, a, rows, c); break;
    case 7: core_exact_kernel<7, CB><<<grid, 256, 0, s>>>(w, a, rows, c); break;
    case 8: core_exact_kernel<8, CB><<<grid, 256, 0, s>>>(w, a, rows, c); break;
    case 9: case 10: case 11:  // 1.5 / 2.5 / 3.5 bits per weight exist for mul1 only
        if constexpr (CB == CB_MUL1) {
            if (w.bits == 9) core_exact_kernel<9, CB><<<grid, 256, 0, s>>>(w, a, rows, c);
            else if (w.bits == 10) core_exact_kernel<10, CB><<<grid, 256, 0, s>>>(w, a, rows, c);
            else core_exact_kernel<11, CB><<<grid, 256, 0, s>>>(w, a, rows, c);
            break;
        }
        return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// ---- decode-rate probe ---------------------------------------------------------------------
// The inner loop of the fused GEMV with nothing around it: two units of the layer's weights sit
// in shared memory, 4 to 32 warps per SM (column tile = warp % 8; the fused GEMV runs sixteen)
// decode them `iters` times with the production device function and feed every tile to the same
// mma as the GEMV.  No global traffic, no barriers, no fold: the clocks per tile measured here
// are the instruction-issue cost of the decoder itself, i.e. the ceiling of every kernel that
// decodes (what the reference measured with modes 0-4 of src/microbench.hip for its own decoder).
namespace {
constexpr int kProbeMaxWarps = 32;
constexpr int kProbeUnits = 2;
}
// kWarps = 16 compiles under the fused GEMV's own thread count (and register room), 32 under
// the device's maximum.
template <int K, int CB, int kWarps>
__global__ void __launch_bounds__(kWarps * 32) decode_rate_kernel(const DeviceWeights w, int iters, float* sink,
                                                                       long long* clocks) {
    extern __shared__ uint32_t probe_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int kUnitWords = unit_bytes(K) / 4;
    const long long have = (long long)w.inputs * w.outputs / 256 * tile_words(K);  // words in the packed stream
    for (int i = threadIdx.x; i < kProbeUnits * kUnitWords; i += blockDim.x) probe_smem[i] = w.packed[i % have];
    __syncthreads();
    const LaneGeom<K> geom(lane);
    const uint32_t b0 = 0x3C003C00u, b1 = 0x3C003800u;  // fixed activation fragments
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
        const uint32_t* tiles = probe_smem + (it & (kProbeUnits - 1)) * kUnitWords + (warp & 7) * tile_words(K);
#pragma unroll
        for (int kt = 0; kt < 8; kt += 2) {
            uint32_t fa[4], fb[4];
            decode_tile_frag<K, CB>(tiles + kt * 8 * tile_words(K), geom, fa);
            decode_tile_frag<K, CB>(tiles + (kt + 1) * 8 * tile_words(K), geom, fb);
            mma_16816(acc[0], fa, b0, b1);
            mma_16816(acc[1], fb, b0, b1);
        }
    }
    const long long t1 = clock64();
    sink[blockIdx.x * blockDim.x + threadIdx.x] =
        acc[0][0] + acc[0][1] + acc[0][2] + acc[0][3] + acc[1][0] + acc[1][1] + acc[1][2] + acc[1][3];
    if (threadIdx.x == 0) clocks[blockIdx.x] = t1 - t0;
}

template <int K, int CB>
static void probe_launch(const DeviceWeights& w, int iters, int warps, float* sink, long long* clocks, int grid, size_t smem,
                         cudaStream_t s) {
    if (warps <= 16) decode_rate_kernel<K, CB, 16><<<grid, warps * 32, smem, s>>>(w, iters, sink, clocks);
    else decode_rate_kernel<K, CB, kProbeMaxWarps><<<grid, warps * 32, smem, s>>>(w, iters, sink, clocks);
}

template <int CB>
static cudaError_t decode_rate_bits(const DeviceWeights& w, int iters, int warps, float* sink, long long* clocks, int grid,
                                    cudaStream_t s) {
    const size_t smem = (size_t)kProbeUnits * unit_bytes(w.bits);
    switch (w.bits) {
    case 1: probe_launch<1, CB>(w, iters, warps, sink, clocks, grid, smem, s); break;
    case 2: probe_launch<2, CB>(w, iters, warps, sink, clocks, grid, smem, s); break;
    case 3: probe_launch<3, CB>(w, iters, warps, sink, clocks, grid, smem, s); break;
    case 4: probe_launch<4, CB>(w, iters, warps, sink, clocks, grid, smem, s); break;
    case 5: probe_launch<5, CB>(w, iters, warps, sink, clocks, grid, smem, s); break;
    case 6: probe_launch<6, CB>(w, iters, warps, sink, clocks, grid, smem, s); break;
    case 7: probe_launch<7, CB>(w, iters, warps, sink, clocks, grid, smem, s); break;
    case 8: probe_launch<8, CB>(w, iters, warps, sink, clocks, grid, smem, s); break;
    case 9: case 10: case 11:
        if constexpr (CB == CB_MUL1) {
            if (w.bits == 9) probe_launch<9, CB>(w, iters, warps, sink, clocks, grid, smem, s);
            else if (w.bits == 10) probe_launch<10, CB>(w, iters, warps, sink, clocks, grid, smem, s);
            else probe_launch<11, CB>(w, iters, warps, sink, clocks, grid, smem, s);
            break;
        }
        return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

// sink: grid * warps * 32 floats, clocks: grid int64 (device memory); clocks[b] = SM clocks CTA b spent in the loop
cudaError_t launch_decode_rate(const DeviceWeights& w, int iters, int warps, int grid, float* sink, long long* clocks,
                               cudaStream_t stream) {
    if (iters < 1 || grid < 1 || warps < 4 || warps > kProbeMaxWarps || warps % 4) return cudaErrorInvalidValue;
    switch (w.codebook) {
    case CB_3INST: return decode_rate_bits<CB_3INST>(w, iters, warps, sink, clocks, grid, stream);
    case CB_MCG: return decode_rate_bits<CB_MCG>(w, iters, warps, sink, clocks, grid, stream);
    case CB_MUL1: return decode_rate_bits<CB_MUL1>(w, iters, warps, sink, clocks, grid, stream);
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_core_exact(const DeviceWeights& w, const uint16_t* core16, int rows, float* core_out,
                              cudaStream_t stream) {
    if (rows < 1 || rows > 64) return cudaErrorInvalidValue;
    switch (w.codebook) {
    case CB_3INST: return core_exact_bits<CB_3INST>(w, core16, rows, core_out, stream);
    case CB_MCG: return core_exact_bits<CB_MCG>(w, core16, rows, core_out, stream);
    case CB_MUL1: return core_exact_bits<CB_MUL1>(w, core16, rows, core_out, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace st
