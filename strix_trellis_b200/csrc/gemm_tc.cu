// Prefill GEMM (rows > 8) on the 5th-generation tensor cores: tcgen05.mma with fp32
// accumulators in tensor memory, trellis tiles decoded on the fly by producer warps
// into the swizzled K-major shared-memory layout the MMA reads, and the output stages
// (H128, svh, bias, alpha/beta) fused into the epilogue.  It stands in for the reference's
// input_transform + wmma tiled core + fused output epilogue (src/wmma_tiled.hip:87-269,
// src/gemm.hip:15-76, src/backend.hip:121-140).
//
// Launches: (1) input stages, writing the RN16 core input as pre-swizzled
// [128 rows x 64 k] tiles so that each tile is ONE contiguous 16 KB bulk copy;
// (2) the persistent GEMM kernel, one CTA per SM, launched programmatically after (1);
// (3) with one row tile only: K is cut into partitions so that every SM has work, and a
// finishing kernel folds their raw accumulators.  CTA tile = 256 rows x 256 columns as
// 2 x (128 x 256) accumulators = all 512 TMEM columns: every decoded weight stage feeds
// 256 rows and every activation tile feeds 256 columns.  K is stepped by 64.
//   warp 0      A producer  : cp.async.bulk of the A tiles of a stage; L2 prefetch of the
//                             CTA's weight words eight K steps ahead
//   warp 1      MMA issuer  : tcgen05.mma (one thread), tcgen05.commit to the barriers
//   warps 2-5   epilogue    : tcgen05.ld -> shared staging -> H128 by warp shuffles -> y
//   warps 6-21  decoders    : one warp per 16-column tile, 4 k-tiles per stage, the ring
//                             words of the next two stages in registers; on the CTA's last
//                             work item they share the epilogue
// Every wait is bounded and reports into the device status word.
#include <cstdlib>

#include "backend.h"
#include "hadamard.cuh"
#include "sync_primitives.cuh"
#include "tcgen05.cuh"
#include "trellis_decode.cuh"

namespace st {

namespace {
constexpr int kBM = 128, kMT = 2, kBN = 256, kBK = 64;
constexpr int kStagesTc = 3;
constexpr int kTileBytes = kBM * kBK * 2;                      // 16 KB: 128 rows x 64 binary16
constexpr int kStageBytesTc = (kMT + kBN / 128) * kTileBytes;  // A0, A1, B (256 rows)
constexpr int kDecodeWarps = 16, kEpiWarps = 4;                // one decode warp per column tile
constexpr int kThreadsTc = (2 + kEpiWarps + kDecodeWarps) * 32;
constexpr int kStagingStride = 129;                            // floats per staged row
constexpr int kStagingBytes = 16 * kStagingStride * 4;         // per epilogue warp, 16 rows at a time
constexpr size_t kSmemTc = 1024 + (size_t)kStagesTc * kStageBytesTc + (size_t)kEpiWarps * kStagingBytes + 128;
constexpr uint32_t kTmemCols = 512;
constexpr int kChunkedMaxRows = 16;  // more rows than this take the tensor-core route
constexpr int kWeightsAhead = 8;  // K steps between the L2 prefetch of weight words and their use
static_assert((size_t)kDecodeWarps * kStagingBytes <= (size_t)kStagesTc * kStageBytesTc,
              "the decoder warps' staging areas of the last work item must fit the idle ring");

struct GemmArgs {
    LinearCall call;
    const unsigned char* a_tiles;  // [M/128 padded][I/64][16 KB]
    int m_pairs;                   // ceil(rows / 256)
    int n_pairs;                   // ceil(column blocks / 2)
    int k_splits;                  // K partitions per tile (1 = the epilogue finishes the outputs)
    float* partials;               // [k_splits][rows padded to 256][N] raw accumulators when k_splits > 1
};
}  // namespace

// ---- launch 1: input stages into pre-swizzled A tiles ------------------------------------
__global__ void input_tiles_kernel(const float* __restrict__ x, int x_dtype, long long x_stride,
                                   const uint16_t* __restrict__ suh, int inputs, int rows, int rows_padded,
                                   unsigned char* __restrict__ a_tiles) {
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = inputs / 128, kt64 = inputs / 64;
    const long long groups = (long long)rows_padded * blocks_per_row;
    pdl_launch_dependents();  // the GEMM may set itself up and decode its first weights meanwhile
    for (long long g = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); g < groups;
         g += (long long)gridDim.x * (blockDim.x >> 5)) {
        const int row = (int)(g / blocks_per_row), blk = (int)(g % blocks_per_row);
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (row < rows) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = blk * 128 + lane + 32 * j;
                v[j] = __half2float(scale_input(load_element(x, x_dtype, (long long)row * x_stride + c), suh[c]));
            }
            hadamard128_warp(v, lane);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = blk * 128 + lane + 32 * j;  // input index
            unsigned char* tile = a_tiles + ((size_t)(row >> 7) * kt64 + (k >> 6)) * kTileBytes;
            *reinterpret_cast<__half*>(tile + sw128_offset(row & 127, k & 63)) = __float2half_rn(v[j]);
        }
    }
}

// ---- launch 2: the GEMM ---------------------------------------------------------------------
template <int K, int CB>
__global__ void __launch_bounds__(kThreadsTc, 1) gemm_tc_kernel(const GemmArgs args) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const LinearCall& c = args.call;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kt64 = c.w.inputs / 64, ktiles16 = c.w.inputs / 16;
    const int nblocks = c.w.outputs / 128;
    // tiles ordered with the row pair fastest: CTAs that run together share a weight stripe
    // work item = (tile, K partition); partitions of a tile are neighbours in the order
    const int splits = args.k_splits;
    const int tiles = args.n_pairs * args.m_pairs * splits;
    const int my_tiles = tiles > (int)blockIdx.x ? (tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    // accumulators (128-row halves) of row tile mp that hold any of the call's rows: the last row
    // tile of a call may need only the first, and then nothing is loaded, multiplied or read back
    // for the second
    auto live_mt = [&](int mp) {
        const int left = c.rows - mp * (kBM * kMT);
        return left > kBM ? kMT : 1;
    };
    auto k_begin_of = [&](int t) { return kt64 * (t % splits) / splits; };
    auto k_end_of = [&](int t) { return kt64 * (t % splits + 1) / splits; };

    unsigned char* ring = smem;
    float* staging = reinterpret_cast<float*>(ring + (size_t)kStagesTc * kStageBytesTc);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(staging) +
                                                 (size_t)kEpiWarps * kStagingBytes);
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    const uint32_t full = smem_u32(bars), empty = smem_u32(bars + kStagesTc), tmem_full = smem_u32(bars + 2 * kStagesTc),
                   tmem_empty = smem_u32(bars + 2 * kStagesTc + 1);

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStagesTc; ++i) {
            // ONE barrier per stage for everything the MMA warp waits for: the activation copies (one
            // arrival + bytes) and the sixteen decoders
            mbar_init(full + 8 * i, 1 + kDecodeWarps);
            mbar_init(empty + 8 * i, 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, kEpiWarps);
        mbar_fence_init();
        s_abort = 0;
    }
    if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = s_tmem_base;
    pdl_launch_dependents();

    // One half-item of the epilogue of work item t: 16 rows x 128 columns of one accumulator leave
    // tensor memory through `stage` (16 x 129 floats of the calling warp); a K partition stores
    // them raw for splitk_finish_kernel, a whole tile gets H128, output signs, bias, alpha/beta.
    // item = accumulator * 4 + column block * 2 + half.
    auto epilogue_half = [&](int t, int item, int quarter, float* stage) {
        const int np = (t / splits) / args.m_pairs, mp = (t / splits) % args.m_pairs;
        const int mt = item >> 2, cb = (item >> 1) & 1, half = item & 1;
        const int nb = np * (kBN / 128) + cb;
        if (mt >= live_mt(mp) || nb >= nblocks) return;  // no rows of the call / padding column block
        float* raw = splits > 1 ? args.partials + (size_t)(t % splits) * args.m_pairs * (kBM * kMT) * c.w.outputs : nullptr;
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + mt * kBN + cb * 128;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + ch * 32, r);
            tmem_ld_wait();
            if ((lane >> 4) == half) {
#pragma unroll
                for (int j = 0; j < 32; ++j) stage[(lane & 15) * kStagingStride + ch * 32 + j] = __uint_as_float(r[j]);
            }
        }
        __syncwarp();
        const int row_base = (mp * kMT + mt) * kBM + quarter * 32 + half * 16;
        if (raw) {
            for (int r1 = 0; r1 < 16; ++r1) {
                const int row = row_base + r1;
                if (row < c.rows) {
                    float* out = raw + (size_t)row * c.w.outputs + nb * 128 + lane;
#pragma unroll
                    for (int j = 0; j < 4; ++j) out[32 * j] = stage[r1 * kStagingStride + lane + 32 * j];
                }
            }
        } else {
            float sv[4], bi[4];  // per-column constants of this lane's four columns
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int cidx = nb * 128 + lane + 32 * j;
                sv[j] = half_bits_to_float(c.w.svh[cidx]);
                bi[j] = c.w.bias ? c.w.bias[cidx] : 0.f;
            }
            for (int r4 = 0; r4 < 16; r4 += 4) {  // four independent rows in flight
                float v[4][4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[u][j] = stage[(r4 + u) * kStagingStride + lane + 32 * j];
#pragma unroll
                for (int u = 0; u < 4; ++u) hadamard128_warp(v[u], lane);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int row = row_base + r4 + u;
                    if (row < c.rows) {
                        const long long out = (long long)row * c.y_stride + nb * 128 + lane;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float value = __fmul_rn(v[u][j], sv[j]);
                            if (c.w.bias) value = __fadd_rn(value, bi[j]);
                            scale_and_store(c.y, c.y_dtype, out + 32 * j, value, c.alpha, c.beta);
                        }
                    }
                }
            }
        }
        __syncwarp();
    };

    if (warp == 0) {
        // ---- A producer ---------------------------------------------------------------
        if (lane == 0) {
            // The decoders read their words straight from global memory, one K step ahead: with
            // weights that no other CTA has touched that is a DRAM round trip per K step.  This
            // thread asks the L2 for the CTA's words kWeightsAhead K steps before they are read
            // (a K step of one 128-column block is one contiguous run of the stream).
            constexpr uint32_t kStepBytes = 4 * 8 * tile_words(K) * 4;
            int plt = -1, pks = 0, pke = 0;
            const unsigned char* pbase[kBN / 128] = {};
            auto prefetch_step = [&]() {
                while (pks == pke) {  // next work item of this CTA
                    if (++plt >= my_tiles) return;
                    const int t = (int)blockIdx.x + plt * (int)gridDim.x;
                    pks = k_begin_of(t);
                    pke = k_end_of(t);
                    for (int cb = 0; cb < kBN / 128; ++cb) {
                        const int nb = ((t / splits) / args.m_pairs) * (kBN / 128) + cb;
                        pbase[cb] = nb < nblocks ? reinterpret_cast<const unsigned char*>(
                                                       c.w.packed + (size_t)nb * ktiles16 * 8 * tile_words(K))
                                                 : nullptr;
                    }
                }
                for (int cb = 0; cb < kBN / 128; ++cb)
                    if (pbase[cb]) bulk_prefetch_l2(pbase[cb] + (size_t)pks * kStepBytes, kStepBytes);
                ++pks;
            };
            for (int i = 0; i < kWeightsAhead; ++i) prefetch_step();
            // Launched programmatically after input_tiles_kernel: everything up to here, and the
            // decoders' first stages (weights are immutable), overlap its tail; only the
            // activation tiles need its memory.  Everything older than that kernel was complete
            // before it started.
            pdl_wait_prior_grid();
            int it = 0;
            for (int lt = 0; lt < my_tiles && !s_abort; ++lt) {
                const int t = (int)blockIdx.x + lt * (int)gridDim.x;
                const int mp = (t / splits) % args.m_pairs;
                const int live = live_mt(mp);
                for (int ks = k_begin_of(t), ke = k_end_of(t); ks < ke; ++ks, ++it) {
                    const int st = it % kStagesTc;
                    if (it >= kStagesTc &&
                        !mbar_wait(empty + 8 * st, (uint32_t)((it / kStagesTc) - 1) & 1, c.status, kTimeoutTensorPipe)) {
                        s_abort = 1;
                        break;
                    }
                    unsigned char* dst = ring + (size_t)st * kStageBytesTc;
                    mbar_expect_tx(full + 8 * st, live * kTileBytes);
                    for (int mt = 0; mt < live; ++mt)
                        bulk_load(smem_u32(dst + mt * kTileBytes),
                                  args.a_tiles + ((size_t)(mp * kMT + mt) * kt64 + ks) * kTileBytes, kTileBytes,
                                  full + 8 * st);
                    prefetch_step();
                }
            }
            // Never leave with a copy still landing in this CTA's shared memory.
            for (int i = (it > kStagesTc ? it - kStagesTc : 0); i < it; ++i)
                mbar_wait(full + 8 * (i % kStagesTc), (uint32_t)(i / kStagesTc) & 1, c.status, kTimeoutDrain);
        }
    } else if (warp == 1) {
        // ---- MMA issuer ---------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16_f32(kBM, kBN);
            int it = 0;
            for (int lt = 0; lt < my_tiles && !s_abort; ++lt) {
                if (lt >= 1 && !mbar_wait(tmem_empty, (uint32_t)(lt - 1) & 1, c.status, kTimeoutTensorPipe)) {
                    s_abort = 1;
                    break;
                }
                tc_fence_after_sync();
                const int t = (int)blockIdx.x + lt * (int)gridDim.x;
                const int kb = k_begin_of(t);
                const int live = live_mt((t / splits) % args.m_pairs);
                for (int ks = kb, ke = k_end_of(t); ks < ke && !s_abort; ++ks, ++it) {
                    const int st = it % kStagesTc;
                    const uint32_t par = (uint32_t)(it / kStagesTc) & 1;
                    if (!mbar_wait(full + 8 * st, par, c.status, kTimeoutTensorPipe)) {
                        s_abort = 1;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t base = smem_u32(ring + (size_t)st * kStageBytesTc);
                    const uint64_t bdesc = umma_desc_k_major_sw128(base + kMT * kTileBytes);
                    for (int mt = 0; mt < live; ++mt) {
                        const uint64_t adesc = umma_desc_k_major_sw128(base + mt * kTileBytes);
#pragma unroll
                        for (int k4 = 0; k4 < kBK / 16; ++k4)  // +32 bytes per 16-element K step
                            umma_f16(tmem_base + mt * kBN, adesc + 2 * k4, bdesc + 2 * k4, idesc, ks != kb || k4 != 0);
                    }
                    umma_commit(empty + 8 * st);  // stage reusable once these MMAs have read it
                }
                umma_commit(tmem_full);  // accumulators of this tile complete
            }
        }
    } else if (warp < 2 + kEpiWarps) {
        // ---- epilogue -------------------------------------------------------------------
        // A lane quarter's work on a tile is eight half-items (accumulator, column block, 16-row
        // half): its one epilogue warp takes them all, except on the CTA's LAST work item, where
        // the four decoder warps of the quarter, idle by then, take a share.
        const int quarter = warp & 3;  // TMEM lanes this warp may read: 32*quarter .. +31
        float* stage = staging + (size_t)(warp - 2) * 16 * kStagingStride;
        for (int lt = 0; lt < my_tiles; ++lt) {
            const int t = (int)blockIdx.x + lt * (int)gridDim.x;
            if (s_abort || !mbar_wait(tmem_full, (uint32_t)lt & 1, c.status, kTimeoutTensorPipe)) {
                s_abort = 1;
                break;
            }
            tc_fence_after_sync();
            if (lt + 1 < my_tiles) {
                for (int item = 0; item < 8; ++item) epilogue_half(t, item, quarter, stage);
                // all four accumulators read: hand tensor memory back to the MMA warp
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_empty);
            } else {
                for (int item = 0; item < 8; item += 5) epilogue_half(t, item, quarter, stage);
                tc_fence_before_sync();
            }
        }
    } else {
        // ---- decoders: trellis tiles -> swizzled K-major B stage -------------------------------
        const int d = warp - (2 + kEpiWarps);  // column tile 0..15 of the 256-column stripe
        const int cb = d >> 3, ct = d & 7;
        const LaneGeom<K> geom(lane);
        const int n0 = d * 16 + (lane >> 2), kq = 2 * (lane & 3);
        const uint32_t o00 = sw128_offset(n0, kq), o01 = sw128_offset(n0, kq + 8);
        const uint32_t o10 = sw128_offset(n0 + 8, kq), o11 = sw128_offset(n0 + 8, kq + 8);
        int iters = 0;
        for (int lt = 0; lt < my_tiles; ++lt) {
            const int t = (int)blockIdx.x + lt * (int)gridDim.x;
            iters += k_end_of(t) - k_begin_of(t);
        }
        // (work item, K step) whose ring words are fetched next
        int flt = 0, fks = 0, fetched = 0;
        const uint32_t* fcol = nullptr;
        bool fvalid = false;
        int fke = 0;  // end of the K range of the work item being fetched
        auto fetch = [&](uint32_t (&w)[4][3]) {
            if (fcol && fks == fke) { ++flt; fcol = nullptr; }
            if (!fcol) {
                const int t = (int)blockIdx.x + flt * (int)gridDim.x;
                fks = k_begin_of(t);
                fke = k_end_of(t);
                const int nb = ((t / splits) / args.m_pairs) * (kBN / 128) + cb;
                fvalid = nb < nblocks;  // a padding stripe decodes nothing
                fcol = c.w.packed + (((size_t)(fvalid ? nb : 0) * ktiles16) * 8 + ct) * tile_words(K);
            }
            const uint32_t* tile = fcol + (size_t)fks * 4 * 8 * tile_words(K);
            if (fvalid) {
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) load_window<K>(tile + (size_t)k4 * 8 * tile_words(K), geom, w[k4]);
            }
            ++fks;
            ++fetched;
        };
        uint32_t cur[4][3] = {}, nxt[4][3] = {}, far[4][3] = {};  // this K step and the next two, in flight
        if (iters > 0) fetch(cur);
        if (iters > 1) fetch(nxt);
        for (int it = 0; it < iters && !s_abort; ++it) {
            const int st = it % kStagesTc;
            if (fetched < iters) fetch(far);  // two K steps ahead: one decode time does not cover an L2 round trip
            if (it >= kStagesTc &&
                !mbar_wait(empty + 8 * st, (uint32_t)((it / kStagesTc) - 1) & 1, c.status, kTimeoutTensorPipe)) {
                s_abort = 1;
                break;
            }
            unsigned char* bt = ring + (size_t)st * kStageBytesTc + kMT * kTileBytes;
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
                uint32_t frag[4];
                decode_words_frag<K, CB>(cur[k4], geom, frag);
                // a K step of 16 elements is two 16-byte chunks: the swizzle XORs the chunk index
                // with the row, so stepping k4 toggles bits 5..6 of the byte offset
                const uint32_t kx = (uint32_t)(k4 * 2) << 4;
                // frag[0]: (n0, k..k+1)  frag[2]: (n0, k+8..)  frag[1]: (n0+8, k..)  frag[3]: (n0+8, k+8..)
                *reinterpret_cast<uint32_t*>(bt + (o00 ^ kx)) = frag[0];
                *reinterpret_cast<uint32_t*>(bt + (o01 ^ kx)) = frag[2];
                *reinterpret_cast<uint32_t*>(bt + (o10 ^ kx)) = frag[1];
                *reinterpret_cast<uint32_t*>(bt + (o11 ^ kx)) = frag[3];
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(full + 8 * st);
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4)
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    cur[k4][j] = nxt[k4][j];
                    nxt[k4][j] = far[k4][j];
                }
        }
        // The CTA's last work item: the ring is idle for good once its MMAs have completed, so
        // this warp takes a staging area there and a share of its lane quarter's epilogue.
        if (my_tiles > 0 && !s_abort && mbar_wait(tmem_full, (uint32_t)(my_tiles - 1) & 1, c.status, kTimeoutTensorPipe)) {
            tc_fence_after_sync();
            float* stage = reinterpret_cast<float*>(ring) + (size_t)d * 16 * kStagingStride;
            const int t = (int)blockIdx.x + (my_tiles - 1) * (int)gridDim.x;
            for (int item = 1 + (d >> 2); item < 8; item += 5) epilogue_half(t, item, warp & 3, stage);
            tc_fence_before_sync();
        }
    }

    // ---- common exit: nobody leaves before every role is done, then TMEM is returned ------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- launch 3 (only with K partitions): fold the raw partial accumulators in ascending K
// order from +0 and apply the output stages; one warp per (row, 128-column block) ------------
__global__ void splitk_finish_kernel(const float* __restrict__ partials, int splits, size_t plane, int rows,
                                     int outputs, const uint16_t* __restrict__ svh, const float* __restrict__ bias,
                                     float alpha, float beta, float* y, int y_dtype, long long y_stride) {
    const int lane = threadIdx.x & 31;
    const int nblocks = outputs / 128;
    const long long items = (long long)rows * nblocks;
    pdl_wait_prior_grid();  // the partial accumulators belong to the GEMM before this launch
    for (long long g = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5); g < items;
         g += (long long)gridDim.x * (blockDim.x >> 5)) {
        const int row = (int)(g / nblocks), nb = (int)(g % nblocks);
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < splits; ++s) {
            const float* src = partials + (size_t)s * plane + (size_t)row * outputs + nb * 128 + lane;
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = __fadd_rn(v[j], src[32 * j]);
        }
        hadamard128_warp(v, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cidx = nb * 128 + lane + 32 * j;
            float value = __fmul_rn(v[j], half_bits_to_float(svh[cidx]));
            if (bias) value = __fadd_rn(value, bias[cidx]);
            scale_and_store(y, y_dtype, (long long)row * y_stride + cidx, value, alpha, beta);
        }
    }
}

// ---- host side ---------------------------------------------------------------------------------
GemmPlan plan_gemm_chunked(const DeviceWeights& w, int rows, int sm_count);
cudaError_t launch_gemm_chunked(const LinearCall& call, int sm_count, void* workspace, bool programmatic_launch,
                                cudaStream_t stream);

// gemm_tc_pair.cu: two CTAs per 512 x 256 tile
int gemm_pair_rows_padded(int rows);
cudaError_t launch_gemm_pair(const LinearCall& call, const unsigned char* a_tiles, int sm_count, cudaStream_t stream);

GemmPlan plan_gemm(const DeviceWeights& w, int rows, int sm_count) {
    // Up to two 8-row chunks of the fused GEMV are faster than the three launches of the
    // tensor-core route (measured on cold weights, K4: 4096 -> 12288 45 against 39 us at 16 rows,
    // but 4096 -> 4096 23 against 31 and 14336 -> 4096 52 against 74); from 17 rows on the
    // tensor-core route wins or ties on every benchmark shape.
    if (rows <= kChunkedMaxRows) return plan_gemm_chunked(w, rows, sm_count);
    GemmPlan plan{};
    const bool pair = rows > kBM * kMT && sm_count >= 2;
    const int rows_padded = pair ? gemm_pair_rows_padded(rows) : (rows + kBM * kMT - 1) / (kBM * kMT) * (kBM * kMT);
    plan.act_bytes = (size_t)rows_padded * w.inputs * 2;
    plan.workspace_bytes = align_up(plan.act_bytes);
    plan.tile_m = pair ? 2 * kBM * kMT : kBM * kMT;
    // One row tile leaves most SMs without a column tile: partition K so that every SM has work.
    plan.k_splits = 1;
    if (!pair && rows_padded == kBM * kMT) {
        const int n_pairs = (w.outputs / 128 + kBN / 128 - 1) / (kBN / 128);
        int splits = sm_count / n_pairs;
        if (splits > 4) splits = 4;
        while (splits > 1 && (w.inputs / kBK) / splits < 8) --splits;  // at least eight K steps per partition
        if (splits > 1) {
            plan.k_splits = splits;
            plan.workspace_bytes += align_up((size_t)splits * rows_padded * w.outputs * sizeof(float));
        }
    }
    plan.tile_n = kBN;
    plan.sm_count = sm_count;
    plan.tensor_core = true;
    return plan;
}

template <int K, int CB>
static cudaError_t launch_tc(const GemmArgs& args, int grid, bool programmatic, cudaStream_t stream) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreadsTc);
    cfg.dynamicSmemBytes = kSmemTc;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<K, CB>, args);
}

// Opt-in dynamic shared memory is a per-device function attribute: set for every instantiation
// when a context is created on a device (configure_device), never on the launch path.
template <int CB>
static cudaError_t configure_gemm_tc_kernels_codebook() {
    cudaError_t e = cudaSuccess;
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<1, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTc);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<2, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTc);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<3, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTc);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<4, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTc);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<5, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTc);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<6, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTc);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<7, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTc);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<8, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTc);
    if constexpr (CB == CB_MUL1) {
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<9, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTc);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<10, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTc);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_kernel<11, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemTc);
    }
    return e;
}
cudaError_t configure_gemm_tc_kernels() {
    cudaError_t e = configure_gemm_tc_kernels_codebook<CB_3INST>();
    if (e == cudaSuccess) e = configure_gemm_tc_kernels_codebook<CB_MCG>();
    if (e == cudaSuccess) e = configure_gemm_tc_kernels_codebook<CB_MUL1>();
    return e;
}

template <int CB>
static cudaError_t launch_tc_bits(const GemmArgs& a, int grid, bool programmatic, cudaStream_t s) {
    switch (a.call.w.bits) {
    case 1: return launch_tc<1, CB>(a, grid, programmatic, s);
    case 2: return launch_tc<2, CB>(a, grid, programmatic, s);
    case 3: return launch_tc<3, CB>(a, grid, programmatic, s);
    case 4: return launch_tc<4, CB>(a, grid, programmatic, s);
    case 5: return launch_tc<5, CB>(a, grid, programmatic, s);
    case 6: return launch_tc<6, CB>(a, grid, programmatic, s);
    case 7: return launch_tc<7, CB>(a, grid, programmatic, s);
    case 8: return launch_tc<8, CB>(a, grid, programmatic, s);
    case 9: case 10: case 11:  // 1.5 / 2.5 / 3.5 bits per weight exist for mul1 only
        if constexpr (CB == CB_MUL1) {
            if (a.call.w.bits == 9) return launch_tc<9, CB>(a, grid, programmatic, s);
            if (a.call.w.bits == 10) return launch_tc<10, CB>(a, grid, programmatic, s);
            return launch_tc<11, CB>(a, grid, programmatic, s);
        }
        return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_gemm(const LinearCall& call, const GemmPlan& plan, void* workspace, bool programmatic_launch,
                        cudaStream_t stream) {
    // The 8-row chunks launch programmatically after whatever precedes them in the stream.  The
    // tensor-core route starts with an ordinary launch (input_tiles_kernel) and chains its own
    // later launches to it programmatically.
    if (!plan.tensor_core) return launch_gemm_chunked(call, plan.sm_count, workspace, programmatic_launch, stream);
    if (!workspace) return cudaErrorInvalidValue;
    const bool pair = plan.tile_m == 2 * kBM * kMT;
    const int m_pairs = (call.rows + kBM * kMT - 1) / (kBM * kMT);
    const int rows_padded = pair ? gemm_pair_rows_padded(call.rows) : m_pairs * kBM * kMT;
    {
        const long long groups = (long long)rows_padded * (call.w.inputs / 128);
        const long long want = (groups + 7) / 8;
        const int grid = streaming_grid(want);
        input_tiles_kernel<<<grid, 256, 0, stream>>>(call.x, call.x_dtype, call.x_stride, call.w.suh, call.w.inputs, call.rows,
                                                     rows_padded, static_cast<unsigned char*>(workspace));
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    if (pair) return launch_gemm_pair(call, static_cast<const unsigned char*>(workspace), plan.sm_count, stream);
    GemmArgs args{};
    args.call = call;
    args.a_tiles = static_cast<const unsigned char*>(workspace);
    args.m_pairs = m_pairs;
    args.n_pairs = (call.w.outputs / 128 + kBN / 128 - 1) / (kBN / 128);
    args.k_splits = plan.k_splits;
    args.partials = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + align_up(plan.act_bytes));
    const long long tiles = (long long)args.n_pairs * m_pairs * plan.k_splits;
    if (tiles > 0x3FFFFFFF) return cudaErrorInvalidValue;
    const int grid = (int)(tiles < plan.sm_count ? tiles : plan.sm_count);
    cudaError_t e;
    switch (call.w.codebook) {
    case CB_3INST: e = launch_tc_bits<CB_3INST>(args, grid, programmatic_launch, stream); break;
    case CB_MCG: e = launch_tc_bits<CB_MCG>(args, grid, programmatic_launch, stream); break;
    case CB_MUL1: e = launch_tc_bits<CB_MUL1>(args, grid, programmatic_launch, stream); break;
    default: return cudaErrorInvalidValue;
    }
    if (e != cudaSuccess || plan.k_splits == 1) return e;
    const long long items = (long long)call.rows * (call.w.outputs / 128);
    const long long want = (items + 7) / 8;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(streaming_grid(want));
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic_launch ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, splitk_finish_kernel, (const float*)args.partials, plan.k_splits,
                              (size_t)rows_padded * call.w.outputs, call.rows, call.w.outputs, call.w.svh, call.w.bias,
                              call.alpha, call.beta, call.y, call.y_dtype, call.y_stride);
}

}  // namespace st
