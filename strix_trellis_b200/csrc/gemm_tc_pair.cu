// Prefill GEMM for more than 256 rows: two CTAs of a cluster work as one tensor-core unit
// (tcgen05 cta_group::2).  The pair owns a 512-row x 256-column tile; each CTA holds 256 rows
// of it as two 128 x 256 f32 accumulators (all 512 columns of its tensor memory), streams its
// own two activation tiles per K step and DECODES ONLY ITS OWN 128 COLUMNS of the weight
// stage -- the MMA reads the other 128 from the partner's shared memory.  Against the
// single-CTA kernel (gemm_tc.cu) every decoded weight feeds twice as many rows, which halves
// the decode work per flop.
//
// Per CTA: warp 0 activation producer (bulk copies), warp 1 MMA issuer (leader CTA) or relay
// (partner CTA: ONE remote arrival per stage once its activation tiles have landed and its
// decoders are done), warps 2-9 epilogue of the CTA's own accumulators (two per tensor-memory
// lane quarter), warps 10-25 decoders (column tile = d % 8, K half = d / 8); on a CTA's last
// tile the decoders, idle by then, take a share of the epilogue with staging areas in the ring.  Barriers another CTA arrives on are waited with cluster scope; a
// tcgen05.commit arrives on both CTAs' barriers at once.  Every wait is bounded and reports
// into the status word; both CTAs meet at a cluster barrier before tensor memory is returned.
#include "backend.h"
#include "hadamard.cuh"
#include "sync_primitives.cuh"
#include "tcgen05.cuh"
#include "trellis_decode.cuh"

namespace st {

namespace {
constexpr int kBM = 128, kMT = 2, kBN = 256, kBK = 64;
constexpr int kStagesP = 3;
constexpr int kTileBytes = kBM * kBK * 2;               // 16 KB: 128 rows x 64 binary16
constexpr int kStageBytesP = (kMT + 1) * kTileBytes;    // A0, A1, this CTA's half of B
constexpr int kDecodeWarps = 16, kEpiWarps = 8;  // two epilogue warps per tensor-memory lane quarter
constexpr int kThreadsP = (2 + kEpiWarps + kDecodeWarps) * 32;
constexpr int kStagingStride = 129;
constexpr int kStagingBytes = 16 * kStagingStride * 4;
static_assert((size_t)kDecodeWarps * kStagingBytes <= (size_t)kStagesP * kStageBytesP, "the decoders' last-tile staging fits the ring");
constexpr size_t kSmemP = 1024 + (size_t)kStagesP * kStageBytesP + (size_t)kEpiWarps * kStagingBytes + 256;
constexpr uint32_t kTmemCols = 512;
constexpr int kWeightsAhead = 8;  // K steps between the L2 prefetch of weight words and their use

struct PairArgs {
    LinearCall call;
    const unsigned char* a_tiles;  // [rows padded to 512 / 128][I/64][16 KB]
    int m_quads;                   // ceil(rows / 512)
    int n_pairs;                   // ceil(column blocks / 2)
};
}  // namespace

template <int K, int CB>
__global__ void __launch_bounds__(kThreadsP, 1) gemm_tc_pair_kernel(const PairArgs args) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const LinearCall& c = args.call;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const int kt64 = c.w.inputs / 64, ktiles16 = c.w.inputs / 16;
    const int nblocks = c.w.outputs / 128;
    const int pair = (int)blockIdx.x >> 1, pairs = (int)gridDim.x >> 1;
    const int tiles = args.n_pairs * args.m_quads;
    const int my_tiles = tiles > pair ? (tiles - pair + pairs - 1) / pairs : 0;

    unsigned char* ring = smem;
    float* staging = reinterpret_cast<float*>(ring + (size_t)kStagesP * kStageBytesP);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(staging) +
                                                 (size_t)kEpiWarps * kStagingBytes);
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    const uint32_t full_a = smem_u32(bars), full_b = smem_u32(bars + kStagesP), peer_a = smem_u32(bars + 2 * kStagesP),
                   empty = smem_u32(bars + 3 * kStagesP), tmem_full = smem_u32(bars + 4 * kStagesP),
                   tmem_empty = smem_u32(bars + 4 * kStagesP + 1);

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStagesP; ++i) {
            mbar_init(full_a + 8 * i, 1);
            mbar_init(full_b + 8 * i, kDecodeWarps);      // this CTA's decoders
            // leader's: ONE barrier per stage for everything its MMA warp waits for -- its own activation
            // copies (one arrival + bytes), its sixteen decoders and the partner's relay
            mbar_init(peer_a + 8 * i, 1 + kDecodeWarps + 1);
            mbar_init(empty + 8 * i, 1);
        }
        mbar_init(tmem_full, 1);
        mbar_init(tmem_empty, 2 * kEpiWarps);              // leader's: the epilogue warps of both CTAs
        mbar_fence_init();
        s_abort = 0;
    }
    // where this CTA's activation copies and decoders report: the leader's merged barrier, or the
    // two barriers the partner's relay waits for
    const uint32_t a_bar = rank == 0 ? peer_a : full_a, b_bar = rank == 0 ? peer_a : full_b;
    if (warp == 1) tmem_alloc_pair(smem_u32(&s_tmem_base), kTmemCols);
    tc_fence_before_sync();
    cluster_sync_all();  // barriers initialised and tensor memory allocated in BOTH CTAs
    tc_fence_after_sync();
    const uint32_t tmem_base = s_tmem_base;

    // One half-item of the epilogue of tile t: 16 rows x 128 columns of one accumulator leave tensor
    // memory through `stage` (16 x 129 floats of the calling warp), then H128, output signs, bias,
    // alpha/beta and the stores.  item = accumulator * 4 + column block * 2 + half.  (As a separate
    // device function it cost a third of the kernel's speed: a call gives the whole kernel a stack frame.)
    auto epilogue_half = [&](int t, int item, int quarter, float* stage) {
        const int np = t / args.m_quads, mq = t % args.m_quads;
        const int mt = item >> 2, cb = (item >> 1) & 1, half = item & 1;
        const int nb = np * (kBN / 128) + cb;
        if (nb >= nblocks) return;  // odd column-block count: second half is padding
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + mt * kBN + cb * 128;
        float sv[4], bi[4];
    #pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cidx = nb * 128 + lane + 32 * j;
            sv[j] = half_bits_to_float(c.w.svh[cidx]);
            bi[j] = c.w.bias ? c.w.bias[cidx] : 0.f;
        }
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
        const int row_base = ((mq * 4 + (int)rank * 2 + mt) * kBM) + quarter * 32 + half * 16;
        for (int r4 = 0; r4 < 16; r4 += 4) {
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
        __syncwarp();
    };


    if (warp == 0) {
        // ---- activation producer: this CTA's two 128-row tiles of every K step -------------
        if (lane == 0) {
            // L2 prefetch of this CTA's weight words kWeightsAhead K steps before its decoders
            // read them (a K step of a 128-column block is one contiguous run of the stream).
            constexpr uint32_t kStepBytes = 4 * 8 * tile_words(K) * 4;
            int plt = -1, pks = kt64;
            const unsigned char* pbase = nullptr;
            auto prefetch_step = [&]() {
                if (pks == kt64) {  // next tile of this pair
                    if (++plt >= my_tiles) { --plt; return; }
                    const int nb = ((pair + plt * pairs) / args.m_quads) * (kBN / 128) + (int)rank;
                    pbase = nb < nblocks ? reinterpret_cast<const unsigned char*>(
                                               c.w.packed + (size_t)nb * ktiles16 * 8 * tile_words(K))
                                         : nullptr;
                    pks = 0;
                }
                if (pbase) bulk_prefetch_l2(pbase + (size_t)pks * kStepBytes, kStepBytes);
                ++pks;
            };
            for (int i = 0; i < kWeightsAhead; ++i) prefetch_step();
            int it = 0;
            for (int lt = 0; lt < my_tiles && !s_abort; ++lt) {
                const int t = pair + lt * pairs;
                const int mq = t % args.m_quads;
                for (int ks = 0; ks < kt64; ++ks, ++it) {
                    const int st = it % kStagesP;
                    if (it >= kStagesP &&
                        !mbar_wait_cluster(empty + 8 * st, (uint32_t)((it / kStagesP) - 1) & 1, c.status, kTimeoutTensorPipe)) {
                        s_abort = 1;
                        break;
                    }
                    unsigned char* dst = ring + (size_t)st * kStageBytesP;
                    mbar_expect_tx(a_bar + 8 * st, kMT * kTileBytes);
#pragma unroll
                    for (int mt = 0; mt < kMT; ++mt)
                        bulk_load(smem_u32(dst + mt * kTileBytes),
                                  args.a_tiles + ((size_t)(mq * 4 + (int)rank * 2 + mt) * kt64 + ks) * kTileBytes,
                                  kTileBytes, a_bar + 8 * st);
                    prefetch_step();
                }
            }
            for (int i = (it > kStagesP ? it - kStagesP : 0); i < it; ++i)  // nothing still landing at exit
                mbar_wait(a_bar + 8 * (i % kStagesP), (uint32_t)(i / kStagesP) & 1, c.status, kTimeoutDrain);
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- MMA issuer (leader CTA only) -------------------------------------------------
            constexpr uint32_t idesc = umma_idesc_f16_f32(2 * kBM, kBN);
            int it = 0;
            for (int lt = 0; lt < my_tiles && !s_abort; ++lt) {
                if (lt >= 1 && !mbar_wait_cluster(tmem_empty, (uint32_t)(lt - 1) & 1, c.status, kTimeoutTensorPipe)) {
                    s_abort = 1;
                    break;
                }
                tc_fence_after_sync();
                for (int ks = 0; ks < kt64 && !s_abort; ++ks, ++it) {
                    const int st = it % kStagesP;
                    const uint32_t par = (uint32_t)(it / kStagesP) & 1;
                    if (!mbar_wait_cluster(peer_a + 8 * st, par, c.status, kTimeoutTensorPipe)) {
                        s_abort = 1;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t base = smem_u32(ring + (size_t)st * kStageBytesP);
                    const uint64_t bdesc = umma_desc_k_major_sw128(base + kMT * kTileBytes);
#pragma unroll
                    for (int mt = 0; mt < kMT; ++mt) {
                        const uint64_t adesc = umma_desc_k_major_sw128(base + mt * kTileBytes);
#pragma unroll
                        for (int k4 = 0; k4 < kBK / 16; ++k4)
                            umma_f16_pair(tmem_base + mt * kBN, adesc + 2 * k4, bdesc + 2 * k4, idesc, (ks | k4) != 0);
                    }
                    umma_commit_pair(empty + 8 * st, 3);  // both CTAs may refill this stage
                }
                umma_commit_pair(tmem_full, 3);           // both CTAs' accumulators of this tile complete
            }
        } else if (lane == 0) {
            // ---- partner CTA: ONE remote arrival per stage, once this CTA's activation tiles have
            // landed and its sixteen decoders have written their half of the weights -------------
            const uint32_t leader_peer_a = map_to_rank(peer_a, 0);
            const int iters = my_tiles * kt64;
            for (int it = 0; it < iters && !s_abort; ++it) {
                const int st = it % kStagesP;
                const uint32_t par = (uint32_t)(it / kStagesP) & 1;
                if (!mbar_wait(full_a + 8 * st, par, c.status, kTimeoutTensorPipe) ||
                    !mbar_wait(full_b + 8 * st, par, c.status, kTimeoutTensorPipe)) {
                    s_abort = 1;
                    break;
                }
                fence_async_smem();
                mbar_arrive_cluster(leader_peer_a + 8 * st);
            }
        }
    } else if (warp < 2 + kEpiWarps) {
        // ---- epilogue of this CTA's 256 rows --------------------------------------------------
        // A lane quarter's work on a tile is eight half-items (accumulator, column block, 16-row
        // half).  On every tile but the last its two epilogue warps take four each; on a CTA's
        // LAST tile the four decoder warps of the quarter, idle by then, take a share too.
        const int quarter = warp & 3, mine = (warp - 2) >> 2;
        float* stage = staging + (size_t)(warp - 2) * 16 * kStagingStride;
        const uint32_t leader_tmem_empty = map_to_rank(tmem_empty, 0);
        for (int lt = 0; lt < my_tiles; ++lt) {
            const int t = pair + lt * pairs;
            if (s_abort || !mbar_wait_cluster(tmem_full, (uint32_t)lt & 1, c.status, kTimeoutTensorPipe)) {
                s_abort = 1;
                break;
            }
            tc_fence_after_sync();
            if (lt + 1 < my_tiles) {
                for (int item = mine; item < 8; item += 2) epilogue_half(t, item, quarter, stage);
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(leader_tmem_empty);  // the leader's MMA warp owns the next tile
            } else {
                for (int item = mine; item < 8; item += 6) epilogue_half(t, item, quarter, stage);
                tc_fence_before_sync();
            }
        }
    } else {
        // ---- decoders: this CTA's 128 columns of the stage, swizzled K-major ---------------------
        const int d = warp - (2 + kEpiWarps);
        const int ct = d & 7, kh = d >> 3;  // column tile, K half (k-tiles 2kh, 2kh+1 of the four)
        const LaneGeom<K> geom(lane);
        const int n0 = ct * 16 + (lane >> 2), kq = 2 * (lane & 3);
        const uint32_t o00 = sw128_offset(n0, kq), o01 = sw128_offset(n0, kq + 8);
        const uint32_t o10 = sw128_offset(n0 + 8, kq), o11 = sw128_offset(n0 + 8, kq + 8);
        const int iters = my_tiles * kt64;
        int flt = 0, fks = 0, fetched = 0;
        const uint32_t* fcol = nullptr;
        bool fvalid = false;
        auto fetch = [&](uint32_t (&w)[2][3]) {
            if (fks == kt64) { fks = 0; ++flt; fcol = nullptr; }
            if (!fcol) {
                const int t = pair + flt * pairs;
                const int nb = (t / args.m_quads) * (kBN / 128) + (int)rank;
                fvalid = nb < nblocks;  // a padding column block decodes nothing
                fcol = c.w.packed + (((size_t)(fvalid ? nb : 0) * ktiles16 + 2 * kh) * 8 + ct) * tile_words(K);
            }
            const uint32_t* tile = fcol + (size_t)fks * 4 * 8 * tile_words(K);
            if (fvalid) {
#pragma unroll
                for (int k2 = 0; k2 < 2; ++k2) load_window<K>(tile + (size_t)k2 * 8 * tile_words(K), geom, w[k2]);
            }
            ++fks;
            ++fetched;
        };
        uint32_t w0[2][3] = {}, w1[2][3] = {}, w2[2][3] = {};  // this stage and the next two, in flight
        if (iters > 0) fetch(w0);
        if (iters > 1) fetch(w1);
        for (int it = 0; it < iters && !s_abort; ++it) {
            const int st = it % kStagesP;
            if (fetched < iters) fetch(w2);
            if (it >= kStagesP &&
                !mbar_wait_cluster(empty + 8 * st, (uint32_t)((it / kStagesP) - 1) & 1, c.status, kTimeoutTensorPipe)) {
                s_abort = 1;
                break;
            }
            unsigned char* bt = ring + (size_t)st * kStageBytesP + kMT * kTileBytes;
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2) {
                uint32_t frag[4];
                decode_words_frag<K, CB>(w0[k2], geom, frag);
                const uint32_t kx = (uint32_t)((2 * kh + k2) * 2) << 4;  // 16 K elements = two 16-byte chunks
                *reinterpret_cast<uint32_t*>(bt + (o00 ^ kx)) = frag[0];
                *reinterpret_cast<uint32_t*>(bt + (o01 ^ kx)) = frag[2];
                *reinterpret_cast<uint32_t*>(bt + (o10 ^ kx)) = frag[1];
                *reinterpret_cast<uint32_t*>(bt + (o11 ^ kx)) = frag[3];
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(b_bar + 8 * st);  // local: the relay (partner) or the MMA warp (leader) waits on it
#pragma unroll
            for (int k2 = 0; k2 < 2; ++k2)
#pragma unroll
                for (int j = 0; j < 3; ++j) { w0[k2][j] = w1[k2][j]; w1[k2][j] = w2[k2][j]; }
        }
        // The CTA's last tile: the ring is idle for good once its MMAs have completed (every copy
        // has landed, both CTAs' reads are done), so this warp takes a staging area there and a
        // share of its lane quarter's epilogue.
        if (my_tiles > 0 && !s_abort &&
            mbar_wait_cluster(tmem_full, (uint32_t)(my_tiles - 1) & 1, c.status, kTimeoutTensorPipe)) {
            tc_fence_after_sync();
            float* stage = reinterpret_cast<float*>(ring) + (size_t)d * 16 * kStagingStride;
            const int t = pair + (my_tiles - 1) * pairs;
            for (int item = 2 + (d >> 2); item < 8; item += 6) epilogue_half(t, item, warp & 3, stage);
            tc_fence_before_sync();
        }
    }

    // ---- common exit: both CTAs are done with each other's memory before anything is freed ----
    tc_fence_before_sync();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// ---- host side ---------------------------------------------------------------------------------
int gemm_pair_rows_padded(int rows) { return (rows + 511) / 512 * 512; }

template <int K, int CB>
static cudaError_t launch_pair(const PairArgs& args, int grid, cudaStream_t stream) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreadsP);
    cfg.dynamicSmemBytes = kSmemP;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel<K, CB>, args);
}

// Opt-in dynamic shared memory is a per-device function attribute: set for every instantiation
// when a context is created on a device (configure_device), never on the launch path.
template <int CB>
static cudaError_t configure_gemm_pair_kernels_codebook() {
    cudaError_t e = cudaSuccess;
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<1, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<2, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<3, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<4, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<5, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<6, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<7, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<8, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP);
    if constexpr (CB == CB_MUL1) {
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<9, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<10, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_pair_kernel<11, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemP);
    }
    return e;
}
cudaError_t configure_gemm_pair_kernels() {
    cudaError_t e = configure_gemm_pair_kernels_codebook<CB_3INST>();
    if (e == cudaSuccess) e = configure_gemm_pair_kernels_codebook<CB_MCG>();
    if (e == cudaSuccess) e = configure_gemm_pair_kernels_codebook<CB_MUL1>();
    return e;
}

template <int CB>
static cudaError_t launch_pair_bits(const PairArgs& a, int grid, cudaStream_t s) {
    switch (a.call.w.bits) {
    case 1: return launch_pair<1, CB>(a, grid, s);
    case 2: return launch_pair<2, CB>(a, grid, s);
    case 3: return launch_pair<3, CB>(a, grid, s);
    case 4: return launch_pair<4, CB>(a, grid, s);
    case 5: return launch_pair<5, CB>(a, grid, s);
    case 6: return launch_pair<6, CB>(a, grid, s);
    case 7: return launch_pair<7, CB>(a, grid, s);
    case 8: return launch_pair<8, CB>(a, grid, s);
    case 9: case 10: case 11:  // 1.5 / 2.5 / 3.5 bits per weight exist for mul1 only
        if constexpr (CB == CB_MUL1) {
            if (a.call.w.bits == 9) return launch_pair<9, CB>(a, grid, s);
            if (a.call.w.bits == 10) return launch_pair<10, CB>(a, grid, s);
            return launch_pair<11, CB>(a, grid, s);
        }
        return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
    }
}

// `a_tiles` holds the pre-swizzled core input for rows padded to a multiple of 512.
cudaError_t launch_gemm_pair(const LinearCall& call, const unsigned char* a_tiles, int sm_count, cudaStream_t stream) {
    PairArgs args{};
    args.call = call;
    args.a_tiles = a_tiles;
    args.m_quads = (call.rows + 511) / 512;
    args.n_pairs = (call.w.outputs / 128 + 1) / 2;
    const long long tiles = (long long)args.n_pairs * args.m_quads;
    if (tiles > 0x3FFFFFFF || sm_count < 2) return cudaErrorInvalidValue;
    const int pairs = (int)(tiles < sm_count / 2 ? tiles : sm_count / 2);
    switch (call.w.codebook) {
    case CB_3INST: return launch_pair_bits<CB_3INST>(args, 2 * pairs, stream);
    case CB_MCG: return launch_pair_bits<CB_MCG>(args, 2 * pairs, stream);
    case CB_MUL1: return launch_pair_bits<CB_MUL1>(args, 2 * pairs, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace st
