// Fused decode GEMV for 1..8 activation rows: input stages (suh scale, RN16, H128,
// RN16), trellis decode, tensor-core dot, split-K fold, output H128, svh, bias and
// alpha/beta in ONE launch.  It stands in for the reference's input_transform +
// gemv_lds_kernel + output_transform sequence (src/backend.hip:102-151,
// src/gemv_lds.hip:93-167, src/transforms.hpp:8-52) and for its fused R1 variants
// (src/gemv_fused.hip:17-129, src/gemv_fused_both.hip:10-93).
//
// Work split ("stream-K"): the weights are one byte stream of units, a unit being the
// 64 tiles of (one 128-column block) x (one H128 block of K), ordered column block
// major -- exactly the prepared layout.  The grid is one persistent CTA per SM and CTA
// c owns the contiguous unit range [c*U/G, (c+1)*U/G): every SM streams the same number
// of bytes (+-1 unit) through a shared-memory ring filled by 1-D bulk copies.  Sixteen
// decode warps: warp (t, g) owns column tile t of the units of parity g, so the two warp
// groups leapfrog through the ring.  A decoded tile is the A operand of mma.sync.m16n8k16 (m = output column), the
// activation rows are the B operand (n = row), so 1..8 rows cost the same tensor work.
//
// Fold: a column block that lies inside one CTA's range is finished by that CTA.  A
// column block shared by several CTAs is finished by the CTA that holds its FIRST K range
// -- the end of that CTA's own unit range, so it gets there when everybody else is done or
// about to be.  The others publish one partial plane each in global scratch, word by word,
// where a word is either the "empty" pattern (all ones, a NaN no sum produces) or a value:
// no flag, no fence, no atomic.  The finishing CTA polls the words (bounded), adds the
// planes in ascending K order from +0 with its own contribution first (never in arrival
// order; the reference's order, src/gemv_fused.hip:81-127), marks them empty again and
// applies the output stages.  Waits only point to higher CTA indices, all CTAs of the grid
// are resident (grid <= SM count), and a wait that runs out reports kTimeoutFold.  All of that is done by
// a separate epilogue warp: decode warps only drop their accumulators into a double-buffered
// shared-memory area and move on, so no decode warp ever waits on global-memory latency.
#include <cstdlib>
#include <type_traits>

#include "backend.h"
#include "gemv_partition.h"
#include "hadamard.cuh"
#include "sync_primitives.cuh"
#include "trellis_decode.cuh"

namespace st {

namespace {
constexpr int kGroups = 2;                       // k-tile parities per column tile
constexpr int kConsumers = 8 * kGroups;          // decode warps
constexpr int kThreads = (kConsumers + 2) * 32;  // + producer warp + epilogue warp
constexpr int kDumpThreads = (kConsumers + 1) * 32;  // decode warps + epilogue warp
constexpr uint32_t kEmptyWord = 0xFFFFFFFFu;      // a partial-plane word nobody has written yet
constexpr int kActBytes = 64 * 1024;             // staged core input per CTA
constexpr size_t kGemvSmemLimit = 200 * 1024;    // dynamic shared memory a launch may ask for
#ifndef ST_GEMV_OCCUPANCY
#define ST_GEMV_OCCUPANCY 1
#endif
#ifndef ST_GEMV_ILP
#define ST_GEMV_ILP 2
#endif
constexpr int kCtasPerSm = ST_GEMV_OCCUPANCY;    // measured: a second resident CTA (the next launch) gains nothing
constexpr int kTilesInFlight = ST_GEMV_ILP;      // independent tile decodes per warp

struct GemvArgs {
    LinearCall call;
    Split split;               // unit range of every CTA (units / grid, units % grid)
    int stages;
    int act_blocks;            // H128 blocks of core input staged at a time
    float* partials;           // [grid][rows][128], every word empty on entry and on exit
#ifdef ST_TIMELINE
    unsigned long long* timeline;
#endif
};

__host__ __device__ inline int stage_bytes(int bits) { return 2048 * bits; }

}  // namespace

// One output row of one column block, by one warp: this CTA's own contribution (`own`, the
// two k-group planes of the shared-memory fold buffer) first, then the planes of CTAs
// first+1 .. last in ascending K order, each polled word by word until it is no longer empty
// (bounded) and marked empty again; then output H128, svh, bias, alpha, beta.
__device__ __forceinline__ void fold_row(const GemvArgs& args, const float* own, int r, int rows, int nb, int first,
                                         int last, int lane, const float (&sv)[4], const float (&bs)[4]) {
    const LinearCall& c = args.call;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
        v[j] = __fadd_rn(0.f, __fadd_rn(own[r * 128 + lane + 32 * j], own[1024 + r * 128 + lane + 32 * j]));
    for (int p0 = first + 1; p0 <= last; p0 += 8) {  // eight planes in flight
        uint32_t t[8][4];
        bool have = false;
        for (uint32_t tries = 0; tries < (1u << 18) && !have; ++tries) {
            bool all = true;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const uint32_t* src =
                    reinterpret_cast<const uint32_t*>(args.partials) + ((size_t)(p0 + q) * rows + r) * 128 + lane;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    t[q][j] = p0 + q <= last ? ld_relaxed_gpu(src + 32 * j) : 0u;
                    all = all && t[q][j] != kEmptyWord;
                }
            }
            have = __all_sync(0xFFFFFFFFu, all);
        }
        if (!have) {  // bounded: report and leave this row unwritten
            if (lane == 0) atomicOr(c.status, kTimeoutFold);
            return;
        }
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            if (p0 + q <= last) {
                uint32_t* src = reinterpret_cast<uint32_t*>(args.partials) + ((size_t)(p0 + q) * rows + r) * 128 + lane;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    v[j] = __fadd_rn(v[j], __uint_as_float(t[q][j]));
                    st_relaxed_gpu(src + 32 * j, kEmptyWord);  // empty again for the next launch
                }
            }
        }
    }
    hadamard128_warp(v, lane);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float* out = c.y + (long long)r * c.y_stride + nb * 128 + lane + 32 * j;
        float value = __fmul_rn(v[j], sv[j]);
        if (c.w.bias) value = __fadd_rn(value, bs[j]);
        value = __fmul_rn(value, c.alpha);
        if (c.beta != 0.0f) value = __fadd_rn(value, __fmul_rn(c.beta, *out));
        *out = value;
    }
}

// MULTI selects the code for more than one activation row (several staging items per warp in
// flight, fold sums in shared memory); the one-row instantiation carries none of it, which
// keeps the latency-critical head and tail of the decode case as short as they can be.
template <int K, int CB, bool MULTI>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) gemv_fused_kernel(const GemvArgs args) {
    extern __shared__ __align__(128) unsigned char smem[];
    const LinearCall& c = args.call;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = c.rows;
    const int hblocks = c.w.inputs / 128;
    const int cta = (int)blockIdx.x;
    const Range mine = cta_range(args.split, cta);
    const int my_units = mine.end - mine.begin;
    const int stages = args.stages;
    constexpr int kStage = 2048 * K;

    // shared memory: [2 x fold 8 KB][barriers 512 B][ring][core input]
    float* fold_base = reinterpret_cast<float*>(smem);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 16384);
    unsigned char* ring = smem + 16384 + 512;
    uint2* act = reinterpret_cast<uint2*>(ring + (size_t)stages * kStage);

    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + stages);
    if ((int)threadIdx.x < stages) {  // one thread per ring slot
        mbar_init(full0 + 8 * threadIdx.x, 1);
        mbar_init(empty0 + 8 * threadIdx.x, 8);
        mbar_fence_init();
    }
    __syncthreads();
#ifdef ST_TIMELINE
    auto stamp = [&](int slot) {
        if (args.timeline && ((threadIdx.x == 0 && slot != 1 && slot != 5) || (slot == 6 && threadIdx.x == 32 * kConsumers) ||
                              ((slot == 1 || slot == 5) && threadIdx.x == 32 * (kConsumers + 1)))) {
            unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            args.timeline[(size_t)blockIdx.x * 8 + slot] = t;
            if (slot == 3) args.timeline[(size_t)blockIdx.x * 8 + 7] = (unsigned long long)clock64();
            if (slot == 4) args.timeline[(size_t)blockIdx.x * 8 + 7] = (unsigned long long)clock64() - args.timeline[(size_t)blockIdx.x * 8 + 7];
        }
    };
#else
    auto stamp = [](int) {};
#endif
    stamp(0);
    pdl_launch_dependents();

    if (warp == kConsumers) {
        // ---- producer: weights are immutable, so this needs no wait on the prior grid ----
        if (lane == 0) {
            const unsigned char* stream =
                reinterpret_cast<const unsigned char*>(c.w.packed) + (size_t)mine.begin * kStage;
            int issued = 0;
            int st = 0;             // ring slot of unit i and the parity of its previous use,
            uint32_t prev_use = 1;  // stepped without divisions
            for (int i = 0; i < my_units; ++i) {
                if (i >= stages && !mbar_wait(empty0 + 8 * st, prev_use, c.status, kTimeoutRingEmpty)) break;
                mbar_expect_tx(full0 + 8 * st, kStage);
                bulk_load(smem_u32(ring + (size_t)st * kStage), stream + (size_t)i * kStage, kStage,
                          full0 + 8 * st);
                issued = i + 1;
                if (++st == stages) { st = 0; prev_use ^= 1; }
            }
            stamp(6);
            // Never leave the CTA with a copy still landing in its shared memory.
            for (int i = (issued > stages ? issued - stages : 0); i < issued; ++i)
                mbar_wait(full0 + 8 * (i % stages), (i / stages) & 1, c.status, kTimeoutDrain);
        }
        return;
    }

    // Segment walk shared by decode and epilogue warps: the CTA's unit range is cut at
    // column-block ends (where a contribution is flushed) and at the staging capacity.
    // Each warp calls it once per segment, in order; the position is carried, not divided out.
    int walk_nb = mine.begin / hblocks, walk_hb0 = mine.begin - walk_nb * hblocks;
    auto segment = [&](int done, int& nb, int& hb0, int& len) {
        nb = walk_nb;
        hb0 = walk_hb0;
        len = my_units - done;
        if (len > hblocks - hb0) len = hblocks - hb0;
        if (len > args.act_blocks) len = args.act_blocks;
        walk_hb0 += len;
        if (walk_hb0 == hblocks) { walk_hb0 = 0; ++walk_nb; }
    };

    if (warp == kConsumers + 1) {
        // ---- epilogue warp: turns dumped accumulators into partial planes or outputs ------
        // Everything a flush needs that does not depend on the accumulators (contributor
        // range, output scales, bias) is resolved BEFORE the wait for the dump, while the
        // decode warps are still busy; after the dump the critical path is one plane write for
        // a contributor and, for the folding CTA, the wait for the others' plane words.
        pdl_wait_prior_grid();  // y and scratch may belong to the prior grid
        int done = 0, flush = 0;
        while (done < my_units) {
            int nb, hb0, len;
            segment(done, nb, hb0, len);
            done += len;
            if (!((hb0 + len == hblocks) || (done == my_units))) continue;
            const int buf = flush & 1;
            const int blk_lo = nb * hblocks, blk_hi = blk_lo + hblocks;
            const bool whole = mine.begin <= blk_lo && mine.end >= blk_hi;
            int first = cta, last = cta;
            if (!whole) contributors(args.split, blk_lo, blk_hi, first, last);
            float sv[4], bs[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int cidx = nb * 128 + lane + 32 * j;
                sv[j] = half_bits_to_float(c.w.svh[cidx]);
                bs[j] = c.w.bias ? c.w.bias[cidx] : 0.0f;
            }
            // A CTA publishes at most one plane per launch: for the block its range begins inside.
            uint32_t* plane = reinterpret_cast<uint32_t*>(args.partials) + (size_t)cta * rows * 128;

            named_barrier(2 + buf, kDumpThreads);  // all decode warps have dumped into `buf`
            const float* f0 = fold_base + buf * 2048;
            if (!whole && cta != first) {
                // contributor: publish the plane word by word (k-groups in ascending order); a
                // real sum never has the empty pattern (an all-ones NaN), so no flag and no fence
                for (int e = lane; e < rows * 128; e += 32)
                    st_relaxed_gpu(plane + e, __float_as_uint(__fadd_rn(f0[e], f0[1024 + e])));
                stamp(1);
            } else {
                // The block is finished here: it lies inside this CTA's range, or this CTA holds
                // its FIRST K range -- the end of its own unit range, so every other contributor
                // finishes at about the same time or earlier.  With several rows and planes to
                // wait for, the decode warps (idle by then) fold one row each instead.
                if (!(MULTI && !whole)) {
                    for (int r = 0; r < rows; ++r) fold_row(args, f0, r, rows, nb, first, last, lane, sv, bs);
                }
            }
            // hand the buffer back (decode warps wait on this before its next reuse)
            asm volatile("bar.arrive %0, %1;" ::"r"(4 + buf), "r"(kDumpThreads) : "memory");
            ++flush;
        }
        stamp(5);
        return;
    }

    // ---- decode warps -------------------------------------------------------------------
    // Resident mode: the whole core input fits the staging area, so every H128 block this
    // CTA's range touches is staged exactly once, at its own slot, before the loop starts.
    // The input scales of a warp's first block are weights (immutable): they are fetched
    // before the wait on the prior grid, so only the activation load follows it.
    const bool resident = MULTI ? hblocks <= args.act_blocks : true;  // the one-row kernel is only launched resident
    const int need = my_units < hblocks ? my_units : hblocks;
    const int hb_first = walk_hb0;
    uint16_t su_first[4] = {0, 0, 0, 0};
    if (resident && warp < rows * need) {
        int hb = hb_first + warp % need;
        if (hb >= hblocks) hb -= hblocks;
#pragma unroll
        for (int j = 0; j < 4; ++j) su_first[j] = c.w.suh[(size_t)hb * 128 + lane + 32 * j];
    }
    pdl_wait_prior_grid();  // x may belong to the prior grid
    stamp(2);
    const int ctile = warp & 7, kgroup = warp >> 3;
    const LaneGeom<K> geom(lane);
    // Row fed by this lane as the B operand.  Rows >= `rows` only reach accumulator
    // columns that are never read, so those lanes may load any valid row.
    const int brow = (lane >> 2) < rows ? (lane >> 2) : rows - 1;
    const uint2* act_lane = act + brow * 32 + (lane & 3);
    __half* act_h = reinterpret_cast<__half*>(act);
    const int col = ctile * 16 + (lane >> 2), r0 = 2 * (lane & 3);

    // (row, H128 block) items through the input stages, written in B-fragment order:
    // act[((slot*rows + r)*8 + kt)*4 + q] = {half2(k0,k0+1), half2(k0+8,k0+9)}, k0 = 2q.
    // A warp keeps four items in flight so that their global loads overlap (eight rows of a
    // 4096-input layer are 256 items, sixteen per warp).  where(item, r, hb, slot) names an item.
    auto stage_items = [&](int n, bool first_scales_ready, auto&& where, auto width) {
        constexpr int kInFlight = decltype(width)::value;
        for (int base = warp; base < n; base += kInFlight * kConsumers) {
            float xv[kInFlight][4];
            uint16_t sc[kInFlight][4];
            int rr[kInFlight], ss[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const int item = base + u * kConsumers;
                if (item < n) {
                    int hb;
                    where(item, rr[u], hb, ss[u]);
                    const float* xr = c.x + (long long)rr[u] * c.x_stride + (size_t)hb * 128;
                    const uint16_t* su = c.w.suh + (size_t)hb * 128;
                    const bool ready = first_scales_ready && item == warp;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        xv[u][j] = xr[lane + 32 * j];
                        sc[u][j] = ready ? su_first[j] : su[lane + 32 * j];
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                if (base + u * kConsumers < n) {
                    float v[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = __half2float(scale_input(xv[u][j], sc[u][j]));
                    hadamard128_warp(v, lane);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int e = lane + 32 * j, kt = e >> 4, kk = e & 15;
                        const int q = (kk & 7) >> 1, hi = kk >> 3, lo = kk & 1;
                        act_h[((((size_t)ss[u] * rows + rr[u]) * 8 + kt) * 4 + q) * 4 + hi * 2 + lo] = __float2half_rn(v[j]);
                    }
                }
            }
        }
    };
    if (resident) {
        auto where = [&](int item, int& r, int& hb, int& slot) {
            r = item / need;
            hb = hb_first + item % need;
            if (hb >= hblocks) hb -= hblocks;
            slot = hb;
        };
        stage_items(rows * need, true, where, std::integral_constant<int, MULTI ? 4 : 1>{});
        named_barrier(1, kConsumers * 32);
    }

    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    bool ok = true;
    int done = 0, flush = 0, final_nb = 0;
    int next = kgroup;  // the unit (relative to the range) this warp decodes next
    int slot = kgroup % stages;
    uint32_t use = (uint32_t)(kgroup / stages) & 1;
    while (done < my_units) {
        int nb, hb0, len;
        segment(done, nb, hb0, len);

        // chunked mode: input stages for H128 blocks [hb0, hb0+len) into slots 0..len-1
        if (!resident) {
            named_barrier(1, kConsumers * 32);  // previous chunk's readers are done
            stage_items(rows * len, false, [&](int item, int& r, int& hb, int& slot) {
                r = item / len;
                slot = item % len;
                hb = hb0 + slot;
            }, std::integral_constant<int, MULTI ? 4 : 1>{});
            named_barrier(1, kConsumers * 32);
        }
        if (done == 0) stamp(3);

        // this warp group takes the units of its parity (ring slots alternate with them)
        for (; next < done + len && ok; next += 2) {
            const int b = next - done, st = slot;
            ok = mbar_wait(full0 + 8 * st, use, c.status, kTimeoutRingFull);
            if (!ok) break;
            slot += 2;  // ring slot and use parity of this warp's next unit, without divisions
            while (slot >= stages) { slot -= stages; use ^= 1; }
            const uint32_t* tiles =
                reinterpret_cast<const uint32_t*>(ring + (size_t)st * kStage) + ctile * (8 * K);
            const uint2* bsrc = act_lane + (size_t)(resident ? hb0 + b : b) * rows * 32;
#pragma unroll
            for (int kt = 0; kt < 8; kt += kTilesInFlight) {  // independent tiles in flight
                uint32_t f[kTilesInFlight][4];
                uint2 bf[kTilesInFlight];
#pragma unroll
                for (int q = 0; q < kTilesInFlight; ++q) {
                    decode_tile_frag<K, CB>(tiles + (kt + q) * 8 * (8 * K), geom, f[q]);
                    bf[q] = bsrc[(kt + q) * 4];
                }
#pragma unroll
                for (int q = 0; q < kTilesInFlight; ++q) mma_16816(acc[q & 1], f[q], bf[q].x, bf[q].y);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * st);
        }
        done += len;
        if (done == my_units) stamp(4);
        if (!((hb0 + len == hblocks) || (done == my_units))) continue;

        // ---- drop this CTA's contribution to column block nb and move on --------------------
        // c0,c1: column ctile*16 + lane/4, rows 2(lane%4), +1; c2,c3: column + 8
        const int buf = flush & 1;
        if (flush >= 2) named_barrier(4 + buf, kDumpThreads);  // epilogue is done with `buf`
        {
            float* g = fold_base + buf * 2048 + kgroup * 1024;
            const float v00 = acc[0][0] + acc[1][0], v01 = acc[0][1] + acc[1][1];
            const float v10 = acc[0][2] + acc[1][2], v11 = acc[0][3] + acc[1][3];
            if (r0 < rows) { g[r0 * 128 + col] = v00; g[r0 * 128 + col + 8] = v10; }
            if (r0 + 1 < rows) { g[(r0 + 1) * 128 + col] = v01; g[(r0 + 1) * 128 + col + 8] = v11; }
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[0][j] = acc[1][j] = 0.f;
        }
        asm volatile("bar.arrive %0, %1;" ::"r"(2 + buf), "r"(kDumpThreads) : "memory");
        ++flush;
        final_nb = nb;
    }

    // ---- several rows: the decode warps finish the CTA's last, shared column block ----------
    // If this CTA folds that block (it holds the block's first K range, other CTAs hold the
    // rest), warp r folds row r -- eight rows wait for their planes side by side instead of one
    // after the other in the epilogue warp.  Every decode warp reaches the barrier, whatever
    // its own waits returned, so it cannot be left short of arrivals.
    if (MULTI && my_units > 0) {
        const int blk_lo = final_nb * hblocks, blk_hi = blk_lo + hblocks;
        if (!(mine.begin <= blk_lo && mine.end >= blk_hi)) {
            int first, last;
            contributors(args.split, blk_lo, blk_hi, first, last);
            if (cta == first) {
                named_barrier(1, kConsumers * 32);  // every decode warp has dumped its accumulators
                if (ok && warp < rows) {
                    float sv[4], bs[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int cidx = final_nb * 128 + lane + 32 * j;
                        sv[j] = half_bits_to_float(c.w.svh[cidx]);
                        bs[j] = c.w.bias ? c.w.bias[cidx] : 0.0f;
                    }
                    fold_row(args, fold_base + ((flush - 1) & 1) * 2048, warp, rows, final_nb, first, last, lane, sv, bs);
                }
            }
        }
    }
}

// ---- host side -------------------------------------------------------------------------
static int gemv_grid(const DeviceWeights& w, int sm_count) {
    const long long units = (long long)(w.inputs / 128) * (w.outputs / 128);
    return (int)(units < sm_count ? units : sm_count);
}

GemvPlan plan_gemv(const DeviceWeights& w, int rows, int sm_count) {
    GemvPlan plan{};
    const int hblocks = w.inputs / 128, nblocks = w.outputs / 128;
    const int grid = gemv_grid(w, sm_count);
    const long long units = (long long)hblocks * nblocks;
    const int per_cta = (int)((units + grid - 1) / grid);
    int act_blocks = kActBytes / (256 * rows);
    if (act_blocks > hblocks) act_blocks = hblocks;
    const int ring_budget = 200 * 1024 - 16384 - 512 - act_blocks * 256 * rows;
    int stages = ring_budget / stage_bytes(w.bits);
    const int want = (128 * 1024) / stage_bytes(w.bits);  // enough bytes in flight per SM to cover HBM latency
    if (stages > want) stages = want;
    if (stages > per_cta) stages = per_cta;
    if (stages > 28) stages = 28;
    if (stages < 1) stages = 1;
    plan.grid = grid;
    plan.act_blocks = act_blocks;
    plan.splits = (grid + nblocks - 1) / nblocks;  // typical K partitions of a column block
    plan.stages = stages;
    plan.smem_bytes = 16384 + 512 + (size_t)stages * stage_bytes(w.bits) + (size_t)act_blocks * 256 * rows;
    plan.counter_bytes = 0;  // the fold needs no counters
    plan.partial_bytes = align_up((size_t)grid * rows * 128 * sizeof(float));
    return plan;
}

template <int K, int CB, bool MULTI>
static cudaError_t launch_rows(const GemvArgs& args, int grid, size_t smem, bool pdl, cudaStream_t stream) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemv_fused_kernel<K, CB, MULTI>, args);
}

template <int K, int CB>
static cudaError_t launch_one(const GemvArgs& args, int grid, size_t smem, bool pdl, cudaStream_t stream) {
    const bool lean = args.call.rows == 1 && args.call.w.inputs / 128 <= args.act_blocks;
    return lean ? launch_rows<K, CB, false>(args, grid, smem, pdl, stream)
                : launch_rows<K, CB, true>(args, grid, smem, pdl, stream);
}

template <int CB>
static cudaError_t launch_bits(const GemvArgs& a, int g, size_t smem, bool pdl, cudaStream_t s) {
    switch (a.call.w.bits) {
    case 1: return launch_one<1, CB>(a, g, smem, pdl, s);
    case 2: return launch_one<2, CB>(a, g, smem, pdl, s);
    case 3: return launch_one<3, CB>(a, g, smem, pdl, s);
    case 4: return launch_one<4, CB>(a, g, smem, pdl, s);
    case 5: return launch_one<5, CB>(a, g, smem, pdl, s);
    case 6: return launch_one<6, CB>(a, g, smem, pdl, s);
    case 7: return launch_one<7, CB>(a, g, smem, pdl, s);
    case 8: return launch_one<8, CB>(a, g, smem, pdl, s);
    default: return cudaErrorInvalidValue;
    }
}

// Opt-in dynamic shared memory is a per-device function attribute: set for every instantiation
// when a context is created on a device (configure_device), never on the launch path.
template <int K, int CB>
static cudaError_t configure_rate() {
    cudaError_t e = cudaFuncSetAttribute(gemv_fused_kernel<K, CB, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kGemvSmemLimit);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemv_fused_kernel<K, CB, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kGemvSmemLimit);
    return e;
}
template <int CB>
static cudaError_t configure_codebook() {
    cudaError_t e = configure_rate<1, CB>();
    if (e == cudaSuccess) e = configure_rate<2, CB>();
    if (e == cudaSuccess) e = configure_rate<3, CB>();
    if (e == cudaSuccess) e = configure_rate<4, CB>();
    if (e == cudaSuccess) e = configure_rate<5, CB>();
    if (e == cudaSuccess) e = configure_rate<6, CB>();
    if (e == cudaSuccess) e = configure_rate<7, CB>();
    if (e == cudaSuccess) e = configure_rate<8, CB>();
    return e;
}
cudaError_t configure_gemv_kernels() {
    cudaError_t e = configure_codebook<CB_3INST>();
    if (e == cudaSuccess) e = configure_codebook<CB_MCG>();
    if (e == cudaSuccess) e = configure_codebook<CB_MUL1>();
    return e;
}

cudaError_t reset_gemv_scratch(void* workspace, const GemvPlan& plan, cudaStream_t stream) {
    const size_t bytes = plan.counter_bytes + plan.partial_bytes;
    if (!bytes) return cudaSuccess;
    return cudaMemsetAsync(workspace, 0xFF, bytes, stream);
}

cudaError_t launch_gemv(const LinearCall& call, const GemvPlan& plan, void* workspace,
                        bool programmatic_launch, cudaStream_t stream) {
    if (call.rows < 1 || call.rows > 8 || !workspace) return cudaErrorInvalidValue;
    GemvArgs args{};
    args.call = call;
    const long long units = (long long)(call.w.inputs / 128) * (call.w.outputs / 128);
    if (units > 0x7FFFFFFF || plan.grid < 1 || plan.grid > units) return cudaErrorInvalidValue;
    args.split = make_split((int)units, plan.grid);
    args.stages = plan.stages;
    args.act_blocks = plan.act_blocks;
    args.partials = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + plan.counter_bytes);
#ifdef ST_TIMELINE
    if (const char* t = getenv("STRIX_TL")) args.timeline = (unsigned long long*)strtoull(t, nullptr, 16);
#endif
    switch (call.w.codebook) {
    case CB_3INST: return launch_bits<CB_3INST>(args, plan.grid, plan.smem_bytes, programmatic_launch, stream);
    case CB_MCG: return launch_bits<CB_MCG>(args, plan.grid, plan.smem_bytes, programmatic_launch, stream);
    case CB_MUL1: return launch_bits<CB_MUL1>(args, plan.grid, plan.smem_bytes, programmatic_launch, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace st
