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
// groups leapfrog through the ring.  A decoded tile is the A operand of mma.sync.m16n8k16
// (m = output column), the activation rows are the B operand (n = row), so 1..8 rows cost
// the same tensor work.
//
// Fold: a column block that lies inside one CTA's range is finished by that CTA.  A
// column block shared by several CTAs is finished by the CTA that holds its FIRST K range
// -- the end of that CTA's own unit range, so it gets there when everybody else is done or
// about to be.  The others publish partial planes in global scratch, word by word, where a
// word is either the "empty" pattern (all ones, a NaN no sum produces) or a value: no flag,
// no fence, no atomic.  The finishing CTA polls the words (bounded), adds the planes in
// ascending K order from +0 with its own contribution first (never in arrival order; the
// reference's order, src/gemv_fused.hip:81-127), marks them empty again and applies the
// output stages.  Waits only point to higher CTA indices, all CTAs of the grid are resident
// (grid <= SM count), and a wait that runs out reports kTimeoutFold.
//
// Two kernels share this design.  gemv_fused_kernel serves 2..8 rows (and one row of a
// layer too wide to stage at once): a separate epilogue warp turns dumped accumulators into
// planes or outputs.  gemv_row_kernel is the one-row decode case, where the head and the
// tail of the launch weigh as much as the loop: contributors publish their planes straight from
// the accumulator registers, and the finishing CTA polls one plane per decode warp.
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
constexpr int kTilesInFlight = 2;                // independent tile decodes per warp

struct GemvArgs {
    LinearCall call;
    Split split;               // unit range of every CTA (units / grid, units % grid)
    int stages;
    int act_blocks;            // H128 blocks of core input staged at a time
    float* partials;           // [grid][rows][128] ([grid][2][128] for the one-row kernel), every word empty on entry and on exit
};

__host__ __device__ inline int stage_bytes(int rate) { return unit_bytes(rate); }

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
        float value = __fmul_rn(v[j], sv[j]);
        if (c.w.bias) value = __fadd_rn(value, bs[j]);
        scale_and_store(c.y, c.y_dtype, (long long)r * c.y_stride + nb * 128 + lane + 32 * j, value, c.alpha, c.beta);
    }
}

// Rows 2..8 (and one row of a layer whose core input does not fit the staging area at once).
template <int K, int CB>
__global__ void __launch_bounds__(kThreads, 1) gemv_fused_kernel(const GemvArgs args) {
    extern __shared__ __align__(128) unsigned char smem[];
    const LinearCall& c = args.call;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows = c.rows;
    const int hblocks = c.w.inputs / 128;
    const int cta = (int)blockIdx.x;
    const Range mine = cta_range(args.split, cta);
    const int my_units = mine.end - mine.begin;
    const int stages = args.stages;
    constexpr int kStage = unit_bytes(K);

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
            } else {
                // The block is finished here: it lies inside this CTA's range, or this CTA holds
                // its FIRST K range -- the end of its own unit range, so every other contributor
                // finishes at about the same time or earlier.  With several rows and planes to
                // wait for, the decode warps (idle by then) fold one row each instead.
                if (whole) {
                    for (int r = 0; r < rows; ++r) fold_row(args, f0, r, rows, nb, first, last, lane, sv, bs);
                }
            }
            // hand the buffer back (decode warps wait on this before its next reuse)
            asm volatile("bar.arrive %0, %1;" ::"r"(4 + buf), "r"(kDumpThreads) : "memory");
            ++flush;
        }
        return;
    }

    // ---- decode warps -------------------------------------------------------------------
    // Resident mode: the whole core input fits the staging area, so every H128 block this
    // CTA's range touches is staged exactly once, at its own slot, before the loop starts.
    // The input scales of a warp's first block are weights (immutable): they are fetched
    // before the wait on the prior grid, so only the activation load follows it.
    const bool resident = hblocks <= args.act_blocks;
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
                    const long long xr = (long long)rr[u] * c.x_stride + (long long)hb * 128;
                    const uint16_t* su = c.w.suh + (size_t)hb * 128;
                    const bool ready = first_scales_ready && item == warp;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        xv[u][j] = load_element(c.x, c.x_dtype, xr + lane + 32 * j);
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
        stage_items(rows * need, true, where, std::integral_constant<int, 4>{});
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
            }, std::integral_constant<int, 4>{});
            named_barrier(1, kConsumers * 32);
        }

        // this warp group takes the units of its parity (ring slots alternate with them)
        for (; next < done + len && ok; next += 2) {
            const int b = next - done, st = slot;
            ok = mbar_wait(full0 + 8 * st, use, c.status, kTimeoutRingFull);
            if (!ok) break;
            slot += 2;  // ring slot and use parity of this warp's next unit, without divisions
            while (slot >= stages) { slot -= stages; use ^= 1; }
            const uint32_t* tiles =
                reinterpret_cast<const uint32_t*>(ring + (size_t)st * kStage) + ctile * tile_words(K);
            const uint2* bsrc = act_lane + (size_t)(resident ? hb0 + b : b) * rows * 32;
#pragma unroll
            for (int kt = 0; kt < 8; kt += kTilesInFlight) {  // independent tiles in flight
                uint32_t f[kTilesInFlight][4];
                uint2 bf[kTilesInFlight];
#pragma unroll
                for (int q = 0; q < kTilesInFlight; ++q) {
                    decode_tile_frag<K, CB>(tiles + (kt + q) * 8 * tile_words(K), geom, f[q]);
                    bf[q] = bsrc[(kt + q) * 4];
                }
#pragma unroll
                for (int q = 0; q < kTilesInFlight; ++q) mma_16816(acc[q & 1], f[q], bf[q].x, bf[q].y);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * st);
        }
        done += len;
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
    if (my_units > 0) {
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


// ---- one activation row -----------------------------------------------------------------
namespace {
constexpr int kRowHeader = 2048 + 8192 + 128 + 512;  // fold buffers, gathered planes, flag, barriers
static_assert(kRowHeader % 128 == 0, "the ring starts on a 128-byte boundary");

__device__ __forceinline__ uint4 ld_relaxed_gpu_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu_v4(uint4* p, uint4 v) {
    asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ bool any_empty(const uint4& a, const uint4& b) {
    return a.x == kEmptyWord || a.y == kEmptyWord || a.z == kEmptyWord || a.w == kEmptyWord ||
           b.x == kEmptyWord || b.y == kEmptyWord || b.z == kEmptyWord || b.w == kEmptyWord;
}

// One warp waits for one contributor's plane: lane l owns columns 4l..4l+3 of both k-group
// halves.  The first load is looked at as soon as it is back: measured on the benchmark shapes,
// most planes are already there when the finishing CTA gets here, and anything that delays the
// first look (pacing the loads, staggering them) costs more than it gains.  Returns the two
// halves (every word a value) and marks the plane empty again; false when the bounded wait
// runs out.
__device__ __forceinline__ bool await_plane(uint4* g0, uint4* g1, int lane, uint4& a, uint4& b) {
    bool have = false;
    for (uint32_t tries = 0; tries < (1u << 20) && !have; ++tries) {
        a = ld_relaxed_gpu_v4(g0 + lane);
        b = ld_relaxed_gpu_v4(g1 + lane);
        have = __all_sync(0xFFFFFFFFu, !any_empty(a, b));
    }
    if (have) {
        const uint4 empty = make_uint4(kEmptyWord, kEmptyWord, kEmptyWord, kEmptyWord);
        st_relaxed_gpu_v4(g0 + lane, empty);  // empty again for the next launch
        st_relaxed_gpu_v4(g1 + lane, empty);
    }
    return have;
}
}  // namespace

// One row, core input resident in shared memory.  Roles: 16 decode warps, one producer warp
// (bulk copies of the weight stream), one epilogue warp (finishes column blocks that lie
// wholly inside this CTA's range while the decode warps go on).
//
// Head: the producer streams weights from the moment the CTA starts (weights are immutable, so
// this does not wait for the previous kernel of the stream); the input scales of a warp's
// H128 block are fetched before the wait on the previous kernel too, so that only the load of
// the activation row and the input stages follow it, then one barrier, then the first mma.
// (Decoding a warp's first tiles into registers while that load is in flight was measured:
// 0.25 us per launch slower, the extra live registers cost more than the overlap gains.)
//
// Tail: a CTA whose range BEGINS inside a column block is a contributor to it: its decode
// warps store their accumulators straight into the CTA's plane in global scratch
// ([cta][k-group][128] floats), no shared-memory hop and no other warp involved.  The CTA whose
// range ENDS inside a block (it holds the block's first K range) finishes it: decode warp p
// waits for plane p (await_plane), the planes meet in shared memory, and warp 0 adds them in
// ascending K order from +0, its own contribution first, then H128, svh, bias, alpha, beta.
template <int K, int CB>
__global__ void __launch_bounds__(kThreads, 1) gemv_row_kernel(const GemvArgs args) {
    extern __shared__ __align__(128) unsigned char smem[];
    const LinearCall& c = args.call;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hblocks = c.w.inputs / 128;
    const int cta = (int)blockIdx.x;
    const Range mine = cta_range(args.split, cta);
    const int my_units = mine.end - mine.begin;
    const int stages = args.stages;
    constexpr int kStage = unit_bytes(K);

    // shared memory: [2 x fold 1 KB][16 gathered planes 8 KB][flag][barriers 512 B][ring][core input]
    float* fold_base = reinterpret_cast<float*>(smem);            // [2 buffers][2 k-groups][128]
    float* gathered = reinterpret_cast<float*>(smem + 2048);      // [16][128]
    int* gave_up = reinterpret_cast<int*>(smem + 2048 + 8192);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2048 + 8192 + 128);
    unsigned char* ring = smem + kRowHeader;
    uint2* act = reinterpret_cast<uint2*>(ring + (size_t)stages * kStage);

    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + stages);
    if ((int)threadIdx.x < stages) {  // one thread per ring slot
        mbar_init(full0 + 8 * threadIdx.x, 1);
        mbar_init(empty0 + 8 * threadIdx.x, 8);
        mbar_fence_init();
    }
    if (threadIdx.x == 0) *gave_up = 0;
    __syncthreads();
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
                bulk_load(smem_u32(ring + (size_t)st * kStage), stream + (size_t)i * kStage, kStage, full0 + 8 * st);
                issued = i + 1;
                if (++st == stages) { st = 0; prev_use ^= 1; }
            }
            // Never leave the CTA with a copy still landing in its shared memory.
            for (int i = (issued > stages ? issued - stages : 0); i < issued; ++i)
                mbar_wait(full0 + 8 * (i % stages), (i / stages) & 1, c.status, kTimeoutDrain);
        }
        return;
    }

    // Walk of the CTA's unit range, cut at column-block ends; shared by decode and epilogue
    // warps (each calls it once per segment, in order).
    int walk_nb = mine.begin / hblocks, walk_hb0 = mine.begin - walk_nb * hblocks;
    auto segment = [&](int done, int& nb, int& hb0, int& len) {
        nb = walk_nb;
        hb0 = walk_hb0;
        len = my_units - done;
        if (len > hblocks - hb0) len = hblocks - hb0;
        walk_hb0 += len;
        if (walk_hb0 == hblocks) { walk_hb0 = 0; ++walk_nb; }
    };
    // A segment [hb0, hb0+len) of block nb ends the block or the range.  It is `whole` when the
    // block lies inside this CTA's range.
    auto is_whole = [&](int nb) { return mine.begin <= nb * hblocks && mine.end >= (nb + 1) * hblocks; };

    if (warp == kConsumers + 1) {
        // ---- epilogue warp: output stages of the blocks that need nobody else ---------------
        // Output scales and bias of every column block this CTA touches are weights, cold in DRAM,
        // and are needed at the very end of a block: ask the L2 for them now.
        for (int nb = mine.begin / hblocks, last = (mine.end - 1) / hblocks; nb <= last && my_units > 0; ++nb) {
            if (lane < 2) prefetch_line_l2(c.w.svh + (size_t)nb * 128 + lane * 64);
            else if (lane < 6 && c.w.bias) prefetch_line_l2(c.w.bias + (size_t)nb * 128 + (lane - 2) * 32);
        }
        pdl_wait_prior_grid();  // y may belong to the prior grid
        int done = 0, flush = 0;
        while (done < my_units) {
            int nb, hb0, len;
            segment(done, nb, hb0, len);
            done += len;
            if (!is_whole(nb)) continue;
            const int buf = flush & 1;
            float sv[4], bs[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int cidx = nb * 128 + lane + 32 * j;
                sv[j] = half_bits_to_float(c.w.svh[cidx]);
                bs[j] = c.w.bias ? c.w.bias[cidx] : 0.0f;
            }
            named_barrier(2 + buf, kDumpThreads);  // all decode warps have dumped into `buf`
            const float* f0 = fold_base + buf * 256;
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = __fadd_rn(0.f, __fadd_rn(f0[lane + 32 * j], f0[128 + lane + 32 * j]));
            hadamard128_warp(v, lane);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float value = __fmul_rn(v[j], sv[j]);
                if (c.w.bias) value = __fadd_rn(value, bs[j]);
                scale_and_store(c.y, c.y_dtype, (long long)nb * 128 + lane + 32 * j, value, c.alpha, c.beta);
            }
            asm volatile("bar.arrive %0, %1;" ::"r"(4 + buf), "r"(kDumpThreads) : "memory");
            ++flush;
        }
        return;
    }

    // ---- decode warps -------------------------------------------------------------------
    const int ctile = warp & 7, kgroup = warp >> 3;
    const LaneGeom<K> geom(lane);
    const int need = my_units < hblocks ? my_units : hblocks;  // H128 blocks of the row this CTA touches
    const int hb_first = walk_hb0;
    int my_hb = hb_first + warp;                               // the block this warp stages (warp < need)
    if (my_hb >= hblocks) my_hb -= hblocks;
    uint16_t su[4] = {0, 0, 0, 0};
    if (warp < need) {  // input scales are weights: fetched before the wait on the prior grid
#pragma unroll
        for (int j = 0; j < 4; ++j) su[j] = c.w.suh[(size_t)my_hb * 128 + lane + 32 * j];
    }
    // The activation row may still be in flight from the prior grid, or cold in DRAM when it came
    // from the host: ask the L2 for this CTA's part of it now, read it after the wait.
    {
        const int x_bytes = c.x_dtype == DT_F32 ? 4 : 2;
        if (lane * 128 < 128 * x_bytes)
            for (int item = warp; item < need; item += kConsumers) {
                int hb = hb_first + item;
                if (hb >= hblocks) hb -= hblocks;
                prefetch_line_l2(reinterpret_cast<const unsigned char*>(c.x) + (size_t)hb * 128 * x_bytes + lane * 128);
            }
    }
    pdl_wait_prior_grid();  // x, y and the scratch may belong to the prior grid
    float xv[4] = {0.f, 0.f, 0.f, 0.f};
    if (warp < need) {
#pragma unroll
        for (int j = 0; j < 4; ++j) xv[j] = load_element(c.x, c.x_dtype, (long long)my_hb * 128 + lane + 32 * j);
    }

    bool ok = true;
    int slot = kgroup % stages;  // ring slot and use parity of the unit this warp decodes next
    uint32_t use = (uint32_t)(kgroup / stages) & 1;

    // input stages of this warp's block, written in B-fragment order:
    // act[(hb*8 + kt)*4 + q] = {half2(k0,k0+1), half2(k0+8,k0+9)}, k0 = 2q
    __half* act_h = reinterpret_cast<__half*>(act);
    for (int item = warp; item < need; item += kConsumers) {
        int hb = hb_first + item;
        if (hb >= hblocks) hb -= hblocks;
        float v[4];
        if (item == warp) {
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = __half2float(scale_input(xv[j], su[j]));
        } else {  // more blocks than warps: the rest comes straight from memory
#pragma unroll
            for (int j = 0; j < 4; ++j)
                v[j] = __half2float(scale_input(load_element(c.x, c.x_dtype, (long long)hb * 128 + lane + 32 * j),
                                                c.w.suh[(size_t)hb * 128 + lane + 32 * j]));
        }
        hadamard128_warp(v, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = lane + 32 * j, kt = e >> 4, kk = e & 15;
            const int q = (kk & 7) >> 1, hi = kk >> 3, lo = kk & 1;
            act_h[(((size_t)hb * 8 + kt) * 4 + q) * 4 + hi * 2 + lo] = __float2half_rn(v[j]);
        }
    }
    named_barrier(1, kConsumers * 32);

    // Only activation row 0 exists: lanes of every row feed it as the B operand; accumulator
    // columns of rows >= 1 are never read.
    const uint2* act_lane = act + (lane & 3);
    const int col = ctile * 16 + (lane >> 2);
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    int done = 0, flush = 0;
    int next = kgroup;  // the unit (relative to the range) this warp decodes next
    while (done < my_units) {
        int nb, hb0, len;
        segment(done, nb, hb0, len);
        for (; next < done + len && ok; next += 2) {
            const int b = next - done, st = slot;
            ok = mbar_wait(full0 + 8 * st, use, c.status, kTimeoutRingFull);
            if (!ok) break;
            slot += 2;
            while (slot >= stages) { slot -= stages; use ^= 1; }
            const uint32_t* tiles = reinterpret_cast<const uint32_t*>(ring + (size_t)st * kStage) + ctile * tile_words(K);
            const uint2* bsrc = act_lane + (size_t)(hb0 + b) * 32;
#pragma unroll
            for (int kt = 0; kt < 8; kt += kTilesInFlight) {
                uint32_t f[kTilesInFlight][4];
                uint2 bf[kTilesInFlight];
#pragma unroll
                for (int q = 0; q < kTilesInFlight; ++q) {
                    decode_tile_frag<K, CB>(tiles + (kt + q) * 8 * tile_words(K), geom, f[q]);
                    bf[q] = bsrc[(kt + q) * 4];
                }
#pragma unroll
                for (int q = 0; q < kTilesInFlight; ++q) mma_16816(acc[q & 1], f[q], bf[q].x, bf[q].y);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * st);
        }
        done += len;

        // ---- this CTA's contribution to column block nb is complete -------------------------
        // row 0 of the accumulators: lanes with lane % 4 == 0 hold columns col (c0) and col+8 (c2)
        const float v_lo = acc[0][0] + acc[1][0], v_hi = acc[0][2] + acc[1][2];
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[0][j] = acc[1][j] = 0.f;
        const int blk_lo = nb * hblocks, blk_hi = blk_lo + hblocks;
        const bool whole = mine.begin <= blk_lo && mine.end >= blk_hi;
        if (!whole && mine.begin > blk_lo) {
            // contributor: publish straight from the registers, k-group planes apart
            if ((lane & 3) == 0) {
                uint32_t* plane = reinterpret_cast<uint32_t*>(args.partials) + ((size_t)cta * 2 + kgroup) * 128;
                st_relaxed_gpu(plane + col, __float_as_uint(v_lo));
                st_relaxed_gpu(plane + col + 8, __float_as_uint(v_hi));
            }
            continue;
        }
        const int buf = flush & 1;
        if (flush >= 2) named_barrier(4 + buf, kDumpThreads);  // the epilogue warp is done with `buf`
        if ((lane & 3) == 0) {
            float* g = fold_base + buf * 256 + kgroup * 128;
            g[col] = v_lo;
            g[col + 8] = v_hi;
        }
        ++flush;
        if (whole) {
            asm volatile("bar.arrive %0, %1;" ::"r"(2 + buf), "r"(kDumpThreads) : "memory");
            continue;
        }

        // ---- this CTA holds the block's first K range: it finishes the block ----------------
        // (the block goes on in later CTAs, so this is the end of the range)
        int first, last;
        contributors(args.split, blk_lo, blk_hi, first, last);
        const int planes = last - cta;
        float sv[4], bs[4], v[4];
        if (warp == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int cidx = nb * 128 + lane + 32 * j;
                sv[j] = half_bits_to_float(c.w.svh[cidx]);
                bs[j] = c.w.bias ? c.w.bias[cidx] : 0.0f;
            }
        }
        for (int base = 0; base < planes; base += kConsumers) {
            const int p = base + warp;
            if (p < planes) {
                uint4* g0 = reinterpret_cast<uint4*>(args.partials + ((size_t)(cta + 1 + p) * 2) * 128);
                uint4 a, bq;
                if (await_plane(g0, g0 + 32, lane, a, bq)) {
                    float4 sum;  // the contributor's own order: k-group 0 + k-group 1
                    sum.x = __fadd_rn(__uint_as_float(a.x), __uint_as_float(bq.x));
                    sum.y = __fadd_rn(__uint_as_float(a.y), __uint_as_float(bq.y));
                    sum.z = __fadd_rn(__uint_as_float(a.z), __uint_as_float(bq.z));
                    sum.w = __fadd_rn(__uint_as_float(a.w), __uint_as_float(bq.w));
                    reinterpret_cast<float4*>(gathered + warp * 128)[lane] = sum;
                } else if (lane == 0) {
                    atomicOr(c.status, kTimeoutFold);
                    *gave_up = 1;
                }
            }
            named_barrier(1, kConsumers * 32);  // planes of this round (and, first time, the dumps) are in shared memory
            if (warp == 0) {
                if (base == 0) {
                    const float* f0 = fold_base + buf * 256;
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = __fadd_rn(0.f, __fadd_rn(f0[lane + 32 * j], f0[128 + lane + 32 * j]));
                }
                const int n = planes - base < kConsumers ? planes - base : kConsumers;
                for (int q = 0; q < n; ++q) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = __fadd_rn(v[j], gathered[q * 128 + lane + 32 * j]);
                }
            }
            if (base + kConsumers < planes) named_barrier(1, kConsumers * 32);  // before `gathered` is reused
        }
        if (warp == 0 && ok && *gave_up == 0) {  // a wait that ran out leaves the block unwritten
            hadamard128_warp(v, lane);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float value = __fmul_rn(v[j], sv[j]);
                if (c.w.bias) value = __fadd_rn(value, bs[j]);
                scale_and_store(c.y, c.y_dtype, (long long)nb * 128 + lane + 32 * j, value, c.alpha, c.beta);
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
    // the one-row kernel: whole row resident, its own (smaller) header and plane layout
    const bool row_kernel = rows == 1 && hblocks <= act_blocks;
    const int header = row_kernel ? kRowHeader : 16384 + 512;
    const int ring_budget = (int)kGemvSmemLimit - header - act_blocks * 256 * rows;
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
    plan.smem_bytes = header + (size_t)stages * stage_bytes(w.bits) + (size_t)act_blocks * 256 * rows;
    plan.counter_bytes = 0;  // the fold needs no counters
    // one plane per CTA and row; the one-row kernel keeps its two k-group halves apart
    plan.partial_bytes = align_up((size_t)grid * (row_kernel ? 2 : rows) * 128 * sizeof(float));
    return plan;
}

template <int K, int CB, bool ROW>
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
    if (ROW) return cudaLaunchKernelEx(&cfg, gemv_row_kernel<K, CB>, args);
    return cudaLaunchKernelEx(&cfg, gemv_fused_kernel<K, CB>, args);
}

template <int K, int CB>
static cudaError_t launch_one(const GemvArgs& args, int grid, size_t smem, bool pdl, cudaStream_t stream) {
    const bool row_kernel = args.call.rows == 1 && args.call.w.inputs / 128 <= args.act_blocks;
    return row_kernel ? launch_rows<K, CB, true>(args, grid, smem, pdl, stream)
                      : launch_rows<K, CB, false>(args, grid, smem, pdl, stream);
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
    case 9: case 10: case 11:  // 1.5 / 2.5 / 3.5 bits per weight exist for mul1 only
        if constexpr (CB == CB_MUL1) {
            if (a.call.w.bits == 9) return launch_one<9, CB>(a, g, smem, pdl, s);
            if (a.call.w.bits == 10) return launch_one<10, CB>(a, g, smem, pdl, s);
            if (a.call.w.bits == 11) return launch_one<11, CB>(a, g, smem, pdl, s);
        }
        return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
    }
}

// Opt-in dynamic shared memory is a per-device function attribute: set for every instantiation
// when a context is created on a device (configure_device), never on the launch path.
template <int K, int CB>
static cudaError_t configure_rate() {
    cudaError_t e = cudaFuncSetAttribute(gemv_row_kernel<K, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kGemvSmemLimit);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemv_fused_kernel<K, CB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
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
    if constexpr (CB == CB_MUL1) {
        if (e == cudaSuccess) e = configure_rate<9, CB>();
        if (e == cudaSuccess) e = configure_rate<10, CB>();
        if (e == cudaSuccess) e = configure_rate<11, CB>();
    }
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
    switch (call.w.codebook) {
    case CB_3INST: return launch_bits<CB_3INST>(args, plan.grid, plan.smem_bytes, programmatic_launch, stream);
    case CB_MCG: return launch_bits<CB_MCG>(args, plan.grid, plan.smem_bytes, programmatic_launch, stream);
    case CB_MUL1: return launch_bits<CB_MUL1>(args, plan.grid, plan.smem_bytes, programmatic_launch, stream);
    default: return cudaErrorInvalidValue;
    }
}

}  // namespace st
