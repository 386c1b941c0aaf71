// Grouped fused linears (see grouped.h).  One CTA = (problem, 128-column block, K
// partition): a producer warp streams the contiguous weight bytes of that partition through
// a shared-memory ring (1-D bulk copies), eight decode warps each own a 16-column tile and
// feed mma.sync.m16n8k16; partial planes go to the problem's scratch and the last CTA of a
// column block to arrive folds them in ascending K order and applies the output stages.
// Same arithmetic per row as the single-layer GEMV; only the work split differs.  Replaces
// the reference's per-expert projection kernels (src/tp_moe.hip:60-164,
// src/tp_fused_device.hpp:19-126) and its grouped strided GEMV (src/dense_r1_group*.hip).
#include "grouped.h"
#include "hadamard.cuh"
#include "sync_primitives.cuh"
#include "trellis_decode.cuh"

namespace st {

namespace {
constexpr int kWarps = 8;
constexpr int kThreadsG = (kWarps + 1) * 32;
constexpr int kMaxStages = 16;
constexpr int kMaxSplits = 16;
constexpr size_t kGroupedSmemLimit = 110 * 1024;  // dynamic shared memory a launch may ask for (two CTAs per SM)

struct GroupedArgs {
    const GroupedProblem* problems;
    int ctas_per_problem;
    int splits;
    int stages;
    int hblocks;
    int stage_stride;  // bytes between ring slots (sized for the largest rate in the group)
    unsigned int* status;
};

// Decode loop of one CTA for rate K.  Returns false when a bounded wait gave up.
template <int K, int CB>
__device__ __forceinline__ bool consume(const unsigned char* ring, int stage_stride, int stages, int nblk, uint32_t full0,
                                        uint32_t empty0, const uint2* act_lane, int rows, int warp, int lane,
                                        unsigned int* status, float (&acc)[2][4]) {
    const LaneGeom<K> geom(lane);
    int st = 0;
    uint32_t use = 0;  // ring slot and use parity of unit i, stepped without divisions
    for (int i = 0; i < nblk; ++i, st = (st + 1 == stages ? 0 : st + 1), use ^= (st == 0)) {
        if (!mbar_wait(full0 + 8 * st, use, status, kTimeoutRingFull)) return false;
        const uint32_t* tiles = reinterpret_cast<const uint32_t*>(ring + (size_t)st * stage_stride) + warp * tile_words(K);
        const uint2* bsrc = act_lane + (size_t)i * rows * 32;
#pragma unroll
        for (int kt = 0; kt < 8; kt += 2) {
            uint32_t fa[4], fb[4];
            decode_tile_frag<K, CB>(tiles + kt * 8 * tile_words(K), geom, fa);
            decode_tile_frag<K, CB>(tiles + (kt + 1) * 8 * tile_words(K), geom, fb);
            const uint2 ba = bsrc[kt * 4], bb = bsrc[(kt + 1) * 4];
            mma_16816(acc[0], fa, ba.x, ba.y);
            mma_16816(acc[1], fb, bb.x, bb.y);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty0 + 8 * st);
    }
    return true;
}
}  // namespace

template <int CB>
__global__ void __launch_bounds__(kThreadsG, 2) grouped_linear_kernel(const GroupedArgs args) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int pidx = blockIdx.x / args.ctas_per_problem, rem = blockIdx.x % args.ctas_per_problem;
    const GroupedProblem& pr = args.problems[pidx];
    // problem tables may have been written by the prior grid (device routing)
    pdl_wait_prior_grid();
    const int rows = pr.rows;
    if (rows == 0) return;
    const DeviceWeights w = pr.w;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb = rem / args.splits, split = rem % args.splits;
    const int hblocks = args.hblocks;
    const int hb_begin = (int)((long long)hblocks * split / args.splits);
    const int hb_end = (int)((long long)hblocks * (split + 1) / args.splits);
    const int nblk = hb_end - hb_begin;
    const int stages = args.stages;
    const int stage_bytes = unit_bytes(w.bits);

    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    unsigned char* ring = smem + 256;
    uint2* act = reinterpret_cast<uint2*>(ring + (size_t)stages * args.stage_stride);
    __shared__ int s_last, s_abort;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kMaxStages);
    if (threadIdx.x == 0) {
        for (int i = 0; i < stages; ++i) {
            mbar_init(full0 + 8 * i, 1);
            mbar_init(empty0 + 8 * i, kWarps);
        }
        mbar_fence_init();
        s_abort = 0;
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kWarps) {
        if (lane == 0) {
            const unsigned char* stream = reinterpret_cast<const unsigned char*>(w.packed) +
                ((size_t)nb * hblocks + hb_begin) * stage_bytes;
            int issued = 0;
            for (int i = 0; i < nblk; ++i) {
                const int st = i % stages;
                if (i >= stages && !mbar_wait(empty0 + 8 * st, (uint32_t)((i / stages) - 1) & 1, args.status, kTimeoutRingEmpty)) {
                    s_abort = 1;
                    break;
                }
                mbar_expect_tx(full0 + 8 * st, stage_bytes);
                bulk_load(smem_u32(ring + (size_t)st * args.stage_stride), stream + (size_t)i * stage_bytes, stage_bytes,
                          full0 + 8 * st);
                issued = i + 1;
            }
            for (int i = (issued > stages ? issued - stages : 0); i < issued; ++i)
                mbar_wait(full0 + 8 * (i % stages), (uint32_t)(i / stages) & 1, args.status, kTimeoutDrain);
        }
    } else {
        // input stages of the gathered rows for this K partition, in B-fragment order
        __half* act_h = reinterpret_cast<__half*>(act);
        for (int item = warp; item < rows * nblk; item += kWarps) {
            const int r = item / nblk, blk = item % nblk;
            const float* xr = pr.x + (long long)pr.x_row[r] * pr.x_stride + (size_t)(hb_begin + blk) * 128;
            const uint16_t* su = w.suh + (size_t)(hb_begin + blk) * 128;
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = __half2float(scale_input(xr[lane + 32 * j], su[lane + 32 * j]));
            hadamard128_warp(v, lane);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int e = lane + 32 * j, kt = e >> 4, kk = e & 15;
                const int q = (kk & 7) >> 1, hi = kk >> 3, lo = kk & 1;
                act_h[((((size_t)blk * rows + r) * 8 + kt) * 4 + q) * 4 + hi * 2 + lo] = __float2half_rn(v[j]);
            }
        }
        named_barrier(1, kWarps * 32);

        float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const int brow = (lane >> 2) < rows ? (lane >> 2) : rows - 1;
        const uint2* act_lane = act + brow * 32 + (lane & 3);
        bool ok;
        switch (w.bits) {
        case 1: ok = consume<1, CB>(ring, args.stage_stride, stages, nblk, full0, empty0, act_lane, rows, warp, lane, args.status, acc); break;
        case 2: ok = consume<2, CB>(ring, args.stage_stride, stages, nblk, full0, empty0, act_lane, rows, warp, lane, args.status, acc); break;
        case 3: ok = consume<3, CB>(ring, args.stage_stride, stages, nblk, full0, empty0, act_lane, rows, warp, lane, args.status, acc); break;
        case 4: ok = consume<4, CB>(ring, args.stage_stride, stages, nblk, full0, empty0, act_lane, rows, warp, lane, args.status, acc); break;
        case 5: ok = consume<5, CB>(ring, args.stage_stride, stages, nblk, full0, empty0, act_lane, rows, warp, lane, args.status, acc); break;
        case 6: ok = consume<6, CB>(ring, args.stage_stride, stages, nblk, full0, empty0, act_lane, rows, warp, lane, args.status, acc); break;
        case 7: ok = consume<7, CB>(ring, args.stage_stride, stages, nblk, full0, empty0, act_lane, rows, warp, lane, args.status, acc); break;
        case 8: ok = consume<8, CB>(ring, args.stage_stride, stages, nblk, full0, empty0, act_lane, rows, warp, lane, args.status, acc); break;
        default:  // half-integer rates exist for mul1 only
            if constexpr (CB == CB_MUL1) {
                if (w.bits == 9) ok = consume<9, CB>(ring, args.stage_stride, stages, nblk, full0, empty0, act_lane, rows, warp, lane, args.status, acc);
                else if (w.bits == 10) ok = consume<10, CB>(ring, args.stage_stride, stages, nblk, full0, empty0, act_lane, rows, warp, lane, args.status, acc);
                else ok = consume<11, CB>(ring, args.stage_stride, stages, nblk, full0, empty0, act_lane, rows, warp, lane, args.status, acc);
            } else {
                ok = false;
            }
            break;
        }
        if (!ok) s_abort = 1;
        const int col = warp * 16 + (lane >> 2), r0 = 2 * (lane & 3);
        float* p = pr.partials + (((size_t)nb * args.splits + split) * rows) * 128;
        const float v00 = acc[0][0] + acc[1][0], v01 = acc[0][1] + acc[1][1];
        const float v10 = acc[0][2] + acc[1][2], v11 = acc[0][3] + acc[1][3];
        if (r0 < rows) { p[r0 * 128 + col] = v00; p[r0 * 128 + col + 8] = v10; }
        if (r0 + 1 < rows) { p[(r0 + 1) * 128 + col] = v01; p[(r0 + 1) * 128 + col + 8] = v11; }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // one release/acquire atomic: the CTA's planes (ordered before it by the barrier) are
        // visible before the count, and the last arriver sees the planes of the others
        unsigned int seen;
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(seen) : "l"(pr.counters + nb) : "memory");
        const int last = (seen == (unsigned int)args.splits - 1);
        if (last) pr.counters[nb] = 0;  // visible at grid end, before any later launch
        s_last = last && !s_abort;
    }
    __syncthreads();
    if (!s_last || warp >= rows) return;
    {
        const int r = warp;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < args.splits; ++s) {
            const float* p = pr.partials + (((size_t)nb * args.splits + s) * rows + r) * 128;
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = __fadd_rn(v[j], __ldcg(p + lane + 32 * j));
        }
        hadamard128_warp(v, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cidx = nb * 128 + lane + 32 * j;
            float* out = pr.y + (long long)pr.y_row[r] * pr.y_stride + cidx;
            *out = finish_output(v[j], w.svh[cidx], w.bias, cidx, 1.0f, 0.0f, out);
        }
    }
}

namespace {
constexpr int kBlocksPerCta = 32;  // H128 blocks of K per CTA: 8 rows x 32 blocks x 256 B = 64 KB of core input

// Among the K partition counts up to `most`, the one with the least estimated time in units of
// one decoded unit on one SM: the CTAs' work spread over the SMs (two CTAs share an SM and its
// issue slots; a CTA costs about one unit beyond its own) plus the half-empty tail of the last
// CTAs.  `problems` is the number of problems the caller EXPECTS to be live.  Fitted to the
// routed-expert block at 1 / 8 / 64 tokens, where 2-4 / 2 / 1 partitions measured best.
int choose_splits(int hblocks, int nblocks, int problems, int sm_count, int most) {
    const int min_splits = (hblocks + kBlocksPerCta - 1) / kBlocksPerCta;
    int splits = min_splits;
    double best = -1.0;
    for (int s = min_splits; s <= hblocks && s <= most; s *= 2) {
        const double ctas = (double)problems * nblocks * s, each = (double)((hblocks + s - 1) / s) + 1.0;
        const double cost = ctas * each / sm_count + 0.5 * each;
        if (best < 0.0 || cost < best) { best = cost; splits = s; }
    }
    return splits;
}

// Everything of a plan that follows from its partition count.
void shape_plan(GroupedPlan& plan, int hblocks, int nblocks, int max_bits, int splits) {
    const int per = (hblocks + splits - 1) / splits;
    int stages = (32 * 1024) / unit_bytes(max_bits);
    if (stages > per) stages = per;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 1) stages = 1;
    plan.splits = splits;
    plan.stages = stages;
    plan.ctas_per_problem = nblocks * splits;
    plan.stage_stride = unit_bytes(max_bits);
    plan.smem_bytes = 256 + (size_t)stages * plan.stage_stride + (size_t)per * 256 * kGroupRows;
}
}  // namespace

GroupedPlan plan_grouped(int inputs, int outputs, int max_bits, int problems, int sm_count, int headroom) {
    GroupedPlan plan{};
    const int hblocks = inputs / 128, nblocks = outputs / 128;
    const int splits = choose_splits(hblocks, nblocks, problems, sm_count, kMaxSplits);
    shape_plan(plan, hblocks, nblocks, max_bits, splits);
    int room = splits * (headroom < 1 ? 1 : headroom);  // partitions the scratch is sized for
    if (room > kMaxSplits) room = kMaxSplits;
    if (room > hblocks) room = hblocks;
    if (room < splits) room = splits;
    plan.scratch_splits = room;
    plan.counter_bytes_per_problem = align_up((size_t)nblocks * sizeof(unsigned int));
    plan.partial_bytes_per_problem = align_up((size_t)nblocks * room * kGroupRows * 128 * sizeof(float));
    return plan;
}

GroupedPlan replan_grouped(const GroupedPlan& sized, int inputs, int outputs, int max_bits, int problems, int sm_count) {
    GroupedPlan plan = sized;  // the scratch figures stay: they describe memory that exists
    const int hblocks = inputs / 128, nblocks = outputs / 128;
    shape_plan(plan, hblocks, nblocks, max_bits, choose_splits(hblocks, nblocks, problems, sm_count, sized.scratch_splits));
    return plan;
}

// Opt-in dynamic shared memory is a per-device function attribute: set when a context is created
// on a device (configure_device), never on the launch path.
cudaError_t configure_grouped_kernels() {
    cudaError_t e = cudaFuncSetAttribute(grouped_linear_kernel<CB_3INST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGroupedSmemLimit);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_linear_kernel<CB_MCG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGroupedSmemLimit);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(grouped_linear_kernel<CB_MUL1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGroupedSmemLimit);
    return e;
}

template <int CB>
static cudaError_t launch_grouped_cb(const GroupedArgs& args, int grid, size_t smem, bool pdl, cudaStream_t stream) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreadsG);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, grouped_linear_kernel<CB>, args);
}

cudaError_t launch_grouped(const GroupedProblem* problems, int problem_count, int inputs, int outputs,
                           int codebook, const GroupedPlan& plan, unsigned int* status, bool programmatic,
                           cudaStream_t stream) {
    if (problem_count <= 0) return cudaSuccess;
    (void)outputs;
    GroupedArgs args{problems, plan.ctas_per_problem, plan.splits, plan.stages, inputs / 128, plan.stage_stride, status};
    const long long grid = (long long)problem_count * plan.ctas_per_problem;
    if (grid > 0x7FFFFFFF || plan.smem_bytes > kGroupedSmemLimit) return cudaErrorInvalidValue;
    switch (codebook) {
    case CB_3INST: return launch_grouped_cb<CB_3INST>(args, (int)grid, plan.smem_bytes, programmatic, stream);
    case CB_MCG: return launch_grouped_cb<CB_MCG>(args, (int)grid, plan.smem_bytes, programmatic, stream);
    case CB_MUL1: return launch_grouped_cb<CB_MUL1>(args, (int)grid, plan.smem_bytes, programmatic, stream);
    default: return cudaErrorInvalidValue;
    }
}

// ---- SwiGLU and routed-expert combine --------------------------------------------------------
__global__ void swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up,
                              float* __restrict__ hidden, long long count, int width, long long out_stride) {
    pdl_wait_prior_grid();  // gate / up come from the launch before
    pdl_launch_dependents();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x) {
        const float g = gate[i];
        const float e = expf(g < 0.0f ? g : -g);  // stable sigmoid
        const float d = __fadd_rn(1.0f, e);
        const float sig = g < 0.0f ? __fdiv_rn(e, d) : __fdiv_rn(1.0f, d);
        hidden[(i / width) * out_stride + (i % width)] = __fmul_rn(__fmul_rn(g, sig), up[i]);
    }
}

// A small kernel of a routed-expert submit: launched programmatically when the context allows
// it, so that it is resident and waiting when the launch before it ends.
template <class... Params, class... Args>
static cudaError_t launch_small(void (*kernel)(Params...), int grid, int block, bool programmatic, cudaStream_t stream,
                                Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

cudaError_t launch_swiglu(const float* gate, const float* up, float* hidden, int rows, int width,
                          long long out_stride, bool programmatic, cudaStream_t stream) {
    const long long count = (long long)rows * width;
    if (count <= 0) return cudaSuccess;
    const long long want = (count + 255) / 256;
    return launch_small(swiglu_kernel, streaming_grid(want), 256, programmatic, stream, gate, up, hidden, count, width,
                        out_stride);
}

// Device-side routing, one CTA.  A row is valid when its ids are in range and distinct and
// its scores are finite and non-negative (src/tp_moe_routes.hpp:46-61); slots of invalid
// rows run nothing.  Valid routes are grouped by expert into problems of up to eight rows,
// so an expert's weights are streamed once per eight routed rows, not once per route.  A
// row's result does not depend on which problem slot or row position carries it.
// Zero-score routes are computed like any other; the combine skips them.
__global__ void __launch_bounds__(1024) moe_route_kernel(const unsigned int* __restrict__ ids,
                                                         const float* __restrict__ scores, int tokens, int top_k,
                                                         const MoeBankEntry* __restrict__ bank, int bank_count,
                                                         const MoeWindow window, GroupedProblem* gate_up,
                                                         GroupedProblem* down, int* row_valid) {
    __shared__ int count[1024], first_problem[1024], cursor[1024], warp_total[32];
    const int tid = threadIdx.x, routes = tokens * top_k;
    count[tid] = 0;
    cursor[tid] = 0;
    pdl_wait_prior_grid();  // ids and scores may come from the launch before
    pdl_launch_dependents();
    __syncthreads();
    for (int t = tid; t < tokens; t += 1024) {
        bool valid = true;
        for (int s = 0; s < top_k && valid; ++s) {
            const unsigned int id = ids[t * top_k + s];
            const float sc = scores[t * top_k + s];
            if (id >= (unsigned int)window.experts_total || !(sc >= 0.0f && sc <= 3.402823466e+38f)) valid = false;
            for (int q = 0; q < s && valid; ++q)
                if (ids[t * top_k + q] == id) valid = false;
        }
        row_valid[t] = valid ? 1 : 0;
        if (valid)
            for (int s = 0; s < top_k; ++s) {  // routes to experts of another rank run nothing here
                const unsigned int e = ids[t * top_k + s] - (unsigned int)window.first_expert;
                if (e < (unsigned int)bank_count) atomicAdd(&count[e], 1);
            }
    }
    __syncthreads();
    const int n = tid < bank_count ? count[tid] : 0;
    const int problems = (n + kGroupRows - 1) / kGroupRows;
    // inclusive scan of problems per expert: within a warp by shuffles, then over the 32 warp totals
    int incl = problems;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int up = __shfl_up_sync(0xFFFFFFFFu, incl, off);
        if ((tid & 31) >= off) incl += up;
    }
    if ((tid & 31) == 31) warp_total[tid >> 5] = incl;
    __syncthreads();
    if (tid < 32) {
        int w = warp_total[tid];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int up = __shfl_up_sync(0xFFFFFFFFu, w, off);
            if (tid >= off) w += up;
        }
        warp_total[tid] = w;
    }
    __syncthreads();
    const int before = (tid >> 5) ? warp_total[(tid >> 5) - 1] : 0;
    const int begin = before + incl - problems, total = warp_total[31];
    first_problem[tid] = begin;
    for (int k = 0; k < problems; ++k) {
        const int q = begin + k;
        const int rows = n - k * kGroupRows < kGroupRows ? n - k * kGroupRows : kGroupRows;
        gate_up[2 * q].rows = gate_up[2 * q + 1].rows = down[q].rows = rows;
        gate_up[2 * q].w = bank[tid].gate;
        gate_up[2 * q + 1].w = bank[tid].up;
        down[q].w = bank[tid].down;
    }
    for (int q = total + tid; q < routes; q += 1024)  // unused slots run nothing
        gate_up[2 * q].rows = gate_up[2 * q + 1].rows = down[q].rows = 0;
    __syncthreads();
    for (int r = tid; r < routes; r += 1024) {
        const int t = r / top_k;
        if (!row_valid[t]) continue;
        const unsigned int local = ids[r] - (unsigned int)window.first_expert;
        if (local >= (unsigned int)bank_count) continue;
        const int e = (int)local;
        const int pos = atomicAdd(&cursor[e], 1);
        const int q = first_problem[e] + pos / kGroupRows, j = pos % kGroupRows;
        gate_up[2 * q].x_row[j] = gate_up[2 * q + 1].x_row[j] = t;
        gate_up[2 * q].y_row[j] = gate_up[2 * q + 1].y_row[j] = r;
        down[q].x_row[j] = down[q].y_row[j] = r;
    }
}

cudaError_t launch_moe_route(const unsigned int* route_ids, const float* route_scores, int tokens, int top_k,
                             const MoeBankEntry* bank, int bank_count, MoeWindow window, GroupedProblem* gate_up,
                             GroupedProblem* down, int* row_valid, bool programmatic, cudaStream_t stream) {
    if (bank_count > 1024 || window.first_expert < 0 || window.experts_total < window.first_expert + bank_count)
        return cudaErrorInvalidValue;
    return launch_small(moe_route_kernel, 1, 1024, programmatic, stream, route_ids, route_scores, tokens, top_k, bank,
                        bank_count, window, gate_up, down, row_valid);
}

__global__ void moe_combine_kernel(const float* __restrict__ each, const float* __restrict__ scores,
                                   const int* __restrict__ row_valid, int tokens, int top_k, int outputs,
                                   float* y, long long y_stride, float alpha, float beta,
                                   const unsigned int* __restrict__ route_ids, int first_expert, int bank_count) {
    pdl_wait_prior_grid();  // the routed rows come from the launch before
    pdl_launch_dependents();
    const long long total = (long long)tokens * outputs;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / outputs), n = (int)(i % outputs);
        float* out = y + (long long)t * y_stride + n;
        if (row_valid && !row_valid[t]) {
            *out = __int_as_float(0x7fc00000);
            continue;
        }
        float sum = 0.0f;
        for (int s = 0; s < top_k; ++s) {  // ascending slot order from +0
            const float score = scores[t * top_k + s];
            if (score == 0.0f) continue;
            if (route_ids && route_ids[t * top_k + s] - (unsigned int)first_expert >= (unsigned int)bank_count) continue;
            sum = __fadd_rn(sum, __fmul_rn(score, each[((long long)t * top_k + s) * outputs + n]));
        }
        float value = __fmul_rn(alpha, sum);
        if (beta != 0.0f) value = __fadd_rn(value, __fmul_rn(beta, *out));
        *out = value;
    }
}

cudaError_t launch_moe_combine(const float* each, const float* scores, const int* row_valid, int tokens,
                               int top_k, int outputs, float* y, long long y_stride, float alpha, float beta,
                               bool programmatic, cudaStream_t stream, const unsigned int* route_ids, int first_expert,
                               int bank_count) {
    const long long total = (long long)tokens * outputs;
    if (total <= 0) return cudaSuccess;
    const long long want = (total + 255) / 256;
    return launch_small(moe_combine_kernel, streaming_grid(want), 256, programmatic, stream, each, scores, row_valid, tokens,
                        top_k, outputs, y, y_stride, alpha, beta, route_ids, first_expert, bank_count);
}

}  // namespace st
