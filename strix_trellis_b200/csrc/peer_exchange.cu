// Exchange between the ranks of one node through peer memory over NVLink: the shard-boundary
// steps of the tensor- and expert-parallel layers (sum of row-parallel outputs, concatenation
// of column-parallel outputs, the two exchanges of an expert-parallel block) as single kernels
// that store straight into the other ranks' memory.  The reference has no inter-rank
// communication at all (README.md:773); its contract for these steps is arithmetic only
// (docs/TP_RANK.md:150-156: sum, concatenate in rank order, combine at the home rank), and that
// contract is what is kept: sums run in ascending rank order from +0 on every rank, so all ranks
// hold the same bits.
//
// Mechanics.  Every rank owns an ARENA (one cudaMalloc) that all other ranks of the node map
// through a CUDA IPC handle.  An arena starts with a control block: an epoch counter per CTA
// slot and, per parity, one flag word per (source rank, CTA slot).  Every exchange kernel runs
// the same number of CTAs on every rank; CTA c
//   1. takes epoch = epoch[c] + 1 (all ranks issue the same sequence of exchanges, so the
//      counters agree without any communication) and uses the data region of parity epoch & 1,
//   2. stores its share of the payload into every destination arena (plain peer stores),
//   3. after a block barrier and a system-scope fence, writes `epoch` into flag
//      [parity][own rank][c] of every rank -- every rank signals every rank, payload or not,
//   4. waits (bounded) until flags [parity][*][c] of its OWN arena hold `epoch`, then reads.
// Alternating parities are what makes the regions reusable: a rank can begin exchange e+2 only
// after it completed e+1, for which every rank had to signal, which each does only after its
// own kernel of exchange e (and everything it enqueued after it) has finished reading.
// No multicast of any kind, no TMA, no spinning without a limit: a wait that runs out sets
// kTimeoutPeer in the context's status word and the kernel ends.
//
// `local_count` consecutive ranks may live in one process on one device (blockIdx.y selects
// the rank a CTA plays).  Production uses one rank per process; hosting all ranks in one
// launch is how the protocol is tested on a single GPU, where kernels that wait for one
// another must not be separate launches.
#include <mutex>

#include "api_internal.h"
#include "sync_primitives.cuh"

using namespace sapi;

namespace {
constexpr int kRanks = STRIX_B200_PEER_MAX_RANKS;
constexpr int kCtas = 32;       // CTA slots of every exchange kernel, per rank
constexpr int kThreads = 256;
constexpr unsigned int kTimeoutPeer = 32u;  // status bit: a peer's flag never arrived
constexpr int kSegments = 3;

struct Control {
    uint32_t epoch[kCtas];
    uint32_t flags[2][kRanks][kCtas];
};
constexpr size_t kControlBytes = (sizeof(Control) + 255) / 256 * 256;
static_assert(kControlBytes == STRIX_B200_PEER_CONTROL_BYTES, "header out of date");

struct PeerView {
    unsigned char* arena[kRanks];  // every rank's arena as mapped into this process
    int world, first_rank;
    unsigned int* status;
    uint32_t wait_polls;  // polls of one wait before it gives up (strix_b200_peer_group_set_wait_polls)
};
constexpr uint32_t kDefaultWaitPolls = 1u << 23;  // several seconds: ranks of one job may be a second apart on the host

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Data that a peer stored: read around the (non-coherent) L1.
__device__ __forceinline__ uint4 ld_sys_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct Turn {
    Control* mine;
    uint32_t epoch;
    int rank;
    __device__ __forceinline__ int parity() const { return (int)(epoch & 1u); }
};

__device__ __forceinline__ Turn exchange_begin(const PeerView& v) {
    __shared__ uint32_t s_epoch;
    Turn t;
    t.rank = v.first_rank + (int)blockIdx.y;
    t.mine = reinterpret_cast<Control*>(v.arena[t.rank]);
    if (threadIdx.x == 0) s_epoch = t.mine->epoch[blockIdx.x] + 1;
    __syncthreads();
    t.epoch = s_epoch;
    return t;
}
// Step 3: everything this CTA stored into other arenas is ordered before the flags.
__device__ __forceinline__ void exchange_signal(const PeerView& v, const Turn& t) {
    __syncthreads();
    if ((int)threadIdx.x < v.world) {
        __threadfence_system();
        Control* there = reinterpret_cast<Control*>(v.arena[threadIdx.x]);
        st_release_sys(&there->flags[t.parity()][t.rank][blockIdx.x], t.epoch);
    }
}
// Step 4, bounded: ranks of one job may be seconds apart on the host (one of them loading or
// checking something), so the limit is several seconds, far beyond any exchange that is going
// to complete; then the status word says so and the CTA skips its reads.
__device__ __forceinline__ bool exchange_wait(const PeerView& v, const Turn& t) {
    __shared__ int s_late;
    if (threadIdx.x == 0) s_late = 0;
    __syncthreads();
    if ((int)threadIdx.x < v.world) {
        const uint32_t* flag = &t.mine->flags[t.parity()][threadIdx.x][blockIdx.x];
        bool seen = false;
        for (uint32_t tries = 0; tries < v.wait_polls && !seen; ++tries) seen = ld_acquire_sys(flag) == t.epoch;
        if (!seen) {
            if (v.status) atomicOr(v.status, kTimeoutPeer);
            s_late = 1;
        }
    }
    __syncthreads();
    return s_late == 0;
}
__device__ __forceinline__ void exchange_end(const Turn& t) {
    __syncthreads();
    if (threadIdx.x == 0) t.mine->epoch[blockIdx.x] = t.epoch;
}

// ---- sum of the ranks' rows ------------------------------------------------------------------
// Small payloads (one to eight rows of a projection's output) are all latency, so this exchange
// does without the flag step: every value travels as an 8-byte word {value, epoch} (8-byte
// stores are not torn), a receiver spins on the words themselves, and the data is there the
// moment it can be trusted -- one NVLink hop instead of payload, fence, flag.  The parities of
// the region alternate as for the other exchanges.
struct ReduceArgs {
    PeerView view;
    float* rows[kRanks];         // per local rank: `count2` pairs of floats, replaced by the sum
    long long count2;
    unsigned long long region;   // byte offset in every arena: [2 parities][world][count2] x 16 bytes
};
__device__ __forceinline__ void st_sys_v4(uint4* p, uint4 v) {
    asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__global__ void __launch_bounds__(kThreads) peer_sum_kernel(const ReduceArgs a) {
    __shared__ int s_late;
    const Turn t = exchange_begin(a.view);
    if (threadIdx.x == 0) s_late = 0;
    float2* y = reinterpret_cast<float2*>(a.rows[blockIdx.y]);
    const long long lane0 = (long long)blockIdx.x * kThreads + threadIdx.x, step = (long long)kCtas * kThreads;
    const long long slot0 = (long long)(a.region / 16) + (long long)t.parity() * a.view.world * a.count2;
    for (long long i = lane0; i < a.count2; i += step) {
        const float2 value = y[i];
        const uint4 word = make_uint4(__float_as_uint(value.x), t.epoch, __float_as_uint(value.y), t.epoch);
        for (int p = 0; p < a.view.world; ++p)
            st_sys_v4(reinterpret_cast<uint4*>(a.view.arena[p]) + slot0 + (long long)t.rank * a.count2 + i, word);
    }
    const uint4* slots = reinterpret_cast<const uint4*>(a.view.arena[t.rank]) + slot0;
    bool late = false;
    for (long long i = lane0; i < a.count2 && !late; i += step) {
        // all ranks' words of this pair are asked for at once; only those that have not landed
        // yet are asked for again
        uint4 part[kRanks];
#pragma unroll
        for (int r = 0; r < kRanks; ++r)
            if (r < a.view.world) part[r] = ld_sys_v4(slots + (long long)r * a.count2 + i);
        float s0 = 0.f, s1 = 0.f;  // ascending rank order from +0, on every rank
#pragma unroll
        for (int r = 0; r < kRanks; ++r) {
            if (r >= a.view.world || late) continue;
            for (uint32_t tries = 0; part[r].y != t.epoch || part[r].w != t.epoch; ++tries) {
                if (tries >= a.view.wait_polls) {  // bounded
                    late = true;
                    break;
                }
                part[r] = ld_sys_v4(slots + (long long)r * a.count2 + i);
            }
            s0 = __fadd_rn(s0, __uint_as_float(part[r].x));
            s1 = __fadd_rn(s1, __uint_as_float(part[r].z));
        }
        if (!late) y[i] = make_float2(s0, s1);
    }
    if (late) {
        if (a.view.status) atomicOr(a.view.status, kTimeoutPeer);
        s_late = 1;
    }
    exchange_end(t);
}

// ---- every rank's block into one matrix on every rank ------------------------------------------
// Up to three matrices of 32-bit words travel in one exchange (an activation matrix with its
// route ids and scores, say); they share the block rows and differ in width.  Rank r's block of
// matrix m is rows[r] x width[m][r] words and lands at (row_at[r], col_at[m][r]) of the
// total_rows x total_cols[m] result.
struct GatherArgs {
    PeerView view;
    int rows[kRanks], row_at[kRanks];  // per global rank
    int total_rows;
    int matrices;
    const uint32_t* block[kSegments][kRanks];  // per local rank: its own block, contiguous
    uint32_t* result[kSegments][kRanks];       // per local rank: private copy of the result, or null (read it in the arena)
    int width[kSegments][kRanks], col_at[kSegments][kRanks];
    int total_cols[kSegments];
    unsigned long long region[kSegments];      // byte offset in every arena: [2 parities][total_rows][total_cols] words
};
__global__ void __launch_bounds__(kThreads) peer_gather_kernel(const GatherArgs a) {
    const Turn t = exchange_begin(a.view);
    const long long lane0 = (long long)blockIdx.x * kThreads + threadIdx.x, step = (long long)kCtas * kThreads;
    for (int m = 0; m < a.matrices; ++m) {
        const int width = a.width[m][t.rank], total = a.total_cols[m];
        const long long words = (long long)a.rows[t.rank] * width;
        const long long base = (long long)(a.region[m] / 4) + (long long)t.parity() * a.total_rows * total;
        const uint32_t* src = a.block[m][blockIdx.y];
        const bool wide = width % 4 == 0 && total % 4 == 0 && a.col_at[m][t.rank] % 4 == 0;
        if (wide) {
            for (long long i = lane0; i < words / 4; i += step) {
                const long long row = (i * 4) / width, col = (i * 4) - row * width;
                const uint4 value = reinterpret_cast<const uint4*>(src)[i];
                const long long at = base + (a.row_at[t.rank] + row) * total + a.col_at[m][t.rank] + col;
                for (int p = 0; p < a.view.world; ++p)
                    *reinterpret_cast<uint4*>(reinterpret_cast<uint32_t*>(a.view.arena[p]) + at) = value;
            }
        } else {
            for (long long i = lane0; i < words; i += step) {
                const long long row = i / width, col = i - row * width;
                const uint32_t value = src[i];
                const long long at = base + (a.row_at[t.rank] + row) * total + a.col_at[m][t.rank] + col;
                for (int p = 0; p < a.view.world; ++p) reinterpret_cast<uint32_t*>(a.view.arena[p])[at] = value;
            }
        }
    }
    exchange_signal(a.view, t);
    if (exchange_wait(a.view, t)) {
        for (int m = 0; m < a.matrices; ++m) {
            uint32_t* out = a.result[m][blockIdx.y];
            if (!out) continue;
            const long long words = (long long)a.total_rows * a.total_cols[m];
            const uint32_t* landed = reinterpret_cast<const uint32_t*>(a.view.arena[t.rank]) + a.region[m] / 4 + (long long)t.parity() * words;
            if (a.total_cols[m] % 4 == 0) {
                // four loads in flight per thread: the copy is latency, not bandwidth
                const uint4* from = reinterpret_cast<const uint4*>(landed);
                uint4* to = reinterpret_cast<uint4*>(out);
                const long long quads = words / 4;
                long long i = lane0;
                for (; i + 3 * step < quads; i += 4 * step) {
                    const uint4 v0 = ld_sys_v4(from + i), v1 = ld_sys_v4(from + i + step);
                    const uint4 v2 = ld_sys_v4(from + i + 2 * step), v3 = ld_sys_v4(from + i + 3 * step);
                    to[i] = v0;
                    to[i + step] = v1;
                    to[i + 2 * step] = v2;
                    to[i + 3 * step] = v3;
                }
                for (; i < quads; i += step) to[i] = ld_sys_v4(from + i);
            } else {
                for (long long i = lane0; i < words; i += step) out[i] = ld_sys_u32(landed + i);
            }
        }
    }
    exchange_end(t);
}

// The same exchange without the fence and the flag step, for results that are copied out anyway:
// every pair of words travels as {word, epoch, word, epoch} (16 bytes, not torn as two 8-byte
// halves), the receiver spins on the words of every rank's block while it copies them out.  The
// region holds [2 parities][total_rows][total_cols] words x 8 bytes.  Widths, column offsets and
// total_cols are even.
__global__ void __launch_bounds__(kThreads) peer_gather_tagged_kernel(const GatherArgs a) {
    __shared__ int s_late;
    const Turn t = exchange_begin(a.view);
    if (threadIdx.x == 0) s_late = 0;
    const long long lane0 = (long long)blockIdx.x * kThreads + threadIdx.x, step = (long long)kCtas * kThreads;
    for (int m = 0; m < a.matrices; ++m) {
        const int width2 = a.width[m][t.rank] / 2, total2 = a.total_cols[m] / 2;
        const long long pairs = (long long)a.rows[t.rank] * width2;
        const long long base = (long long)(a.region[m] / 16) + (long long)t.parity() * a.total_rows * total2;
        const uint2* src = reinterpret_cast<const uint2*>(a.block[m][blockIdx.y]);
        for (long long i = lane0; i < pairs; i += step) {
            const long long row = i / width2, col2 = i - row * width2;
            const uint2 value = src[i];
            const uint4 word = make_uint4(value.x, t.epoch, value.y, t.epoch);
            const long long at = base + (a.row_at[t.rank] + row) * total2 + a.col_at[m][t.rank] / 2 + col2;
            for (int p = 0; p < a.view.world; ++p) st_sys_v4(reinterpret_cast<uint4*>(a.view.arena[p]) + at, word);
        }
    }
    bool late = false;
    for (int m = 0; m < a.matrices && !late; ++m) {
        const int total2 = a.total_cols[m] / 2;
        const uint4* landed = reinterpret_cast<const uint4*>(a.view.arena[t.rank]) + a.region[m] / 16 +
                              (long long)t.parity() * a.total_rows * total2;
        uint2* out = reinterpret_cast<uint2*>(a.result[m][blockIdx.y]);
        for (int r = 0; r < a.view.world && !late; ++r) {  // rank r's block, wherever it lands
            const int width2 = a.width[m][r] / 2;
            const long long pairs = (long long)a.rows[r] * width2;
            const long long origin = (long long)a.row_at[r] * total2 + a.col_at[m][r] / 2;
            for (long long i0 = lane0; i0 < pairs && !late; i0 += 4 * step) {
                uint4 part[4];   // four pairs asked for at once; those not landed yet are asked for again
                long long at[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const long long i = i0 + u * step;
                    const long long row = i / width2;
                    at[u] = origin + row * total2 + (i - row * width2);
                    if (i < pairs) part[u] = ld_sys_v4(landed + at[u]);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (i0 + u * step >= pairs || late) continue;
                    for (uint32_t tries = 0; part[u].y != t.epoch || part[u].w != t.epoch; ++tries) {
                        if (tries >= a.view.wait_polls) {  // bounded
                            late = true;
                            break;
                        }
                        part[u] = ld_sys_v4(landed + at[u]);
                    }
                    if (!late) out[at[u]] = make_uint2(part[u].x, part[u].z);
                }
            }
        }
    }
    if (late) {
        if (a.view.status) atomicOr(a.view.status, kTimeoutPeer);
        s_late = 1;
    }
    exchange_end(t);
}

// ---- routed rows back to the home rank of their token -----------------------------------------
// Tokens are laid out rank-major: token t lives on rank t / tokens_per_rank.  A rank that owns
// the expert of route (t, s) -- id inside its window [first_expert, first_expert + experts) --
// and finds the token's row valid stores the route's output row into the home rank's arena at
// [(t % tokens_per_rank) * top_k + s].
struct ReturnArgs {
    PeerView view;
    const float* each[kRanks];       // per local rank: [tokens * top_k][width] rows this rank computed
    const uint32_t* ids[kRanks];     // per local rank: [tokens][top_k] global expert ids
    const int* row_valid[kRanks];    // per local rank: [tokens]
    int first_expert[kRanks], experts[kRanks];  // per local rank: its window
    int tokens, tokens_per_rank, top_k, width4;
    unsigned long long region;       // byte offset in every arena: [2 parities][tokens_per_rank*top_k][width] floats
};
__global__ void __launch_bounds__(kThreads) peer_return_kernel(const ReturnArgs a) {
    const Turn t = exchange_begin(a.view);
    const int local = blockIdx.y;
    const long long rows_home = (long long)a.tokens_per_rank * a.top_k;
    const long long base4 = (long long)(a.region / 16) + (long long)t.parity() * rows_home * a.width4;
    for (int route = blockIdx.x; route < a.tokens * a.top_k; route += kCtas) {
        const int token = route / a.top_k, slot = route - token * a.top_k;
        if (!a.row_valid[local][token]) continue;
        const uint32_t id = ld_sys_u32(a.ids[local] + route);
        if (id - (uint32_t)a.first_expert[local] >= (uint32_t)a.experts[local]) continue;
        const int home = token / a.tokens_per_rank;
        if (home >= a.view.world) continue;
        const long long at = base4 + ((long long)(token - home * a.tokens_per_rank) * a.top_k + slot) * a.width4;
        const uint4* src = reinterpret_cast<const uint4*>(a.each[local]) + (long long)route * a.width4;
        uint4* dst = reinterpret_cast<uint4*>(a.view.arena[home]) + at;
        for (int i = threadIdx.x; i < a.width4; i += kThreads) dst[i] = src[i];
    }
    exchange_signal(a.view, t);
    (void)exchange_wait(a.view, t);  // the rows of this rank's tokens have landed when the kernel ends
    exchange_end(t);
}

}  // namespace

struct strix_b200_peer_group_impl {
    strix_context owner = nullptr;
    PeerView view{};
    int local_count = 0;
    uint64_t arena_bytes = 0;
    bool mapped[kRanks] = {};  // arenas opened through an IPC handle (closed on destroy)
};

namespace {
strix_status group_call(strix_b200_peer_group g, const strix_stream* stream, cudaStream_t& cs) {
    if (!g) return STRIX_ERROR_INVALID_ARGUMENT;
    const strix_status s = context_check(g->owner);
    if (s != STRIX_SUCCESS) return s;
    // Exchanges are enqueued on hot paths and inside stream captures: the stream descriptor is
    // checked for its header only, as plan submits do with their frozen stream.
    const strix_status h = header(stream);
    if (h != STRIX_SUCCESS) return h;
    cs = static_cast<cudaStream_t>(stream->hip_stream);
    return STRIX_SUCCESS;
}
bool region_fits(strix_b200_peer_group g, uint64_t region, uint64_t bytes) {
    return region >= kControlBytes && region % 256 == 0 && bytes <= g->arena_bytes && region <= g->arena_bytes - bytes;
}
}  // namespace

extern "C" {

strix_status strix_b200_peer_arena_create(strix_context c, uint64_t bytes, void** arena, unsigned char* handle) {
    if (arena) *arena = nullptr;
    if (!arena || !handle || bytes < kControlBytes || bytes > SIZE_MAX) return STRIX_ERROR_INVALID_ARGUMENT;
    const strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    static_assert(sizeof(cudaIpcMemHandle_t) == STRIX_B200_PEER_HANDLE_BYTES, "handle size");
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, (size_t)bytes);  // epochs and flags start at zero
    cudaIpcMemHandle_t h{};
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        if (p) (void)cudaFree(p);
        return cuda_status(e);
    }
    std::memcpy(handle, &h, sizeof h);
    *arena = p;
    return STRIX_SUCCESS;
}

strix_status strix_b200_peer_arena_destroy(strix_context c, void* arena) {
    const strix_status s = context_check(c);
    if (s != STRIX_SUCCESS || !arena) return s != STRIX_SUCCESS ? s : STRIX_ERROR_INVALID_ARGUMENT;
    return cuda_status(cudaFree(arena));
}

strix_status strix_b200_peer_group_create(strix_context c, void* const* local_arenas, uint32_t local_count,
                                          uint32_t first_rank, uint64_t arena_bytes, const unsigned char* handles,
                                          uint32_t world, strix_b200_peer_group* out) {
    if (out) *out = nullptr;
    if (!out || !local_arenas || world < 1 || world > (uint32_t)kRanks || local_count < 1 ||
        first_rank + local_count > world || arena_bytes < kControlBytes)
        return STRIX_ERROR_INVALID_ARGUMENT;
    if (local_count < world && !handles) return STRIX_ERROR_INVALID_ARGUMENT;
    const strix_status s = context_check(c);
    if (s != STRIX_SUCCESS) return s;
    strix_b200_peer_group_impl* g = new (std::nothrow) strix_b200_peer_group_impl;
    if (!g) return STRIX_ERROR_OUT_OF_MEMORY;
    g->owner = c;
    g->local_count = (int)local_count;
    g->arena_bytes = arena_bytes;
    g->view.world = (int)world;
    g->view.first_rank = (int)first_rank;
    g->view.status = c->status;
    g->view.wait_polls = kDefaultWaitPolls;
    cudaError_t e = cudaSuccess;
    for (uint32_t r = 0; r < world && e == cudaSuccess; ++r) {
        if (r >= first_rank && r < first_rank + local_count) {
            if (!local_arenas[r - first_rank]) e = cudaErrorInvalidValue;
            g->view.arena[r] = static_cast<unsigned char*>(local_arenas[r - first_rank]);
            continue;
        }
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles + (size_t)r * STRIX_B200_PEER_HANDLE_BYTES, sizeof h);
        void* p = nullptr;
        e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e == cudaSuccess) {
            g->view.arena[r] = static_cast<unsigned char*>(p);
            g->mapped[r] = true;
        }
    }
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        for (int r = 0; r < kRanks; ++r)
            if (g->mapped[r]) (void)cudaIpcCloseMemHandle(g->view.arena[r]);
        delete g;
        return cuda_status(e);
    }
    *out = g;
    return STRIX_SUCCESS;
}

strix_status strix_b200_peer_group_set_wait_polls(strix_b200_peer_group g, uint32_t polls) {
    if (!g || polls == 0) return STRIX_ERROR_INVALID_ARGUMENT;
    g->view.wait_polls = polls;
    return STRIX_SUCCESS;
}

strix_status strix_b200_peer_group_destroy(strix_b200_peer_group g) {
    if (!g) return STRIX_ERROR_INVALID_ARGUMENT;
    const strix_status s = context_check(g->owner);
    if (s != STRIX_SUCCESS) return s;
    for (int r = 0; r < kRanks; ++r)
        if (g->mapped[r]) (void)cudaIpcCloseMemHandle(g->view.arena[r]);
    delete g;
    return STRIX_SUCCESS;
}

strix_status strix_b200_peer_sum(strix_b200_peer_group g, float* const* rows, uint64_t count, uint64_t region,
                                 const strix_stream* stream) {
    cudaStream_t cs{};
    const strix_status s = group_call(g, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    if (!rows || count % 2 || count > (1ull << 40)) return STRIX_ERROR_INVALID_ARGUMENT;
    if (!count) return STRIX_SUCCESS;
    if (!region_fits(g, region, 2ull * g->view.world * count * 8)) return STRIX_ERROR_INSUFFICIENT_BUFFER;
    ReduceArgs a{};
    a.view = g->view;
    a.count2 = (long long)(count / 2);
    a.region = region;
    for (int i = 0; i < g->local_count; ++i) {
        if (!rows[i] || reinterpret_cast<uintptr_t>(rows[i]) % 8) return STRIX_ERROR_INVALID_ARGUMENT;
        a.rows[i] = rows[i];
    }
    peer_sum_kernel<<<dim3(kCtas, g->local_count), kThreads, 0, cs>>>(a);
    return cuda_status(cudaGetLastError());
}

strix_status strix_b200_peer_gather(strix_b200_peer_group g, const strix_b200_peer_gather_desc* d,
                                    const strix_stream* stream) {
    cudaStream_t cs{};
    strix_status s = group_call(g, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (d->matrices < 1 || d->matrices > (uint32_t)kSegments || (d->flags & ~(uint32_t)STRIX_B200_PEER_GATHER_TAGGED))
        return STRIX_ERROR_INVALID_ARGUMENT;
    const bool tagged = (d->flags & STRIX_B200_PEER_GATHER_TAGGED) != 0;
    GatherArgs a{};
    a.view = g->view;
    a.matrices = (int)d->matrices;
    uint64_t total_rows = 0;
    for (int r = 0; r < g->view.world; ++r) {
        if (d->rows[r] > INT_MAX || d->row_at[r] > INT_MAX) return STRIX_ERROR_INVALID_ARGUMENT;
        a.rows[r] = (int)d->rows[r];
        a.row_at[r] = (int)d->row_at[r];
        total_rows = std::max<uint64_t>(total_rows, (uint64_t)d->row_at[r] + d->rows[r]);
    }
    if (total_rows > INT_MAX) return STRIX_ERROR_INVALID_ARGUMENT;
    a.total_rows = (int)total_rows;
    for (int m = 0; m < a.matrices; ++m) {
        const strix_b200_peer_matrix& mx = d->matrix[m];
        if (mx.total_cols < 1 || mx.total_cols > INT_MAX) return STRIX_ERROR_INVALID_ARGUMENT;
        a.total_cols[m] = (int)mx.total_cols;
        a.region[m] = mx.region;
        if (!region_fits(g, mx.region, 2ull * total_rows * mx.total_cols * (tagged ? 8 : 4)))
            return STRIX_ERROR_INSUFFICIENT_BUFFER;
        if (tagged && mx.total_cols % 2) return STRIX_ERROR_INVALID_ARGUMENT;
        for (int r = 0; r < g->view.world; ++r) {
            if ((uint64_t)mx.col_at[r] + mx.width[r] > mx.total_cols) return STRIX_ERROR_INVALID_ARGUMENT;
            if (tagged && (mx.width[r] % 2 || mx.col_at[r] % 2)) return STRIX_ERROR_INVALID_ARGUMENT;
            a.width[m][r] = (int)mx.width[r];
            a.col_at[m][r] = (int)mx.col_at[r];
        }
        for (int i = 0; i < g->local_count; ++i) {
            const int r = g->view.first_rank + i;
            if ((!mx.block[i] && a.rows[r] && a.width[m][r]) || reinterpret_cast<uintptr_t>(mx.block[i]) % 16 ||
                reinterpret_cast<uintptr_t>(mx.result[i]) % 16)
                return STRIX_ERROR_INVALID_ARGUMENT;
            if (tagged && !mx.result[i]) return STRIX_ERROR_INVALID_ARGUMENT;  // tagged words are of no use in place
            a.block[m][i] = static_cast<const uint32_t*>(mx.block[i]);
            a.result[m][i] = static_cast<uint32_t*>(mx.result[i]);
        }
    }
    if (tagged) peer_gather_tagged_kernel<<<dim3(kCtas, g->local_count), kThreads, 0, cs>>>(a);
    else peer_gather_kernel<<<dim3(kCtas, g->local_count), kThreads, 0, cs>>>(a);
    return cuda_status(cudaGetLastError());
}

strix_status strix_b200_peer_return_routes(strix_b200_peer_group g, const strix_b200_peer_return_desc* d,
                                           const strix_stream* stream) {
    cudaStream_t cs{};
    strix_status s = group_call(g, stream, cs);
    if (s != STRIX_SUCCESS) return s;
    s = header(d);
    if (s != STRIX_SUCCESS) return s;
    if (d->tokens_per_rank < 1 || d->top_k < 1 || d->top_k > STRIX_B200_MOE_MAX_TOP_K || d->width < 4 || d->width % 4 ||
        d->width > INT_MAX || d->tokens > STRIX_B200_MOE_MAX_ROWS ||
        (uint64_t)d->tokens_per_rank * g->view.world < d->tokens)
        return STRIX_ERROR_INVALID_ARGUMENT;
    if (!region_fits(g, d->region, 2ull * d->tokens_per_rank * d->top_k * d->width * 4)) return STRIX_ERROR_INSUFFICIENT_BUFFER;
    ReturnArgs a{};
    a.view = g->view;
    a.tokens = (int)d->tokens;
    a.tokens_per_rank = (int)d->tokens_per_rank;
    a.top_k = (int)d->top_k;
    a.width4 = (int)(d->width / 4);
    a.region = d->region;
    for (int i = 0; i < g->local_count; ++i) {
        if (!d->each[i] || !d->ids[i] || !d->row_valid[i] || reinterpret_cast<uintptr_t>(d->each[i]) % 16)
            return STRIX_ERROR_INVALID_ARGUMENT;
        a.each[i] = d->each[i];
        a.ids[i] = d->ids[i];
        a.row_valid[i] = d->row_valid[i];
        a.first_expert[i] = (int)d->first_expert[i];
        a.experts[i] = (int)d->experts[i];
    }
    peer_return_kernel<<<dim3(kCtas, g->local_count), kThreads, 0, cs>>>(a);
    return cuda_status(cudaGetLastError());
}

}  // extern "C"
