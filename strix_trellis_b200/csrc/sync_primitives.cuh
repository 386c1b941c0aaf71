// mbarrier / bulk-copy / programmatic-launch primitives for sm_100a, every wait bounded.
#pragma once
#include <stdint.h>

namespace st {

// Bits OR-ed into the context's device status word when a bounded wait gives up
// (host code reads the word with strix_b200_device_status).
enum : unsigned int {
    kTimeoutRingFull = 1u,    // consumer waited for a weight stage that never landed
    kTimeoutRingEmpty = 2u,   // producer waited for a stage that was never released
    kTimeoutDrain = 4u,       // copies still in flight at kernel exit
    kTimeoutTensorPipe = 8u,  // tcgen05 pipeline barrier
    kTimeoutFold = 16u,       // split-K fold waited for a partial plane that never arrived
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// Hardware-suspended wait: the thread sleeps inside try_wait for up to ~2 us per call,
// so a waiting warp costs no issue slots.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(2000u) : "memory");
    return ok != 0;
}
// Bounded: gives up after about a quarter of a second and reports it in `status`.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned int* status,
                                          unsigned int fail_bit) {
    for (uint32_t i = 0; i < (1u << 17); ++i)
        if (mbar_try(bar, parity)) return true;
    if (status) atomicOr(status, fail_bit);
    return false;
}
// Cluster-scope variants for barriers that another CTA of the cluster arrives on.
constexpr uint32_t kClusterWaitHintNs = 100;  // suspend-time hint of one try_wait
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(kClusterWaitHintNs) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, unsigned int* status,
                                                  unsigned int fail_bit) {
    for (uint32_t i = 0; i < (1u << 21); ++i)  // short sleeps: about the same quarter second in total
        if (mbar_try_cluster(bar, parity)) return true;
    if (status) atomicOr(status, fail_bit);
    return false;
}
// Arrive on a barrier given by its shared::cluster address (see map_to_rank).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Word-granular publication between CTAs of one grid: a 32-bit word is either the "empty"
// pattern or a value, so neither a fence nor a flag is needed around it.
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.  Source,
// destination and size are multiples of 16 bytes.  No multicast.
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes,
                                          uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Asks the L2 to fetch `bytes` (a multiple of 16) at the 16-byte aligned `src`; nothing waits
// for it and nothing depends on it.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
// Asks the L2 for the 128-byte line that holds `p`.  The L2 is the point of coherence of the
// device, so a line fetched early and written by another SM afterwards is still read correctly
// from the L2 later.
__device__ __forceinline__ void prefetch_line_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p) : "memory");
}
// Programmatic dependent launch: let the next grid of the stream start its
// independent prologue, and wait for the previous grid's memory before touching
// anything it may have written.  Both are no-ops for an ordinary launch.
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait_prior_grid() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- thread-block cluster: barrier and distributed shared memory -------------------
__device__ __forceinline__ void cluster_sync_all() {
    __syncwarp();  // the .aligned forms need the whole warp converged
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
    return out;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

// Not volatile: the compiler may interleave independent decodes around it.
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

}  // namespace st
