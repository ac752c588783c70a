// Thin inline-PTX wrappers for the sm_100a features the skinny GEMM uses: mbarrier, TMA tiled
// loads, tcgen05 (TMEM allocation, MMA, commit, load), thread-block-cluster barriers and
// distributed shared memory, programmatic dependent launch. Nothing here is generic: each
// wrapper is the one form of the instruction this library issues.
#pragma once

#include <cuda.h>
#include <stdint.h>

namespace hfrk {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(arrivals) : "memory");
}

// Makes freshly initialised barriers visible to the async proxy (TMA, tcgen05.commit) and to the
// other CTAs of a cluster.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// One 2-D tiled load into this CTA's shared memory; completion is counted in bytes on `bar`.
// x is the innermost (contiguous) coordinate and must be a multiple of 16 elements for 8-bit data.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar,
                                            int x, int y, uint64_t l2_policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y),
          "l"(l2_policy)
        : "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t result_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem),
                 "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish_alloc_permit() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns)
                 : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tcgen05_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (the layout a TMA load with CU_TENSOR_MAP_SWIZZLE_128B and a 128-byte inner box
// produces). Eight rows form one 1024-byte swizzle group; groups follow each other at 1024 bytes.
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4 (unused here, 1)
//   bits [32,46) stride byte offset >> 4   bits [46,48) descriptor version (1 on sm_100)
//   bits [61,64) layout type (2 = 128-byte swizzle)
__device__ __forceinline__ uint64_t umma_desc_kmajor_sw128(uint32_t tile_smem) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((tile_smem & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor for tcgen05.mma kind::f8f6f4, e4m3 x e4m3 -> f32, both operands K-major.
//   bits [4,6) D format (1 = f32)   [7,10) A format (0 = e4m3)   [10,13) B format (0 = e4m3)
//   bit 15 / 16 A / B major (0 = K)  [17,23) N >> 3               [24,29) M >> 4
__host__ __device__ constexpr uint32_t umma_idesc_e4m3_f32(int mma_m, int mma_n) {
    return (1u << 4) | (0u << 7) | (0u << 10) | (static_cast<uint32_t>(mma_n >> 3) << 17) |
           (static_cast<uint32_t>(mma_m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_f8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
        "}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives once on `bar` when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// Each thread of the warp reads 16 consecutive 32-bit columns of its own TMEM lane
// (lane = 32 * (warp index % 4) + lane id, encoded in bits [31:16] of taddr by the caller).
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
          "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- clusters / DSMEM
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Execution-only cluster barrier: orders nothing in memory. Enough to keep a CTA alive until its
// peers have finished reading its shared memory (their loads have returned before they arrive).
__device__ __forceinline__ void cluster_sync_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t dsmem_map(uint32_t local_smem, uint32_t cta_rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem), "r"(cta_rank));
    return remote;
}

__device__ __forceinline__ float dsmem_ld_f32(uint32_t cluster_addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr) : "memory");
    return v;
}

// Split cluster barrier: arrive early (non-blocking), wait later.
__device__ __forceinline__ void cluster_arrive_release() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}

// Arrival without memory ordering: for threads that have written nothing the peers will read.
__device__ __forceinline__ void cluster_arrive_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}

__device__ __forceinline__ void cluster_wait_acquire() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Bulk copy from this CTA's shared memory into a peer's (addresses from dsmem_map); the bytes
// are counted on the PEER's mbarrier. Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void dsmem_bulk_copy(uint32_t dst_cluster_addr, uint32_t src_cta_addr, uint32_t bytes,
                                                uint32_t peer_bar_cluster_addr) {
    asm volatile(
        "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_cluster_addr), "r"(src_cta_addr), "r"(bytes), "r"(peer_bar_cluster_addr)
        : "memory");
}

// Asynchronous stores from registers into a peer's shared memory (addresses from dsmem_map). Each
// store adds its own size to the transaction count of the PEER's mbarrier when it has landed, so
// the receiver learns from one barrier that every sender's data is there. No staging in shared
// memory, no proxy fence and no copy engine on the way.
__device__ __forceinline__ void st_async_b32(uint32_t dst_cluster_addr, uint32_t a, uint32_t peer_bar_cluster_addr) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(dst_cluster_addr), "r"(a), "r"(peer_bar_cluster_addr)
                 : "memory");
}

__device__ __forceinline__ void st_async_v2_b32(uint32_t dst_cluster_addr, uint32_t a, uint32_t b,
                                                uint32_t peer_bar_cluster_addr) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];"
                 ::"r"(dst_cluster_addr), "r"(a), "r"(b), "r"(peer_bar_cluster_addr)
                 : "memory");
}

__device__ __forceinline__ void st_async_v4_b32(uint32_t dst_cluster_addr, uint32_t a, uint32_t b, uint32_t c,
                                                uint32_t d, uint32_t peer_bar_cluster_addr) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(dst_cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(peer_bar_cluster_addr)
                 : "memory");
}

// The issuing thread's bulk copies have finished READING their source.
__device__ __forceinline__ void bulk_copies_source_done() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- programmatic dependent launch
// Both are no-ops when the grid was launched without the programmatic-serialisation attribute.
__device__ __forceinline__ void pdl_wait_prior_grids() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

}  // namespace hfrk
