// Thin inline-PTX layer over the Blackwell (sm_100a) tensor-core path: mbarriers with bounded
// waits, cp.async staging, tensor-memory allocation, shared-memory matrix descriptors, the
// block-scaled tcgen05.mma (kind::mxf8f6f4, one UE8M0 scale per 32 K-elements) and TMEM loads.
//
// Every wait in this file is bounded: a waiter that runs out of time reports failure to its caller,
// which raises NVMOE_STATUS_WAIT_EXPIRED and winds the kernel down; nothing here can spin forever.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace nvmoe {
namespace tc {

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier --------------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  `abort_flag` (shared memory) lets one role tell the others that it gave up, so
// that a broken pipeline unwinds in one timeout instead of one per role.  Returns false when the
// wait expired (after `limit` clock cycles) or was aborted.
constexpr long long kDefaultWaitCycles = 4000000000ll;  // about two seconds at B200 clocks
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - start > limit) {
            *abort_flag = 1u;
            return false;
        }
    }
}

// The same wait for a whole warp: one lane polls, the verdict is shared, so that a waiting warp
// costs one polling thread instead of thirty-two.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, long long limit) {
    uint32_t ok = 0u;
    if ((threadIdx.x & 31u) == 0u) ok = mbar_wait(bar, parity, abort_flag, limit) ? 1u : 0u;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0u;
}

// Wind-down wait: for a role that is leaving after the pipeline was aborted and must first see what it
// has in flight (bulk copies, tensor-core operations) finish.  It ignores the abort flag, which is set
// by then, and gives up after `limit` cycles on its own; what it waits for completes within
// microseconds unless the barrier also counts arrivals that an aborted role will never make, in which
// case the time spent here is itself the grace period for the copies.
__device__ __forceinline__ bool mbar_wait_winddown(uint64_t* bar, uint32_t parity, long long limit) {
    const long long start = clock64();
    for (;;) {
        for (int i = 0; i < 64; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - start > limit) return false;
    }
}
constexpr long long kWinddownCycles = 4000000ll;  // about two milliseconds

// ---- generic-proxy staging into shared memory ---------------------------------------------------

// src_bytes < size zero-fills the rest (src_bytes == 0 reads nothing)
__device__ __forceinline__ void cp_async_8(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// mbarrier arrival that fires once every cp.async this thread issued so far has landed; it counts
// as one of the arrivals the barrier was initialised with (.noinc)
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// makes this thread's generic-proxy writes to shared memory visible to the async proxy (tcgen05)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- TMA (async proxy) --------------------------------------------------------------------------------

// one arrival that also announces `bytes` of bulk-copy traffic the barrier must see before it completes
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// 3-D tiled load; the box lands swizzled (and, for the padded 4-bit type, spread into 16-byte slots)
// and the barrier is credited with the GLOBAL bytes of the box
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void* tensor_map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst_smem), "l"(tensor_map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}
// 2-D tiled load (byte tensors: the barrier is credited with the bytes of the whole box, rows and
// columns past the tensor's edge included - they arrive as zeros)
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void* tensor_map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst_smem), "l"(tensor_map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}
// linear copy of `bytes` (a multiple of 16, both addresses 16-byte aligned) credited to the barrier
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// a tensor map that a kernel wrote (tensormap_publish) must be acquired by the thread that uses it
__device__ __forceinline__ void tensormap_acquire(const void* tensor_map) {
    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(tensor_map) : "memory");
}
// patch the global address of a 128-byte tensor map held in shared memory (one thread)
__device__ __forceinline__ void tensormap_replace_address(void* smem_map, const void* global_address) {
    asm volatile("tensormap.replace.tile.global_address.shared::cta.b1024.b64 [%0], %1;" ::"r"(smem_u32(smem_map)),
                 "l"(global_address)
                 : "memory");
}
// copy the patched map to global memory with the release the TMA unit needs (whole warp)
__device__ __forceinline__ void tensormap_publish(void* global_map, const void* smem_map) {
    asm volatile("tensormap.cp_fenceproxy.global.shared::cta.tensormap::generic.release.gpu.sync.aligned [%0], [%1], 128;"
                 ::"l"(global_map), "r"(smem_u32(smem_map))
                 : "memory");
}

// ---- tensor memory ----------------------------------------------------------------------------------

// whole-warp instructions
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// arrive on `bar` once every tcgen05 operation this thread issued so far has completed
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ---- descriptors ------------------------------------------------------------------------------------

// K-major operand tile, 128-byte swizzle: rows of 128 bytes, 16-byte chunks XOR-ed with (row & 7),
// groups of 8 rows 1024 bytes apart.  The tile base must be 1024-byte aligned.
__device__ __forceinline__ uint64_t desc_k_major_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);        // start address
    d |= (uint64_t)1u << 16;                            // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024u >> 4) << 32;                  // stride byte offset between 8-row groups
    d |= (uint64_t)1u << 46;                            // descriptor version of sm_100
    d |= (uint64_t)2u << 61;                            // SWIZZLE_128B
    return d;
}
// 32 rows x 16 bytes, no swizzle: the source of a scale-factor copy
__device__ __forceinline__ uint64_t desc_scale_block(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
    d |= (uint64_t)(128u >> 4) << 32;                   // 8 rows x 16 bytes between row groups
    d |= (uint64_t)1u << 46;
    return d;
}
__device__ __forceinline__ uint32_t swizzle128_offset(uint32_t row, uint32_t chunk16) {
    return row * 128u + ((chunk16 ^ (row & 7u)) << 4);
}

enum : uint32_t { kFmtE4M3 = 0u, kFmtE2M1 = 5u };
// Instruction descriptor of tcgen05.mma.kind::mxf8f6f4.block_scale, UE8M0 scales, K-major A and B.
__host__ __device__ constexpr uint32_t idesc_mxf8f6f4(uint32_t a_format, uint32_t b_format, uint32_t m, uint32_t n) {
    return (a_format << 7) | (b_format << 10) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24);
}
// which of the four scale bytes of a TMEM column this MMA reads, for A and for B
__device__ __forceinline__ uint32_t idesc_with_scale_ids(uint32_t idesc, uint32_t a_id, uint32_t b_id) {
    return idesc | (b_id << 4) | (a_id << 29);
}

// ---- instructions issued by one thread ----------------------------------------------------------------

// shared memory (32 rows x 16 bytes) -> 4 TMEM columns, replicated into all four lane quadrants
__device__ __forceinline__ void tc_copy_scales(uint32_t taddr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] with per-32-element UE8M0 scales read from TMEM
__device__ __forceinline__ void tc_mma_block_scaled(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}

// ---- TMEM -> registers (whole warp; lane i of warp w reads TMEM lane 32*(w%4)+i) ------------------------

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// named barrier over a subset of the block's warps
__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace tc
}  // namespace nvmoe
