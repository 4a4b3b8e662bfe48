// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the GEMM uses: mbarriers with
// bounded waits, TMA tiled loads (never multicast), tensor-memory allocation, tcgen05 MMA issue,
// commit and accumulator loads, and the shared-memory / instruction descriptors they consume.
#pragma once
#include <cstdint>
#include <cuda.h>

namespace tts::b200::ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("{\n\t.reg .b64 state;\n\tmbarrier.arrive.shared::cta.b64 state, [%0];\n\t}" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 state;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 state, [%0], %1;\n\t}" ::"r"(bar),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return done != 0;
}
// Wait with a limit. Returns false once `*abort_flag` is set by anyone or the limit passes (in
// which case it sets the flag itself), so a wrong phase or a lost copy ends the kernel with an
// error status instead of hanging the GPU. The limit is counted on the SM's own cycle counter
// (about two seconds at 2 GHz); the global nanosecond timer is far too slow to read in a hot loop.
constexpr long long kWaitLimitCycles = 4000000000ll;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          long long limit = kWaitLimitCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 0) {
            if (*abort_flag) return false;
            if (clock64() - start > limit) {
                *abort_flag = 1;
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------- thread-block clusters
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Hardware barrier over every thread of every CTA in the cluster; release/acquire makes shared
// memory written before it visible to the peers that read it afterwards.
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// Split form of the same barrier: arrive early, wait only where the peers' progress is needed.
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t addr, uint32_t value) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(value) : "memory");
}
// Programmatic dependent launch: let the next kernel in the stream start its prologue now, and
// block until everything the previous kernel wrote is visible. Both are no-ops for a kernel that
// was launched without the programmatic-serialization attribute.
__device__ __forceinline__ void launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void wait_for_upstream() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Address of the same shared-memory location in the CTA with rank `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr), "r"(rank));
    return remote;
}
__device__ __forceinline__ uint4 ld_cluster_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared::cluster.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr)
                 : "memory");
    return v;
}

// ---------------------------------------------------------------- TMA (2-D tiled load, no multicast)
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// x is the innermost coordinate (bytes along K here); it must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x,
                                                 int y, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
                 "[%0], [%1, {%3, %4}], [%2], %5;" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "l"(policy)
                 : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// ---------------------------------------------------------------- tensor memory
// One full warp allocates `columns` (power of two, 32..512) and writes the base address to smem.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives on `bar` once every MMA issued so far by this thread has finished.
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// This warp's 32 lanes x 16 consecutive 32-bit columns starting at `taddr`.
__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                   "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
                   "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_load_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster act as one MMA unit: each holds 128 rows of A and half of B in its own shared
// memory and 128 accumulator rows in its own tensor memory; the even CTA issues the instruction.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
// TMA load whose completion is signalled on a barrier that may live in the peer CTA (`bar` is a
// shared::cluster address). No multicast: each CTA fetches only its own half.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void mma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
                 "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// Arrives on the barrier at the same shared-memory offset in every CTA named by `cta_mask` once
// all MMAs issued so far by this thread have finished (a commit is not a load: multicast is fine).
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(cta_mask)
                 : "memory");
}
// Arrive on a barrier given by a shared::cluster address (own CTA or a peer).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory operand descriptor for a K-major tile whose rows are 128 bytes, laid down by TMA
// with the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset), the leading
// offset is unused for this layout, descriptor version 1, layout code 2 (128B swizzle).
// Stepping along K inside the swizzled row is a plain byte offset on the start address.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= uint64_t((smem_addr & 0x3ffffu) >> 4);
    d |= uint64_t(1) << 16;
    d |= uint64_t(1024 >> 4) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(2) << 61;
    return d;
}
// The same descriptor as two 32-bit halves. Only the low half (start address) changes from tile to
// tile and from K step to K step, so an issue loop that carries the halves separately keeps the high
// half loop-invariant and steps the low half with 32-bit adds.
constexpr uint32_t kDescHiK128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_lo_k128(uint32_t smem_addr) {
    return ((smem_addr & 0x3ffffu) >> 4) | (1u << 16);
}
__device__ __forceinline__ void mma_i8_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, p;\n\t}" ::"r"(d_tmem),
                 "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiK128)
                 : "memory");
}
__device__ __forceinline__ void mma_f8_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %3, p;\n\t}" ::"r"(d_tmem),
                 "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiK128)
                 : "memory");
}
// The four MMAs that consume one 128-byte K block (32 bytes of K each: +2 descriptor units per
// step), issued from one instruction block so that no other code separates them. `accumulate`
// applies to the first; the other three always add to it (the instruction descriptor is never zero,
// which is what the second predicate test relies on).
#define B200Q_MMA_K128(NAME, GROUP, KIND)                                                                      \
    __device__ __forceinline__ void NAME(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,         \
                                         uint32_t accumulate) {                                                \
        asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t.reg .b32 al, bl;\n\t"                      \
                     "setp.ne.b32 p, %4, 0;\n\t"                                                               \
                     "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"                                      \
                     "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %3, p;\n\t"                 \
                     "setp.ne.b32 p, %3, 0;\n\t"                                                               \
                     "add.u32 al, %1, 2;\n\tadd.u32 bl, %2, 2;\n\t"                                            \
                     "mov.b64 da, {al, %5};\n\tmov.b64 db, {bl, %5};\n\t"                                      \
                     "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %3, p;\n\t"                 \
                     "add.u32 al, %1, 4;\n\tadd.u32 bl, %2, 4;\n\t"                                            \
                     "mov.b64 da, {al, %5};\n\tmov.b64 db, {bl, %5};\n\t"                                      \
                     "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %3, p;\n\t"                 \
                     "add.u32 al, %1, 6;\n\tadd.u32 bl, %2, 6;\n\t"                                            \
                     "mov.b64 da, {al, %5};\n\tmov.b64 db, {bl, %5};\n\t"                                      \
                     "tcgen05.mma.cta_group::" GROUP ".kind::" KIND " [%0], da, db, %3, p;\n\t}" ::"r"(d_tmem),  \
                     "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHiK128)                        \
                     : "memory");                                                                              \
    }
B200Q_MMA_K128(mma_i8_k128, "1", "i8")
B200Q_MMA_K128(mma_f8_k128, "1", "f8f6f4")
B200Q_MMA_K128(mma_i8_pair_k128, "2", "i8")
B200Q_MMA_K128(mma_f8_pair_k128, "2", "f8f6f4")
#undef B200Q_MMA_K128
// Named hardware barrier 4 over 64 threads (the MMA warp and its waiter warp) that also ANDs one
// predicate per thread: how a waiter tells the issuer "the barriers you need have completed" without
// the issuer touching shared memory.
__device__ __forceinline__ bool pair_barrier_and(bool ok) {
    uint32_t all;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.and.pred p, 4, 64, q;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(all)
                 : "r"(uint32_t(ok))
                 : "memory");
    return all != 0;
}
// The same over any named barrier: every one of the `threads` participants learns whether all of
// them passed `ok`. Used where several warps must agree to leave a loop together, because a warp
// that left alone would strand its siblings at their next named barrier.
__device__ __forceinline__ bool barrier_and(uint32_t id, uint32_t threads, bool ok) {
    uint32_t all;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %3, 0;\n\tbar.red.and.pred p, %1, %2, q;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(all)
                 : "r"(id), "r"(threads), "r"(uint32_t(ok))
                 : "memory");
    return all != 0;
}
// One lane of a converged warp; the same lane every time for the same mask.
__device__ __forceinline__ bool elect_one() {
    uint32_t elected;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    return elected != 0;
}
// Instruction descriptor: D format at bits 4-5 (1 = f32, 2 = s32), A/B formats at 7-9 / 10-12,
// both operands K-major, N>>3 at bits 17-22, M>>4 at bits 24-28.
__host__ __device__ constexpr uint32_t idesc_i8(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
__host__ __device__ constexpr uint32_t idesc_e4m3(int m, int n) {
    return (1u << 4) | (0u << 7) | (0u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}
} // namespace tts::b200::ptx
