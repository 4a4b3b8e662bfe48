// Compute-bound K-group W8A8 GEMM (group_int8 / group_fp8 prefill) for sm_100a: persistent CTAs over
// 128-channel x 128-token tiles, K-group size 128 on BOTH operands.
//
// Arithmetic (reference grouped_gemm, src/ops/kernels/quant/quant_grouped.cu:16-169): every K block
// of 128 is its own integer/fp8 dot product p_g, and out[m,n] = D(sum_g float(p_g) * (sx_g[m] *
// sw_g[n])) (+ fp32 residual). The tensor cores therefore produce one 128x128 partial tile per K
// block, and CUDA cores rescale and add it; that second part is what bounds this kernel.
//
//   warp 0  : TMA producer. Per K block one pipeline stage (weights 128x128 B + tokens 128x128 B,
//             128-byte swizzle) and one slot of a small scale ring (sx_g row slice and sw_g row slice
//             of that K block, 2 x 512 B, brought in as plain 2-D TMA boxes of the group-major arrays).
//   warp 1  : MMA issuer, whole warp in the loop, elected lane issues. Four accumulators of 128
//             columns rotate through tensor memory, so the tensor cores run up to four K blocks
//             ahead of the rescale. It never tests an mbarrier itself: a test between MMA issues
//             costs the issuing warp about 200 cycles, two per K block would double its loop.
//   warp 10 : waiter. Tests "accumulator free" and "stage full" for the next K block and hands the
//             result to warp 1 through a named hardware barrier (64 threads), which is free.
//   warps 2-9: per K block, pull the accumulator into registers (lane = channel, 64 tokens per
//             thread), hand the buffer back at once, then result += float(p) * (sx * sw) with packed
//             two-wide fp32 instructions; INT8 partials are converted with the exact
//             add-a-magic-constant trick (|p| <= 128 * 127^2 < 2^22) instead of the slow conversion
//             pipe. After the last K block the 64 results per thread go out through the same
//             shared-memory patches as the per-row prefill kernel (coalesced 8-byte row stores).
// Every wait is bounded; on expiry the CTA flags the status word and runs to the common exit.
#pragma once
#include "kernels/quant_prefill_sm100.cuh"

namespace tts::b200 {

constexpr int kGroupedStages = 5;
constexpr int kGroupedAccumulators = 4;
constexpr int kScaleSlots = 8;
constexpr int kGroupedThreads = kGemmThreads + 32; // + the waiter warp
constexpr int kScaleSlotBytes = 2 * kGroupedTokens * 4; // sx_g slice then sw_g slice of one K block
constexpr size_t kGroupedSmem = 1024 + size_t(kGroupedStages) * (kBlockChannels + kGroupedTokens) * kBlockK +
                                size_t(kScaleSlots) * kScaleSlotBytes + kPrefillPatchBytes;

namespace ptx {
// Two fp32 lanes in one 64-bit register, and the packed arithmetic Blackwell has for them.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
} // namespace ptx

template <Type F>
__global__ void __launch_bounds__(kGroupedThreads, 1)
w8a8_tcgen05_prefill_grouped(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                             const __grid_constant__ CUtensorMap map_sw, const __grid_constant__ CUtensorMap map_sx,
                             const __grid_constant__ PrefillArgs a) {
    constexpr bool kInt = F == Type::I8;
    constexpr int BN = kGroupedTokens;
    constexpr int kWeightBytes = kBlockChannels * kBlockK, kTokenBytes = BN * kBlockK;
    constexpr int kStageBytes = kWeightBytes + kTokenBytes;
    constexpr uint32_t kRingBytes = kGroupedStages * kStageBytes;
    constexpr uint32_t kScaleBytes = kScaleSlots * kScaleSlotBytes;
    constexpr uint32_t kIdesc = kInt ? ptx::idesc_i8(kBlockChannels, BN) : ptx::idesc_e4m3(kBlockChannels, BN);

    extern __shared__ uint8_t dynamic_smem[];
    __shared__ alignas(8) uint64_t full_bar[kGroupedStages], empty_bar[kGroupedStages];
    __shared__ alignas(8) uint64_t acc_full[kGroupedAccumulators], acc_empty[kGroupedAccumulators];
    __shared__ alignas(8) uint64_t scale_full[kScaleSlots], scale_empty[kScaleSlots];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ alignas(16) float ones[16];

    const uint32_t raw_base = ptx::smem_u32(dynamic_smem);
    const uint32_t tiles_base = (raw_base + 1023u) & ~1023u;
    uint8_t *aligned = dynamic_smem + (tiles_base - raw_base);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (a.n + kBlockChannels - 1) / kBlockChannels, m_tiles = (a.m + BN - 1) / BN;
    const int tiles = n_tiles * m_tiles;
    const int kb_count = (a.k + kBlockK - 1) / kBlockK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kGroupedStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < kGroupedAccumulators; ++b) {
            ptx::mbar_init(ptx::smem_u32(&acc_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&acc_empty[b]), kEpilogueThreads / 32);
        }
        for (int s = 0; s < kScaleSlots; ++s) {
            ptx::mbar_init(ptx::smem_u32(&scale_full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&scale_empty[s]), kEpilogueThreads / 32);
        }
        abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    if (threadIdx.x < 16) ones[threadIdx.x] = 1.f;
    if (warp == 1) ptx::tmem_alloc(ptx::smem_u32(&tmem_slot), 512);
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = tmem_slot;
    volatile int *abort_ptr = &abort_flag;
    ptx::launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::prefetch_tensormap(&map_w);
            ptx::prefetch_tensormap(&map_x);
            ptx::prefetch_tensormap(&map_sw);
            ptx::prefetch_tensormap(&map_sx);
            ptx::wait_for_upstream();
            int stage = 0, slot = 0;
            uint32_t phase = 0, slot_phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int n0 = (tile % n_tiles) * kBlockChannels, m0 = (tile / n_tiles) * BN;
                for (int kb = 0; kb < kb_count; ++kb) {
                    if (!ptx::mbar_wait(ptx::smem_u32(&scale_empty[slot]), slot_phase ^ 1u, abort_ptr)) { ok = false; break; }
                    const uint32_t scale_bar = ptx::smem_u32(&scale_full[slot]);
                    const uint32_t scale_dst = tiles_base + kRingBytes + uint32_t(slot) * kScaleSlotBytes;
                    ptx::mbar_arrive_expect_tx(scale_bar, kScaleSlotBytes);
                    ptx::tma_load_2d(scale_dst, &map_sx, scale_bar, m0, kb);
                    ptx::tma_load_2d(scale_dst + BN * 4, &map_sw, scale_bar, n0, kb);
                    if (++slot == kScaleSlots) { slot = 0; slot_phase ^= 1u; }
                    if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_ptr)) { ok = false; break; }
                    const uint32_t bar = ptx::smem_u32(&full_bar[stage]);
                    const uint32_t dst = tiles_base + uint32_t(stage) * kStageBytes;
                    ptx::mbar_arrive_expect_tx(bar, kStageBytes);
                    ptx::tma_load_2d(dst, &map_w, bar, kb * kBlockK, n0);
                    ptx::tma_load_2d(dst + kWeightBytes, &map_x, bar, kb * kBlockK, m0);
                    if (++stage == kGroupedStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1 || warp == 10) {
        // ------------------------------------------------------------ MMA issuer (1) and its waiter (10)
        // Both walk the same K-block sequence and meet once per K block at named barrier 4, which also
        // carries the waiter's verdict. Neither leaves its loop early, so the barrier counts always
        // match; after a failed wait the abort flag makes every later wait return at once and the
        // issuer stops issuing.
        int stage = 0;
        uint32_t phase = 0, count = 0; // count: K blocks so far, over all tiles
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
            for (int kb = 0; kb < kb_count; ++kb, ++count) {
                const uint32_t buffer = count % kGroupedAccumulators;
                if (warp == 10) {
                    const uint32_t use = (count / kGroupedAccumulators) & 1u;
                    const bool ready = ptx::mbar_wait(ptx::smem_u32(&acc_empty[buffer]), use ^ 1u, abort_ptr) &&
                                       ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_ptr);
                    (void)ptx::pair_barrier_and(ready);
                } else {
                    const bool ready = ptx::pair_barrier_and(true);
                    ptx::tcgen05_fence_after();
                    const uint32_t tile_smem = tiles_base + uint32_t(stage) * kStageBytes;
                    const uint32_t lo_w = ptx::smem_desc_lo_k128(tile_smem), lo_x = ptx::smem_desc_lo_k128(tile_smem + kWeightBytes);
                    const uint32_t d = tmem_base + buffer * uint32_t(BN);
                    if (ready && ptx::elect_one()) {
                        if (kInt) ptx::mma_i8_k128(d, lo_w, lo_x, kIdesc, 0u);
                        else ptx::mma_f8_k128(d, lo_w, lo_x, kIdesc, 0u);
                        ptx::tcgen05_commit(ptx::smem_u32(&empty_bar[stage]));
                        ptx::tcgen05_commit(ptx::smem_u32(&acc_full[buffer]));
                    }
                    __syncwarp();
                }
                if (++stage == kGroupedStages) { stage = 0; phase ^= 1u; }
            }
        }
    } else {
        // ------------------------------------------------------------ rescale + epilogue warps
        const int quadrant = warp & 3, half = (warp - 2) >> 2;
        const uint32_t lane_base = tmem_base + (uint32_t(quadrant * 32) << 16);
        const float *__restrict__ residual = a.residual_f32;
        const float *scales = reinterpret_cast<const float *>(aligned + kRingBytes);
        uint16_t *patches = reinterpret_cast<uint16_t *>(aligned + kRingBytes + kScaleBytes);
        const uint64_t magic2 = ptx::pack2(-12582912.f, -12582912.f);
        ptx::wait_for_upstream();
        uint32_t count = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            const int n0 = (tile % n_tiles) * kBlockChannels, m0 = (tile / n_tiles) * BN;
            const int valid_tokens = min(BN, a.m - m0);
            uint64_t result[32]; // [chunk 0..3][pair 0..7]: tokens (2*k + half)*16 + 2*pair, +1
#pragma unroll
            for (int i = 0; i < 32; ++i) result[i] = 0ull;
#pragma unroll 1
            for (int kb = 0; kb < kb_count; ++kb, ++count) {
                const uint32_t buffer = count % kGroupedAccumulators, use = (count / kGroupedAccumulators) & 1u;
                const uint32_t slot = count % kScaleSlots, slot_use = (count / kScaleSlots) & 1u;
                if (!ptx::mbar_wait(ptx::smem_u32(&acc_full[buffer]), use, abort_ptr)) { ok = false; break; }
                ptx::tcgen05_fence_after();
                uint32_t r[4][16];
#pragma unroll
                for (int k = 0; k < 4; ++k) ptx::tmem_load16(lane_base + buffer * uint32_t(BN) + uint32_t((2 * k + half) * 16), r[k]);
                ptx::tmem_load_wait();
                // Everything is in registers: the tensor cores may have the buffer back.
                ptx::tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&acc_empty[buffer]));
                if (!ptx::mbar_wait(ptx::smem_u32(&scale_full[slot]), slot_use, abort_ptr)) { ok = false; break; }
                const float *slot_scales = scales + slot * (kScaleSlotBytes / 4);
                const float scale_w = slot_scales[BN + quadrant * 32 + lane];
                const uint64_t scale_w2 = ptx::pack2(scale_w, scale_w);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float4 *sx4 = reinterpret_cast<const float4 *>(slot_scales + (2 * k + half) * 16);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 sx = sx4[q];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int i = 4 * q + 2 * h;
                            uint64_t p;
                            if (kInt) {
                                // float(int) exactly: bits(2^23 + 2^22 + p) read as fp32, minus that constant.
                                p = ptx::add2(ptx::pack2(__uint_as_float(r[k][i] + 0x4B400000u), __uint_as_float(r[k][i + 1] + 0x4B400000u)), magic2);
                            } else {
                                p = ptx::pack2(__uint_as_float(r[k][i]), __uint_as_float(r[k][i + 1]));
                            }
                            const uint64_t s = ptx::mul2(h ? ptx::pack2(sx.z, sx.w) : ptx::pack2(sx.x, sx.y), scale_w2);
                            result[k * 8 + i / 2] = ptx::fma2(p, s, result[k * 8 + i / 2]);
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&scale_empty[slot]));
            }
            // All eight warps decide together whether the tile is stored (a warp that left alone would
            // strand the three that share its staging patch); the same barrier keeps two consecutive
            // tiles from meeting in one patch.
            ok = ptx::barrier_and(1, kEpilogueThreads, ok && !*abort_ptr);
            if (!ok) break;
            // ---- tile finished: 16-token chunks out through the staging patches.
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int chunk = 2 * k + half;
                if (chunk * 16 < valid_tokens) { // uniform over the four warps that share the chunk
                    uint32_t words[16];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float lo, hi;
                        ptx::unpack2(result[k * 8 + j], lo, hi);
                        words[2 * j] = __float_as_uint(lo);
                        words[2 * j + 1] = __float_as_uint(hi);
                    }
                    prefill_store_chunk<false>(a, words, ones, 1.f, residual, m0 + chunk * 16, n0, valid_tokens - chunk * 16,
                                               quadrant, lane, half, patches + ((half * 2 + (k & 1)) * 16 * kBlockChannels));
                }
            }
        }
        ptx::tcgen05_fence_before();
    }

    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc(tmem_base, 512);
    }
    if (threadIdx.x == 0 && abort_flag) atomicExch(a.status, 1 + int(blockIdx.x));
}
} // namespace tts::b200
