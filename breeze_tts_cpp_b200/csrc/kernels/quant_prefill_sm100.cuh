// Compute-bound (prefill) variant of the W8A8 GEMM for sm_100a: persistent CTAs, 128-channel x
// 256-token tiles, two accumulators in tensor memory so that the dequant epilogue of tile i runs
// while the tensor cores work on tile i+1.
//
// Same orientation and arithmetic as the weight-streaming kernel (quant_linear_sm100.cuh): 128
// weight channels are the MMA M rows, 256 tokens the MMA N columns, K in 128-byte swizzled TMA
// boxes; out[m,n] = D((float(acc) * sx[m]) * sw[n]) (+ fp32 residual), per-row scales only.
// Replaces the reference's compute-bound paths: CUTLASS SM80 `Sm80Gemm`
// (src/ops/kernels/quant/quant_gemm_sm80.cu:14-82) and the SM90a WGMMA family
// (quant_gemm_sm90.cu:16-69), neither of which uses Blackwell's tensor memory.
//
// Roles (320 threads): warp 0 = TMA producer, warp 1 = MMA issuer and tensor-memory owner,
// warps 2-9 = epilogue (two warps per 32-lane quadrant, alternating 16-token chunks).
// Tiles are dealt round-robin: tile = blockIdx.x + i * gridDim.x, channel tile fastest, so the CTAs
// running at any moment share a few activation row blocks and the whole weight matrix through L2.
#pragma once
#include "kernels/quant_linear_sm100.cuh"

namespace tts::b200 {

constexpr int kPrefillStages = 4;
constexpr int kPrefillPatchBytes = 2 * 2 * 16 * kBlockChannels * 2; // two chunk groups x two parities x [16][128] 16-bit

struct PrefillArgs {
    int m, n, k;
    const float *sx, *sw;
    void *out;
    int out_type; // Type::BF16 or Type::F16
    const float *residual_f32;
    int *status;
};

// One 16-token chunk of a tile's epilogue, executed by the four warps (one per tensor-memory lane
// quadrant) that share a chunk. Phase 1, lane = channel: accumulator -> (acc*sx)*sw (+ fp32 residual)
// -> 16-bit, written to a small shared-memory patch [token][channel]. After a 128-thread barrier,
// phase 2, lane = four consecutive channels: every warp copies four token rows of the patch to
// global memory as 8-byte stores, 256 contiguous bytes per row. The patch is double-buffered so one
// barrier per chunk suffices. `r` holds the chunk's 16 accumulator words of this lane.
template <bool kInt>
__device__ __forceinline__ void prefill_store_chunk(const PrefillArgs &a, const uint32_t (&r)[16], const float *sx_chunk,
                                                    float scale_w, const float *__restrict__ residual, int m_first,
                                                    int n_tile0, int valid_rows, int quadrant, int lane, int group,
                                                    uint16_t *patch /* [16][128] of this group and parity */) {
    const int channel = quadrant * 32 + lane, n = n_tile0 + channel;
    const bool bf16_out = a.out_type == int(Type::BF16);
    // All loads (activation scales from shared memory, residuals from global memory) come first: a
    // load may not be moved above an earlier store it might alias, so interleaving them with the patch
    // stores would serialise sixteen round trips.
    float scale_x[16], skip[16];
    {
        const float4 *sx4 = reinterpret_cast<const float4 *>(sx_chunk);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 v = sx4[q];
            scale_x[4 * q] = v.x; scale_x[4 * q + 1] = v.y; scale_x[4 * q + 2] = v.z; scale_x[4 * q + 3] = v.w;
        }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i)
        skip[i] = (residual && n < a.n && i < valid_rows) ? __ldg(residual + size_t(m_first + i) * a.n + n) : 0.f;
    uint16_t bits[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float acc = kInt ? float(int(r[i])) : __uint_as_float(r[i]);
        float value = __fmul_rn(__fmul_rn(acc, scale_x[i]), scale_w);
        if (residual) value = __fadd_rn(value, skip[i]);
        if (bf16_out) { __nv_bfloat16 b = __float2bfloat16_rn(value); bits[i] = *reinterpret_cast<uint16_t *>(&b); }
        else { __half h = __float2half_rn(value); bits[i] = *reinterpret_cast<uint16_t *>(&h); }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) patch[i * kBlockChannels + channel] = bits[i];
    if (group == 0) asm volatile("bar.sync 2, 128;" ::: "memory");
    else asm volatile("bar.sync 3, 128;" ::: "memory");
    const int n4 = n_tile0 + lane * 4;
    if (n4 < a.n) {
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
            const int i = quadrant * 4 + rr;
            if (i < valid_rows) {
                const uint2 four = *reinterpret_cast<const uint2 *>(patch + i * kBlockChannels + lane * 4);
                *reinterpret_cast<uint2 *>(static_cast<uint16_t *>(a.out) + size_t(m_first + i) * a.n + n4) = four;
            }
        }
    }
}

template <Type F>
__global__ void __launch_bounds__(kGemmThreads, 1)
w8a8_tcgen05_prefill(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                     const PrefillArgs a) {
    constexpr bool kInt = F == Type::I8;
    constexpr int BN = kPrefillTokens;
    constexpr int kWeightBytes = kBlockChannels * kBlockK, kTokenBytes = BN * kBlockK;
    constexpr int kStageBytes = kWeightBytes + kTokenBytes;
    constexpr uint32_t kRingBytes = kPrefillStages * kStageBytes; // the epilogue's staging patches follow the ring
    constexpr uint32_t kIdesc = kInt ? ptx::idesc_i8(kBlockChannels, BN) : ptx::idesc_e4m3(kBlockChannels, BN);

    extern __shared__ uint8_t dynamic_smem[];
    __shared__ alignas(8) uint64_t full_bar[kPrefillStages], empty_bar[kPrefillStages], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ alignas(16) float sx_tile[2][BN]; // activation scales of the tile in each accumulator

    const uint32_t raw_base = ptx::smem_u32(dynamic_smem);
    const uint32_t tiles_base = (raw_base + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (a.n + kBlockChannels - 1) / kBlockChannels, m_tiles = (a.m + BN - 1) / BN;
    const int tiles = n_tiles * m_tiles;
    const int kb_count = (a.k + kBlockK - 1) / kBlockK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPrefillStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&acc_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&acc_empty[b]), kEpilogueThreads / 32);
        }
        abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
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
            ptx::wait_for_upstream();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                const int n0 = (tile % n_tiles) * kBlockChannels, m0 = (tile / n_tiles) * BN;
                for (int kb = 0; kb < kb_count; ++kb) {
                    if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_ptr)) { ok = false; break; }
                    const uint32_t bar = ptx::smem_u32(&full_bar[stage]);
                    const uint32_t dst = tiles_base + uint32_t(stage) * kStageBytes;
                    ptx::mbar_arrive_expect_tx(bar, kStageBytes);
                    ptx::tma_load_2d(dst, &map_w, bar, kb * kBlockK, n0);
                    ptx::tma_load_2d(dst + kWeightBytes, &map_x, bar, kb * kBlockK, m0);
                    if (++stage == kPrefillStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp runs the loop (warp-uniform stage arithmetic); one elected lane issues the
        // four MMAs of a K block from a single instruction block and commits.
        {
            int stage = 0, local = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
                const int buffer = local & 1;
                // The epilogue must have drained this accumulator (two tiles ago).
                ok = __all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&acc_empty[buffer]), ((uint32_t(local) >> 1) & 1u) ^ 1u, abort_ptr));
                if (!ok) break;
                ptx::tcgen05_fence_after();
                const uint32_t d = tmem_base + uint32_t(buffer * BN);
                for (int kb = 0; kb < kb_count; ++kb) {
                    ok = __all_sync(0xffffffffu, ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_ptr));
                    if (!ok) break;
                    ptx::tcgen05_fence_after();
                    const uint32_t tile_smem = tiles_base + uint32_t(stage) * kStageBytes;
                    const uint32_t lo_w = ptx::smem_desc_lo_k128(tile_smem), lo_x = ptx::smem_desc_lo_k128(tile_smem + kWeightBytes);
                    if (ptx::elect_one()) {
                        if (kInt) ptx::mma_i8_k128(d, lo_w, lo_x, kIdesc, uint32_t(kb > 0));
                        else ptx::mma_f8_k128(d, lo_w, lo_x, kIdesc, uint32_t(kb > 0));
                        ptx::tcgen05_commit(ptx::smem_u32(&empty_bar[stage]));
                    }
                    __syncwarp();
                    if (++stage == kPrefillStages) { stage = 0; phase ^= 1u; }
                }
                if (ok && ptx::elect_one()) ptx::tcgen05_commit(ptx::smem_u32(&acc_full[buffer]));
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps
        const int e_thread = threadIdx.x - 64;
        const int quadrant = warp & 3, half = (warp - 2) >> 2;
        const uint32_t lane_base = tmem_base + (uint32_t(quadrant * 32) << 16);
        const float *__restrict__ residual = a.residual_f32;
        uint16_t *patches = reinterpret_cast<uint16_t *>(dynamic_smem + (tiles_base - raw_base) + kRingBytes);
        ptx::wait_for_upstream();
        int local = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
            const int buffer = local & 1;
            const int n0 = (tile % n_tiles) * kBlockChannels, m0 = (tile / n_tiles) * BN;
            const int valid_tokens = min(BN, a.m - m0);
            const int n = n0 + quadrant * 32 + lane;
            const float scale_w = n < a.n ? a.sw[n] : 0.f;
            // Stage this tile's activation scales while the tensor cores are still busy with it.
            sx_tile[buffer][e_thread] = e_thread < valid_tokens ? a.sx[m0 + e_thread] : 0.f;
            // One barrier publishes the scales and makes the verdict of the wait common to all eight
            // warps: they leave the loop together or not at all.
            if (!ptx::barrier_and(1, kEpilogueThreads, ptx::mbar_wait(ptx::smem_u32(&acc_full[buffer]), (uint32_t(local) >> 1) & 1u, abort_ptr)))
                break;
            ptx::tcgen05_fence_after();
#pragma unroll 1
            for (int chunk = half; chunk < BN / 16; chunk += 2) {
                if (chunk * 16 >= valid_tokens) break;
                uint32_t r[16];
                ptx::tmem_load16(lane_base + uint32_t(buffer * BN + chunk * 16), r);
                ptx::tmem_load_wait();
                prefill_store_chunk<kInt>(a, r, &sx_tile[buffer][chunk * 16], scale_w, residual, m0 + chunk * 16, n0,
                                          valid_tokens - chunk * 16, quadrant, lane, half,
                                          patches + ((half * 2 + ((chunk >> 1) & 1)) * 16 * kBlockChannels));
            }
            // This warp has read everything it needs from the accumulator: hand it back.
            ptx::tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&acc_empty[buffer]));
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
