// Compute-bound W8A8 GEMM on CTA pairs (tcgen05 cta_group::2): two SMs share one 256-channel x
// 256-token tile. Each CTA of the pair loads 128 weight rows and only HALF of the token rows into its
// own shared memory and keeps 128 accumulator rows in its own tensor memory; the even CTA issues the
// M=256 x N=256 MMAs for both. Compared with one-CTA 128x256 tiles this cuts the bytes every SM pulls
// from L2 per MMA by a third, which is what bounds 8-bit GEMMs at these K (the tensor pipe needs
// 96 B/clk/SM of operands otherwise).
//
// Same arithmetic as quant_prefill_sm100.cuh: out[m,n] = D((float(acc) * sx[m]) * sw[n]) (+ fp32
// residual), per-row scales. Persistent clusters, two accumulators in tensor memory so the epilogue
// of tile i overlaps the MMAs of tile i+1. No TMA multicast: each CTA issues its own loads; the loads
// carry the cta_group::2 qualifier only so that they can signal the barrier in the leader CTA.
// Replaces reference quant_gemm_sm80.cu:14-82 / quant_gemm_sm90.cu:16-69 for compute-bound shapes.
//
// Two orientations of the same tile (`TokensAsRows`): with the CHANNELS as the MMA's M rows (A = weight tile), as
// in the weight-streaming kernel, the epilogue transposes 16-token chunks through shared-memory patches and
// stores 256 contiguous bytes per row; with the TOKENS as M rows (A = activation tile) a CTA's tensor memory holds
// 128 token rows x 256 channels, every epilogue thread owns one token row, reads 32 consecutive channels per
// round and stores them straight from registers: no transposition, no barrier per chunk, fewer instructions per
// output. The loads are the same in both. Measured (bursts, M=8192): tokens-as-rows is 3-15 % faster up to 4096
// output channels and 4 % slower on the 12288-channel gate+up output, so the launcher picks by output width.
//
// Barrier protocol (L = leader, even rank; P = peer):
//   full[s]      in L : L's producer arrives with expect_tx for BOTH CTAs' bytes; both producers'
//                       TMA loads complete their bytes on it.
//   empty[s]     in L and P : one multicast tcgen05.commit after the MMAs that read stage s.
//   acc_full[b]  in L and P : multicast commit after the last MMA of a tile.
//   acc_empty[b] in L : 16 arrivals (8 epilogue warps of each CTA, the peer's arrive remotely).
// Every wait is bounded; on expiry the CTA flags the status word and runs to the common exit.
#pragma once
#include "kernels/quant_prefill_sm100.cuh"

namespace tts::b200 {

constexpr int kPairStages = 6;

template <Type F, bool TokensAsRows = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
w8a8_tcgen05_prefill_pair(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                          const PrefillArgs a) {
    constexpr bool kInt = F == Type::I8;
    constexpr int BN = kPrefillTokens;               // tokens per tile (MMA N)
    constexpr int kHalfTokens = BN / 2;               // token rows this CTA loads
    constexpr int kWeightBytes = kBlockChannels * kBlockK, kTokenBytes = kHalfTokens * kBlockK;
    constexpr int kStageBytes = kWeightBytes + kTokenBytes; // per CTA
    constexpr uint32_t kRingBytes = kPairStages * kStageBytes; // the epilogue's staging patches follow the ring
    constexpr uint32_t kIdesc = kInt ? ptx::idesc_i8(2 * kBlockChannels, BN) : ptx::idesc_e4m3(2 * kBlockChannels, BN);

    extern __shared__ uint8_t dynamic_smem[];
    __shared__ alignas(8) uint64_t full_bar[kPairStages], empty_bar[kPairStages], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ alignas(16) float sx_tile[2][BN]; // per accumulator: activation scales (channels as rows) or weight scales (tokens as rows)

    const uint32_t raw_base = ptx::smem_u32(dynamic_smem);
    const uint32_t tiles_base = (raw_base + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const bool leader = rank == 0;
    const int pair_tiles_n = (a.n + 2 * kBlockChannels - 1) / (2 * kBlockChannels), m_tiles = (a.m + BN - 1) / BN;
    const int tiles = pair_tiles_n * m_tiles;
    const int clusters = gridDim.x / 2, cluster_id = blockIdx.x / 2;
    const int kb_count = (a.k + kBlockK - 1) / kBlockK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairStages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&acc_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&acc_empty[b]), 2 * (kEpilogueThreads / 32));
        }
        abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    if (warp == 1) ptx::tmem_alloc_pair(ptx::smem_u32(&tmem_slot), 512);
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::cluster_sync(); // both CTAs' barriers are initialised before either signals the other
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = tmem_slot;
    volatile int *abort_ptr = &abort_flag;
    ptx::launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            ptx::prefetch_tensormap(&map_w);
            ptx::prefetch_tensormap(&map_x);
            ptx::wait_for_upstream();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < tiles && ok; tile += clusters) {
                const int n0 = (tile % pair_tiles_n) * 2 * kBlockChannels + int(rank) * kBlockChannels;
                const int m0 = (tile / pair_tiles_n) * BN + int(rank) * kHalfTokens;
                for (int kb = 0; kb < kb_count; ++kb) {
                    if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_ptr)) { ok = false; break; }
                    const uint32_t leader_full = ptx::map_to_rank(ptx::smem_u32(&full_bar[stage]), 0);
                    const uint32_t dst = tiles_base + uint32_t(stage) * kStageBytes;
                    if (leader) ptx::mbar_arrive_expect_tx(ptx::smem_u32(&full_bar[stage]), 2 * kStageBytes);
                    ptx::tma_load_2d_pair(dst, &map_w, leader_full, kb * kBlockK, n0);
                    ptx::tma_load_2d_pair(dst + kWeightBytes, &map_x, leader_full, kb * kBlockK, m0);
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        // The whole warp runs the loop (warp-uniform stage arithmetic); one elected lane issues the
        // four MMAs of a K block from a single instruction block and commits.
        if (leader) {
            int stage = 0, local = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = cluster_id; tile < tiles && ok; tile += clusters, ++local) {
                const int buffer = local & 1;
                ok = ptx::mbar_wait(ptx::smem_u32(&acc_empty[buffer]), ((uint32_t(local) >> 1) & 1u) ^ 1u, abort_ptr);
                ok = __all_sync(0xffffffffu, ok);
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
                        const uint32_t lo_a = TokensAsRows ? lo_x : lo_w, lo_b = TokensAsRows ? lo_w : lo_x;
                        if (kInt) ptx::mma_i8_pair_k128(d, lo_a, lo_b, kIdesc, uint32_t(kb > 0));
                        else ptx::mma_f8_pair_k128(d, lo_a, lo_b, kIdesc, uint32_t(kb > 0));
                        ptx::tcgen05_commit_pair(ptx::smem_u32(&empty_bar[stage]), 3);
                    }
                    __syncwarp();
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
                if (ok && ptx::elect_one()) ptx::tcgen05_commit_pair(ptx::smem_u32(&acc_full[buffer]), 3);
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue warps (both CTAs)
        const int e_thread = threadIdx.x - 64;
        const int quadrant = warp & 3, half = (warp - 2) >> 2;
        const uint32_t lane_base = tmem_base + (uint32_t(quadrant * 32) << 16);
        const float *__restrict__ residual = a.residual_f32;
        uint16_t *patches = reinterpret_cast<uint16_t *>(dynamic_smem + (tiles_base - raw_base) + kRingBytes);
        ptx::wait_for_upstream();
        int local = 0;
        if constexpr (TokensAsRows) {
            // lane = token row of this CTA's half, columns = the tile's 256 channels; the two warps of a lane
            // quadrant alternate 32-channel column groups.
            const bool bf16_out = a.out_type == int(Type::BF16);
            for (int tile = cluster_id; tile < tiles; tile += clusters, ++local) {
                const int buffer = local & 1;
                const int n0 = (tile % pair_tiles_n) * 2 * kBlockChannels;
                const int token = (tile / pair_tiles_n) * BN + int(rank) * kHalfTokens + quadrant * 32 + lane;
                const bool token_ok = token < a.m;
                const int valid_channels = min(2 * kBlockChannels, a.n - n0); // a multiple of 16 (the launcher requires it)
                const float scale_x = token_ok ? a.sx[token] : 0.f;
                sx_tile[buffer][e_thread] = e_thread < valid_channels ? a.sw[n0 + e_thread] : 0.f;
                if (!ptx::barrier_and(1, kEpilogueThreads, ptx::mbar_wait(ptx::smem_u32(&acc_full[buffer]), (uint32_t(local) >> 1) & 1u, abort_ptr)))
                    break;
                ptx::tcgen05_fence_after();
                const size_t row = size_t(token_ok ? token : 0) * a.n + n0;
                const float *__restrict__ skip_row = residual ? residual + row : nullptr;
                uint16_t *out_row = static_cast<uint16_t *>(a.out) + row;
#pragma unroll 1
                for (int group = half; group < 2 * kBlockChannels / 32; group += 2) {
                    const int c0 = group * 32;
                    if (c0 >= valid_channels) break; // warp-uniform
                    uint32_t r[2][16];
                    ptx::tmem_load16(lane_base + uint32_t(buffer * BN + c0), r[0]);
                    ptx::tmem_load16(lane_base + uint32_t(buffer * BN + c0 + 16), r[1]);
                    ptx::tmem_load_wait();
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int c = c0 + 16 * h;
                        if (c >= valid_channels) break;
                        float value[16];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float4 sw = *reinterpret_cast<const float4 *>(&sx_tile[buffer][c + 4 * q]); // broadcast read
                            const float w4[4] = {sw.x, sw.y, sw.z, sw.w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float acc = kInt ? float(int(r[h][4 * q + i])) : __uint_as_float(r[h][4 * q + i]);
                                value[4 * q + i] = __fmul_rn(__fmul_rn(acc, scale_x), w4[i]);
                            }
                        }
                        if (skip_row && token_ok) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const float4 s4 = __ldg(reinterpret_cast<const float4 *>(skip_row + c + 4 * q));
                                value[4 * q] = __fadd_rn(value[4 * q], s4.x); value[4 * q + 1] = __fadd_rn(value[4 * q + 1], s4.y);
                                value[4 * q + 2] = __fadd_rn(value[4 * q + 2], s4.z); value[4 * q + 3] = __fadd_rn(value[4 * q + 3], s4.w);
                            }
                        }
                        if (token_ok) {
                            uint32_t packed[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) packed[i] = pack16(value[2 * i], value[2 * i + 1], bf16_out ? int(Type::BF16) : int(Type::F16));
                            *reinterpret_cast<uint4 *>(out_row + c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                            *reinterpret_cast<uint4 *>(out_row + c + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        }
                    }
                }
                ptx::tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_rank(ptx::smem_u32(&acc_empty[buffer]), 0));
            }
        } else
        for (int tile = cluster_id; tile < tiles; tile += clusters, ++local) {
            const int buffer = local & 1;
            const int n0 = (tile % pair_tiles_n) * 2 * kBlockChannels + int(rank) * kBlockChannels;
            const int m0 = (tile / pair_tiles_n) * BN;
            const int valid_tokens = min(BN, a.m - m0);
            const int n = n0 + quadrant * 32 + lane;
            const float scale_w = n < a.n ? a.sw[n] : 0.f;
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
            // Hand the accumulator back to the leader's MMA issuer (remote arrive from the peer CTA).
            ptx::tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::map_to_rank(ptx::smem_u32(&acc_empty[buffer]), 0));
        }
        ptx::tcgen05_fence_before();
    }

    // Neither CTA may leave while the other can still signal its barriers or read its shared memory.
    __syncthreads();
    ptx::cluster_sync();
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, 512);
    }
    if (threadIdx.x == 0 && abort_flag) atomicExch(a.status, 1 + int(blockIdx.x));
}
} // namespace tts::b200
