// W8A8 GEMM + dequant epilogue for sm_100a: tcgen05 MMA (kind::i8 / kind::f8f6f4), accumulators in
// tensor memory, operands brought in by TMA with the 128-byte swizzle, split-K with an in-kernel,
// fixed-order reduction.
//
// Orientation: the 128-row MMA operand is a slab of 128 output channels of the weight matrix
// W[N,K]; the MMA "N" operand is a tile of BN tokens of X[M,K]. Both are K-contiguous exactly as
// the reference stores them, so no repacking is needed. One accumulator lane = one output channel,
// one accumulator column = one token; a warp storing one token writes 32 consecutive channels.
//
//   per-row scales : out[m,n] = D((float(acc) * sx[m]) * sw[n])
//                    (reference order: src/ops/kernels/quant/quant_gemm_sm80.cu:22-29)
//   K groups       : r += float(p_g) * (sx[g,m] * sw[g,n]) for g ascending, out = D(r)
//                    (reference: src/ops/kernels/quant/quant_grouped.cu:85-168); every group of
//                    128, 64 or 32 along K (the narrower of the two operands' group widths, as in
//                    the reference, :185-199) accumulates into a fresh tensor-memory buffer that the
//                    epilogue warps drain and rescale while the next group's MMAs run. A 128-byte K
//                    block is four 32-byte MMAs, so it splits into one, two or four such units.
//   split-K        : the splits of one output tile form a thread-block cluster. Token rows are dealt
//                    to the CTAs in blocks of 16; every CTA pushes its partial rows straight from
//                    tensor memory into the owner's shared memory (one slot per split, remote
//                    stores over distributed shared memory), one cluster barrier later the owner
//                    sums its slots in split order and finishes the rows. No workspace traffic, no
//                    second launch (replaces reference quant_reduce.cuh:9-29), deterministic.
//   launch overlap : the kernel starts under programmatic dependent launch: barriers, tensor
//                    memory and the first pipeline stages of WEIGHT tiles are set up while the
//                    producer of the activations is still running; only the activation tiles, the
//                    scales and the residual wait for it.
//   epilogue       : accumulators leave tensor memory lane-per-channel, are transposed through
//                    shared memory, and are finished token-row-wise so that every global access
//                    (fp32 residual, bias, bf16 store) is a coalesced 16-byte vector.
#pragma once
#include "kernels/sm100_ptx.cuh"
#include "kernels/quant_linear_geometry.h"
#include "kernels/sequence_finish.cuh"
#include "core/tensor.h"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tts::b200 {

constexpr int kGemmThreads = 320;   // warp 0 TMA, warp 1 MMA + TMEM, warps 2-9 epilogue
constexpr int kEpilogueThreads = 256;

// Workspace carve-up (owner zeroes the first kWorkspaceHeader bytes once). The GEMM itself needs
// no scratch; only the status word lives here.
constexpr size_t kStatusOffset = 16384;    // int status[4]: nonzero after a bounded wait gave up
constexpr size_t kWorkspaceHeader = 32768;

struct FusedEpilogue {
    const void *bias = nullptr;         // [N], output dtype
    const void *residual = nullptr;     // [M, residual_ld], output dtype
    const float *residual_f32 = nullptr; // [M, N] fp32, added before the first rounding
    float value_scale = 1.f, residual_scale = 1.f, output_scale = 1.f, alpha = .1f;
    int activation = 0;                 // ops::Activation
    int residual_ld = 0;
    int chain = 0;                      // nonzero when anything beyond residual_f32 is requested
};

struct GemmArgs {
    int m, n, k;
    const float *sx, *sw;
    void *out;
    int out_type; // Type::BF16, Type::F16, or Type::I32 (raw accumulators, per-row INT8 only)
    int input_group, weight_group;
    int splits, stages;
    int tile_region; // bytes of shared memory holding the pipeline stages (and, unsplit, the transposed tile)
    int owned_passes; // split-K: 16-row passes each CTA of the cluster may own (slots per split)
    int vector_io;   // every global row touched by the epilogue is 16-byte aligned
    int *status;
    // Failure-path exercise (host-side injection, see quant_linear_inject_wait_expiry): the first weight
    // barrier expects `expiry_extra_bytes` more than its copy delivers, and every wait gives up after
    // `wait_limit_cycles` (0 = the regular limit). Both zero in normal operation.
    int expiry_extra_bytes;
    long long wait_limit_cycles;
    FusedEpilogue ep;
};

__device__ __forceinline__ float round_to(float v, int type) {
    return type == int(Type::F16) ? __half2float(__float2half_rn(v)) : __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float load_as(const void *p, size_t i, int type) {
    return type == int(Type::F16) ? __half2float(static_cast<const __half *>(p)[i])
                                  : __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
}
// Post-GEMM chain on one rounded value; rounding points follow the reference's separate pass
// (src/ops/kernels/sequence/sequence_internal.cuh:52-74; the activations are the finishing pass's own
// instruction sequences, so GEMM + fused chain equals GEMM followed by that pass bit for bit). `bias` and `skip` are already fp32
// (0 when absent). Deliberately not inlined: the transcendental activations are large, and eight
// inlined copies per row pushed the common no-chain path out of the instruction cache.
__device__ __noinline__ float finish_chain(const FusedEpilogue &e, int type, float value, float bias, float skip) {
    value = round_to(value, type);
    if (e.bias) value = round_to(__fadd_rn(value, bias), type);
    if (e.residual || e.value_scale != 1.f)
        value = round_to(__fmaf_rn(e.value_scale, value, __fmul_rn(e.residual_scale, skip)), type); // contracted as in the reference's finishing pass
    if (e.activation || e.output_scale != 1.f)
        value = finish_activation(round_to(__fmul_rn(value, e.output_scale), type), e.activation, e.alpha);
    return value;
}
__device__ __forceinline__ uint32_t pack16(float lo, float hi, int type) {
    if (type == int(Type::F16)) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&b);
}

template <Type F, bool Grouped, int BN>
__global__ void __launch_bounds__(kGemmThreads, (!Grouped && BN <= 64) ? 2 : 1)
w8a8_tcgen05_gemm(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                  const __grid_constant__ GemmArgs a) {
    constexpr bool kInt = F == Type::I8;
    constexpr bool kIntAcc = kInt && !Grouped; // partial tiles / raw outputs carry int32 bit patterns
    constexpr int kWeightBytes = kBlockChannels * kBlockK, kTokenBytes = BN * kBlockK;
    constexpr int kStageBytes = kWeightBytes + kTokenBytes;
    // K-group mode gives every K block its own accumulator for as long as tensor memory lasts (512
    // columns: 32 buffers at BN=16 ... 4 at BN=128) and reuses them round-robin after that.
    constexpr int kAccBuffers = Grouped ? (512 / BN > 32 ? 32 : 512 / BN) : 1;
    constexpr int kAccColumns = Grouped ? kAccBuffers * BN : BN;
    constexpr uint32_t kTmemColumns = kAccColumns <= 32 ? 32 : kAccColumns <= 64 ? 64 : kAccColumns <= 128 ? 128
                                      : kAccColumns <= 256 ? 256 : 512;
    constexpr uint32_t kIdesc = kInt ? ptx::idesc_i8(kBlockChannels, BN) : ptx::idesc_e4m3(kBlockChannels, BN);
    constexpr int kChunks = BN / 16;               // 16-token column chunks of the accumulator
    constexpr int kMyChunks = (kChunks + 1) / 2;   // two epilogue warps share a lane quadrant
    constexpr uint32_t kPassBytes = kRowsPerPass * kBlockChannels * 4;

    extern __shared__ uint8_t dynamic_smem[];
    __shared__ alignas(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_full[kAccBuffers], acc_empty[kAccBuffers], x_full;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    __shared__ float sx_tile[BN]; // per-row activation scales of this token tile

    // Dynamic shared memory, 1024-byte aligned for the swizzled TMA boxes:
    //   [pipeline stages | split-K slots pushed by the cluster peers | K-group scales]
    // Unsplit launches reuse the stage memory for the transposed tile once the last MMA retired;
    // split launches must not, because peers push while this CTA may still be in its main loop.
    const uint32_t raw_base = ptx::smem_u32(dynamic_smem);
    const uint32_t tiles_base = (raw_base + 1023u) & ~1023u;
    uint8_t *tiles_ptr = dynamic_smem + (tiles_base - raw_base);
    const int splits = a.splits;
    const uint32_t reduce_bytes = splits > 1 ? uint32_t(splits * a.owned_passes) * kPassBytes : 0u;
    const uint32_t reduce_base = tiles_base + uint32_t(a.tile_region);
    uint8_t *reduce_ptr = tiles_ptr + a.tile_region;
    float *scale_smem = reinterpret_cast<float *>(reduce_ptr + reduce_bytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = splits > 1 ? int(ptx::cluster_ctarank()) : 0; // cluster = (1,1,splits): rank == blockIdx.z
    const int n0 = blockIdx.x * kBlockChannels, m0 = blockIdx.y * BN;
    const int kb_total = (a.k + kBlockK - 1) / kBlockK;
    const int kb_begin = int(int64_t(kb_total) * split / splits);
    const int kb_end = int(int64_t(kb_total) * (split + 1) / splits);
    const int kb_count = kb_end - kb_begin;
    // K-group mode: accumulation units per 128-byte K block (1, 2 or 4) and MMAs per unit.
    const int unit_k = Grouped ? min(a.input_group ? a.input_group : kBlockK, a.weight_group ? a.weight_group : kBlockK) : kBlockK;
    const int units = kBlockK / unit_k, unit_mmas = 4 / units;
    const int tile_linear = blockIdx.y * gridDim.x + blockIdx.x;
    const int valid_tokens = min(BN, a.m - m0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
        }

        for (int b = 0; b < kAccBuffers; ++b) {
            ptx::mbar_init(ptx::smem_u32(&acc_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&acc_empty[b]), kEpilogueThreads / 32);
        }
        ptx::mbar_init(ptx::smem_u32(&x_full), 1);
        abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    if (warp == 1) ptx::tmem_alloc(ptx::smem_u32(&tmem_slot), kTmemColumns);
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = tmem_slot;
    volatile int *abort_ptr = &abort_flag;
    const long long wait_limit = a.wait_limit_cycles > 0 ? a.wait_limit_cycles : ptx::kWaitLimitCycles;
    // The next kernel in the stream may begin its own prologue; peers learn that this CTA is running.
    ptx::launch_dependents();
    if (splits > 1) ptx::cluster_arrive();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::prefetch_tensormap(&map_w);
            ptx::prefetch_tensormap(&map_x);
            // Weights do not depend on the upstream kernel: fill the ring with weight tiles first
            // (one barrier per stage), then wait for upstream and add the activation tiles of all
            // those stages under ONE barrier. A barrier test between MMA issues costs the issuing
            // thread about 200 cycles, so the burst over the prefetched stages must not need any.
            // Weights are streamed once: they are marked first-to-evict so that the few megabytes of
            // activations the chain keeps passing from kernel to kernel stay in L2.
            const uint64_t stream_once = ptx::policy_evict_first();
            const int ahead = min(a.stages, kb_count);
            for (int i = 0; i < ahead; ++i) {
                const uint32_t bar = ptx::smem_u32(&full_bar[i]);
                ptx::mbar_arrive_expect_tx(bar, kWeightBytes + (i == 0 ? uint32_t(a.expiry_extra_bytes) : 0u));
                ptx::tma_load_2d_hint(tiles_base + uint32_t(i) * kStageBytes, &map_w, bar, (kb_begin + i) * kBlockK, n0, stream_once);
            }
            ptx::wait_for_upstream();
            ptx::mbar_arrive_expect_tx(ptx::smem_u32(&x_full), uint32_t(ahead) * kTokenBytes);
            for (int i = 0; i < ahead; ++i)
                ptx::tma_load_2d(tiles_base + uint32_t(i) * kStageBytes + kWeightBytes, &map_x,
                                 ptx::smem_u32(&x_full), (kb_begin + i) * kBlockK, m0);
            int stage = ahead == a.stages ? 0 : ahead;
            uint32_t phase = ahead == a.stages ? 1u : 0u;
            for (int kb = kb_begin + ahead; kb < kb_end; ++kb) {
                if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_ptr, wait_limit)) break;
                const uint32_t bar = ptx::smem_u32(&full_bar[stage]);
                const uint32_t dst = tiles_base + uint32_t(stage) * kStageBytes;
                ptx::mbar_arrive_expect_tx(bar, kStageBytes);
                ptx::tma_load_2d_hint(dst, &map_w, bar, kb * kBlockK, n0, stream_once);
                ptx::tma_load_2d(dst + kWeightBytes, &map_x, bar, kb * kBlockK, m0);
                if (++stage == a.stages) { stage = 0; phase ^= 1u; }
            }
        }
        if (splits > 1) ptx::cluster_wait();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp runs the loop so that stage indices and descriptors stay warp-uniform (the
        // tensor-core instructions take them from uniform registers); one elected lane issues.
        {
            // The weight tiles of the prefetched stages land while the upstream kernel still runs:
            // collect those barriers now, off the critical path, then wait once for the activations.
            const int ahead = min(a.stages, kb_count);
            bool ok = true;
            for (int i = 0; i < ahead && ok; ++i) ok = ptx::mbar_wait(ptx::smem_u32(&full_bar[i]), 0u, abort_ptr, wait_limit);
            ok = ok && ptx::mbar_wait(ptx::smem_u32(&x_full), 0u, abort_ptr, wait_limit);
            ok = __all_sync(0xffffffffu, ok);
            // The prefetched stages need no barrier at all any more, so their MMAs go out back to back
            // (any shared-memory access between MMA issues stalls the issuing warp for a couple of
            // hundred cycles). Stage i holds K block i here; in K-group mode K block i also has
            // accumulator i to itself while fresh accumulators last.
            // Narrow K groups: the MMAs of one 128-byte K block go to `units` accumulators, `unit_mmas`
            // each; every accumulator reports on its own barrier.
            auto issue_units = [&](uint32_t lo_w, uint32_t lo_x, uint32_t d_first, int buffer_first) {
                for (int u = 0; u < units; ++u) {
                    for (int s = 0; s < unit_mmas; ++s) {
                        const uint32_t step = uint32_t(2 * (u * unit_mmas + s)); // 32 bytes of K = 2 descriptor units
                        if (kInt) ptx::mma_i8_lo(d_first + uint32_t(u * BN), lo_w + step, lo_x + step, kIdesc, uint32_t(s > 0));
                        else ptx::mma_f8_lo(d_first + uint32_t(u * BN), lo_w + step, lo_x + step, kIdesc, uint32_t(s > 0));
                    }
                    ptx::tcgen05_commit(ptx::smem_u32(&acc_full[buffer_first + u]));
                }
            };
            int first = 0;
            if (ok) {
                const int burst = Grouped ? min(ahead, kAccBuffers / units) : ahead;
                ptx::tcgen05_fence_after();
                for (int it = 0; it < burst; ++it) {
                    const uint32_t tile = tiles_base + uint32_t(it) * kStageBytes;
                    const uint32_t lo_w = ptx::smem_desc_lo_k128(tile), lo_x = ptx::smem_desc_lo_k128(tile + kWeightBytes);
                    const uint32_t d = tmem_base + (Grouped ? uint32_t(it * units * BN) : 0u);
                    if (ptx::elect_one()) {
                        if (!Grouped || units == 1) {
                            const uint32_t accumulate = Grouped ? 0u : uint32_t(it > 0);
                            if (kInt) ptx::mma_i8_k128(d, lo_w, lo_x, kIdesc, accumulate);
                            else ptx::mma_f8_k128(d, lo_w, lo_x, kIdesc, accumulate);
                        } else {
                            issue_units(lo_w, lo_x, d, it * units);
                        }
                        // Only a stage that will be refilled needs to report that its MMAs retired.
                        if (it + a.stages < kb_count) ptx::tcgen05_commit(ptx::smem_u32(&empty_bar[it]));
                        if (Grouped && units == 1) ptx::tcgen05_commit(ptx::smem_u32(&acc_full[it]));
                    }
                    __syncwarp();
                }
                first = burst;
            }
            int stage = first == a.stages ? 0 : first;
            uint32_t phase = first == a.stages ? 1u : 0u;
            // Refilled stages arrive at the rate memory delivers them, one barrier each.
            for (int it = first; it < kb_count && ok; ++it) {
                const int buffer = Grouped ? (it * units) % kAccBuffers : 0;
                if (Grouped && it * units >= kAccBuffers) // the epilogue drained these accumulators' previous groups
                    for (int u = 0; u < units && ok; ++u)
                        ok = ptx::mbar_wait(ptx::smem_u32(&acc_empty[buffer + u]),
                                            (uint32_t((it * units + u) / kAccBuffers) & 1u) ^ 1u, abort_ptr, wait_limit);
                if (it >= ahead) ok = ok && ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_ptr, wait_limit);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ptx::tcgen05_fence_after();
                const uint32_t tile = tiles_base + uint32_t(stage) * kStageBytes;
                const uint32_t lo_w = ptx::smem_desc_lo_k128(tile), lo_x = ptx::smem_desc_lo_k128(tile + kWeightBytes);
                const uint32_t d = tmem_base + uint32_t(buffer * BN);
                if (ptx::elect_one()) {
                    if (!Grouped || units == 1) {
                        const uint32_t accumulate = Grouped ? 0u : uint32_t(it > 0);
                        if (kInt) ptx::mma_i8_k128(d, lo_w, lo_x, kIdesc, accumulate);
                        else ptx::mma_f8_k128(d, lo_w, lo_x, kIdesc, accumulate);
                    } else {
                        issue_units(lo_w, lo_x, d, buffer);
                    }
                    if (it + a.stages < kb_count) ptx::tcgen05_commit(ptx::smem_u32(&empty_bar[stage]));
                    if (Grouped && units == 1) ptx::tcgen05_commit(ptx::smem_u32(&acc_full[buffer]));
                }
                __syncwarp();
                if (++stage == a.stages) { stage = 0; phase ^= 1u; }
            }
            if (ptx::elect_one()) {
                if (!Grouped) ptx::tcgen05_commit(ptx::smem_u32(&acc_full[0]));
            }
            __syncwarp();
        }
        if (splits > 1) ptx::cluster_wait();
    } else {
        // ------------------------------------------------------------ epilogue warps (8 warps)
        const int e_thread = threadIdx.x - 64;
        const int quadrant = warp & 3;      // tensor-memory lanes this warp may read
        const int half = (warp - 2) >> 2;   // the two warps of a quadrant take alternate 16-token chunks
        const int channel_in_tile = quadrant * 32 + lane;
        const uint32_t lane_base = tmem_base + (uint32_t(quadrant * 32) << 16);
        uint32_t *tile_words = reinterpret_cast<uint32_t *>(tiles_ptr);
        bool ok = true;

        // Phase-2 ownership of this thread: 8 consecutive channels of one token row per pass.
        const int j = e_thread & 15, row_in_pass = e_thread >> 4;
        const int n = n0 + 8 * j;
        const bool columns_ok = n < a.n;
        const FusedEpilogue &e = a.ep;
        const int type = a.out_type;
        const int passes = (valid_tokens + kRowsPerPass - 1) / kRowsPerPass;
        // Static operands (weights' scales, bias) are fetched before anything else so their latency
        // hides behind the main loop.
        float sw8[8], bias8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            sw8[i] = (!Grouped && columns_ok) ? a.sw[n + i] : 1.f;
            bias8[i] = (e.bias && columns_ok) ? load_as(e.bias, n + i, type) : 0.f;
        }
        // K-group mode: the weights' group scales of this CTA's K range are static too, one entry per
        // accumulation unit (a unit past the end of K, whose accumulator holds zeros, takes scale 1).
        const int unit_count = kb_count * units;
        float *sx_smem = scale_smem, *sw_smem = scale_smem + size_t(unit_count) * BN;
        if constexpr (Grouped) {
            for (int i = e_thread; i < unit_count * kBlockChannels; i += kEpilogueThreads) {
                const int unit = i / kBlockChannels, channel = n0 + i % kBlockChannels, k0 = kb_begin * kBlockK + unit * unit_k;
                sw_smem[i] = (a.weight_group && channel < a.n && k0 < a.k) ? a.sw[size_t(k0 / a.weight_group) * a.n + channel] : 1.f;
            }
        }
        ptx::wait_for_upstream(); // activation scales, residuals and the output buffer belong to upstream
        float first_residual[8];
        {
            const int c = split * kRowsPerPass + row_in_pass; // first pass this CTA owns
#pragma unroll
            for (int i = 0; i < 8; ++i) first_residual[i] = 0.f;
            if (e.residual_f32 && columns_ok && c < valid_tokens) {
                const float *src = e.residual_f32 + size_t(m0 + c) * a.n + n;
                if (a.vector_io) {
                    const float4 lo = *reinterpret_cast<const float4 *>(src), hi = *reinterpret_cast<const float4 *>(src + 4);
                    first_residual[0] = lo.x; first_residual[1] = lo.y; first_residual[2] = lo.z; first_residual[3] = lo.w;
                    first_residual[4] = hi.x; first_residual[5] = hi.y; first_residual[6] = hi.z; first_residual[7] = hi.w;
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) first_residual[i] = src[i];
                }
            }
        }

        // ---- phase 1: accumulators (one lane = one channel) -> [token][channel] rows, either in this
        // CTA's shared memory (unsplit) or pushed into the owning peer's slot for this split.
        auto emit_chunk = [&](int chunk, const uint32_t (&words)[16]) {
            if (splits == 1) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (chunk * 16 + i < valid_tokens) tile_words[(chunk * 16 + i) * kBlockChannels + channel_in_tile] = words[i];
            } else {
                const int owner = chunk % splits, local_pass = chunk / splits;
                const uint32_t slot = reduce_base + uint32_t(split * a.owned_passes + local_pass) * kPassBytes +
                                      uint32_t(channel_in_tile) * 4u;
                const uint32_t remote = ptx::map_to_rank(slot, uint32_t(owner));
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if (chunk * 16 + i < valid_tokens) ptx::st_cluster_u32(remote + uint32_t(i) * (kBlockChannels * 4u), words[i]);
            }
        };

        if constexpr (!Grouped) {
            for (int c = e_thread; c < BN; c += kEpilogueThreads) sx_tile[c] = c < valid_tokens ? a.sx[m0 + c] : 0.f;
            ok = ptx::mbar_wait(ptx::smem_u32(&acc_full[0]), 0, abort_ptr, wait_limit);
            ptx::tcgen05_fence_after();
            if (splits > 1) ptx::cluster_wait(); // every peer is running: its shared memory may be written
            if (ok) {
                // Two chunks per round: both loads are in flight before the single wait.
#pragma unroll 1
                for (int chunk = half; chunk < kChunks; chunk += 4) {
                    if (chunk * 16 >= valid_tokens) break;
                    const bool second = chunk + 2 < kChunks && (chunk + 2) * 16 < valid_tokens;
                    uint32_t r0[16], r1[16];
                    ptx::tmem_load16(lane_base + uint32_t(chunk * 16), r0);
                    if (second) ptx::tmem_load16(lane_base + uint32_t((chunk + 2) * 16), r1);
                    ptx::tmem_load_wait();
                    emit_chunk(chunk, r0);
                    if (second) emit_chunk(chunk + 2, r1);
                }
            }
        } else {
            // Stage the activations' group scales of this split (the weights' were staged before the wait):
            // sx_g[unit][token], each operand indexed by its own group width.
            for (int i = e_thread; i < unit_count * BN; i += kEpilogueThreads) {
                const int unit = i / BN, token = i % BN, k0 = kb_begin * kBlockK + unit * unit_k;
                sx_smem[i] = (a.input_group && token < valid_tokens && k0 < a.k)
                                 ? a.sx[size_t(k0 / a.input_group) * a.m + m0 + token] : 1.f;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            float result[kMyChunks * 16];
#pragma unroll
            for (int c = 0; c < kMyChunks * 16; ++c) result[c] = 0.f;
#pragma unroll 1
            for (int it = 0; it < unit_count && ok; ++it) {
                const int buffer = it % kAccBuffers;
                ok = ptx::mbar_wait(ptx::smem_u32(&acc_full[buffer]), uint32_t(it / kAccBuffers) & 1u, abort_ptr, wait_limit);
                if (!ok) break;
                ptx::tcgen05_fence_after();
                const float scale_w = sw_smem[it * kBlockChannels + channel_in_tile];
                const float *scale_x = sx_smem + it * BN;
                uint32_t r[kMyChunks][16];
#pragma unroll
                for (int k = 0; k < kMyChunks; ++k)
                    if (2 * k + half < kChunks) ptx::tmem_load16(lane_base + uint32_t(buffer * BN + (2 * k + half) * 16), r[k]);
                ptx::tmem_load_wait();
                // Everything this warp needs is in registers: hand the buffer back before the arithmetic.
                ptx::tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&acc_empty[buffer]));
#pragma unroll
                for (int k = 0; k < kMyChunks; ++k) {
                    if (2 * k + half < kChunks) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            // |p| <= 128*127^2 < 2^24, so the int -> float conversion is exact.
                            const float p = kInt ? float(int(r[k][i])) : __uint_as_float(r[k][i]);
                            result[k * 16 + i] = fmaf(p, scale_x[(2 * k + half) * 16 + i] * scale_w, result[k * 16 + i]);
                        }
                    }
                }
            }
            if (splits > 1) ptx::cluster_wait();
            if (ok) {
                // Outer scales exist only when just one operand carries K-group scales.
                const int channel = n0 + channel_in_tile;
                const float outer_w = (!a.weight_group && channel < a.n) ? a.sw[channel] : 1.f;
#pragma unroll
                for (int k = 0; k < kMyChunks; ++k) {
                    const int chunk = 2 * k + half;
                    if (chunk < kChunks && chunk * 16 < valid_tokens) {
                        uint32_t words[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int c = chunk * 16 + i;
                            const float outer = (a.input_group || c >= valid_tokens) ? 1.f : a.sx[m0 + c];
                            words[i] = __float_as_uint(result[k * 16 + i] * (outer * outer_w));
                        }
                        emit_chunk(chunk, words);
                    }
                }
            }
        }
        ptx::tcgen05_fence_before();

        // ---- phase boundary: rows are where their finisher will read them.
        if (splits > 1) ptx::cluster_sync();
        else asm volatile("bar.sync 1, 256;" ::: "memory");

        // ---- phase 2: finish token rows; every global access is a 16-byte vector on a 256-byte row.
        // The common case (bf16 out, aligned rows, nothing but an optional fp32 residual) takes a lean
        // loop; everything else takes the general loop below it.
        const bool lean = type == int(Type::BF16) && a.vector_io && !e.chain;
        if (ok && !*abort_ptr && columns_ok && lean) {
            const float *__restrict__ residual = e.residual_f32; // never aliases the output rows
            uint16_t *__restrict__ out16 = static_cast<uint16_t *>(a.out);
            const size_t slot_stride = size_t(a.owned_passes) * kPassBytes;
#pragma unroll 2
            for (int local_pass = 0;; ++local_pass) {
                const int pass = local_pass * splits + split;
                if (pass >= passes) break;
                const int c = pass * kRowsPerPass + row_in_pass;
                if (c >= valid_tokens) continue;
                const size_t at = size_t(m0 + c) * a.n + n;
                float r8[8];
                if (residual && local_pass > 0) {
                    const float4 lo = *reinterpret_cast<const float4 *>(residual + at), hi = *reinterpret_cast<const float4 *>(residual + at + 4);
                    r8[0] = lo.x; r8[1] = lo.y; r8[2] = lo.z; r8[3] = lo.w; r8[4] = hi.x; r8[5] = hi.y; r8[6] = hi.z; r8[7] = hi.w;
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) r8[i] = first_residual[i];
                }
                uint32_t raw[8];
                if (splits == 1) {
                    const uint8_t *src = tiles_ptr + size_t(c * kBlockChannels + 8 * j) * 4;
                    const uint4 lo = *reinterpret_cast<const uint4 *>(src), hi = *reinterpret_cast<const uint4 *>(src + 16);
                    raw[0] = lo.x; raw[1] = lo.y; raw[2] = lo.z; raw[3] = lo.w; raw[4] = hi.x; raw[5] = hi.y; raw[6] = hi.z; raw[7] = hi.w;
                } else {
                    const uint8_t *src = reduce_ptr + size_t(local_pass) * kPassBytes + size_t(row_in_pass * kBlockChannels + 8 * j) * 4;
#pragma unroll
                    for (int i = 0; i < 8; ++i) raw[i] = 0u;
                    for (int s = 0; s < splits; ++s) {
                        const uint4 lo = *reinterpret_cast<const uint4 *>(src + s * slot_stride);
                        const uint4 hi = *reinterpret_cast<const uint4 *>(src + s * slot_stride + 16);
                        const uint32_t part[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            raw[i] = kIntAcc ? uint32_t(int(raw[i]) + int(part[i]))
                                             : __float_as_uint(__fadd_rn(__uint_as_float(raw[i]), __uint_as_float(part[i])));
                    }
                }
                const float scale_x = sx_tile[Grouped ? 0 : c];
                float value[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float acc = kIntAcc ? float(int(raw[i])) : __uint_as_float(raw[i]);
                    value[i] = Grouped ? acc : __fmul_rn(__fmul_rn(acc, scale_x), sw8[i]);
                    if (residual) value[i] = __fadd_rn(value[i], r8[i]);
                }
                uint4 packed;
                {
                    __nv_bfloat162 b0 = __floats2bfloat162_rn(value[0], value[1]), b1 = __floats2bfloat162_rn(value[2], value[3]);
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(value[4], value[5]), b3 = __floats2bfloat162_rn(value[6], value[7]);
                    packed = make_uint4(*reinterpret_cast<uint32_t *>(&b0), *reinterpret_cast<uint32_t *>(&b1),
                                        *reinterpret_cast<uint32_t *>(&b2), *reinterpret_cast<uint32_t *>(&b3));
                }
                *reinterpret_cast<uint4 *>(out16 + at) = packed;
            }
        } else if (ok && !*abort_ptr && columns_ok) {
            for (int local_pass = 0;; ++local_pass) {
                const int pass = local_pass * splits + split;
                if (pass >= passes) break;
                const int c = pass * kRowsPerPass + row_in_pass;
                if (c >= valid_tokens) continue;
                const int m = m0 + c;
                uint32_t raw[8];
                if (splits == 1) {
                    const uint8_t *src = tiles_ptr + size_t(c * kBlockChannels + 8 * j) * 4;
                    const uint4 lo = *reinterpret_cast<const uint4 *>(src), hi = *reinterpret_cast<const uint4 *>(src + 16);
                    raw[0] = lo.x; raw[1] = lo.y; raw[2] = lo.z; raw[3] = lo.w;
                    raw[4] = hi.x; raw[5] = hi.y; raw[6] = hi.z; raw[7] = hi.w;
                } else {
                    // Slots of this pass, one per split, summed in split order (deterministic).
                    const uint8_t *src = reduce_ptr + size_t(local_pass) * kPassBytes + size_t(row_in_pass * kBlockChannels + 8 * j) * 4;
                    const size_t slot_stride = size_t(a.owned_passes) * kPassBytes;
#pragma unroll
                    for (int i = 0; i < 8; ++i) raw[i] = 0u; // int 0 and +0.f share this pattern
                    for (int s = 0; s < splits; ++s) {
                        const uint4 lo = *reinterpret_cast<const uint4 *>(src + s * slot_stride);
                        const uint4 hi = *reinterpret_cast<const uint4 *>(src + s * slot_stride + 16);
                        const uint32_t part[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            raw[i] = kIntAcc ? uint32_t(int(raw[i]) + int(part[i]))
                                             : __float_as_uint(__fadd_rn(__uint_as_float(raw[i]), __uint_as_float(part[i])));
                    }
                }
                const size_t at = size_t(m) * a.n + n;
                if (type == int(Type::I32)) {
                    uint32_t *dst = static_cast<uint32_t *>(a.out) + at;
                    if (a.vector_io) {
                        *reinterpret_cast<uint4 *>(dst) = make_uint4(raw[0], raw[1], raw[2], raw[3]);
                        *reinterpret_cast<uint4 *>(dst + 4) = make_uint4(raw[4], raw[5], raw[6], raw[7]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) dst[i] = raw[i];
                    }
                    continue;
                }
                float value[8];
                const float scale_x = sx_tile[Grouped ? 0 : c];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float acc = kIntAcc ? float(int(raw[i])) : __uint_as_float(raw[i]);
                    value[i] = Grouped ? acc : __fmul_rn(__fmul_rn(acc, scale_x), sw8[i]);
                }
                if (e.residual_f32) {
                    float r8[8];
                    if (local_pass == 0) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) r8[i] = first_residual[i];
                    } else if (a.vector_io) {
                        const float4 lo = *reinterpret_cast<const float4 *>(e.residual_f32 + at);
                        const float4 hi = *reinterpret_cast<const float4 *>(e.residual_f32 + at + 4);
                        r8[0] = lo.x; r8[1] = lo.y; r8[2] = lo.z; r8[3] = lo.w;
                        r8[4] = hi.x; r8[5] = hi.y; r8[6] = hi.z; r8[7] = hi.w;
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) r8[i] = e.residual_f32[at + i];
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) value[i] = __fadd_rn(value[i], r8[i]);
                }
                if (e.chain) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float skip = e.residual ? load_as(e.residual, size_t(m) * e.residual_ld + n + i, type) : 0.f;
                        value[i] = finish_chain(e, type, value[i], bias8[i], skip);
                    }
                }
                uint16_t *dst = static_cast<uint16_t *>(a.out) + at;
                const uint4 packed = make_uint4(pack16(value[0], value[1], type), pack16(value[2], value[3], type),
                                                pack16(value[4], value[5], type), pack16(value[6], value[7], type));
                if (a.vector_io) {
                    *reinterpret_cast<uint4 *>(dst) = packed;
                } else {
                    dst[0] = uint16_t(packed.x); dst[1] = uint16_t(packed.x >> 16);
                    dst[2] = uint16_t(packed.y); dst[3] = uint16_t(packed.y >> 16);
                    dst[4] = uint16_t(packed.z); dst[5] = uint16_t(packed.z >> 16);
                    dst[6] = uint16_t(packed.w); dst[7] = uint16_t(packed.w >> 16);
                }
            }
        }
    }
    if (warp < 2 && splits > 1) ptx::cluster_sync(); // the producer/MMA warps' share of the phase barrier

    __syncthreads(); // tensor memory is drained and nobody else will touch this CTA's shared memory
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemColumns);
    }
    if (threadIdx.x == 0 && abort_flag) atomicExch(a.status, 1 + tile_linear);
}
} // namespace tts::b200
