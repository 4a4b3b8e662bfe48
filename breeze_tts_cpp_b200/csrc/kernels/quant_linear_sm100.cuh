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
//   K128 groups    : r += float(p_g) * (sx[g,m] * sw[g,n]) for g ascending, out = D(r)
//                    (reference: src/ops/kernels/quant/quant_grouped.cu:85-168); every K block
//                    accumulates into a fresh tensor-memory buffer that the epilogue warps drain
//                    and rescale while the next block's MMAs run.
//   split-K        : every split writes its partial tile to the workspace; the last one to arrive
//                    (an atomic ticket, no spinning) sums the partials in split order and runs the
//                    epilogue, then resets the ticket
//                    (replaces reference quant_reduce.cuh:9-29, a second launch).
#pragma once
#include "kernels/sm100_ptx.cuh"
#include "core/tensor.h"
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tts::b200 {

constexpr int kBlockChannels = 128; // MMA M: weight rows per tile
constexpr int kBlockK = 128;        // bytes of K per pipeline stage (one 128B-swizzled TMA box)
constexpr int kMaxStages = 12;
constexpr int kGemmThreads = 192;   // warp 0 TMA, warp 1 MMA + TMEM, warps 2-5 epilogue

// Workspace carve-up (owner zeroes the first kWorkspaceHeader bytes once):
constexpr size_t kTicketBytes = 16384;     // int tickets, one per output tile
constexpr size_t kStatusOffset = 16384;    // int status[4]: nonzero after a bounded wait gave up
constexpr size_t kWorkspaceHeader = 32768; // split-K partials start here

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
    float *partials; // 4-byte partial sums (int32 bit patterns or fp32)
    int *tickets;
    int *status;
    FusedEpilogue ep;
};

__device__ __forceinline__ float round_to(float v, int type) {
    return type == int(Type::F16) ? __half2float(__float2half_rn(v)) : __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ float load_as(const void *p, size_t i, int type) {
    return type == int(Type::F16) ? __half2float(static_cast<const __half *>(p)[i])
                                  : __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
}
// reference: src/ops/kernels/common/activation.cuh:5-27
__device__ __forceinline__ float activate(float x, int kind, float alpha) {
    switch (kind) {
    case 1: return fmaxf(x, 0.f);
    case 2: return x >= 0 ? x : x * alpha;
    case 3: return x / (1.f + expf(-x));
    case 4: return .5f * x * (1.f + erff(x * .7071067811865475f));
    case 5: return .5f * x * (1.f + tanhf(.7978845608028654f * (x + .044715f * x * x * x)));
    case 7: return tanhf(x);
    case 8: return 1.f / (1.f + expf(-x));
    default: return x;
    }
}

// Dequantized fp32 value -> stored element, with the optional chain whose rounding points follow
// the reference's post-GEMM pass (src/ops/kernels/sequence/sequence_internal.cuh:52-74).
__device__ __forceinline__ void store_output(const GemmArgs &a, float value, int m, int n) {
    const size_t at = size_t(m) * a.n + n;
    const FusedEpilogue &e = a.ep;
    if (e.residual_f32) value = __fadd_rn(value, e.residual_f32[at]);
    if (e.chain) {
        const int t = a.out_type;
        value = round_to(value, t);
        if (e.bias) value = round_to(__fadd_rn(value, load_as(e.bias, n, t)), t);
        if (e.residual || e.value_scale != 1.f) {
            float skip = e.residual ? load_as(e.residual, size_t(m) * e.residual_ld + n, t) : 0.f;
            value = round_to(__fadd_rn(__fmul_rn(e.value_scale, value), __fmul_rn(e.residual_scale, skip)), t);
        }
        if (e.activation || e.output_scale != 1.f)
            value = activate(round_to(__fmul_rn(value, e.output_scale), t), e.activation, e.alpha);
    }
    if (a.out_type == int(Type::F16)) static_cast<__half *>(a.out)[at] = __float2half_rn(value);
    else static_cast<__nv_bfloat16 *>(a.out)[at] = __float2bfloat16_rn(value);
}

template <Type F, bool Grouped, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
w8a8_tcgen05_gemm(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                  const GemmArgs a) {
    constexpr bool kInt = F == Type::I8;
    constexpr bool kIntAcc = kInt && !Grouped; // partials / raw outputs carry int32 bit patterns
    constexpr int kWeightBytes = kBlockChannels * kBlockK, kTokenBytes = BN * kBlockK;
    constexpr int kStageBytes = kWeightBytes + kTokenBytes;
    constexpr int kAccColumns = Grouped ? 2 * BN : BN;
    constexpr uint32_t kTmemColumns = kAccColumns <= 32 ? 32 : kAccColumns <= 64 ? 64 : kAccColumns <= 128 ? 128
                                      : kAccColumns <= 256 ? 256 : 512;
    constexpr uint32_t kIdesc = kInt ? ptx::idesc_i8(kBlockChannels, BN) : ptx::idesc_e4m3(kBlockChannels, BN);

    extern __shared__ uint8_t dynamic_smem[];
    __shared__ alignas(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag, last_flag;

    const uint32_t raw_base = ptx::smem_u32(dynamic_smem);
    const uint32_t tiles_base = (raw_base + 1023u) & ~1023u;
    uint8_t *tiles_ptr = dynamic_smem + (tiles_base - raw_base);
    float *scale_smem = reinterpret_cast<float *>(tiles_ptr + size_t(a.stages) * kStageBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kBlockChannels, m0 = blockIdx.y * BN, split = blockIdx.z;
    const int kb_total = (a.k + kBlockK - 1) / kBlockK;
    const int kb_begin = int(int64_t(kb_total) * split / a.splits);
    const int kb_end = int(int64_t(kb_total) * (split + 1) / a.splits);
    const int kb_count = kb_end - kb_begin;
    const int tile_linear = blockIdx.y * gridDim.x + blockIdx.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            ptx::mbar_init(ptx::smem_u32(&full_bar[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&acc_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&acc_empty[b]), 4);
        }
        abort_flag = 0;
        last_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    if (warp == 1) ptx::tmem_alloc(ptx::smem_u32(&tmem_slot), kTmemColumns);
    ptx::tcgen05_fence_before();
    __syncthreads();
    ptx::tcgen05_fence_after();
    const uint32_t tmem_base = tmem_slot;
    volatile int *abort_ptr = &abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::prefetch_tensormap(&map_w);
            ptx::prefetch_tensormap(&map_x);
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = kb_begin; kb < kb_end; ++kb) {
                if (!ptx::mbar_wait(ptx::smem_u32(&empty_bar[stage]), phase ^ 1u, abort_ptr)) break;
                const uint32_t bar = ptx::smem_u32(&full_bar[stage]);
                const uint32_t dst = tiles_base + uint32_t(stage) * kStageBytes;
                ptx::mbar_arrive_expect_tx(bar, kStageBytes);
                ptx::tma_load_2d(dst, &map_w, bar, kb * kBlockK, n0);
                ptx::tma_load_2d(dst + kWeightBytes, &map_x, bar, kb * kBlockK, m0);
                if (++stage == a.stages) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int it = 0; it < kb_count; ++it) {
                const int buffer = Grouped ? (it & 1) : 0;
                if (Grouped && !ptx::mbar_wait(ptx::smem_u32(&acc_empty[buffer]), ((uint32_t(it) >> 1) & 1u) ^ 1u, abort_ptr))
                    break;
                if (!ptx::mbar_wait(ptx::smem_u32(&full_bar[stage]), phase, abort_ptr)) break;
                ptx::tcgen05_fence_after();
                const uint32_t tile = tiles_base + uint32_t(stage) * kStageBytes;
                const uint64_t desc_w = ptx::smem_desc_k128(tile), desc_x = ptx::smem_desc_k128(tile + kWeightBytes);
                const uint32_t d = tmem_base + uint32_t(buffer * BN);
#pragma unroll
                for (int step = 0; step < kBlockK / 32; ++step) {
                    const uint32_t accumulate = Grouped ? (step > 0) : (it > 0 || step > 0);
                    // 32 bytes of K per MMA: +2 in the descriptor's 16-byte address units.
                    if (kInt) ptx::mma_i8(d, desc_w + uint64_t(step * 2), desc_x + uint64_t(step * 2), kIdesc, accumulate);
                    else ptx::mma_f8(d, desc_w + uint64_t(step * 2), desc_x + uint64_t(step * 2), kIdesc, accumulate);
                }
                ptx::tcgen05_commit(ptx::smem_u32(&empty_bar[stage]));
                if (Grouped) ptx::tcgen05_commit(ptx::smem_u32(&acc_full[buffer]));
                if (++stage == a.stages) { stage = 0; phase ^= 1u; }
            }
            if (!Grouped) ptx::tcgen05_commit(ptx::smem_u32(&acc_full[0]));
        }
    } else {
        // ------------------------------------------------------------ epilogue warps
        const int quadrant = warp & 3;             // tensor-memory lanes this warp may read
        const int channel_in_tile = quadrant * 32 + lane;
        const int n = n0 + channel_in_tile;
        const int epi_thread = threadIdx.x - 64;
        const uint32_t lane_base = tmem_base + (uint32_t(quadrant * 32) << 16);
        const int valid_tokens = min(BN, a.m - m0);
        const bool channel_ok = n < a.n;
        float *my_partials = a.partials + (size_t(tile_linear) * a.splits + split) * BN * kBlockChannels;
        bool ok = true;

        if constexpr (!Grouped) {
            ok = ptx::mbar_wait(ptx::smem_u32(&acc_full[0]), 0, abort_ptr);
            ptx::tcgen05_fence_after();
            const float scale_w = channel_ok ? a.sw[n] : 0.f;
            if (ok) {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    if (c0 >= valid_tokens) break;
                    uint32_t r[16];
                    ptx::tmem_load16(lane_base + uint32_t(c0), r);
                    ptx::tmem_load_wait();
                    if (a.splits > 1) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (c0 + i < valid_tokens)
                                __stcg(reinterpret_cast<uint32_t *>(my_partials) + size_t(c0 + i) * kBlockChannels + channel_in_tile, r[i]);
                    } else if (channel_ok) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int m = m0 + c0 + i;
                            if (c0 + i < valid_tokens) {
                                if (a.out_type == int(Type::I32)) {
                                    static_cast<uint32_t *>(a.out)[size_t(m) * a.n + n] = r[i];
                                } else {
                                    float acc = kInt ? float(int(r[i])) : __uint_as_float(r[i]);
                                    store_output(a, __fmul_rn(__fmul_rn(acc, a.sx[m]), scale_w), m, n);
                                }
                            }
                        }
                    }
                }
            }
        } else {
            // Stage this split's group scales once: sx_g[block][token], sw_g[block][channel].
            float *sx_smem = scale_smem, *sw_smem = scale_smem + size_t(kb_count) * BN;
            for (int i = epi_thread; i < kb_count * BN; i += 128) {
                int block = i / BN, token = i % BN;
                sx_smem[i] = (a.input_group && token < valid_tokens)
                                 ? a.sx[size_t(kb_begin + block) * a.m + m0 + token] : 1.f;
            }
            for (int i = epi_thread; i < kb_count * kBlockChannels; i += 128) {
                int block = i / kBlockChannels, channel = n0 + i % kBlockChannels;
                sw_smem[i] = (a.weight_group && channel < a.n) ? a.sw[size_t(kb_begin + block) * a.n + channel] : 1.f;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            float result[BN];
#pragma unroll
            for (int c = 0; c < BN; ++c) result[c] = 0.f;
#pragma unroll 1
            for (int it = 0; it < kb_count && ok; ++it) {
                const int buffer = it & 1;
                ok = ptx::mbar_wait(ptx::smem_u32(&acc_full[buffer]), (uint32_t(it) >> 1) & 1u, abort_ptr);
                if (!ok) break;
                ptx::tcgen05_fence_after();
                const float scale_w = sw_smem[it * kBlockChannels + channel_in_tile];
                const float *scale_x = sx_smem + it * BN;
#pragma unroll
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t r[16];
                    ptx::tmem_load16(lane_base + uint32_t(buffer * BN + c0), r);
                    ptx::tmem_load_wait();
                    if (c0 + 16 >= BN) {
                        // Last chunk read: hand the buffer back before doing the arithmetic.
                        ptx::tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&acc_empty[buffer]));
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        // |p| <= 128*127^2 < 2^24, so the int -> float conversion is exact.
                        float p = kInt ? float(int(r[i])) : __uint_as_float(r[i]);
                        result[c0 + i] = fmaf(p, scale_x[c0 + i] * scale_w, result[c0 + i]);
                    }
                }
            }
            if (ok) {
                float outer_w = (!a.weight_group && channel_ok) ? a.sw[n] : 1.f;
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    if (c < valid_tokens) {
                        const int m = m0 + c;
                        float value = result[c] * ((a.input_group ? 1.f : a.sx[m]) * outer_w);
                        if (a.splits > 1) __stcg(my_partials + size_t(c) * kBlockChannels + channel_in_tile, value);
                        else if (channel_ok) store_output(a, value, m, n);
                    }
                }
            }
        }

        if (a.splits > 1) {
            // Publish the partial tile, take a ticket; the last split to arrive reduces all of them.
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (epi_thread == 0) {
                int ticket = atomicAdd(a.tickets + tile_linear, 1);
                int last = ticket == a.splits - 1;
                if (last) a.tickets[tile_linear] = 0; // self-resetting for the next launch / graph replay
                last_flag = last;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (last_flag && ok && !*abort_ptr) {
                __threadfence();
                const float *tile_partials = a.partials + size_t(tile_linear) * a.splits * BN * kBlockChannels;
                const float scale_w = (!Grouped && channel_ok) ? a.sw[n] : 0.f;
                for (int c = 0; c < valid_tokens; ++c) {
                    const int m = m0 + c;
                    const size_t at = size_t(c) * kBlockChannels + channel_in_tile;
                    if (kIntAcc) {
                        int sum = 0;
                        for (int s = 0; s < a.splits; ++s)
                            sum += int(__ldcg(reinterpret_cast<const uint32_t *>(tile_partials) + size_t(s) * BN * kBlockChannels + at));
                        if (channel_ok) {
                            if (a.out_type == int(Type::I32)) static_cast<int *>(a.out)[size_t(m) * a.n + n] = sum;
                            else store_output(a, __fmul_rn(__fmul_rn(float(sum), a.sx[m]), scale_w), m, n);
                        }
                    } else {
                        float sum = 0.f;
                        for (int s = 0; s < a.splits; ++s)
                            sum = __fadd_rn(sum, __ldcg(tile_partials + size_t(s) * BN * kBlockChannels + at));
                        if (channel_ok)
                            store_output(a, Grouped ? sum : __fmul_rn(__fmul_rn(sum, a.sx[m]), scale_w), m, n);
                    }
                }
            }
        }
        ptx::tcgen05_fence_before();
    }

    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemColumns);
    }
    if (threadIdx.x == 0 && abort_flag) atomicExch(a.status, 1 + tile_linear);
}
} // namespace tts::b200
