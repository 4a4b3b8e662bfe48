// Device-side arithmetic shared by every quantize producer: scale rule, byte encoders, the
// matched sign-flip + 128-point Hadamard rotation, and the tail that turns eight-wide fp32 register
// tiles into one-byte values plus fp32 scales in the RowScaledView layouts.
//
// The numbers follow the reference's rules exactly so INT8 bytes and scales are bit-identical:
//   scale   = amax == 0 ? 1 : max(amax / range, FLT_MIN), true IEEE division
//             (reference: src/ops/kernels/quant/quant_format.cuh:62-64)
//   inverse = 1 / scale (IEEE), q = encode(x * inverse)
//   INT8    : clamp to ±127, round half to even (quant_format.cuh:37-47)
//   FP8     : e4m3, round to nearest even, saturate to ±448 (quant_format.cuh:12-17)
//   rotation: sign from an integer hash of the absolute column, butterflies with strides
//             1,2,4,...,64 in that order, each (a,b)->(a+b,a-b), then ×2^-3.5
//             (src/ops/kernels/quant/quant_device.cuh:96-125)
// Every product is an explicit round-to-nearest multiply so no FMA contraction can change a bit.
#pragma once
#include "core/tensor.h"
#include <cfloat>
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace tts::b200 {

template <Type F> struct Codec;
template <> struct Codec<Type::I8> {
    static constexpr float range = 127.f;
    __device__ static __forceinline__ uint32_t one(float x) {
        x = fminf(127.f, fmaxf(-127.f, x));
        return uint32_t(__float2int_rn(x)) & 0xffu;
    }
    // Four consecutive values -> four packed bytes (little endian: first value in the low byte).
    __device__ static __forceinline__ uint32_t four(float a, float b, float c, float d) {
        return one(a) | (one(b) << 8) | (one(c) << 16) | (one(d) << 24);
    }
};
template <> struct Codec<Type::FP8> {
    static constexpr float range = 448.f;
    __device__ static __forceinline__ uint32_t one(float x) {
        return uint32_t(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
    }
    __device__ static __forceinline__ uint32_t four(float a, float b, float c, float d) {
        uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
        uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
        return lo | (hi << 16);
    }
};

template <Type F> __device__ __forceinline__ float quant_scale(float amax) {
    return amax == 0.f ? 1.f : fmaxf(__fdiv_rn(amax, Codec<F>::range), FLT_MIN);
}

__device__ __forceinline__ float rotation_sign(uint32_t column) {
    uint32_t h = column * 0x45d9f3bu;
    h = (h ^ (h >> 16)) * 0x45d9f3bu;
    return ((h ^ (h >> 16)) & 1u) ? 1.f : -1.f;
}

// Eight consecutive 16-bit elements -> fp32. `aligned` selects one 128-bit load; otherwise (odd
// pointers, ragged row ends) elements are fetched one by one and missing ones read as zero.
template <class T> __device__ __forceinline__ void load8(const T *p, int remaining, bool aligned, float (&v)[8]) {
    if (aligned && remaining >= 8) {
        uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = float(e[i]);
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = i < remaining ? float(p[i]) : 0.f;
    }
}

// Register form of eight 16-bit elements and its conversion; lets a kernel issue all of its
// 128-bit loads back to back before the first conversion waits on one of them.
template <class T> __device__ __forceinline__ void unpack8(uint4 raw, float (&v)[8]) {
    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = float(e[i]);
}

template <Type F> __device__ __forceinline__ void store8(unsigned char *q, int remaining, bool aligned,
                                                        const float (&v)[8], float inverse) {
    uint32_t lo = Codec<F>::four(__fmul_rn(v[0], inverse), __fmul_rn(v[1], inverse),
                                 __fmul_rn(v[2], inverse), __fmul_rn(v[3], inverse));
    uint32_t hi = Codec<F>::four(__fmul_rn(v[4], inverse), __fmul_rn(v[5], inverse),
                                 __fmul_rn(v[6], inverse), __fmul_rn(v[7], inverse));
    if (aligned && remaining >= 8) {
        *reinterpret_cast<uint2 *>(q) = make_uint2(lo, hi);
    } else {
        uint64_t both = uint64_t(lo) | (uint64_t(hi) << 32);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < remaining) q[i] = (unsigned char)(both >> (8 * i));
    }
}

// In place: the 8 values of this lane are columns [column, column+8) of a 128-wide block that the
// 16 lanes sharing (lane & ~15) hold together. All 32 lanes of the warp must call this.
__device__ __forceinline__ void hadamard128(float (&v)[8], int column) {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], rotation_sign(uint32_t(column + i)));
#pragma unroll
    for (int span = 1; span < 8; span <<= 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (!(i & span)) {
                float a = v[i], b = v[i | span];
                v[i] = __fadd_rn(a, b);
                v[i | span] = __fsub_rn(a, b);
            }
        }
    }
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int span = 1; span < 16; span <<= 1) {
        const bool upper = lane & span;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float other = __shfl_xor_sync(0xffffffffu, v[i], span);
            v[i] = upper ? __fsub_rn(other, v[i]) : __fadd_rn(v[i], other);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fmul_rn(v[i], 0.08838834764831845f);
}

__device__ __forceinline__ float abs_max8(const float (&v)[8]) {
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
    return m;
}

// Max over the whole CTA of a value that is never negative and never NaN (an absolute maximum built with
// fmaxf). `slots` must hold one float per warp. Exact, so the order is irrelevant; such floats order like their
// bit patterns, which lets one warp-reduce instruction replace five shuffle rounds.
template <int Threads> __device__ __forceinline__ float cta_max(float v, float *slots) {
    v = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(v)));
    if (!(threadIdx.x & 31)) slots[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = 0.f;
#pragma unroll
    for (int w = 0; w < Threads / 32; ++w) r = fmaxf(r, slots[w]);
    __syncthreads();
    return r;
}

// Max over the `lanes` consecutive lanes (4, 8 or 16) that share one K group of 8*lanes columns.
__device__ __forceinline__ float group_max(float v, int lanes) {
    for (int d = 1; d < lanes; d <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}

// Tail shared by the standalone quantizer and the fused producers.
// The CTA holds one row (or one shard of it): thread t, item j owns columns
// ((j*parts + shard)*Threads + t)*8 .. +7, already converted (and produced) in fp32.
//   group == 0 : one scale per row at scales[row]; needs parts == 1.
//   group  > 0 : one scale per K group at scales[(column/group)*rows + row].
template <Type F, int Threads, int Items, bool Rotate>
__device__ __forceinline__ void quantize_tail(float (&v)[Items][8], unsigned char *out, float *scales,
                                              int row, int rows, int cols, int group, int shard,
                                              int parts, bool aligned, float *slots) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < Items; ++j) {
        int column = ((j * parts + shard) * Threads + int(threadIdx.x)) * 8;
        if (Rotate) hadamard128(v[j], column);
        if (!group && column < cols) amax = fmaxf(amax, abs_max8(v[j]));
    }
    if (!group) {
        float step = quant_scale<F>(cta_max<Threads>(amax, slots));
        float inverse = __fdiv_rn(1.f, step);
        if (!threadIdx.x && !shard) scales[row] = step;
#pragma unroll
        for (int j = 0; j < Items; ++j) {
            int column = ((j * parts + shard) * Threads + int(threadIdx.x)) * 8;
            if (column < cols)
                store8<F>(out + size_t(row) * cols + column, cols - column, aligned, v[j], inverse);
        }
        return;
    }
    const int lanes = group >> 3;
#pragma unroll
    for (int j = 0; j < Items; ++j) {
        int column = ((j * parts + shard) * Threads + int(threadIdx.x)) * 8;
        float gmax = group_max(column < cols ? abs_max8(v[j]) : 0.f, lanes);
        if (column < cols) {
            float step = quant_scale<F>(gmax);
            if (!(column & (group - 1))) scales[size_t(column / group) * rows + row] = step;
            store8<F>(out + size_t(row) * cols + column, cols - column, aligned, v[j],
                      __fdiv_rn(1.f, step));
        }
    }
}
} // namespace tts::b200
