// Stage 1 (and the stage-3 producer) of the quantized linear path: dynamic per-token quantization
// of a 16-bit [rows,K] matrix to one-byte values plus fp32 scales, optionally after the matched
// H128 rotation and optionally with K-group scales. One pass over HBM: each thread keeps its
// 128-bit loads in registers across the amax reduction, so the row is read once and written once.
//
// Replaces the reference launcher `launch_row_quantize`
// (src/ops/kernels/quant/row_quantize.cu:167-193) and the four kernels behind it
// (:24-37 scalar, :42-87 register-cached, :90-115 rotated per-row, :145-165 K-group).
#include "kernels/row_quantize.h"
#include "kernels/quant_codec.cuh"
#include "kernels/launch.cuh"
#include <stdexcept>

namespace tts {
namespace b200 {
namespace {
constexpr int kThreads = 256;

// Register-resident rows: K <= Items * 2048 * parts.
template <Type F, class T, int Items, bool Rotate>
__global__ void __launch_bounds__(kThreads)
row_quantize_cached(const T *__restrict__ x, unsigned char *__restrict__ q, float *__restrict__ scales,
                    int rows, int cols, int stride, int group, int parts, bool aligned) {
    __shared__ float slots[kThreads / 32];
    pdl_launch_dependents();
    pdl_wait_upstream();
    const int row = blockIdx.x / parts, shard = blockIdx.x % parts;
    const T *source = x + size_t(row) * stride;
    float v[Items][8];
    if (aligned) {
        // All loads of the row shard are issued before the first value is used.
        uint4 raw[Items];
#pragma unroll
        for (int j = 0; j < Items; ++j) {
            int column = ((j * parts + shard) * kThreads + int(threadIdx.x)) * 8;
            raw[j] = column < cols ? *reinterpret_cast<const uint4 *>(source + column) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < Items; ++j) unpack8<T>(raw[j], v[j]);
    } else {
#pragma unroll
        for (int j = 0; j < Items; ++j) {
            int column = ((j * parts + shard) * kThreads + int(threadIdx.x)) * 8;
            if (column < cols) {
                load8(source + column, cols - column, false, v[j]);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[j][i] = 0.f;
            }
        }
    }
    quantize_tail<F, kThreads, Items, Rotate>(v, q, scales, row, rows, cols, group, shard, parts,
                                              aligned, slots);
}

// Arbitrarily wide rows with one scale per row: two passes over the row (the second one mostly
// served by L2), the rotation recomputed rather than spilled.
template <Type F, class T, bool Rotate>
__global__ void __launch_bounds__(kThreads)
row_quantize_wide(const T *__restrict__ x, unsigned char *__restrict__ q, float *__restrict__ scales,
                  int cols, int stride, bool aligned) {
    __shared__ float slots[kThreads / 32];
    pdl_launch_dependents();
    pdl_wait_upstream();
    const int row = blockIdx.x;
    const T *source = x + size_t(row) * stride;
    const int padded = (cols + kThreads * 8 - 1) / (kThreads * 8) * (kThreads * 8);
    float amax = 0.f, v[8];
    for (int column = threadIdx.x * 8; column < padded; column += kThreads * 8) {
        load8(source + (column < cols ? column : 0), column < cols ? cols - column : 0, aligned, v);
        if (Rotate) hadamard128(v, column);
        if (column < cols) amax = fmaxf(amax, abs_max8(v));
    }
    float step = quant_scale<F>(cta_max<kThreads>(amax, slots));
    float inverse = __fdiv_rn(1.f, step);
    if (!threadIdx.x) scales[row] = step;
    for (int column = threadIdx.x * 8; column < padded; column += kThreads * 8) {
        load8(source + (column < cols ? column : 0), column < cols ? cols - column : 0, aligned, v);
        if (Rotate) hadamard128(v, column);
        if (column < cols)
            store8<F>(q + size_t(row) * cols + column, cols - column, aligned, v, inverse);
    }
}

// Long batches with one scale per row: one WARP per row, eight rows per CTA. The row stays in the
// lane's registers (up to 16 128-bit loads, all issued before the first use) and the amax needs only a
// warp reduction, so no CTA-wide barrier sits between the read and the write; with thousands of rows
// this keeps far more bytes in flight per SM than one small CTA per row. Max is exact, so the bytes
// and scales are the same as the CTA-per-row kernel's.
// `Resident` = CTAs per multiprocessor the register budget is cut for. More resident warps beat a spill-free
// kernel once there are rows enough to fill them (M=8192: K=2048 11.2 -> 9.5 us = 0.81 of the measured HBM rate
// with three CTAs; K=4096 14.4 -> 11.5 us with two); short batches keep the unconstrained kernel.
template <Type F, class T, int Loads, int Resident>
__global__ void __launch_bounds__(kThreads, Resident)
row_quantize_warp_rows(const T *__restrict__ x, unsigned char *__restrict__ q, float *__restrict__ scales, int rows,
                       int cols, int stride) {
    pdl_launch_dependents();
    pdl_wait_upstream();
    const int row = blockIdx.x * (kThreads / 32) + int(threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const T *source = x + size_t(row) * stride;
    uint4 raw[Loads];
#pragma unroll
    for (int j = 0; j < Loads; ++j) {
        const int column = (j * 32 + lane) * 8;
        raw[j] = column < cols ? *reinterpret_cast<const uint4 *>(source + column) : make_uint4(0, 0, 0, 0);
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < Loads; ++j) {
        float v[8];
        unpack8<T>(raw[j], v);
        amax = fmaxf(amax, abs_max8(v));
    }
    amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax))); // non-negative floats order like their bits
    const float step = quant_scale<F>(amax), inverse = __fdiv_rn(1.f, step);
    if (!lane) scales[row] = step;
#pragma unroll
    for (int j = 0; j < Loads; ++j) {
        const int column = (j * 32 + lane) * 8;
        if (column < cols) {
            float v[8];
            unpack8<T>(raw[j], v);
            store8<F>(q + size_t(row) * cols + column, 8, true, v, inverse);
        }
    }
}

template <Type F, class T, bool Rotate>
void launch_typed(const T *x, unsigned char *q, float *scales, int rows, int cols, int stride,
                  int group, int multiprocessors, cudaStream_t stream) {
    const bool aligned = cols % 8 == 0 && stride % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(q) % 8 == 0;
    const int chunks = (cols + kThreads * 8 - 1) / (kThreads * 8); // 2048-column slabs per row
    if (!group && !Rotate && aligned && cols <= 4096 && rows >= 8 * multiprocessors) {
        const dim3 grid(unsigned((rows + kThreads / 32 - 1) / (kThreads / 32)));
#define B200Q_WARP_ROWS(L, R)                                                                                          \
    launch_pdl("row quantize launch", row_quantize_warp_rows<F, T, L, R>, grid, dim3(kThreads), 0, stream, x, q, scales,   \
               rows, cols, stride)
        const int loads = (cols + 255) / 256;
        const bool many = rows >= 24 * multiprocessors; // three CTAs of eight rows on every multiprocessor
        if (loads <= 4) B200Q_WARP_ROWS(4, 1);
        else if (loads <= 8) { if (many) B200Q_WARP_ROWS(8, 3); else B200Q_WARP_ROWS(8, 1); }
        else B200Q_WARP_ROWS(16, 2);
#undef B200Q_WARP_ROWS
        return;
    }
    int parts = 1;
    if (group) {
        // K groups never cross a 2048-column slab, so slabs of one row can go to different CTAs.
        // Spread short batches over the machine; long batches keep whole rows per CTA.
        while (parts < chunks && int64_t(rows) * parts * 2 <= multiprocessors) parts *= 2;
        if (chunks > 4 * parts) parts = (chunks + 3) / 4;
    } else if (chunks > 4) {
        launch_pdl("row quantize launch", row_quantize_wide<F, T, Rotate>, dim3(rows), dim3(kThreads), 0, stream, x, q, scales,
                   cols, stride, aligned);
        return;
    }
    const int items = (chunks + parts - 1) / parts;
    const unsigned grid = unsigned(rows) * unsigned(parts);
#define B200Q_LAUNCH(I)                                                                            \
    launch_pdl("row quantize launch", row_quantize_cached<F, T, I, Rotate>, dim3(grid), dim3(kThreads), 0, stream, x, q, \
               scales, rows, cols, stride, group, parts, aligned)
    switch (items) {
    case 1: B200Q_LAUNCH(1); break;
    case 2: B200Q_LAUNCH(2); break;
    case 3: B200Q_LAUNCH(3); break;
    default: B200Q_LAUNCH(4); break;
    }
#undef B200Q_LAUNCH
}

template <Type F, class T>
void launch_rotation(const T *x, unsigned char *q, float *scales, int rows, int cols, int stride,
                     int group, int rotation, int sms, cudaStream_t stream) {
    if (rotation) launch_typed<F, T, true>(x, q, scales, rows, cols, stride, group, sms, stream);
    else launch_typed<F, T, false>(x, q, scales, rows, cols, stride, group, sms, stream);
}
} // namespace
} // namespace b200

void launch_row_quantize(TensorView source, RowScaledView destination, cudaStream_t stream,
                         int multiprocessors) {
    destination.validate();
    if ((source.type != Type::BF16 && source.type != Type::F16) || !source.data ||
        !destination.values.data || !destination.scales.data || source.rows < 1 || source.cols < 1 ||
        source.rows != destination.values.rows || source.cols != destination.values.cols)
        throw std::invalid_argument("row quantization shape/type mismatch");
    if (int64_t(source.rows) * ((source.cols + 2047) / 2048) > INT32_MAX)
        throw std::invalid_argument("quantization grid exceeds capacity");
    if (multiprocessors <= 0) multiprocessors = 148;
    auto *q = destination.values.ptr<unsigned char>();
    auto *s = destination.scales.ptr<float>();
    const int rows = source.rows, cols = source.cols, ld = source.ld();
    const int group = destination.group_size, rotation = destination.rotation_size;
    const bool fp8 = destination.values.type == Type::FP8;
    if (source.type == Type::F16) {
        auto *x = source.ptr<const __half>();
        if (fp8) b200::launch_rotation<Type::FP8>(x, q, s, rows, cols, ld, group, rotation, multiprocessors, stream);
        else b200::launch_rotation<Type::I8>(x, q, s, rows, cols, ld, group, rotation, multiprocessors, stream);
    } else {
        auto *x = source.ptr<const __nv_bfloat16>();
        if (fp8) b200::launch_rotation<Type::FP8>(x, q, s, rows, cols, ld, group, rotation, multiprocessors, stream);
        else b200::launch_rotation<Type::I8>(x, q, s, rows, cols, ld, group, rotation, multiprocessors, stream);
    }
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess)
        throw std::runtime_error(std::string("row quantize launch: ") + cudaGetErrorString(status));
}
} // namespace tts
