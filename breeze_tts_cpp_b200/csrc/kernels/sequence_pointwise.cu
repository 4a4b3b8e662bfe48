// The projection epilogue as passes of their own, for the cases the GEMM's fused epilogue does not
// take (per-sequence gate / condition, pre-activation copy, sequence-tail masking, indexed or
// repeated rows, Mish):
//   launch_pointwise           y = finish(x), in place or not
//   launch_pointwise_quantize  finish(x) rounded to storage, optionally retained, then quantized per
//                              row / per K group (optionally rotated) in the same pass
// Replaces the reference kernels `pointwise_row_kernel` / `pointwise_kernel` and
// `pointwise_quantize_kernel` (src/ops/kernels/sequence/sequence_pointwise.cu:8-45,148-265) and their
// launchers (:283-357). Each thread owns eight consecutive columns (one 128-bit load per operand);
// the quantizing pass keeps a whole row in the registers of one CTA across the amax reduction, so a
// row is read once and written once. Compile with --fmad=false: the rounding points are explicit.
#include "kernels/sequence_pointwise.h"
#include "kernels/launch.cuh"
#include "kernels/quant_codec.cuh"
#include "kernels/sequence_finish.cuh"
#include <stdexcept>
#include <string>

namespace tts {
namespace b200 {
namespace {
constexpr int kThreads = 256;

// Eight consecutive elements of an epilogue operand as fp32 (zeros when the operand is absent).
template <class T>
__device__ __forceinline__ void operand8(const FinishOperand &o, int row, int col, int remaining, float (&v)[8]) {
    if (!o.data) {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = 0.f;
        return;
    }
    const T *p = static_cast<const T *>(o.data) + size_t(o.rows == 1 ? 0 : row) * o.stride + col;
    load8(p, remaining, (reinterpret_cast<uintptr_t>(p) & 15) == 0, v);
}

// finish() of eight consecutive columns of one row; `raw` receives the pre-activation values.
template <class T>
__device__ __forceinline__ void finish8(const FinishArgs &f, const FinishRow &r, int row, int col, int remaining,
                                        const float (&x)[8], float (&out)[8]) {
    T *raw = f.raw ? static_cast<T *>(f.raw) + size_t(row) * f.raw_stride + col : nullptr;
    if (r.masked) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            out[i] = 0.f;
            if (raw && i < remaining) raw[i] = T(0.f);
        }
        return;
    }
    float bias[8], gate[8], skip[8], condition[8];
    operand8<T>(f.bias, 0, col, remaining, bias);
    operand8<T>(f.gate, r.sequence, col, remaining, gate);
    operand8<T>(f.condition, r.sequence, col, remaining, condition);
    if (f.residual.data && r.residual >= 0 && r.residual < f.residual.rows) {
        operand8<T>(f.residual, r.residual, col, remaining, skip);
    } else {
        const float fill = f.residual.data && r.residual >= 0 ? nanf("") : 0.f; // a row index past the end poisons the row
#pragma unroll
        for (int i = 0; i < 8; ++i) skip[i] = fill;
    }
    float before[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float value = round_storage<T>(__fadd_rn(x[i], bias[i]));
        if (f.gate.data) value = round_storage<T>(__fmul_rn(value, gate[i]));
        value = round_storage<T>(__fmaf_rn(f.value_scale, value, __fmul_rn(f.residual_scale, skip[i])));
        if (f.condition.data) value = round_storage<T>(__fadd_rn(value, condition[i]));
        before[i] = value;
        out[i] = finish_activation(round_storage<T>(__fmul_rn(value, f.output_scale)), f.activation, f.alpha);
    }
    if (raw) {
        if ((reinterpret_cast<uintptr_t>(raw) & 15) == 0 && remaining >= 8) {
            uint4 packed;
            T *e = reinterpret_cast<T *>(&packed);
#pragma unroll
            for (int i = 0; i < 8; ++i) e[i] = T(before[i]);
            *reinterpret_cast<uint4 *>(raw) = packed;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i < remaining) raw[i] = T(before[i]);
        }
    }
}

template <class T> __device__ __forceinline__ void store16(T *p, int remaining, const float (&v)[8]) {
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0 && remaining >= 8) {
        uint4 packed;
        T *e = reinterpret_cast<T *>(&packed);
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = T(v[i]);
        *reinterpret_cast<uint4 *>(p) = packed;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < remaining) p[i] = T(v[i]);
    }
}

template <class T> __device__ __forceinline__ void input8(const T *x, int x_rows, int x_stride, int input_row, int col,
                                                           int remaining, float (&v)[8]) {
    const T *p = x + size_t(x_rows == 1 ? 0 : input_row) * x_stride + col;
    load8(p, remaining, (reinterpret_cast<uintptr_t>(p) & 15) == 0, v);
}

template <class T>
__global__ void __launch_bounds__(kThreads)
pointwise_finish(const T *__restrict__ x, int x_rows, int x_stride, T *y, int y_stride, int rows, int cols, int repeat,
                 FinishArgs f) {
    pdl_launch_dependents();
    pdl_wait_upstream();
    const int packets = (cols + 7) / 8;
    const int64_t index = int64_t(blockIdx.x) * kThreads + threadIdx.x;
    if (index >= int64_t(rows) * packets) return;
    const int row = int(index / packets), col = int(index % packets) * 8, remaining = cols - col;
    float in[8], out[8];
    input8(x, x_rows, x_stride, row / repeat, col, remaining, in);
    const FinishRow r = finish_row(f, row);
    finish8<T>(f, r, row, col, remaining, in, out);
    store16(y + size_t(row) * y_stride + col, remaining, out);
}

// One CTA holds a row (K-group mode: one 2048-column-slab shard of it): finish, round, retain, quantize.
template <Type F, class T, int Items, bool Rotate>
__global__ void __launch_bounds__(kThreads)
pointwise_finish_quantize(const T *__restrict__ x, int x_rows, int x_stride, T *retained, int retained_stride,
                          unsigned char *__restrict__ q, float *__restrict__ scales, int rows, int cols, int repeat,
                          int group, int parts, FinishArgs f) {
    __shared__ float slots[kThreads / 32];
    pdl_launch_dependents();
    pdl_wait_upstream();
    const int row = blockIdx.x / parts, shard = blockIdx.x % parts;
    const FinishRow r = finish_row(f, row);
    float v[Items][8];
#pragma unroll
    for (int j = 0; j < Items; ++j) {
        const int col = ((j * parts + shard) * kThreads + int(threadIdx.x)) * 8;
        if (col < cols) {
            float in[8];
            input8(x, x_rows, x_stride, row / repeat, col, cols - col, in);
            finish8<T>(f, r, row, col, cols - col, in, v[j]);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[j][i] = i < cols - col ? round_storage<T>(v[j][i]) : 0.f;
            if (retained) store16(retained + size_t(row) * retained_stride + col, cols - col, v[j]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[j][i] = 0.f;
        }
    }
    const bool aligned = cols % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0;
    quantize_tail<F, kThreads, Items, Rotate>(v, q, scales, row, rows, cols, group, shard, parts, aligned, slots);
}

// Rows wider than one CTA's registers, one scale per row: the chain is evaluated twice (first for the
// amax, then for the bytes; the second pass also writes `retained` and `raw`).
template <Type F, class T>
__global__ void __launch_bounds__(kThreads)
pointwise_finish_quantize_wide(const T *__restrict__ x, int x_rows, int x_stride, T *retained, int retained_stride,
                               unsigned char *__restrict__ q, float *__restrict__ scales, int cols, int repeat, FinishArgs f) {
    __shared__ float slots[kThreads / 32];
    pdl_launch_dependents();
    pdl_wait_upstream();
    const int row = blockIdx.x;
    const FinishRow r = finish_row(f, row);
    FinishArgs quiet = f;
    quiet.raw = nullptr;
    float amax = 0.f;
    for (int col = threadIdx.x * 8; col < cols; col += kThreads * 8) {
        float in[8], out[8];
        input8(x, x_rows, x_stride, row / repeat, col, cols - col, in);
        finish8<T>(quiet, r, row, col, cols - col, in, out);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i < cols - col) amax = fmaxf(amax, fabsf(round_storage<T>(out[i])));
    }
    const float step = quant_scale<F>(cta_max<kThreads>(amax, slots));
    const float inverse = __fdiv_rn(1.f, step);
    if (!threadIdx.x) scales[row] = step;
    const bool aligned = cols % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0;
    for (int col = threadIdx.x * 8; col < cols; col += kThreads * 8) {
        float in[8], out[8];
        input8(x, x_rows, x_stride, row / repeat, col, cols - col, in);
        finish8<T>(f, r, row, col, cols - col, in, out);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = round_storage<T>(out[i]);
        if (retained) store16(retained + size_t(row) * retained_stride + col, cols - col, out);
        store8<F>(q + size_t(row) * cols + col, cols - col, aligned, out, inverse);
    }
}

template <Type F, class T, bool Rotate>
void launch_quantize(TensorView x, TensorView retained, RowScaledView out, const ops::Epilogue &e, int sms,
                     cudaStream_t stream) {
    const int rows = out.values.rows, cols = out.values.cols, group = out.group_size;
    const int chunks = (cols + kThreads * 8 - 1) / (kThreads * 8);
    auto *q = out.values.ptr<unsigned char>();
    auto *s = out.scales.ptr<float>();
    const FinishArgs f(e);
    int parts = 1;
    if (group) {
        // K groups never cross a 2048-column slab, so the slabs of a row may go to different CTAs.
        while (parts < chunks && int64_t(rows) * parts * 2 <= sms) parts *= 2;
        if (chunks > 4 * parts) parts = (chunks + 3) / 4;
    } else if (chunks > 4) {
        if constexpr (!Rotate)
            launch_pdl("finish+quantize launch", pointwise_finish_quantize_wide<F, T>, dim3(rows), dim3(kThreads), 0, stream,
                       x.ptr<const T>(), x.rows, x.ld(), retained.ptr<T>(), retained.ld(), q, s, cols, e.input_repeat, f);
        return;
    }
    const int items = (chunks + parts - 1) / parts;
    const unsigned grid = unsigned(rows) * unsigned(parts);
#define B200Q_RUN(I)                                                                                                  \
    launch_pdl("finish+quantize launch", pointwise_finish_quantize<F, T, I, Rotate>, dim3(grid), dim3(kThreads), 0, stream, \
               x.ptr<const T>(), x.rows, x.ld(), retained.ptr<T>(), retained.ld(), q, s, rows, cols, e.input_repeat, group,   \
               parts, f)
    switch (items) {
    case 1: B200Q_RUN(1); break;
    case 2: B200Q_RUN(2); break;
    case 3: B200Q_RUN(3); break;
    default: B200Q_RUN(4); break;
    }
#undef B200Q_RUN
}
} // namespace
} // namespace b200

void launch_pointwise(TensorView x, TensorView y, const ops::Epilogue &e, cudaStream_t stream) {
    if (y.type != Type::BF16 && y.type != Type::F16)
        throw std::invalid_argument("the finishing pass runs on F16 or BF16 rows");
    const int64_t packets = int64_t(y.rows) * ((y.cols + 7) / 8);
    if (packets > int64_t(INT32_MAX) * b200::kThreads) throw std::invalid_argument("finishing pass grid exceeds capacity");
    const dim3 grid(unsigned((packets + b200::kThreads - 1) / b200::kThreads));
    const b200::FinishArgs f(e);
    if (y.type == Type::F16)
        b200::launch_pdl("finishing pass launch", b200::pointwise_finish<__half>, grid, dim3(b200::kThreads), 0, stream,
                         x.ptr<const __half>(), x.rows, x.ld(), y.ptr<__half>(), y.ld(), y.rows, y.cols, e.input_repeat, f);
    else
        b200::launch_pdl("finishing pass launch", b200::pointwise_finish<__nv_bfloat16>, grid, dim3(b200::kThreads), 0, stream,
                         x.ptr<const __nv_bfloat16>(), x.rows, x.ld(), y.ptr<__nv_bfloat16>(), y.ld(), y.rows, y.cols,
                         e.input_repeat, f);
}

void launch_pointwise_quantize(TensorView x, RowScaledView q, const ops::Epilogue &e, TensorView retained,
                               int multiprocessors, cudaStream_t stream) {
    if (multiprocessors <= 0) multiprocessors = 148;
    if (int64_t(q.values.rows) * ((q.values.cols + 2047) / 2048) > INT32_MAX)
        throw std::invalid_argument("quantization grid exceeds capacity");
    const bool fp8 = q.values.type == Type::FP8, rotate = q.rotation_size != 0;
    auto run = [&](auto tag) {
        using T = decltype(tag);
        if (fp8) {
            if (rotate) b200::launch_quantize<Type::FP8, T, true>(x, retained, q, e, multiprocessors, stream);
            else b200::launch_quantize<Type::FP8, T, false>(x, retained, q, e, multiprocessors, stream);
        } else {
            if (rotate) b200::launch_quantize<Type::I8, T, true>(x, retained, q, e, multiprocessors, stream);
            else b200::launch_quantize<Type::I8, T, false>(x, retained, q, e, multiprocessors, stream);
        }
    };
    if (x.type == Type::F16) run(__half{});
    else run(__nv_bfloat16{});
}
} // namespace tts
