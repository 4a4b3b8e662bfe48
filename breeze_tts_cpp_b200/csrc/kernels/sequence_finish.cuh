// The projection epilogue as device code: bias, per-sequence gate, (indexed) residual, per-sequence
// condition, optional pre-activation copy, sequence-tail masking and activation, each step rounded
// to the storage type exactly where the reference rounds
// (src/ops/kernels/sequence/sequence_internal.cuh:31-74, activations
// src/ops/kernels/common/activation.cuh:5-27). Shared by the separate finishing pass and by the
// finish-and-quantize pass. Every product, sum and fused multiply-add is written out explicitly.
#pragma once
#include "ops/epilogue.h"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace tts::b200 {

// A borrowed [rows, cols] operand of the epilogue; rows == 1 broadcasts row 0.
struct FinishOperand {
    const void *data = nullptr;
    int stride = 0, rows = 0;
    FinishOperand() = default;
    explicit FinishOperand(const TensorView &v) : data(v.data), stride(v.ld()), rows(v.rows) {}
    template <class T> __device__ __forceinline__ float get(int row, int col) const {
        return data ? float(static_cast<const T *>(data)[size_t(rows == 1 ? 0 : row) * stride + col]) : 0.f;
    }
};

struct FinishArgs {
    FinishOperand bias, residual, gate, condition;
    void *raw = nullptr;
    int raw_stride = 0;
    int rows_per_sequence = 1, valid_rows_per_sequence = 0;
    float value_scale = 1.f, output_scale = 1.f, residual_scale = 1.f, alpha = .1f;
    int activation = 0;
    const int *residual_rows = nullptr;
    FinishArgs() = default;
    explicit FinishArgs(const ops::Epilogue &e)
        : bias(e.bias), residual(e.residual), gate(e.gate), condition(e.condition), raw(e.raw.data),
          raw_stride(e.raw.ld()), rows_per_sequence(e.rows_per_sequence),
          valid_rows_per_sequence(e.valid_rows_per_sequence), value_scale(e.value_scale), output_scale(e.output_scale),
          residual_scale(e.residual_scale), alpha(e.alpha), activation(int(e.activation)), residual_rows(e.residual_rows) {}
};

template <class T> __device__ __forceinline__ float round_storage(float v);
template <> __device__ __forceinline__ float round_storage<__nv_bfloat16>(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}
template <> __device__ __forceinline__ float round_storage<__half>(float v) { return __half2float(__float2half_rn(v)); }

__device__ __forceinline__ float finish_activation(float x, int kind, float alpha) {
    switch (kind) {
    case 1: return fmaxf(x, 0.f);
    case 2: return x >= 0 ? x : __fmul_rn(x, alpha);
    case 3: return __fdiv_rn(x, __fadd_rn(1.f, expf(-x)));
    case 4: return __fmul_rn(__fmul_rn(.5f, x), __fadd_rn(1.f, erff(__fmul_rn(x, .7071067811865475f))));
    case 5: {
        // The reference's finishing pass is compiled with multiply-add contraction: the cubic term and x meet
        // in one fused operation. The hardware's approximate tanh as there (activation.cuh:16-17).
        const float inner = __fmaf_rn(__fmul_rn(__fmul_rn(.044715f, x), x), x, x);
        float t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(__fmul_rn(.7978845608028654f, inner)));
        return __fmul_rn(__fmul_rn(.5f, x), __fadd_rn(1.f, t));
    }
    case 6: return __fmul_rn(x, tanhf(x > 20.f ? x : log1pf(expf(x))));
    case 7: return tanhf(x);
    case 8: return __fdiv_rn(1.f, __fadd_rn(1.f, expf(-x)));
    default: return x;
    }
}

// What one output row needs besides its column: its sequence and the row its residual comes from.
struct FinishRow {
    int sequence, residual;
    bool masked;
};
__device__ __forceinline__ FinishRow finish_row(const FinishArgs &f, int row) {
    FinishRow r;
    r.sequence = row / f.rows_per_sequence;
    r.residual = f.residual_rows ? f.residual_rows[row] : row;
    r.masked = f.valid_rows_per_sequence && row % f.rows_per_sequence >= f.valid_rows_per_sequence;
    return r;
}

// The finished value of element (row, col) before the final rounding of the caller; `raw` receives the
// pre-activation value. reference: Finish::apply, sequence_internal.cuh:52-74.
template <class T>
__device__ __forceinline__ float finish_apply(const FinishArgs &f, const FinishRow &r, float value, int row, int col) {
    T *raw = f.raw ? static_cast<T *>(f.raw) + size_t(row) * f.raw_stride + col : nullptr;
    if (r.masked) {
        if (raw) *raw = T(0.f);
        return 0.f;
    }
    value = round_storage<T>(__fadd_rn(value, f.bias.template get<T>(0, col)));
    if (f.gate.data) value = round_storage<T>(__fmul_rn(value, f.gate.template get<T>(r.sequence, col)));
    float skip = 0.f;
    if (f.residual.data && r.residual >= 0)
        skip = r.residual < f.residual.rows ? f.residual.template get<T>(r.residual, col) : nanf("");
    // The reference's finishing pass is built with multiply-add contraction: `value_scale * value + scale * skip`
    // is one product rounded, then a fused multiply-add (found by comparing with its kernels on scales that
    // are not powers of two).
    value = round_storage<T>(__fmaf_rn(f.value_scale, value, __fmul_rn(f.residual_scale, skip)));
    if (f.condition.data) value = round_storage<T>(__fadd_rn(value, f.condition.template get<T>(r.sequence, col)));
    if (raw) *raw = T(value);
    return finish_activation(round_storage<T>(__fmul_rn(value, f.output_scale)), f.activation, f.alpha);
}
} // namespace tts::b200
