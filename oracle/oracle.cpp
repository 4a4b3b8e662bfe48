// TEST INFRASTRUCTURE ONLY — scalar CPU restatement of the reference's quantized-linear math.
// See oracle.h for who may load this and for the "parity unpinned" statement.
//
// Each function names the reference lines it follows (paths inside the reference project).
// Build with -ffp-contract=off: the reference compiles its producers and its GEMV with
// --fmad=false (CMakeLists.txt:94-105), so a*b+c is two roundings there and must be two here.
#include "oracle.h"
#include <algorithm>
#include <cfloat>
#include <chrono>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>
#include <cuda_fp8.h>

namespace {
enum { BF16 = 0, F32 = 1, I32 = 2, FP8 = 3, I8 = 4, F16 = 5 };

inline uint32_t bits_of(float x) { uint32_t u; std::memcpy(&u, &x, 4); return u; }
inline float float_of(uint32_t u) { float x; std::memcpy(&x, &u, 4); return x; }

uint16_t f32_to_f16(float x) {
    uint32_t u = bits_of(x), sign = (u >> 16) & 0x8000u, mag = u & 0x7fffffffu;
    if (mag > 0x7f800000u) return uint16_t(sign | 0x7e00u);
    if (mag >= 0x477ff000u) return uint16_t(sign | 0x7c00u); // >= 65520 rounds to infinity
    if (mag < 0x33000001u) return uint16_t(sign); // below half of the smallest subnormal (ties to even -> 0)
    int exponent = int(mag >> 23) - 127;
    uint32_t mantissa = (mag & 0x7fffffu) | 0x800000u;
    int shift = exponent < -14 ? 13 + (-14 - exponent) : 13;
    uint32_t kept = mantissa >> shift, rest = mantissa & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rest > half || (rest == half && (kept & 1))) ++kept;
    uint32_t result = exponent < -14 ? kept : ((uint32_t(exponent + 15) << 10) + (kept - 0x400u));
    return uint16_t(sign | result);
}
inline float load16(uint16_t v, int type) {
    return type == F16 ? oracle_f16_to_f32(v) : oracle_bf16_to_f32(v);
}
inline uint16_t store16(float v, int type) {
    return type == F16 ? f32_to_f16(v) : oracle_f32_to_bf16(v);
}
inline float round16(float v, int type) { return load16(store16(v, type), type); }
inline uint8_t encode(float x, int format) {
    return format == I8 ? oracle_int8_encode(x) : oracle_fp8_e4m3_encode(x);
}
inline float decode(uint8_t q, int format) {
    return format == I8 ? float(int8_t(q)) : oracle_fp8_e4m3_decode(q);
}

// The tail every producer shares: given one row already in fp32 (rotated or not), write bytes and
// scales. reference: quant_device.cuh:63-88 (K groups), :158-195 (rotated, per-row),
// row_quantize.cu:24-37 (per-row).
void encode_row(const float *row_values, int row, int rows, int cols, uint8_t *values, float *scales,
                int format, int group) {
    if (!group) {
        float amax = 0.f;
        for (int c = 0; c < cols; ++c) amax = std::fmax(amax, std::fabs(row_values[c]));
        float step = oracle_scale(amax, format), inverse = 1.f / step;
        scales[row] = step;
        for (int c = 0; c < cols; ++c) values[size_t(row) * cols + c] = encode(row_values[c] * inverse, format);
        return;
    }
    for (int first = 0; first < cols; first += group) {
        int last = std::min(cols, first + group);
        float amax = 0.f;
        for (int c = first; c < last; ++c) amax = std::fmax(amax, std::fabs(row_values[c]));
        float step = oracle_scale(amax, format), inverse = 1.f / step;
        scales[size_t(first / group) * rows + row] = step;
        for (int c = first; c < last; ++c) values[size_t(row) * cols + c] = encode(row_values[c] * inverse, format);
    }
}
void rotate_row(float *values, int cols) {
    for (int c = 0; c + 128 <= cols; c += 128) oracle_rotate128(values + c, c);
}

// reference: src/ops/kernels/common/activation.cuh:5-27 (the CPU uses libm where the GPU uses
// fast intrinsics; that difference is why activations are compared with a tolerance).
float activate(float x, int kind, float alpha) {
    switch (kind) {
    case 1: return std::fmax(x, 0.f);
    case 2: return x >= 0 ? x : x * alpha;
    case 3: return x / (1.f + std::exp(-x));
    case 4: return .5f * x * (1.f + std::erf(x * .7071067811865475f));
    case 5: return .5f * x * (1.f + std::tanh(.7978845608028654f * (x + .044715f * x * x * x)));
    case 6: return x * std::tanh(x > 20.f ? x : std::log1p(std::exp(x)));
    case 7: return std::tanh(x);
    case 8: return 1.f / (1.f + std::exp(-x));
    default: return x;
    }
}

template <class Body> void parallel_for(int count, int threads, Body body) {
    threads = std::max(1, std::min(threads, count));
    if (threads == 1) { body(0, count); return; }
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) {
        int first = int(int64_t(count) * t / threads), last = int(int64_t(count) * (t + 1) / threads);
        pool.emplace_back([=] { body(first, last); });
    }
    for (auto &t : pool) t.join();
}
} // namespace

extern "C" {
uint16_t oracle_f32_to_bf16(float x) {
    uint32_t u = bits_of(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return uint16_t(u >> 16);
}
float oracle_bf16_to_f32(uint16_t x) { return float_of(uint32_t(x) << 16); }
float oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = uint32_t(h & 0x8000u) << 16, exponent = (h >> 10) & 0x1f, mantissa = h & 0x3ffu;
    if (exponent == 0x1f) return float_of(sign | 0x7f800000u | (mantissa << 13));
    if (!exponent) {
        float magnitude = std::ldexp(float(mantissa), -24);
        return sign ? -magnitude : magnitude;
    }
    return float_of(sign | ((exponent + 112) << 23) | (mantissa << 13));
}

// e4m3: 1 sign, 4 exponent (bias 7), 3 mantissa bits; no infinity, 0x7f is NaN, largest finite 448.
// Round to nearest even, then saturate (reference: quant_format.cuh:12-17 via cuda_fp8.h).
uint8_t oracle_fp8_e4m3_encode(float x) {
    uint8_t sign = (bits_of(x) >> 31) ? 0x80 : 0;
    float a = std::fabs(x);
    if (std::isnan(a)) return uint8_t(sign | 0x7f);
    if (a > 448.f) return uint8_t(sign | 0x7e);
    if (a < 0.015625f) // below the smallest normal 2^-6: multiples of 2^-9
        return uint8_t(sign | uint8_t(std::nearbyint(a * 512.f)));
    int exponent;
    float fraction = std::frexp(a, &exponent); // a = fraction * 2^exponent, fraction in [0.5,1)
    int m = int(std::nearbyint((fraction * 2.f - 1.f) * 8.f)), e = exponent - 1;
    if (m == 8) { m = 0; ++e; }
    int code = ((e + 7) << 3) | m;
    return uint8_t(sign | std::min(code, 0x7e));
}
float oracle_fp8_e4m3_decode(uint8_t q) {
    int e = (q >> 3) & 0xf, m = q & 7;
    float a;
    if (e == 0xf && m == 7) a = NAN;
    else if (!e) a = std::ldexp(float(m), -9);
    else a = std::ldexp(1.f + m / 8.f, e - 7);
    return (q & 0x80) ? -a : a;
}
uint8_t oracle_fp8_e4m3_encode_toolkit(float x) {
    return uint8_t(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}
// reference: quant_format.cuh:37-47 — clamp first, then nearbyint (ties to even).
uint8_t oracle_int8_encode(float x) {
    x = std::fmin(127.f, std::fmax(-127.f, x));
    return uint8_t(int8_t(int(std::nearbyint(x))));
}
// reference: quant_format.cuh:62-64.
float oracle_scale(float amax, int format) {
    float range = format == I8 ? 127.f : 448.f;
    return amax == 0.f ? 1.f : std::fmax(amax / range, FLT_MIN);
}
// reference: quant_device.cuh:100-104.
float oracle_rotation_sign(uint32_t column) {
    uint32_t h = column * 0x45d9f3bu;
    h = (h ^ (h >> 16)) * 0x45d9f3bu;
    return ((h ^ (h >> 16)) & 1u) ? 1.f : -1.f;
}
// reference: quant_device.cuh:96-125. Strides 1,2,...,64 in that order; (a,b) -> (a+b, a-b) with
// `a` the element whose index bit is clear; then the 2^-3.5 factor.
void oracle_rotate128(float *v, int column) {
    for (int i = 0; i < 128; ++i) v[i] = v[i] * oracle_rotation_sign(uint32_t(column + i));
    for (int span = 1; span < 128; span *= 2)
        for (int i = 0; i < 128; ++i)
            if (!(i & span)) {
                float a = v[i], b = v[i | span];
                v[i] = a + b;
                v[i | span] = a - b;
            }
    for (int i = 0; i < 128; ++i) v[i] *= 0.08838834764831845f;
}

// reference: row_quantize.cu:167-193 and the kernels it launches.
void oracle_row_quantize(const uint16_t *source, int source_type, int rows, int cols, int stride,
                         uint8_t *values, float *scales, int format, int group, int rotation) {
    if (!stride) stride = cols;
    std::vector<float> row(cols);
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < cols; ++c) row[c] = load16(source[size_t(r) * stride + c], source_type);
        if (rotation) rotate_row(row.data(), cols);
        encode_row(row.data(), r, rows, cols, values, scales, format, group);
    }
}

void oracle_int8_accumulate(const int8_t *xq, const int8_t *wq, int m, int n, int k, int32_t *acc) {
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j) {
            int32_t sum = 0;
            for (int c = 0; c < k; ++c) sum += int32_t(xq[size_t(i) * k + c]) * int32_t(wq[size_t(j) * k + c]);
            acc[size_t(i) * n + j] = sum;
        }
}

// Per-row scales : D((float(acc)*sx[m])*sw[n])            reference: quant_gemm_sm80.cu:22-29
// K-group scales : r += float(p_g) * (sx[g,m]*sw[g,n]), g ascending, then D(r)
//                                                          reference: quant_grouped.cu:85-168
// FP8 products are accumulated in fp32 in ascending k; the GPU order is implementation defined,
// which is why FP8 outputs are compared with a tolerance.
// Epilogue chain after the 16-bit store (each step rounded to the output type):
//   +bias, value_scale*v + residual_scale*skip, activation(v*output_scale)
//                                                          reference: sequence_internal.cuh:52-74
// residual_f32 is the synthetic decode variant: one rounding of (gemm + residual).
void oracle_quant_linear(const uint8_t *xq, const float *sx, const uint8_t *wq, const float *sw, int m,
                         int n, int k, int input_group, int weight_group, int format, int output_type,
                         uint16_t *output, float *exact, const oracle_epilogue *ep, int threads) {
    const bool grouped = input_group || weight_group;
    const int group = grouped ? std::min(input_group ? input_group : weight_group,
                                         weight_group ? weight_group : input_group) : k;
    // FP8 operands are decoded once through a 256-entry table; the products are then plain fp32.
    std::vector<float> xf_store, wf_store;
    if (format == FP8) {
        float table[256];
        for (int q = 0; q < 256; ++q) table[q] = oracle_fp8_e4m3_decode(uint8_t(q));
        xf_store.resize(size_t(m) * k);
        wf_store.resize(size_t(n) * k);
        for (size_t i = 0; i < xf_store.size(); ++i) xf_store[i] = table[xq[i]];
        for (size_t i = 0; i < wf_store.size(); ++i) wf_store[i] = table[wq[i]];
    }
    const float *xf = xf_store.data(), *wf = wf_store.data();
    parallel_for(n, threads, [=](int first, int last) {
        for (int j = first; j < last; ++j)
            for (int i = 0; i < m; ++i) {
                const uint8_t *a = xq + size_t(i) * k, *b = wq + size_t(j) * k;
                const float *af = xf + size_t(i) * k, *bf = wf + size_t(j) * k;
                float value;
                if (!grouped) {
                    if (format == I8) {
                        int32_t sum = 0;
                        for (int c = 0; c < k; ++c) sum += int32_t(int8_t(a[c])) * int32_t(int8_t(b[c]));
                        value = (float(sum) * sx[i]) * sw[j];
                    } else {
                        float sum = 0.f;
                        for (int c = 0; c < k; ++c) sum = std::fma(af[c], bf[c], sum);
                        value = (sum * sx[i]) * sw[j];
                    }
                } else {
                    float result = 0.f;
                    for (int g0 = 0; g0 < k; g0 += group) {
                        int g1 = std::min(k, g0 + group);
                        float partial;
                        if (format == I8) {
                            int32_t sum = 0;
                            for (int c = g0; c < g1; ++c) sum += int32_t(int8_t(a[c])) * int32_t(int8_t(b[c]));
                            partial = float(sum);
                        } else {
                            partial = 0.f;
                            for (int c = g0; c < g1; ++c) partial = std::fma(af[c], bf[c], partial);
                        }
                        float scale = (input_group ? sx[size_t(g0 / input_group) * m + i] : 1.f) *
                                      (weight_group ? sw[size_t(g0 / weight_group) * n + j] : 1.f);
                        result = std::fma(partial, scale, result);
                    }
                    float outer = input_group ? 1.f : sx[i];
                    if (!weight_group) outer *= sw[j];
                    value = result * outer;
                }
                size_t at = size_t(i) * n + j;
                if (ep && ep->residual_f32) value = value + ep->residual_f32[at];
                float stored = round16(value, output_type);
                if (ep) {
                    if (ep->bias) { value = stored + load16(ep->bias[j], output_type); stored = round16(value, output_type); }
                    if (ep->residual || ep->value_scale != 1.f) {
                        float skip = ep->residual ? load16(ep->residual[at], output_type) : 0.f;
                        // the reference's finishing pass contracts this into product + fused multiply-add
                        value = std::fma(ep->value_scale, stored, ep->residual_scale * skip);
                        stored = round16(value, output_type);
                    }
                    if (ep->activation || ep->output_scale != 1.f) {
                        float scaled = round16(stored * ep->output_scale, output_type);
                        value = activate(scaled, ep->activation, ep->alpha);
                        stored = round16(value, output_type);
                    }
                }
                if (exact) exact[at] = value;
                output[at] = store16(value, output_type);
            }
    });
}

// reference: quant_norm.cu:14-123. 256 threads, 8 values per thread and item; the sum of squares
// is accumulated per thread over its pairs, reduced by a shuffle-down tree inside each warp and
// serially over the 8 warp partials. The GPU uses the approximate rsqrtf, the CPU a correctly
// rounded 1/sqrt: bytes can differ by one step where a normalized value sits on a rounding edge.
void oracle_quantized_norm(uint16_t *residual, const uint16_t *update, const uint16_t *weight,
                           const uint16_t *update_scale, int rows, int cols, int type, float epsilon,
                           int gemma, uint16_t *normalized, uint8_t *values, float *scales, int format,
                           int group, int rotation) {
    std::vector<float> row(cols);
    for (int r = 0; r < rows; ++r) {
        uint16_t *x = residual + size_t(r) * cols;
        if (update)
            for (int c = 0; c < cols; ++c) {
                float u = load16(update[size_t(r) * cols + c], type);
                if (update_scale) u = round16(u * load16(update_scale[c], type), type);
                x[c] = store16(float(double(load16(x[c], type)) + double(u)), type);
            }
        float thread_sum[256] = {};
        const int items = (2048 + 2047) / 2048;
        for (int t = 0; t < 256; ++t)
            for (int j = 0; j < items; ++j) {
                int c0 = (t + j * 256) * 8;
                for (int p = 0; p < 4; ++p) {
                    float fx = c0 + 2 * p < cols ? load16(x[c0 + 2 * p], type) : 0.f;
                    float fy = c0 + 2 * p + 1 < cols ? load16(x[c0 + 2 * p + 1], type) : 0.f;
                    thread_sum[t] += fx * fx + fy * fy;
                }
            }
        float total = 0.f;
        for (int w = 0; w < 8; ++w) {
            float lane[32];
            for (int l = 0; l < 32; ++l) lane[l] = thread_sum[w * 32 + l];
            for (int d = 16; d; d /= 2) {
                float next[32];
                for (int l = 0; l < 32; ++l) next[l] = lane[l] + (l + d < 32 ? lane[l + d] : lane[l]);
                std::memcpy(lane, next, sizeof(lane));
            }
            total += lane[0];
        }
        float inv_norm = 1.f / std::sqrt(total / cols + epsilon);
        for (int c = 0; c < cols; ++c) {
            float f = load16(x[c], type), w = load16(weight[c], type);
            float v = gemma ? round16((f * inv_norm) * (w + 1.f), type)
                            : round16(round16(f * inv_norm, type) * w, type);
            row[c] = v;
            if (normalized) normalized[size_t(r) * cols + c] = store16(v, type);
        }
        if (rotation) rotate_row(row.data(), cols);
        encode_row(row.data(), r, rows, cols, values, scales, format, group);
    }
}

// reference: quant_gated.cu:9-85. act(gate) rounded to storage, times up in storage arithmetic.
void oracle_quantized_gated(const uint16_t *input, int rows, int width, int type, int kind,
                            uint16_t *activated, uint8_t *values, float *scales, int format, int group,
                            int rotation) {
    std::vector<float> row(width);
    for (int r = 0; r < rows; ++r) {
        const uint16_t *gate = input + size_t(r) * width * 2, *up = gate + width;
        for (int c = 0; c < width; ++c) {
            float g = load16(gate[c], type);
            float a = kind == 0 ? g / (1.f + std::exp(-g))
                                : .5f * g * (1.f + std::tanh(.7978845608028654f * (g + .044715f * g * g * g)));
            float v = round16(round16(a, type) * load16(up[c], type), type);
            row[c] = v;
            if (activated) activated[size_t(r) * width + c] = store16(v, type);
        }
        if (rotation) rotate_row(row.data(), width);
        encode_row(row.data(), r, rows, width, values, scales, format, group);
    }
}

// ------------------------------------------------------------------------------------------------
// The row-wise operators around the projections.
//
// reference: Finish::apply, src/ops/kernels/sequence/sequence_internal.cuh:52-74. Every step is
// rounded to the storage type; `value_scale * value + scale * skip` is one rounded product and a
// fused multiply-add (that file is built with contraction on). The transcendental activations use
// libm here and device intrinsics there (tanh-GELU: the hardware's approximate tanh), which is why
// they are compared with a tolerance.
namespace {
inline float operand(const uint16_t *base, int rows, int row, int col, int cols, int type) {
    return base ? load16(base[size_t(rows == 1 ? 0 : row) * cols + col], type) : 0.f;
}
float finish_apply(const oracle_finish &f, int type, float value, int row, int col, int cols) {
    uint16_t *raw = f.raw ? f.raw + size_t(row) * cols + col : nullptr;
    const int per_sequence = std::max(1, f.rows_per_sequence);
    if (f.valid_rows_per_sequence && row % per_sequence >= f.valid_rows_per_sequence) {
        if (raw) *raw = store16(0.f, type);
        return 0.f;
    }
    const int sequence = row / per_sequence;
    value = round16(value + operand(f.bias, 1, 0, col, cols, type), type);
    if (f.gate) value = round16(value * operand(f.gate, f.gate_rows, sequence, col, cols, type), type);
    const int r = f.residual_index ? f.residual_index[row] : row;
    float skip = 0.f;
    if (f.residual && r >= 0) skip = r < f.residual_rows ? operand(f.residual, f.residual_rows, r, col, cols, type) : std::nanf("");
    value = round16(std::fma(f.value_scale, value, f.residual_scale * skip), type);
    if (f.condition) value = round16(value + operand(f.condition, f.condition_rows, sequence, col, cols, type), type);
    if (raw) *raw = store16(value, type);
    return activate(round16(value * f.output_scale, type), f.activation, f.alpha);
}
// Sum of 256 per-thread partials in the order of a block reduction made of warp shuffle-down trees
// (distances 1, 2, 4, 8, 16) followed by thread 0 adding the eight warp results in order.
float block_sum_256(const float *thread_value) {
    float total = 0.f;
    for (int w = 0; w < 8; ++w) {
        float lane[32];
        for (int l = 0; l < 32; ++l) lane[l] = thread_value[w * 32 + l];
        for (int d = 1; d < 32; d *= 2) {
            float next[32];
            for (int l = 0; l < 32; ++l) next[l] = (l + d < 32 ? lane[l + d] : lane[l]) + lane[l];
            std::memcpy(lane, next, sizeof(lane));
        }
        total = w ? total + lane[0] : lane[0];
    }
    return total;
}
// reference: NormRow::load / ::transform and the statistics of norm_kernel,
// src/ops/kernels/sequence/sequence_norm.cu:36-57, 64-204. Thread t of 256 owns columns t, t+256, ...;
// the variance accumulates fma(delta, delta, sum); the CPU's 1/sqrt stands in for rsqrtf.
struct NormRowOracle {
    const oracle_norm &n;
    const uint16_t *input;
    int row, sequence, cols, type;
    NormRowOracle(const oracle_norm &n, const uint16_t *x, int x_rows, int row, int cols, int type)
        : n(n), input(x + size_t(x_rows == 1 ? 0 : row) * cols), row(row), sequence(row / std::max(1, n.rows_per_sequence)),
          cols(cols), type(type) {}
    float load(int c) const {
        float value = round16(load16(input[c], type) + operand(n.projection_bias, 1, 0, c, cols, type), type);
        if (n.gate) value = round16(value * operand(n.gate, n.gate_rows, sequence, c, cols, type), type);
        return round16(value + operand(n.residual, n.residual_rows, row, c, cols, type), type);
    }
    float transform(int c, float value, float mean, float inverse) const {
        value = (value - mean) * inverse;
        if (n.weight) value = value * load16(n.weight[c], type);
        value = round16(value + operand(n.bias, 1, 0, c, cols, type), type);
        if (n.scale) value = round16(value * round16(1.f + operand(n.scale, n.scale_rows, sequence, c, cols, type), type), type);
        return round16(value + operand(n.shift, n.shift_rows, sequence, c, cols, type), type);
    }
    void statistics(std::vector<float> &loaded, float &mean, float &inverse) const {
        loaded.resize(cols);
        float partial[256];
        for (int t = 0; t < 256; ++t) {
            float sum = 0.f;
            for (int c = t; c < cols; c += 256) { loaded[c] = load(c); sum += loaded[c]; }
            partial[t] = sum;
        }
        mean = block_sum_256(partial) / float(cols);
        for (int t = 0; t < 256; ++t) {
            float sum = 0.f;
            for (int c = t; c < cols; c += 256) { float delta = loaded[c] - mean; sum = std::fma(delta, delta, sum); }
            partial[t] = sum;
        }
        inverse = 1.f / std::sqrt(block_sum_256(partial) / float(cols) + n.eps);
    }
};
} // namespace

// reference: pointwise, src/ops/kernels/sequence/sequence_pointwise.cu:332-357 (dense rows).
void oracle_pointwise(const uint16_t *x, int x_rows, int rows, int cols, int type, const oracle_finish *f, uint16_t *y) {
    const int repeat = std::max(1, f->input_repeat);
    for (int r = 0; r < rows; ++r)
        for (int c = 0; c < cols; ++c) {
            float value = load16(x[size_t(x_rows == 1 ? 0 : r / repeat) * cols + c], type);
            y[size_t(r) * cols + c] = store16(finish_apply(*f, type, value, r, c, cols), type);
        }
}

// reference: pointwise_quantize_kernel, sequence_pointwise.cu:149-265: the finished row, rounded to
// storage (and kept in `retained`), goes through the producers' common quantizing tail.
void oracle_pointwise_quantize(const uint16_t *x, int x_rows, int rows, int cols, int type, const oracle_finish *f,
                               uint16_t *retained, uint8_t *values, float *scales, int format, int group, int rotation) {
    const int repeat = std::max(1, f->input_repeat);
    std::vector<float> row(cols);
    for (int r = 0; r < rows; ++r) {
        for (int c = 0; c < cols; ++c) {
            float value = load16(x[size_t(x_rows == 1 ? 0 : r / repeat) * cols + c], type);
            row[c] = round16(finish_apply(*f, type, value, r, c, cols), type);
            if (retained) retained[size_t(r) * cols + c] = store16(row[c], type);
        }
        if (rotation) rotate_row(row.data(), cols);
        encode_row(row.data(), r, rows, cols, values, scales, format, group);
    }
}

// reference: norm_kernel<T, RowOutput>, sequence_norm.cu:64-204, launcher :412-440. `source_rows` (optional)
// gathers input rows; every index must be valid here.
void oracle_layer_norm_quantize(const uint16_t *x, int x_rows, int rows, int cols, int type, const oracle_norm *n,
                                uint16_t *normalized, uint16_t *raw, uint8_t *values, float *scales, int format, int group,
                                int rotation) {
    std::vector<float> loaded, row(cols);
    for (int out = 0; out < rows; ++out) {
        const int source = n->source_rows ? n->source_rows[out] : out;
        NormRowOracle fusion(*n, x, x_rows, source, cols, type);
        float mean, inverse;
        fusion.statistics(loaded, mean, inverse);
        for (int c = 0; c < cols; ++c) {
            row[c] = fusion.transform(c, loaded[c], mean, inverse);
            if (raw) raw[size_t(out) * cols + c] = store16(loaded[c], type);
            if (normalized) normalized[size_t(out) * cols + c] = store16(row[c], type);
        }
        if (rotation) rotate_row(row.data(), cols);
        encode_row(row.data(), out, rows, cols, values, scales, format, group);
    }
}

// reference: norm_project_kernel<T, QuantProjection>, sequence_norm.cu:261-370, launcher :518-575 (K <= 512,
// per-row scales). INT8 dot products are exact; FP8 ones are added by 32 lanes that stride K four bytes at a
// time, fused multiply-add per element, then a shuffle-down tree 16, 8, 4, 2, 1; the result is
// ((acc * sw[n]) * step), rounded to storage and finished.
void oracle_normalized_linear(const uint16_t *x, int rows, int cols, int type, const oracle_norm *n, const uint8_t *wq,
                              const float *sw, int channels, int format, const oracle_finish *f, uint16_t *out,
                              uint8_t *encoded, float *encoded_scales, uint16_t *normalized, uint16_t *raw) {
    std::vector<float> loaded, rounded(cols), activation(cols);
    std::vector<uint8_t> bytes(cols);
    for (int r = 0; r < rows; ++r) {
        NormRowOracle fusion(*n, x, rows, r, cols, type);
        float mean, inverse, amax = 0.f;
        fusion.statistics(loaded, mean, inverse);
        for (int c = 0; c < cols; ++c) {
            rounded[c] = fusion.transform(c, loaded[c], mean, inverse);
            amax = std::fmax(amax, std::fabs(rounded[c]));
            if (raw) raw[size_t(r) * cols + c] = store16(loaded[c], type);
            if (normalized) normalized[size_t(r) * cols + c] = store16(rounded[c], type);
        }
        const float step = oracle_scale(amax, format), reciprocal = 1.f / step;
        if (encoded_scales) encoded_scales[r] = step;
        for (int c = 0; c < cols; ++c) {
            bytes[c] = encode(rounded[c] * reciprocal, format);
            activation[c] = decode(bytes[c], format);
            if (encoded) encoded[size_t(r) * cols + c] = bytes[c];
        }
        for (int j = 0; j < channels; ++j) {
            const uint8_t *w = wq + size_t(j) * cols;
            float result;
            if (format == I8) {
                int32_t acc = 0;
                for (int c = 0; c < cols; ++c) acc += int32_t(int8_t(bytes[c])) * int32_t(int8_t(w[c]));
                result = (float(acc) * sw[j]) * step;
            } else {
                float lane[32];
                for (int l = 0; l < 32; ++l) {
                    float acc = 0.f;
                    for (int c = l * 4; c < cols; c += 128)
                        for (int i = 0; i < 4 && c + i < cols; ++i) acc = std::fma(activation[c + i], decode(w[c + i], format), acc);
                    lane[l] = acc;
                }
                for (int d = 16; d; d /= 2)
                    for (int l = 0; l + d < 32 && l < d; ++l) lane[l] = lane[l] + lane[l + d];
                result = (lane[0] * sw[j]) * step;
            }
            out[size_t(r) * channels + j] = store16(finish_apply(*f, type, round16(result, type), r, j, channels), type);
        }
    }
}

double oracle_time_linear(const uint16_t *x, const uint8_t *wq, const float *sw, int m, int n, int k,
                          int n_slice, int format, int group, int rotation, uint16_t *output,
                          const float *residual_f32, int threads) {
    std::vector<uint8_t> xq(size_t(m) * k);
    std::vector<float> sx(group ? size_t((k + group - 1) / group) * m : size_t(m));
    auto start = std::chrono::steady_clock::now();
    parallel_for(m, threads, [&](int first, int last) {
        // Rows are independent; each thread quantizes a slice with the row count of the whole
        // batch so K-group scales land in their group-major slots.
        std::vector<float> row(k);
        for (int r = first; r < last; ++r) {
            for (int c = 0; c < k; ++c) row[c] = oracle_bf16_to_f32(x[size_t(r) * k + c]);
            if (rotation) rotate_row(row.data(), k);
            encode_row(row.data(), r, m, k, xq.data(), sx.data(), format, group);
        }
    });
    oracle_epilogue ep{};
    ep.value_scale = ep.residual_scale = ep.output_scale = 1.f;
    ep.residual_f32 = residual_f32;
    // Only the leading n_slice channels; scales keep the full-width layout.
    if (n_slice == n || !group) {
        oracle_quant_linear(xq.data(), sx.data(), wq, sw, m, n_slice == n ? n : n_slice, k, group, group,
                            format, BF16, output, nullptr, residual_f32 && n_slice == n ? &ep : nullptr, threads);
    } else {
        std::vector<float> sw_slice(size_t((k + group - 1) / group) * n_slice);
        for (int g = 0; g < (k + group - 1) / group; ++g)
            for (int j = 0; j < n_slice; ++j) sw_slice[size_t(g) * n_slice + j] = sw[size_t(g) * n + j];
        oracle_quant_linear(xq.data(), sx.data(), wq, sw_slice.data(), m, n_slice, k, group, group, format,
                            BF16, output, nullptr, nullptr, threads);
    }
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - start).count();
}
int oracle_hardware_threads(void) { return int(std::max(1u, std::thread::hardware_concurrency())); }
}
