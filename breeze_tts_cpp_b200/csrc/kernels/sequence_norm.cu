// LayerNorm fused with quantization, and the fused LayerNorm + quantize + projection for narrow
// models (K <= 512), as sm_100a kernels behind the reference's operators.
//
// Replaces the reference's `norm_kernel<T, RowOutput>` (src/ops/kernels/sequence/sequence_norm.cu:64-204,
// launcher :412-440) and `norm_project_kernel<T, QuantProjection>` (:261-370, launcher :518-575).
// The statistics keep the reference's arithmetic so that the bytes match it: thread t sums columns
// t, t+256, ... in that order, warps are reduced by a shuffle-down tree with distances 1, 2, 4, 8, 16,
// thread 0 adds the eight warp sums in order, the variance accumulates fma(delta, delta, sum), the
// norm uses the hardware reciprocal square root, and every storage rounding point of the row
// pipeline (projection bias, gate, residual, weight, bias, scale, shift) is kept. The quantizing tail
// then works on eight consecutive columns per thread (128-bit accesses); maxima are exact, so the
// regrouping changes no bit. Compile with --fmad=false: contractions are written out.
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
constexpr int kCached = 8; // strided values a thread keeps between the two statistics passes (2048 columns)

struct NormArgs {
    FinishOperand input, weight, bias, projection, residual, gate, shift, scale;
    void *output = nullptr, *raw = nullptr;
    int output_stride = 0, raw_stride = 0, rows_per_sequence = 1, input_rows = 0;
    const int *source_rows = nullptr;
    float eps = 0.f;
};

template <class T> struct NormRow {
    const T *input, *projection, *residual, *gate, *weight, *bias, *scale, *shift;
    template <class U> __device__ static const U *row_of(const FinishOperand &o, int row) {
        return o.data ? static_cast<const U *>(o.data) + size_t(o.rows == 1 ? 0 : row) * o.stride : nullptr;
    }
    __device__ NormRow(const NormArgs &a, int row) {
        const int sequence = row / a.rows_per_sequence;
        input = row_of<T>(a.input, row);
        projection = row_of<T>(a.projection, 0);
        residual = row_of<T>(a.residual, row);
        gate = row_of<T>(a.gate, sequence);
        weight = row_of<T>(a.weight, 0);
        bias = row_of<T>(a.bias, 0);
        scale = row_of<T>(a.scale, sequence);
        shift = row_of<T>(a.shift, sequence);
    }
    __device__ __forceinline__ static float read(const T *p, int c) { return p ? float(p[c]) : 0.f; }
    // The value that is normalized: input + projection bias, times gate, plus residual, rounded to
    // storage after every step (reference: NormRow::load, sequence_norm.cu:43-47).
    __device__ __forceinline__ float load(int c) const {
        float value = round_storage<T>(__fadd_rn(float(input[c]), read(projection, c)));
        if (gate) value = round_storage<T>(__fmul_rn(value, float(gate[c])));
        return round_storage<T>(__fadd_rn(value, read(residual, c)));
    }
    // reference: NormRow::transform, sequence_norm.cu:48-57
    __device__ __forceinline__ float transform(int c, float value, float mean, float inverse) const {
        value = __fmul_rn(__fsub_rn(value, mean), inverse);
        if (weight) value = __fmul_rn(value, float(weight[c]));
        value = round_storage<T>(__fadd_rn(value, read(bias, c)));
        if (scale) value = round_storage<T>(__fmul_rn(value, round_storage<T>(__fadd_rn(1.f, float(scale[c])))));
        return round_storage<T>(__fadd_rn(value, read(shift, c)));
    }
};

// Sum over the CTA in the order of a block reduction built from warp shuffle-down trees: the result is
// returned to every thread.
__device__ __forceinline__ float block_sum(float v, float *slots, float *broadcast) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) v = __fadd_rn(__shfl_down_sync(0xffffffffu, v, d), v);
    if (!(threadIdx.x & 31)) slots[threadIdx.x >> 5] = v;
    __syncthreads();
    if (!threadIdx.x) {
        float total = slots[0];
#pragma unroll
        for (int w = 1; w < kThreads / 32; ++w) total = __fadd_rn(total, slots[w]);
        *broadcast = total;
    }
    __syncthreads();
    return *broadcast;
}

// Mean and reciprocal standard deviation of one row.
template <class T>
__device__ __forceinline__ void row_statistics(const NormRow<T> &row, int cols, float eps, float *slots, float *shared,
                                               float &mean, float &inverse) {
    float cached[kCached], sum = 0.f;
#pragma unroll
    for (int i = 0; i < kCached; ++i) {
        const int c = int(threadIdx.x) + i * kThreads;
        cached[i] = c < cols ? row.load(c) : 0.f;
        sum = __fadd_rn(sum, cached[i]);
    }
    for (int c = int(threadIdx.x) + kCached * kThreads; c < cols; c += kThreads) sum = __fadd_rn(sum, row.load(c));
    mean = __fdiv_rn(block_sum(sum, slots, shared), float(cols));
    sum = 0.f;
#pragma unroll
    for (int i = 0; i < kCached; ++i) {
        if (int(threadIdx.x) + i * kThreads < cols) {
            const float delta = __fsub_rn(cached[i], mean);
            sum = __fmaf_rn(delta, delta, sum);
        }
    }
    for (int c = int(threadIdx.x) + kCached * kThreads; c < cols; c += kThreads) {
        const float delta = __fsub_rn(row.load(c), mean);
        sum = __fmaf_rn(delta, delta, sum);
    }
    inverse = rsqrtf(__fadd_rn(__fdiv_rn(block_sum(sum, slots, shared + 1), float(cols)), eps));
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

template <Type F, class T, int Items, bool Rotate>
__global__ void __launch_bounds__(kThreads)
layer_norm_quantize_rows(NormArgs a, unsigned char *__restrict__ q, float *__restrict__ scales, int rows, int cols, int group) {
    __shared__ float slots[kThreads / 32];
    __shared__ float shared[2];
    pdl_launch_dependents();
    pdl_wait_upstream();
    const int output_row = blockIdx.x;
    const int row = a.source_rows ? a.source_rows[output_row] : output_row;
    T *output = a.output ? static_cast<T *>(a.output) + size_t(output_row) * a.output_stride : nullptr;
    T *raw = a.raw ? static_cast<T *>(a.raw) + size_t(output_row) * a.raw_stride : nullptr;
    const bool aligned = cols % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0;
    float v[Items][8];
    if (row < 0 || row >= a.input_rows) {
        // A gathered row that does not exist poisons its output (reference: sequence_norm.cu:74-84).
        for (int c = threadIdx.x; c < cols; c += kThreads) {
            if (output) output[c] = T(nanf(""));
            q[size_t(output_row) * cols + c] = (unsigned char)Codec<F>::one(nanf(""));
        }
        const int groups = group ? (cols + group - 1) / group : 1;
        for (int g = threadIdx.x; g < groups; g += kThreads) scales[size_t(g) * rows + output_row] = 1.f;
        return;
    }
    const NormRow<T> fusion(a, row);
    float mean, inverse;
    row_statistics(fusion, cols, a.eps, slots, shared, mean, inverse);
#pragma unroll
    for (int j = 0; j < Items; ++j) {
        const int col = (j * kThreads + int(threadIdx.x)) * 8;
        float before[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const bool inside = col + i < cols;
            before[i] = inside ? fusion.load(col + i) : 0.f;
            v[j][i] = inside ? fusion.transform(col + i, before[i], mean, inverse) : 0.f;
        }
        if (col < cols) {
            if (raw) store16(raw + col, cols - col, before);
            if (output) store16(output + col, cols - col, v[j]);
        }
    }
    quantize_tail<F, kThreads, Items, Rotate>(v, q, scales, output_row, rows, cols, group, 0, 1, aligned, slots);
}

template <Type F, class T, bool Rotate>
void launch_norm(const NormArgs &a, RowScaledView out, cudaStream_t stream) {
    const int rows = out.values.rows, cols = out.values.cols;
    auto *q = out.values.ptr<unsigned char>();
    auto *s = out.scales.ptr<float>();
#define B200Q_RUN(I)                                                                                                 \
    launch_pdl("layer norm + quantize launch", layer_norm_quantize_rows<F, T, I, Rotate>, dim3(rows), dim3(kThreads), 0, \
               stream, a, q, s, rows, cols, out.group_size)
    switch ((cols + kThreads * 8 - 1) / (kThreads * 8)) {
    case 1: B200Q_RUN(1); break;
    case 2: B200Q_RUN(2); break;
    case 3: B200Q_RUN(3); break;
    case 4: B200Q_RUN(4); break;
    default: throw std::invalid_argument("layer norm + quantize holds rows of up to 8192 columns");
    }
#undef B200Q_RUN
}

// ---------------------------------------------------------------- norm + quantize + projection, K <= 512
constexpr int kProjectionValues = 2;               // columns per thread: K <= 512
constexpr int kChannelsPerWarp = 8, kChannelsPerBlock = (kThreads / 32) * kChannelsPerWarp;

struct ProjectionArgs {
    const unsigned char *weight;
    const float *weight_scales;
    unsigned char *encoded;
    float *encoded_scales;
    void *output;
    int output_stride, channels, cols;
};

// Grid (ceil(N / 64), rows). Every CTA of a row normalizes and quantizes the row into shared memory
// (the first one also stores the row-level results), then each warp produces eight output channels:
// lanes stride the K axis four bytes at a time exactly as the reference's warp does, so FP8 sums are
// added in the same order; INT8 sums are exact integers.
template <Type F, class T>
__global__ void __launch_bounds__(kThreads)
norm_quantize_project(NormArgs a, ProjectionArgs p, FinishArgs finish) {
    __shared__ float slots[kThreads / 32];
    __shared__ float shared[3];
    __shared__ __align__(16) T activation[kThreads * kProjectionValues]; // FP8: decoded values; INT8: the bytes
    pdl_launch_dependents();
    pdl_wait_upstream();
    const int row = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, cols = p.cols;
    const NormRow<T> fusion(a, row);
    float values[kProjectionValues], sum = 0.f;
#pragma unroll
    for (int i = 0; i < kProjectionValues; ++i) {
        const int c = int(threadIdx.x) + i * kThreads;
        values[i] = c < cols ? fusion.load(c) : 0.f;
        sum = __fadd_rn(sum, values[i]);
    }
    const float mean = __fdiv_rn(block_sum(sum, slots, shared), float(cols));
    sum = 0.f;
#pragma unroll
    for (int i = 0; i < kProjectionValues; ++i)
        if (int(threadIdx.x) + i * kThreads < cols) {
            const float delta = __fsub_rn(values[i], mean);
            sum = __fmaf_rn(delta, delta, sum);
        }
    const float inverse = rsqrtf(__fadd_rn(__fdiv_rn(block_sum(sum, slots, shared + 1), float(cols)), a.eps));
    float rounded[kProjectionValues], amax = 0.f;
    T *normalized = a.output ? static_cast<T *>(a.output) + size_t(row) * a.output_stride : nullptr;
    T *raw = a.raw ? static_cast<T *>(a.raw) + size_t(row) * a.raw_stride : nullptr;
#pragma unroll
    for (int i = 0; i < kProjectionValues; ++i) {
        const int c = int(threadIdx.x) + i * kThreads;
        rounded[i] = 0.f;
        if (c < cols) {
            rounded[i] = fusion.transform(c, values[i], mean, inverse);
            amax = fmaxf(amax, fabsf(rounded[i]));
            if (!blockIdx.x) {
                if (raw) raw[c] = T(values[i]);
                if (normalized) normalized[c] = T(rounded[i]);
            }
        }
    }
    const float step = quant_scale<F>(cta_max<kThreads>(amax, slots));
    const float reciprocal = __fdiv_rn(1.f, step);
    if (!threadIdx.x && !blockIdx.x && p.encoded_scales) p.encoded_scales[row] = step;
#pragma unroll
    for (int i = 0; i < kProjectionValues; ++i) {
        const int c = int(threadIdx.x) + i * kThreads;
        if (c < cols) {
            const unsigned char byte = (unsigned char)Codec<F>::one(__fmul_rn(rounded[i], reciprocal));
            if (F == Type::I8) {
                reinterpret_cast<unsigned char *>(activation)[c] = byte;
            } else {
                const __half_raw decoded = __nv_cvt_fp8_to_halfraw(byte, __NV_E4M3);
                activation[c] = T(__half2float(__half(decoded)));
            }
            if (!blockIdx.x && p.encoded) p.encoded[size_t(row) * cols + c] = byte;
        }
    }
    __syncthreads();
    const FinishRow finish_of_row = finish_row(finish, row);
    T *out = static_cast<T *>(p.output) + size_t(row) * p.output_stride;
#pragma unroll 1
    for (int k = 0; k < kChannelsPerWarp; ++k) {
        const int channel = (blockIdx.x * (kThreads / 32) + warp) * kChannelsPerWarp + k;
        if (channel >= p.channels) break; // warp-uniform
        const unsigned char *w = p.weight + size_t(channel) * cols;
        float result;
        if (F == Type::I8) {
            int acc = 0;
            for (int c = lane * 4; c < cols; c += 128)
                acc = __dp4a(*reinterpret_cast<const int *>(reinterpret_cast<const unsigned char *>(activation) + c),
                             *reinterpret_cast<const int *>(w + c), acc);
            acc = __reduce_add_sync(0xffffffffu, acc);
            result = __fmul_rn(__fmul_rn(float(acc), p.weight_scales[channel]), step);
        } else {
            float acc = 0.f;
            for (int c = lane * 4; c < cols; c += 128) {
                const unsigned packed = *reinterpret_cast<const unsigned *>(w + c);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const __half_raw decoded = __nv_cvt_fp8_to_halfraw((packed >> (8 * i)) & 0xffu, __NV_E4M3);
                    acc = __fmaf_rn(float(activation[c + i]), __half2float(__half(decoded)), acc);
                }
            }
#pragma unroll
            for (int d = 16; d; d >>= 1) acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, d));
            result = __fmul_rn(__fmul_rn(acc, p.weight_scales[channel]), step);
        }
        if (!lane) out[channel] = T(finish_apply<T>(finish, finish_of_row, round_storage<T>(result), row, channel));
    }
}

NormArgs norm_args(TensorView x, TensorView weight, TensorView bias, float eps, const ops::NormFusion &f, TensorView output) {
    NormArgs a;
    a.input = FinishOperand(x);
    a.weight = FinishOperand(weight);
    a.bias = FinishOperand(bias);
    a.projection = FinishOperand(f.projection_bias);
    a.residual = FinishOperand(f.residual);
    a.gate = FinishOperand(f.gate);
    a.shift = FinishOperand(f.shift);
    a.scale = FinishOperand(f.scale);
    a.output = output.data;
    a.output_stride = output.ld();
    a.raw = f.raw.data;
    a.raw_stride = f.raw.ld();
    a.rows_per_sequence = f.rows_per_sequence;
    a.input_rows = x.rows;
    a.source_rows = f.source_rows;
    a.eps = eps;
    return a;
}
} // namespace
} // namespace b200

void launch_layer_norm_quantize(TensorView x, RowScaledView q, TensorView weight, TensorView bias, float eps,
                                const ops::NormFusion &f, TensorView retained, cudaStream_t stream) {
    const b200::NormArgs a = b200::norm_args(x, weight, bias, eps, f, retained);
    const bool fp8 = q.values.type == Type::FP8, rotate = q.rotation_size != 0;
    auto run = [&](auto tag) {
        using T = decltype(tag);
        if (fp8) {
            if (rotate) b200::launch_norm<Type::FP8, T, true>(a, q, stream);
            else b200::launch_norm<Type::FP8, T, false>(a, q, stream);
        } else {
            if (rotate) b200::launch_norm<Type::I8, T, true>(a, q, stream);
            else b200::launch_norm<Type::I8, T, false>(a, q, stream);
        }
    };
    if (x.type == Type::F16) run(__half{});
    else run(__nv_bfloat16{});
}

void launch_normalized_quantized_linear(TensorView x, TensorView normalized, TensorView norm_weight, TensorView norm_bias,
                                        float eps, const ops::NormFusion &f, RowScaledView weight, TensorView output,
                                        const ops::Epilogue &e, RowScaledView encoded, cudaStream_t stream) {
    const b200::NormArgs a = b200::norm_args(x, norm_weight, norm_bias, eps, f, normalized);
    b200::ProjectionArgs p{weight.values.ptr<unsigned char>(), weight.scales.ptr<float>(), encoded.values.ptr<unsigned char>(),
                           encoded.scales.ptr<float>(), output.data, output.ld(), weight.values.rows, weight.values.cols};
    const dim3 grid(unsigned((p.channels + b200::kChannelsPerBlock - 1) / b200::kChannelsPerBlock), unsigned(x.rows));
    const b200::FinishArgs finish(e);
    auto run = [&](auto tag) {
        using T = decltype(tag);
        if (weight.values.type == Type::FP8)
            b200::launch_pdl("norm + quantize + projection launch", b200::norm_quantize_project<Type::FP8, T>, grid,
                             dim3(b200::kThreads), 0, stream, a, p, finish);
        else
            b200::launch_pdl("norm + quantize + projection launch", b200::norm_quantize_project<Type::I8, T>, grid,
                             dim3(b200::kThreads), 0, stream, a, p, finish);
    };
    if (x.type == Type::F16) run(__half{});
    else run(__nv_bfloat16{});
}
} // namespace tts
