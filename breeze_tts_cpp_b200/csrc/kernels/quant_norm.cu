// Fused producer of the QKV / gate-up activations: x += update (optionally scaled, written back),
// RMSNorm, then per-row / K-group / rotated quantization of the normalized 16-bit value, all with
// the row held in registers (one 128-bit load and one 64-bit store per thread).
//
// Replaces the reference kernel `residual_rms_quantize` (src/ops/kernels/quant/quant_norm.cu:14-123).
// Rounding points and reduction order are kept so the bytes match that kernel bit for bit:
// the residual sum and the weight product happen in storage precision, squares are summed per
// thread over its four pairs, then a shuffle-down tree per warp, then serially over the eight
// warps; the norm uses the hardware reciprocal square root. Compile with --fmad=false.
#include "kernels/quant_norm.h"
#include "kernels/quant_codec.cuh"
#include "kernels/launch.cuh"
#include <stdexcept>
#include <string>

namespace tts {
namespace b200 {
namespace {
constexpr int kThreads = 256;
template <class T> struct Pair16;
template <> struct Pair16<__nv_bfloat16> {
    using P = __nv_bfloat162;
    __device__ static float2 unpack(P v) { return __bfloat1622float2(v); }
    __device__ static P pack(float x, float y) { return __floats2bfloat162_rn(x, y); }
};
template <> struct Pair16<__half> {
    using P = __half2;
    __device__ static float2 unpack(P v) { return __half22float2(v); }
    __device__ static P pack(float x, float y) { return __floats2half2_rn(x, y); }
};

template <class T> __device__ __forceinline__ uint4 load_raw8(const T *p, int remaining, bool aligned) {
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (aligned && remaining >= 8) return *reinterpret_cast<const uint4 *>(p);
    T *e = reinterpret_cast<T *>(&raw);
    for (int i = 0; i < 8; ++i)
        if (i < remaining) e[i] = p[i];
    return raw;
}
template <class T> __device__ __forceinline__ void store_raw8(T *p, uint4 raw, int remaining, bool aligned) {
    if (aligned && remaining >= 8) {
        *reinterpret_cast<uint4 *>(p) = raw;
        return;
    }
    const T *e = reinterpret_cast<const T *>(&raw);
    for (int i = 0; i < 8; ++i)
        if (i < remaining) p[i] = e[i];
}

template <Type F, class T, bool Add, bool Rotate>
__global__ void __launch_bounds__(kThreads)
rms_quantize(T *__restrict__ x, const T *__restrict__ update, const T *__restrict__ weight,
             const T *__restrict__ update_scale, unsigned char *__restrict__ out, float *__restrict__ scales,
             int rows, int cols, float eps, bool gemma, int group, bool aligned) {
    using M = Pair16<T>;
    using P = typename M::P;
    __shared__ float slots[kThreads / 32];
    pdl_launch_dependents();
    const int row = blockIdx.x, column = threadIdx.x * 8;
    uint4 value = make_uint4(0, 0, 0, 0), w = make_uint4(0, 0, 0, 0);
    if (column < cols) w = load_raw8(weight + column, cols - column, aligned); // static: may precede the wait
    pdl_wait_upstream();
    if (column < cols) {
        const int remaining = cols - column;
        value = load_raw8(x + size_t(row) * cols + column, remaining, aligned);
        if (Add) {
            uint4 u = load_raw8(update + size_t(row) * cols + column, remaining, aligned);
            uint4 s = update_scale ? load_raw8(update_scale + column, remaining, aligned) : make_uint4(0, 0, 0, 0);
            P *vp = reinterpret_cast<P *>(&value), *up = reinterpret_cast<P *>(&u), *sp = reinterpret_cast<P *>(&s);
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                P b = up[p];
                if (update_scale) b = __hmul2(b, sp[p]);
                vp[p] = __hadd2(vp[p], b);
            }
            store_raw8(x + size_t(row) * cols + column, value, remaining, aligned);
        }
    }
    float sum = 0.f;
    {
        const P *vp = reinterpret_cast<const P *>(&value);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            float2 f = M::unpack(vp[p]);
            sum = __fadd_rn(sum, __fadd_rn(__fmul_rn(f.x, f.x), __fmul_rn(f.y, f.y)));
        }
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, d));
    if (!(threadIdx.x & 31)) slots[threadIdx.x >> 5] = sum;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int p = 0; p < kThreads / 32; ++p) total = __fadd_rn(total, slots[p]);
    __syncthreads();
    const float inv_norm = rsqrtf(__fadd_rn(__fdiv_rn(total, float(cols)), eps));
    float v[1][8];
    {
        const P *vp = reinterpret_cast<const P *>(&value), *wp = reinterpret_cast<const P *>(&w);
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            float2 f = M::unpack(vp[p]);
            P normalized;
            if (gemma) {
                float2 wf = M::unpack(wp[p]);
                normalized = M::pack(__fmul_rn(__fmul_rn(f.x, inv_norm), __fadd_rn(wf.x, 1.f)),
                                     __fmul_rn(__fmul_rn(f.y, inv_norm), __fadd_rn(wf.y, 1.f)));
            } else {
                normalized = __hmul2(M::pack(__fmul_rn(f.x, inv_norm), __fmul_rn(f.y, inv_norm)), wp[p]);
            }
            float2 r = M::unpack(normalized);
            v[0][2 * p] = column < cols ? r.x : 0.f;
            v[0][2 * p + 1] = column < cols ? r.y : 0.f;
        }
    }
    quantize_tail<F, kThreads, 1, Rotate>(v, out, scales, row, rows, cols, group, 0, 1, aligned, slots);
}

template <Type F, class T>
void launch(T *x, const T *update, const T *weight, const T *update_scale, unsigned char *q, float *s, int rows,
            int cols, float eps, bool gemma, int group, int rotation, cudaStream_t stream) {
    const bool aligned = cols % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(weight) % 16 == 0 && reinterpret_cast<uintptr_t>(q) % 8 == 0 &&
                         (!update || reinterpret_cast<uintptr_t>(update) % 16 == 0) &&
                         (!update_scale || reinterpret_cast<uintptr_t>(update_scale) % 16 == 0);
#define B200Q_RUN(ADD, ROT)                                                                        \
    launch_pdl("quantized norm launch", rms_quantize<F, T, ADD, ROT>, dim3(rows), dim3(kThreads), 0, stream, x, update,   \
               weight, update_scale, q, s, rows, cols, eps, gemma, group, aligned)
    if (update) { if (rotation) B200Q_RUN(true, true); else B200Q_RUN(true, false); }
    else { if (rotation) B200Q_RUN(false, true); else B200Q_RUN(false, false); }
#undef B200Q_RUN
}
} // namespace
} // namespace b200

void launch_quantized_norm(TensorView residual, TensorView update, TensorView weight, RowScaledView output,
                           float epsilon, bool gemma, TensorView update_scale, cudaStream_t stream) {
    output.validate();
    // reference: quant_norm.cu:170-180
    if ((residual.type != Type::BF16 && residual.type != Type::F16) || !residual.data || !weight.data ||
        !output.values.data || !output.scales.data || !residual.dense() || residual.cols < 1 ||
        residual.cols > 2048 || residual.rows < 1 || residual.cols != output.values.cols ||
        residual.rows != output.values.rows || weight.type != residual.type || !weight.dense() ||
        weight.numel() != size_t(residual.cols) ||
        (update.data && (update.type != residual.type || update.rows != residual.rows ||
                         update.cols != residual.cols || !update.dense())) ||
        (update_scale.data && (update_scale.type != residual.type || !update_scale.dense() ||
                               update_scale.numel() != size_t(residual.cols))))
        throw std::invalid_argument("quantized RMS shape/type mismatch");
    auto *q = output.values.ptr<unsigned char>();
    auto *s = output.scales.ptr<float>();
    const bool fp8 = output.values.type == Type::FP8;
    auto run = [&](auto tag) {
        using T = decltype(tag);
        if (fp8)
            b200::launch<Type::FP8, T>(residual.ptr<T>(), update.ptr<const T>(), weight.ptr<const T>(),
                                       update_scale.ptr<const T>(), q, s, residual.rows, residual.cols, epsilon, gemma,
                                       output.group_size, output.rotation_size, stream);
        else
            b200::launch<Type::I8, T>(residual.ptr<T>(), update.ptr<const T>(), weight.ptr<const T>(),
                                      update_scale.ptr<const T>(), q, s, residual.rows, residual.cols, epsilon, gemma,
                                      output.group_size, output.rotation_size, stream);
    };
    if (residual.type == Type::F16) run(__half{});
    else run(__nv_bfloat16{});
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) throw std::runtime_error(std::string("quantized norm launch: ") + cudaGetErrorString(status));
}
} // namespace tts
