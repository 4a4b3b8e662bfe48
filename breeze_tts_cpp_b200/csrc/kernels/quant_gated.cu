// Fused producer of the down-projection activation: act(gate) * up over a [rows, 2K] matrix,
// rounded to storage precision at the reference's two points, then per-row / K-group / rotated
// quantization — one read of the gate/up row, one write of bytes and scales.
//
// Replaces the reference kernel `vector_gated_quantize` (src/ops/kernels/quant/quant_gated.cu:18-85).
// SiLU uses the same scaled fast divide and fast exponential (quant_gated.cu:9-16) so INT8 bytes
// match that kernel bit for bit. Compile with --fmad=false.
// In K-group mode the 2048-column slabs of one row are independent and are spread over several
// CTAs for short batches; with one scale per row the CTA holds the whole row (K <= 8192).
#include "kernels/quant_gated.h"
#include "kernels/quant_codec.cuh"
#include "kernels/launch.cuh"
#include <stdexcept>
#include <string>

namespace tts {
namespace b200 {
namespace {
constexpr int kThreads = 256;
template <int Kind> __device__ __forceinline__ float gate_activation(float x) {
    if (Kind == 0) return __fdividef(__fmul_rn(x, 0x1p-16f), __fmul_rn(__fadd_rn(1.f, __expf(-x)), 0x1p-16f));
    float cube = __fmul_rn(__fmul_rn(__fmul_rn(.044715f, x), x), x);
    float t = tanhf(__fmul_rn(.7978845608028654f, __fadd_rn(x, cube)));
    return __fmul_rn(__fmul_rn(.5f, x), __fadd_rn(1.f, t));
}
template <class T> __device__ __forceinline__ float round16(float v);
template <> __device__ __forceinline__ float round16<__nv_bfloat16>(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}
template <> __device__ __forceinline__ float round16<__half>(float v) { return __half2float(__float2half_rn(v)); }

template <Type F, class T, int Kind, int Items, bool Rotate, int Threads = kThreads>
__global__ void __launch_bounds__(Threads)
gated_quantize(const T *__restrict__ input, unsigned char *__restrict__ out, float *__restrict__ scales, int rows,
               int cols, int group, int parts, bool aligned) {
    constexpr int kThreads = Threads; // shadows the file-wide default inside this kernel
    __shared__ float slots[kThreads / 32];
    pdl_launch_dependents();
    pdl_wait_upstream();
    const int row = blockIdx.x / parts, shard = blockIdx.x % parts;
    const T *gate = input + size_t(row) * cols * 2, *up = gate + cols;
    float v[Items][8];
    if (aligned) {
        // All loads of the row shard are issued before the first value is used.
        uint4 raw_gate[Items], raw_up[Items];
#pragma unroll
        for (int j = 0; j < Items; ++j) {
            const int column = ((j * parts + shard) * kThreads + int(threadIdx.x)) * 8;
            raw_gate[j] = raw_up[j] = make_uint4(0, 0, 0, 0);
            if (column < cols) {
                raw_gate[j] = *reinterpret_cast<const uint4 *>(gate + column);
                raw_up[j] = *reinterpret_cast<const uint4 *>(up + column);
            }
        }
#pragma unroll
        for (int j = 0; j < Items; ++j) {
            float g[8], u[8];
            unpack8<T>(raw_gate[j], g);
            unpack8<T>(raw_up[j], u);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[j][i] = round16<T>(__fmul_rn(round16<T>(gate_activation<Kind>(g[i])), u[i]));
        }
    } else {
#pragma unroll
        for (int j = 0; j < Items; ++j) {
            const int column = ((j * parts + shard) * kThreads + int(threadIdx.x)) * 8;
            if (column < cols) {
                float g[8], u[8];
                load8(gate + column, cols - column, false, g);
                load8(up + column, cols - column, false, u);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    // Both operands are storage-precision values, so the fp32 product is exact and
                    // one rounding reproduces the packed 16-bit multiply.
                    v[j][i] = round16<T>(__fmul_rn(round16<T>(gate_activation<Kind>(g[i])), u[i]));
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) v[j][i] = 0.f;
            }
        }
    }
    quantize_tail<F, kThreads, Items, Rotate>(v, out, scales, row, rows, cols, group, shard, parts, aligned, slots);
}

template <Type F, class T, int Kind, bool Rotate>
void launch_items(const T *x, unsigned char *q, float *s, int rows, int cols, int group, int sms, cudaStream_t stream) {
    const bool aligned = cols % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(q) % 8 == 0;
    const int chunks = (cols + kThreads * 8 - 1) / (kThreads * 8);
    // K-group slabs of a row are independent, so short batches spread them over several CTAs. With
    // one scale per row the CTA keeps the whole row: joining CTAs through a cluster barrier was
    // measured slower than the three 128-bit loads per thread it saves.
    int parts = 1;
    if (group)
        while (parts < chunks && parts < 8 && int64_t(rows) * parts <= 2 * sms) parts *= 2;
    // Short batches with one scale per row (decode): the CTA that holds a row is alone on its multiprocessor, and
    // with 256 threads the activation arithmetic of 6144 columns is three dependent rounds on two warps per
    // scheduler. One value group per thread on a CTA three or four times as wide hides those latencies.
    if (!group && aligned && chunks > 1 && chunks <= 4 && rows <= sms) {
        const int threads = chunks * kThreads;
#define B200Q_WIDE(N)                                                                                                   \
    launch_pdl("quantized gated launch", gated_quantize<F, T, Kind, 1, Rotate, N>, dim3(unsigned(rows)), dim3(N), 0, stream, x, \
               q, s, rows, cols, group, 1, aligned)
        if (threads == 512) B200Q_WIDE(512);
        else if (threads == 768) B200Q_WIDE(768);
        else B200Q_WIDE(1024);
#undef B200Q_WIDE
        return;
    }
    const int items = (chunks + parts - 1) / parts;
    const unsigned grid = unsigned(rows) * unsigned(parts);
#define B200Q_RUN(I)                                                                                                  \
    launch_pdl("quantized gated launch", gated_quantize<F, T, Kind, I, Rotate>, dim3(grid), dim3(kThreads), 0, stream, x, \
               q, s, rows, cols, group, parts, aligned)
    switch (items) {
    case 1: B200Q_RUN(1); break;
    case 2: B200Q_RUN(2); break;
    case 3: B200Q_RUN(3); break;
    default: B200Q_RUN(4); break;
    }
#undef B200Q_RUN
}
template <Type F, class T>
void launch_kind(const T *x, unsigned char *q, float *s, int rows, int cols, int group, int rotation, int kind, int sms,
                 cudaStream_t stream) {
    if (kind == 0) {
        if (rotation) launch_items<F, T, 0, true>(x, q, s, rows, cols, group, sms, stream);
        else launch_items<F, T, 0, false>(x, q, s, rows, cols, group, sms, stream);
    } else {
        if (rotation) launch_items<F, T, 1, true>(x, q, s, rows, cols, group, sms, stream);
        else launch_items<F, T, 1, false>(x, q, s, rows, cols, group, sms, stream);
    }
}
} // namespace
} // namespace b200

bool quant_gated_supports_clusters(int device) {
    int supported = 0;
    cudaDeviceGetAttribute(&supported, cudaDevAttrClusterLaunch, device);
    return supported != 0;
}

void launch_quantized_gated(TensorView input, RowScaledView output, int kind, cudaStream_t stream,
                            int multiprocessors, bool clusters) {
    (void)clusters; // sm_100 always has cluster launch; the flag is kept for signature compatibility
    output.validate();
    const int width = output.values.cols;
    // reference: quant_gated.cu:183-187
    if ((input.type != Type::BF16 && input.type != Type::F16) || !input.data || !output.values.data ||
        !output.scales.data || !input.dense() || input.rows != output.values.rows ||
        input.cols != int64_t(2) * width || kind < 0 || kind > 1 || width < 1 || width > 8192 || input.rows < 1)
        throw std::invalid_argument("quantized gated shape/type mismatch");
    if (multiprocessors <= 0) multiprocessors = 148;
    auto *q = output.values.ptr<unsigned char>();
    auto *s = output.scales.ptr<float>();
    const bool fp8 = output.values.type == Type::FP8;
    auto run = [&](auto tag) {
        using T = decltype(tag);
        if (fp8)
            b200::launch_kind<Type::FP8, T>(input.ptr<const T>(), q, s, input.rows, width, output.group_size,
                                            output.rotation_size, kind, multiprocessors, stream);
        else
            b200::launch_kind<Type::I8, T>(input.ptr<const T>(), q, s, input.rows, width, output.group_size,
                                           output.rotation_size, kind, multiprocessors, stream);
    };
    if (input.type == Type::F16) run(__half{});
    else run(__nv_bfloat16{});
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) throw std::runtime_error(std::string("quantized gated launch: ") + cudaGetErrorString(status));
}
} // namespace tts
