// Host launchers of the quantized GEMM. Signatures follow the reference's
// (src/ops/kernels/quant/quant_dispatch.h:7-17) so `QuantizedGemm` and any direct caller can
// switch without edits; `LinearKind::Tcgen05` is the only kind this build executes.
#pragma once
#include "core/quantization.h"
#include <cuda.h>
#include <cuda_runtime.h>

namespace tts {
namespace ops { struct Epilogue; }

void grouped_quant_gemm(KernelProblem, const void *input, const float *input_scales,
                        const void *weights, const float *weight_scales, void *output,
                        cudaStream_t, Type format, Type output_type, int tokens = 16, int splits = 1,
                        void *workspace = nullptr, size_t workspace_bytes = 0);
void launch_quant_linear(LinearPath config, KernelProblem shape, const void *input,
                         const float *input_scales, const void *weights, const float *weight_scales,
                         void *output, void *workspace, size_t workspace_bytes, cudaStream_t stream,
                         Type format = Type::FP8, Type output_type = Type::BF16,
                         const ops::Epilogue *finish = nullptr, const struct WeightMaps *prepared = nullptr);
// Initialization only; the fused finish needs no extra resources on this path.
KernelResources quant_linear_finish_resources(LinearPath, Type format, Type output_type);

// --- additions of this build -------------------------------------------------------------------
// The TMA descriptor of a weight matrix, built once while plans are prepared and handed to
// `launch_quant_linear` through its last, optional argument; a launch whose weights it does not
// describe (or that passes none) builds the descriptor itself.
struct WeightMaps {
    CUtensorMap values;
    const void *weights = nullptr;
    int channels = 0, reduction = 0;
};
WeightMaps quant_linear_weight_maps(const void *weights, int channels, int reduction);
// Tile/split choice for a problem with the B200 chip model: tokens = token tile (16..256),
// channels = 128, splits = split-K. Shorthand for `select_linear` (ops/quantization_policy.h).
LinearPath select_tcgen05_path(KernelProblem, Type format, int multiprocessors, size_t workspace_bytes);
// Bytes of caller workspace a path needs (header + split-K partials).
size_t quant_linear_workspace_bytes(LinearPath, KernelProblem);
// One-time set-up per device and process: raises the dynamic shared-memory limit of every kernel
// instance and resolves the driver entry point for tensor maps. Call before stream capture.
void quant_linear_initialize(int device);
// Zeroes the ticket/status header of a fresh workspace (asynchronously on `stream`).
void quant_linear_reset_workspace(void *workspace, size_t workspace_bytes, cudaStream_t stream);
// Failure-path exercise without a GPU fault: the NEXT weight-streaming GEMM launched from this thread
// arms its first weight barrier for `extra_bytes` more than its (fully completing) copy delivers and
// lets every device-side wait give up after `limit_cycles` SM cycles, so the kernel runs to its normal
// teardown, stores nothing and raises the status word. One-shot; nothing is left in flight.
void quant_linear_inject_wait_expiry(int extra_bytes, long long limit_cycles);
// Blocking read of the status word: 0 = clean, otherwise 1 + index of the tile whose bounded wait gave up.
int quant_linear_status(const void *workspace, cudaStream_t stream);
} // namespace tts
