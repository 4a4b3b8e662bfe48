// Plan cache + dispatch of the quantized GEMM. Public surface identical to the reference class
// (src/ops/cuda/quantization.h:15-42): prepare / prepare_finish before seal(), linear /
// linear_finish afterwards; a shape that was not prepared throws instead of tuning at serve time.
// The cuBLASLt handle of the reference constructor is accepted and ignored: every format runs on
// this library's own tcgen05 kernels.
#pragma once
#include "core/buffer.h"
#include "core/quantization.h"
#include <cuda_runtime_api.h>
#include <memory>

namespace tts {
namespace ops { struct NormFusion; struct Epilogue; }
struct QkvProjectionOutput;
struct QuantCacheStats {
    SelectionStats selection;
    size_t prepared_plans = 0;
};
class QuantizedGemm {
    struct Impl;
    std::unique_ptr<Impl> impl;

  public:
    QuantizedGemm(cudaStream_t stream, void *library_handle, Buffer &workspace, Type format = Type::FP8);
    ~QuantizedGemm();
    QuantizedGemm(const QuantizedGemm &) = delete;
    void seal();
    QuantCacheStats cache_stats() const;
    void prepare(int rows, int output_channels, int input_channels, Type output_type = Type::BF16,
                 QuantizationGroups groups = {});
    // Addition: builds the TMA descriptor of a quantized weight matrix ahead of time (before seal()),
    // so that no launch has to encode it. Views that are not one-byte dense matrices are ignored.
    void prepare_weight(TensorView quantized_values);
    void prepare_finish(int rows, int output_channels, int input_channels, Type output_type,
                        const ops::Epilogue &, QuantizationGroups groups = {});
    void linear(RowScaledView input, RowScaledView weight, TensorView output);
    // True when the epilogue ran inside the GEMM; false leaves it to the caller's separate pass.
    bool linear_finish(RowScaledView input, RowScaledView weight, TensorView output, const ops::Epilogue &);
    // Fused LayerNorm + quantize + projection for K <= 512 with per-row scales; false = not taken, which
    // by contract leaves the caller's two-step path responsible.
    bool normalized_linear(TensorView input, TensorView normalized, TensorView norm_weight,
                           TensorView norm_bias, float epsilon, const ops::NormFusion &,
                           RowScaledView weight, TensorView output, const ops::Epilogue &,
                           RowScaledView encoded = {}, const QkvProjectionOutput *writeback = nullptr);
    // Additions: the chosen path of a prepared shape, and the device status word.
    LinearPath planned_path(int rows, int output_channels, int input_channels, Type output_type,
                            QuantizationGroups groups = {}) const;
    int status() const;
};
} // namespace tts
