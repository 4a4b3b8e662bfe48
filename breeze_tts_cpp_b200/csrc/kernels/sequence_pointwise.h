// Launchers of the epilogue passes (finish, finish + quantize) and of LayerNorm + quantize and the
// fused norm + quantize + projection. The callers in ops/ validate shapes and aliasing first.
#pragma once
#include "core/quantization.h"
#include "ops/sequence.h"
#include <cuda_runtime_api.h>

namespace tts {
void launch_pointwise(TensorView x, TensorView y, const ops::Epilogue &, cudaStream_t);
void launch_pointwise_quantize(TensorView x, RowScaledView quantized, const ops::Epilogue &, TensorView retained,
                               int multiprocessors, cudaStream_t);
void launch_layer_norm_quantize(TensorView x, RowScaledView quantized, TensorView weight, TensorView bias, float eps,
                                const ops::NormFusion &, TensorView retained, cudaStream_t);
// Fused LayerNorm + per-row quantize + projection + finish for K <= 512 (one launch). `encoded`
// optionally receives the quantized rows, `normalized` the 16-bit normalized rows.
void launch_normalized_quantized_linear(TensorView x, TensorView normalized, TensorView norm_weight, TensorView norm_bias,
                                        float eps, const ops::NormFusion &, RowScaledView weight, TensorView output,
                                        const ops::Epilogue &, RowScaledView encoded, cudaStream_t);
} // namespace tts
