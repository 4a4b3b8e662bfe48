// Semantic operators of the quantized linear path, as free functions over views — the level the
// reference's layers call (src/ops/storage.h:12, src/ops/basic.h:11,25-26,33-35, src/ops/linear.h:11-14).
#pragma once
#include "core/quantization.h"
#include "ops/epilogue.h"
#include "ops/sequence.h"
#include <variant>

namespace tts {
struct QkvProjectionOutput;
}
namespace tts::ops {
using LinearOperand = std::variant<TensorView, RowScaledView>;

// Dynamic per-row (or per-K-group, optionally rotated) quantization of a 16-bit matrix.
void quantize_rows(TensorView input, RowScaledView output);
// output[M,N] = dequant(input[M,K] x weight[N,K]^T); the shape must have been prepared.
void matmul(RowScaledView input, RowScaledView weight, TensorView output);
void prepare_quantized(TensorView weight, int rows, int output_channels, int input_channels, Type type,
                       const Epilogue &epilogue = {}, QuantizationGroups groups = {});
// Residual add (written back) + RMSNorm + quantize; feeds QKV and gate/up.
void quantized_norm(TensorView input, TensorView update, TensorView weight, RowScaledView output, float epsilon,
                    bool gemma = false, TensorView scale = {});
// act(gate) * up on [rows, 2K] + quantize; feeds the down projection. kind 0 = SiLU, 1 = tanh-GELU.
void quantized_gated(TensorView input, RowScaledView output, int kind);
// Quantized Linear: quantizes a dense activation into `scratch` when needed, runs the GEMM and
// applies bias + epilogue inside it. With `quantized_output`, the finished rows are re-quantized
// for the next layer and `output` is scratch.
void linear(const LinearOperand &input, const LinearOperand &weight, TensorView bias, TensorView output,
            Epilogue = {}, RowScaledView scratch = {}, RowScaledView quantized_output = {});
// LayerNorm + quantize + projection + finish in one launch for narrow rows (K <= 512, per-row scales).
// False means "not taken": the caller runs layer_norm_quantize + linear instead, exactly as with the
// reference (src/ops/linear.h:15-18). The attention write-back argument is accepted and declined.
bool normalized_linear(TensorView input, const LinearOperand &weight, TensorView bias, TensorView normalized,
                       TensorView output, TensorView norm_weight, TensorView norm_bias, float epsilon,
                       const NormFusion &fusion, Epilogue = {}, const QkvProjectionOutput *writeback = nullptr,
                       RowScaledView quantized_output = {});
void seal(int device);
} // namespace tts::ops
