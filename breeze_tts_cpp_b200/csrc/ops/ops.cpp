#include "ops/ops.h"
#include "ops/context.h"
#include "kernels/row_quantize.h"
#include "kernels/quant_norm.h"
#include "kernels/quant_gated.h"

namespace tts::ops {
// reference: src/ops/basic.cpp:69-78
void quantize_rows(TensorView input, RowScaledView output) {
    output.validate();
    if ((input.type != Type::BF16 && input.type != Type::F16) || input.rows < 1 || input.cols < 1 || !input.data ||
        !output.values.data || !output.scales.data || input.rows != output.values.rows ||
        input.cols != output.values.cols)
        throw std::invalid_argument("quantization source/destination shape/type mismatch");
    auto &gpu = execution_context(input, {output.values, output.scales});
    launch_row_quantize(input, output, gpu.stream, gpu.multiprocessors);
}
// reference: src/ops/basic.cpp:64-67
void matmul(RowScaledView input, RowScaledView weight, TensorView output) {
    auto &gpu = execution_context(output, {input.values, input.scales, weight.values, weight.scales});
    if (!gpu.quantization) throw std::logic_error("context was created without a quantization mode");
    gpu.quantization->linear(input, weight, output);
}
// reference: src/ops/basic.cpp:48-53
void prepare_quantized(TensorView weight, int rows, int output_channels, int input_channels, Type type,
                       const Epilogue &epilogue, QuantizationGroups groups) {
    auto &gpu = execution_context(weight);
    if (!gpu.quantization) throw std::logic_error("context was created without a quantization mode");
    gpu.quantization->prepare(rows, output_channels, input_channels, type, groups);
    if (weight.rows == output_channels && weight.cols == input_channels) gpu.quantization->prepare_weight(weight);
    gpu.quantization->prepare_finish(rows, output_channels, input_channels, type, epilogue, groups);
}
// reference: src/ops/basic.cpp:54-58
void quantized_norm(TensorView input, TensorView update, TensorView weight, RowScaledView output, float epsilon,
                    bool gemma, TensorView scale) {
    auto &gpu = execution_context(input, {update, weight, output.values, output.scales, scale});
    launch_quantized_norm(input, update, weight, output, epsilon, gemma, scale, gpu.stream);
}
// reference: src/ops/basic.cpp:59-63
void quantized_gated(TensorView input, RowScaledView output, int kind) {
    auto &gpu = execution_context(input, {output.values, output.scales});
    launch_quantized_gated(input, output, kind, gpu.stream, gpu.multiprocessors, gpu.quant_gated_clusters);
}
void seal(int device) {
    auto &gpu = execution_context(device);
    gpu.plans_sealed = true;
    if (gpu.quantization) gpu.quantization->seal();
}

// reference: src/ops/linear.cpp:26-83, quantized-weight branch. The dense BF16 branch of the
// reference is a different subsystem and is not provided here. An epilogue the GEMM can apply rides
// in its own epilogue; any other legal epilogue runs as the separate finishing pass the reference
// uses (src/ops/linear.cpp:76-82), fused with the re-quantization when `quantized_output` is asked for.
void linear(const LinearOperand &input, const LinearOperand &weight, TensorView bias, TensorView output, Epilogue e,
            RowScaledView scratch, RowScaledView quantized_output) {
    auto &gpu = execution_context(output, {bias, e.residual, e.gate, e.condition, e.raw, e.residual_f32,
                                           scratch.values, scratch.scales, quantized_output.values,
                                           quantized_output.scales});
    const auto *matrix = std::get_if<RowScaledView>(&weight);
    if (!matrix) throw std::invalid_argument("this library only executes quantized weights");
    if (!gpu.quantization) throw std::logic_error("context was created without a quantization mode");
    if (e.bias.data) throw std::invalid_argument("linear already owns its bias");
    for (const TensorView &source : {bias, e.residual, e.gate, e.condition})
        if (source.overlaps(output))
            throw std::invalid_argument("linear epilogue source aliases its projection output");
    e.bias = bias;
    if (quantized_output.values.data) validate_pointwise_quantize(output, quantized_output, e);
    matrix->validate();
    RowScaledView activation;
    if (const auto *dense = std::get_if<TensorView>(&input)) {
        quantize_rows(*dense, scratch);
        activation = scratch;
    } else {
        activation = std::get<RowScaledView>(input);
    }
    if (activation.values.cols != matrix->values.cols || output.rows != activation.values.rows ||
        output.cols != matrix->values.rows || !output.dense())
        throw std::invalid_argument("quantized linear dimensions/layout mismatch");
    if (plain(e)) {
        gpu.quantization->linear(activation, *matrix, output);
        if (quantized_output.values.data) quantize_rows(output, quantized_output);
        return;
    }
    if (gpu.quantization->linear_finish(activation, *matrix, output, e)) {
        if (quantized_output.values.data) quantize_rows(output, quantized_output);
        return;
    }
    if (e.residual_f32.data) throw std::invalid_argument("an fp32 residual needs an epilogue the GEMM can fuse");
    gpu.quantization->linear(activation, *matrix, output);
    if (quantized_output.values.data) pointwise_quantize(output, quantized_output, e, {}, gpu.multiprocessors);
    else pointwise(output, output, e);
}

// reference: ops::normalized_linear, src/ops/linear.cpp:84-126 (quantized-weight branch).
bool normalized_linear(TensorView input, const LinearOperand &weight, TensorView bias, TensorView normalized,
                       TensorView output, TensorView norm_weight, TensorView norm_bias, float epsilon,
                       const NormFusion &fusion, Epilogue e, const QkvProjectionOutput *writeback,
                       RowScaledView quantized_output) {
    auto &gpu = execution_context(input, {bias, normalized, output, norm_weight, norm_bias, fusion.residual,
                                          fusion.projection_bias, fusion.raw, fusion.gate, fusion.shift, fusion.scale,
                                          e.residual, e.gate, e.condition, e.raw, quantized_output.values,
                                          quantized_output.scales});
    if (e.bias.data) throw std::invalid_argument("linear already owns its bias");
    for (const TensorView &source : {bias, e.residual, e.gate, e.condition})
        if (source.overlaps(output))
            throw std::invalid_argument("linear epilogue source aliases its projection output");
    if (e.packed || e.condition_sources || e.output_rows) return false;
    const auto *quantized = std::get_if<RowScaledView>(&weight);
    if (!quantized) throw std::invalid_argument("this library only executes quantized weights");
    if (!gpu.quantization) throw std::logic_error("context was created without a quantization mode");
    if (writeback) return false; // the fused Q/K/V cache write-back belongs to the attention subsystem
    auto project = [&](const Epilogue &epilogue) {
        return gpu.quantization->normalized_linear(input, normalized, norm_weight, norm_bias, epsilon, fusion, *quantized,
                                                   output, epilogue, {}, nullptr);
    };
    if (quantized_output.values.data) {
        e.bias = bias;
        validate_pointwise_quantize(output, quantized_output, e);
        if (quantized_output.values.type == quantized->values.type && project(e)) {
            quantize_rows(output, quantized_output);
        } else {
            if (!project({})) return false;
            pointwise_quantize(output, quantized_output, e, {}, gpu.multiprocessors);
        }
        return true;
    }
    e.bias = bias;
    return project(e);
}
} // namespace tts::ops
