// Quantized Linear layer: holds a RowScaledView weight (+ optional bias) and runs
// quantize -> GEMM -> fused epilogue through the op layer. Public methods follow the reference's
// `tts::Linear` (src/layers/linear.h:11-76) for the quantized case; construction from a checkpoint
// (`Weights`) and the `ForwardContext` plumbing are the reference engine's own and are replaced
// here by `Linear::quantize`, which performs the load-time step of `Weights::quantized`
// (src/io/weights.cpp:80-87,133-154): concatenate the source matrices by rows and quantize them
// on the device into storage the layer owns.
#pragma once
#include "core/buffer.h"
#include "layers/quantization.h"
#include "ops/ops.h"
#include <memory>
#include <vector>

namespace tts {
class Linear {
    RowScaledView weight_;
    TensorView bias_;
    Type activation_type_ = Type::BF16;
    std::shared_ptr<Buffer> values_, scales_; // set when the layer owns its quantized weight

  public:
    using Workspace = QuantizationWorkspace;
    Linear(RowScaledView weight, Type activation_type, TensorView bias = {});
    // Load-time quantization of one or several [N_i, K] 16-bit matrices fused by rows (Q,K,V -> QKV;
    // gate, up -> gate_up). Must run under an ExecutionScope; the kernels run on the context's stream.
    static Linear quantize(const std::vector<TensorView> &parts, Quantization mode, TensorView bias = {});

    Type activation_type() const { return activation_type_; }
    bool is_quantized() const { return true; }
    int input_channels() const { return weight_.values.cols; }
    int output_channels() const { return weight_.values.rows; }
    TensorView bias() const { return bias_; }
    RowScaledView weight() const { return weight_; }
    QuantizationGroups quantization_layout() const {
        return {weight_.group_size, weight_.group_size, weight_.rotation_size};
    }
    Workspace::Capacity workspace_capacity() const {
        return Workspace::Capacity::matrix(input_channels(), weight_.group_size);
    }
    // Plans for every row-capacity class up to max_rows (reference: src/layers/linear.cpp:132-148).
    void prepare_range(int max_rows, ops::Activation activation = ops::Activation::Identity) const;
    RowScaledView quantized_view(const Workspace &workspace, int rows) const;
    // Already-quantized activation -> output (no epilogue, no bias).
    void project(RowScaledView input, TensorView output) const;
    // Dense activation: quantize into the workspace, GEMM, bias + epilogue fused; with
    // quantized_output the finished rows are re-quantized for the next layer.
    void forward(Workspace &workspace, TensorView input, TensorView output, ops::Epilogue epilogue = {},
                 RowScaledView quantized_output = {}) const;
};
} // namespace tts
