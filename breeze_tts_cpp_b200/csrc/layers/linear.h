// Quantized Linear layer: holds a RowScaledView weight (+ optional bias) and runs
// quantize -> GEMM -> fused epilogue through the op layer. Public methods follow the reference's
// `tts::Linear` (src/layers/linear.h:11-76) for the quantized case; construction from a checkpoint
// (`Weights`) is the reference engine's own and is replaced here by `Linear::quantize`, which
// performs the load-time step of `Weights::quantized`
// (src/io/weights.cpp:80-87,133-154): concatenate the source matrices by rows and quantize them
// on the device into storage the layer owns.
#pragma once
#include "core/buffer.h"
#include "core/forward_context.h"
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
    void project(Workspace &workspace, TensorView input, TensorView output) const; // no bias, no epilogue

    // Phase-switched calls (reference: src/layers/linear.cpp:49-88): Prepare plans every row class up to
    // context.max_rows and sizes the layer's own activation scratch; Execute runs; Plan and Capture
    // launch nothing. The first form takes its output from the context's scratch arena.
    TensorView forward(TensorView input, ForwardContext &context, const ops::Epilogue &finish = {}) const;
    TensorView forward(TensorView input, TensorView output, ForwardContext &context, const ops::Epilogue &finish = {}) const;
    TensorView project(TensorView input, TensorView output, ForwardContext &context) const;
    // `segments` is a host I32 [S, 3] list of (first input row, row count, first output row); zero
    // segments or one contiguous cover runs the whole batch at once (reference: linear.cpp:89-121).
    TensorView forward_segments(TensorView input, TensorView segments, TensorView output, ForwardContext &context) const;

    // LayerNorm of the input fused with its quantization into the workspace (reference: linear.cpp:177-185).
    RowScaledView normalize_input(Workspace &workspace, TensorView input, TensorView norm_weight, TensorView norm_bias,
                                  float epsilon, const ops::NormFusion &fusion, TensorView retained = {}) const;
    // LayerNorm + projection: one fused launch when the shape allows it, else normalize_input followed
    // by the projection (reference: linear.cpp:195-214). Always true for a quantized layer without write-back.
    bool normalized_forward(Workspace &workspace, TensorView input, TensorView normalized, TensorView output,
                            TensorView norm_weight, TensorView norm_bias, float epsilon, const ops::NormFusion &fusion,
                            ops::Epilogue epilogue = {}, const QkvProjectionOutput *writeback = nullptr,
                            RowScaledView quantized_output = {}) const;

  private:
    TensorView apply_context(TensorView input, TensorView output, ForwardContext &context, TensorView bias,
                             const ops::Epilogue &finish) const;
    void validate_types(TensorView input, TensorView output) const;
    Workspace &context_workspace(const ForwardContext &context) const;
    mutable std::shared_ptr<Workspace> context_workspace_; // made in Prepare, reused by every Execute
    mutable int context_rows_ = 0;
};
} // namespace tts
