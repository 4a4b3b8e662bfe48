#include "layers/linear.h"
#include "ops/context.h"

namespace tts {
Linear::Linear(RowScaledView weight, Type activation_type, TensorView bias)
    : weight_(weight), bias_(bias), activation_type_(activation_type) {
    weight_.validate();
    if (activation_type != Type::BF16 && activation_type != Type::F16)
        throw std::invalid_argument("quantized Linear activations must be F16 or BF16");
    if (bias.data && (bias.type != activation_type || bias.numel() != size_t(weight.values.rows)))
        throw std::invalid_argument("Linear bias mismatch");
}

Linear Linear::quantize(const std::vector<TensorView> &parts, Quantization mode, TensorView bias) {
    if (parts.empty()) throw std::invalid_argument("Linear::quantize needs at least one matrix");
    const int columns = parts.front().cols;
    const Type source_type = parts.front().type;
    int rows = 0;
    for (const auto &p : parts) {
        if (p.cols != columns || p.type != source_type || !p.data) throw std::invalid_argument("fused Linear parts differ in K or dtype");
        rows += p.rows;
    }
    const auto groups = quantization_groups(mode);
    const Type format = quantized_type(mode);
    const int device = parts.front().device;
    auto shape = quantization_scale_shape(rows, columns, groups.weight);
    auto values = std::make_shared<Buffer>(size_t(rows) * columns);
    auto scales = std::make_shared<Buffer>(shape.numel() * sizeof(float));
    RowScaledView whole{values->view(rows, columns, format), scales->view(shape.rows, shape.cols, Type::F32),
                        groups.weight, groups.rotation};
    if (parts.size() == 1 || !groups.weight) {
        // Per-row scales: each part fills its own row range of values and scales.
        int first = 0;
        for (const auto &p : parts) {
            RowScaledView slice{whole.values.slice(first, p.rows),
                                groups.weight ? whole.scales : whole.scales.slice(first, p.rows), groups.weight,
                                groups.rotation};
            ops::quantize_rows(p, slice);
            first += p.rows;
        }
    } else {
        // K-group scales are group-major over all N rows, so the parts are first gathered into one
        // contiguous 16-bit matrix (load time only) and quantized in a single pass.
        auto &gpu = execution_context(device);
        Buffer gathered(size_t(rows) * columns * bytes(source_type));
        size_t offset = 0;
        for (const auto &p : parts) {
            if (!p.dense()) throw std::invalid_argument("fused K-group parts must be dense");
            if (cudaMemcpyAsync(static_cast<char *>(gathered.data()) + offset, p.data, p.size(), cudaMemcpyDeviceToDevice,
                                gpu.stream) != cudaSuccess)
                throw std::runtime_error("gathering fused weight parts failed");
            offset += p.size();
        }
        ops::quantize_rows(gathered.view(rows, columns, source_type), whole);
    }
    // The GEMM prefetches weight tiles and weight scales ahead of its wait on the preceding kernel,
    // so a weight must be complete on the device before the first GEMM that uses it is enqueued.
    if (cudaStreamSynchronize(execution_context(device).stream) != cudaSuccess)
        throw std::runtime_error("weight quantization failed");
    Linear layer(whole, source_type, bias);
    layer.values_ = values;
    layer.scales_ = scales;
    return layer;
}

void Linear::prepare_range(int max_rows, ops::Activation activation) const {
    if (max_rows < 1) throw std::invalid_argument("Linear::prepare_range needs a positive row bound");
    ops::Epilogue finish;
    finish.activation = activation;
    const auto layout = quantization_layout();
    // One plan per capacity class: walk the classes upward until max_rows is covered.
    for (int rows = 1;;) {
        const int capacity = row_capacity(rows);
        ops::prepare_quantized(weight_.values, capacity, output_channels(), input_channels(), activation_type_, finish,
                               layout);
        if (capacity >= max_rows) break;
        rows = capacity + 1;
    }
}

RowScaledView Linear::quantized_view(const Workspace &workspace, int rows) const {
    return workspace.view(rows, input_channels(), weight_.values.type, quantization_layout());
}

void Linear::project(RowScaledView input, TensorView output) const { ops::matmul(input, weight_, output); }

void Linear::validate_types(TensorView input, TensorView output) const {
    if (input.type != activation_type_ || output.type != activation_type_)
        throw std::invalid_argument("linear activation dtype mismatch");
}

void Linear::forward(Workspace &workspace, TensorView input, TensorView output, ops::Epilogue epilogue,
                     RowScaledView quantized_output) const {
    if (input.type != activation_type_ || output.type != activation_type_ || input.cols != input_channels() ||
        output.cols != output_channels() || input.rows != output.rows)
        throw std::invalid_argument("Linear activation shape/type mismatch");
    ops::linear(input, weight_, bias_, output, epilogue, quantized_view(workspace, input.rows), quantized_output);
}

void Linear::project(Workspace &workspace, TensorView input, TensorView output) const {
    validate_types(input, output);
    ops::linear(input, weight_, {}, output, {}, quantized_view(workspace, input.rows));
}

Linear::Workspace &Linear::context_workspace(const ForwardContext &context) const {
    if (!context_workspace_ || context_rows_ < context.max_rows) {
        if (context.mode != ForwardContext::Prepare)
            throw std::logic_error("linear was not prepared for this many rows before execution");
        context_workspace_ = std::make_shared<Workspace>(context.max_rows, workspace_capacity());
        context_rows_ = context.max_rows;
    }
    return *context_workspace_;
}

TensorView Linear::apply_context(TensorView input, TensorView output, ForwardContext &context, TensorView bias,
                                 const ops::Epilogue &finish) const {
    validate_types(input, output);
    if (input.rows < 1 || input.rows > context.max_rows || input.cols != input_channels() || output.rows != input.rows ||
        output.cols != output_channels())
        throw std::invalid_argument("linear input shape/type");
    if (context.mode == ForwardContext::Prepare) {
        context_workspace(context);
        if (input.data && output.data) prepare_range(context.max_rows, finish.activation);
    } else if (context.mode == ForwardContext::Execute) {
        ops::linear(input, weight_, bias, output, finish, quantized_view(context_workspace(context), input.rows));
    }
    return output;
}

TensorView Linear::forward(TensorView input, ForwardContext &context, const ops::Epilogue &finish) const {
    TensorView output = context.tensor({context.max_rows, output_channels()}, activation_type_).slice(0, input.rows);
    return forward(input, output, context, finish);
}
TensorView Linear::forward(TensorView input, TensorView output, ForwardContext &context, const ops::Epilogue &finish) const {
    return apply_context(input, output, context, bias_, finish);
}
TensorView Linear::project(TensorView input, TensorView output, ForwardContext &context) const {
    return apply_context(input, output, context, {}, {});
}

TensorView Linear::forward_segments(TensorView input, TensorView segments, TensorView output, ForwardContext &context) const {
    if (context.mode == ForwardContext::Plan || context.mode == ForwardContext::Capture) return output;
    if (context.mode == ForwardContext::Prepare) {
        context_workspace(context);
        if (input.data && output.data) prepare_range(context.max_rows);
        return output;
    }
    if (segments.device != -1 || segments.type != Type::I32 || segments.cols != 3)
        throw std::invalid_argument("projection segments must contain host I32 row ranges");
    Workspace &workspace = context_workspace(context);
    int contiguous_rows = 0;
    for (int index = 0; index < segments.rows; ++index) {
        const int *range = segments.ptr<int>() + size_t(index) * segments.ld();
        if (range[0] != contiguous_rows || range[2] != contiguous_rows) break;
        contiguous_rows += range[1];
    }
    if (!segments.rows || (contiguous_rows == input.rows && output.rows == input.rows)) {
        forward(workspace, input, output);
        return output;
    }
    for (int index = 0; index < segments.rows; ++index) {
        const int *range = segments.ptr<int>() + size_t(index) * segments.ld();
        forward(workspace, input.slice(range[0], range[1]), output.slice(range[2], range[1]));
    }
    return output;
}

RowScaledView Linear::normalize_input(Workspace &workspace, TensorView input, TensorView norm_weight, TensorView norm_bias,
                                      float epsilon, const ops::NormFusion &fusion, TensorView retained) const {
    if (input.type != activation_type_ || input.cols != input_channels())
        throw std::invalid_argument("linear normalization input mismatch");
    RowScaledView output = quantized_view(workspace, input.rows);
    ops::layer_norm_quantize(input, output, norm_weight, norm_bias, epsilon, fusion, retained);
    return output;
}

bool Linear::normalized_forward(Workspace &workspace, TensorView input, TensorView normalized, TensorView output,
                                TensorView norm_weight, TensorView norm_bias, float epsilon, const ops::NormFusion &fusion,
                                ops::Epilogue epilogue, const QkvProjectionOutput *writeback,
                                RowScaledView quantized_output) const {
    validate_types(input, output);
    if (writeback) return false;
    if (ops::normalized_linear(input, weight_, bias_, normalized, output, norm_weight, norm_bias, epsilon, fusion, epilogue,
                               nullptr, quantized_output))
        return true;
    RowScaledView normalized_input = normalize_input(workspace, input, norm_weight, norm_bias, epsilon, fusion, normalized);
    ops::linear(normalized_input, weight_, bias_, output, epilogue, {}, quantized_output);
    return true;
}
} // namespace tts
