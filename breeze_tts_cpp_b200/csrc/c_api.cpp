// extern "C" edge of the library: POD structs in, status code + message out. Exceptions never
// cross this boundary (same convention as the reference's bindings/c_api.cpp:25-40).
#include "b200q.h"
#include "c_api_convert.h"
#include "kernels/quant_dispatch.h"
#include "ops/context.h"
#include "ops/ops.h"
#include "layers/linear.h"
#include "ops/quantization_policy.h"
#include <vector>
#include <cstdio>
#include <cstring>
#include <exception>
#include <memory>

struct b200q_context {
    std::unique_ptr<tts::CudaContext> gpu;
};
struct b200q_linear_layer {
    std::unique_ptr<tts::Linear> layer;
    std::unique_ptr<tts::QuantizationWorkspace> scratch;
    int max_rows = 0;
};

namespace {
using namespace tts;
void copy_error(char *error, size_t capacity, const char *message) {
    if (error && capacity) std::snprintf(error, capacity, "%s", message);
}
template <class Body> int guarded(char *error, size_t capacity, Body &&body) {
    try {
        body();
        if (error && capacity) error[0] = 0;
        return 0;
    } catch (const std::exception &e) {
        copy_error(error, capacity, e.what());
    } catch (...) {
        copy_error(error, capacity, "unknown error");
    }
    return -1;
}
CudaContext &context_of(b200q_context *c) {
    if (!c || !c->gpu) throw std::invalid_argument("null b200q context");
    return *c->gpu;
}
using capi::epilogue_of;
using capi::fusion_of;
using capi::scaled_of;
using capi::type_of;
using capi::view_of;
void put_path(b200q_path *out, LinearPath p) {
    if (out) *out = {int32_t(p.kind), p.tokens, p.channels, p.splits};
}
} // namespace

extern "C" {
const char *b200q_version(void) { return "b200q 0.1 sm_100a; quantization=int8,fp8,group_int8,group_fp8"; }

int b200q_context_create(int32_t device, void *stream, void *workspace, size_t workspace_bytes,
                         const char *quantization, b200q_context **out, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        if (!out) throw std::invalid_argument("null output handle");
        auto mode = quantization_from_string(quantization ? quantization : "");
        if (mode == Quantization::None) throw std::invalid_argument("quantization must be int8, fp8, group_int8 or group_fp8");
        auto holder = std::make_unique<b200q_context>();
        holder->gpu = std::make_unique<CudaContext>(device, mode, static_cast<cudaStream_t>(stream), workspace, workspace_bytes);
        *out = holder.release();
    });
}
void b200q_context_destroy(b200q_context *c) { delete c; }

int b200q_row_quantize(b200q_context *c, const b200q_tensor *source, const b200q_row_scaled *destination,
                       char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        ops::quantize_rows(view_of(source), scaled_of(destination));
    });
}
int b200q_quantized_norm(b200q_context *c, const b200q_tensor *residual, const b200q_tensor *update,
                         const b200q_tensor *weight, const b200q_row_scaled *output, float epsilon, int32_t gemma,
                         const b200q_tensor *update_scale, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        ops::quantized_norm(view_of(residual), view_of(update), view_of(weight), scaled_of(output), epsilon,
                            gemma != 0, view_of(update_scale));
    });
}
int b200q_quantized_gated(b200q_context *c, const b200q_tensor *input, const b200q_row_scaled *output, int32_t kind,
                          char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        ops::quantized_gated(view_of(input), scaled_of(output), kind);
    });
}
int b200q_prepare(b200q_context *c, int32_t rows, int32_t channels, int32_t reduction, int32_t output_type,
                  int32_t activation_group, int32_t weight_group, b200q_path *chosen, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        auto &gpu = context_of(c);
        ExecutionScope scope(gpu);
        QuantizationGroups groups{activation_group, weight_group, 0};
        gpu.quantization->prepare(rows, channels, reduction, type_of(output_type), groups);
        put_path(chosen, gpu.quantization->planned_path(rows, channels, reduction, type_of(output_type), groups));
    });
}
int b200q_prepare_weight(b200q_context *c, const b200q_row_scaled *weight, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        auto &gpu = context_of(c);
        ExecutionScope scope(gpu);
        auto w = scaled_of(weight);
        w.validate();
        if (w.values.device != gpu.device) throw std::invalid_argument("operand is not on the context's device");
        gpu.quantization->prepare_weight(w.values);
    });
}
int b200q_seal(b200q_context *c, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        auto &gpu = context_of(c);
        ExecutionScope scope(gpu);
        ops::seal(gpu.device);
    });
}
int b200q_linear(b200q_context *c, const b200q_row_scaled *input, const b200q_row_scaled *weight,
                 const b200q_tensor *output, const b200q_epilogue *epilogue, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        auto &gpu = context_of(c);
        ExecutionScope scope(gpu);
        if (!epilogue) {
            ops::matmul(scaled_of(input), scaled_of(weight), view_of(output));
            return;
        }
        auto e = epilogue_of(epilogue);
        if (!gpu.quantization->linear_finish(scaled_of(input), scaled_of(weight), view_of(output), e))
            throw std::invalid_argument("epilogue cannot be fused, or the shape was not prepared");
    });
}
int b200q_quant_linear(b200q_context *c, const b200q_path *path, const b200q_row_scaled *input,
                       const b200q_row_scaled *weight, const b200q_tensor *output, const b200q_epilogue *epilogue,
                       char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        auto &gpu = context_of(c);
        ExecutionScope scope(gpu);
        if (!path) throw std::invalid_argument("null path");
        auto x = scaled_of(input), w = scaled_of(weight);
        auto y = view_of(output);
        x.validate();
        w.validate();
        if (x.values.type != w.values.type || x.values.cols != w.values.cols || x.rotation_size != w.rotation_size ||
            y.rows != x.values.rows || y.cols != w.values.rows || !y.dense() || !y.data)
            throw std::invalid_argument("quantized linear dimensions/type mismatch");
        for (const TensorView *v : {&x.values, &x.scales, &w.values, &w.scales, &y})
            if (v->device != gpu.device) throw std::invalid_argument("operand is not on the context's device");
        ops::Epilogue e = epilogue_of(epilogue);
        launch_quant_linear({static_cast<LinearKind>(path->kind), path->tokens, path->channels, path->splits},
                            {y.rows, y.cols, x.values.cols, x.group_size, w.group_size}, x.values.data,
                            x.scales.ptr<float>(), w.values.data, w.scales.ptr<float>(), y.data,
                            gpu.gemm_workspace.data(), gpu.gemm_workspace.size(), gpu.stream, x.values.type, y.type,
                            epilogue ? &e : nullptr);
    });
}
int b200q_select_path(b200q_context *c, int32_t rows, int32_t channels, int32_t reduction, int32_t activation_group,
                      int32_t weight_group, b200q_path *chosen, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        auto &gpu = context_of(c);
        put_path(chosen, select_tcgen05_path({rows, channels, reduction, activation_group, weight_group},
                                             quantized_type(gpu.mode), gpu.multiprocessors, gpu.gemm_workspace.size()));
    });
}
int b200q_linear_forward(b200q_context *c, const b200q_tensor *input, const b200q_row_scaled *weight,
                         const b200q_row_scaled *scratch, const b200q_tensor *output, const b200q_epilogue *epilogue,
                         const b200q_row_scaled *quantized_output, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        ops::Epilogue e = epilogue_of(epilogue);
        TensorView bias = e.bias;
        e.bias = {};
        ops::linear(view_of(input), scaled_of(weight), bias, view_of(output), e, scaled_of(scratch),
                    quantized_output ? scaled_of(quantized_output) : RowScaledView{});
    });
}
int b200q_pointwise(b200q_context *c, const b200q_tensor *x, const b200q_tensor *y, const b200q_epilogue *epilogue,
                    char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        ops::pointwise(view_of(x), view_of(y), epilogue_of(epilogue));
    });
}
int b200q_pointwise_quantize(b200q_context *c, const b200q_tensor *x, const b200q_row_scaled *quantized,
                             const b200q_epilogue *epilogue, const b200q_tensor *retained, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        ops::pointwise_quantize(view_of(x), scaled_of(quantized), epilogue_of(epilogue), view_of(retained));
    });
}
int b200q_layer_norm_quantize(b200q_context *c, const b200q_tensor *x, const b200q_row_scaled *quantized,
                              const b200q_tensor *weight, const b200q_tensor *bias, float epsilon,
                              const b200q_norm_fusion *fusion, const b200q_tensor *retained, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        ops::layer_norm_quantize(view_of(x), scaled_of(quantized), view_of(weight), view_of(bias), epsilon,
                                 fusion_of(fusion), view_of(retained));
    });
}
int b200q_normalized_linear(b200q_context *c, const b200q_tensor *input, const b200q_row_scaled *weight,
                            const b200q_tensor *bias, const b200q_tensor *normalized, const b200q_tensor *output,
                            const b200q_tensor *norm_weight, const b200q_tensor *norm_bias, float epsilon,
                            const b200q_norm_fusion *fusion, const b200q_epilogue *epilogue,
                            const b200q_row_scaled *quantized_output, int32_t *taken, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        ops::Epilogue e = epilogue_of(epilogue);
        if (e.bias.data) throw std::invalid_argument("linear already owns its bias");
        const bool done = ops::normalized_linear(view_of(input), scaled_of(weight), view_of(bias), view_of(normalized),
                                                 view_of(output), view_of(norm_weight), view_of(norm_bias), epsilon,
                                                 fusion_of(fusion), e, nullptr,
                                                 quantized_output ? scaled_of(quantized_output) : RowScaledView{});
        if (taken) *taken = done ? 1 : 0;
    });
}
int b200q_linear_layer_create(b200q_context *c, const b200q_tensor *parts, int32_t part_count, const b200q_tensor *bias,
                              b200q_linear_layer **out, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        auto &gpu = context_of(c);
        ExecutionScope scope(gpu);
        if (!out || !parts || part_count < 1) throw std::invalid_argument("invalid layer arguments");
        std::vector<TensorView> views;
        for (int i = 0; i < part_count; ++i) views.push_back(view_of(parts + i));
        auto holder = std::make_unique<b200q_linear_layer>();
        holder->layer = std::make_unique<Linear>(Linear::quantize(views, gpu.mode, view_of(bias)));
        *out = holder.release();
    });
}
void b200q_linear_layer_destroy(b200q_linear_layer *l) { delete l; }
int b200q_linear_layer_prepare(b200q_context *c, b200q_linear_layer *l, int32_t max_rows, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        if (!l || !l->layer) throw std::invalid_argument("null layer");
        l->layer->prepare_range(max_rows);
        l->scratch = std::make_unique<QuantizationWorkspace>(max_rows, l->layer->workspace_capacity());
        l->max_rows = max_rows;
    });
}
int b200q_linear_layer_forward(b200q_context *c, b200q_linear_layer *l, const b200q_tensor *input, const b200q_tensor *output,
                               const b200q_epilogue *epilogue, const b200q_row_scaled *quantized_output, char *error,
                               size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        if (!l || !l->layer) throw std::invalid_argument("null layer");
        if (!l->scratch) throw std::logic_error("layer was not prepared before execution");
        ops::Epilogue e = epilogue_of(epilogue);
        if (e.bias.data) throw std::invalid_argument("linear already owns its bias");
        l->layer->forward(*l->scratch, view_of(input), view_of(output), e,
                          quantized_output ? scaled_of(quantized_output) : RowScaledView{});
    });
}
int b200q_linear_layer_apply(b200q_context *c, b200q_linear_layer *l, int32_t mode, int32_t max_rows, const b200q_tensor *input,
                             const b200q_tensor *output, const b200q_epilogue *epilogue, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        if (!l || !l->layer) throw std::invalid_argument("null layer");
        if (mode < 0 || mode > int(ForwardContext::Execute) || max_rows < 1) throw std::invalid_argument("invalid forward phase");
        ForwardContext context(1, max_rows, max_rows);
        context.mode = static_cast<ForwardContext::Mode>(mode);
        ops::Epilogue e = epilogue_of(epilogue);
        if (e.bias.data) throw std::invalid_argument("linear already owns its bias");
        l->layer->forward(view_of(input), view_of(output), context, e);
    });
}
int b200q_linear_layer_forward_segments(b200q_context *c, b200q_linear_layer *l, int32_t mode, int32_t max_rows,
                                        const b200q_tensor *input, const int32_t *segments, int32_t segment_count,
                                        const b200q_tensor *output, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        if (!l || !l->layer) throw std::invalid_argument("null layer");
        if (mode < 0 || mode > int(ForwardContext::Execute) || max_rows < 1 || segment_count < 0 || (segment_count && !segments))
            throw std::invalid_argument("invalid forward phase or segments");
        ForwardContext context(1, max_rows, max_rows);
        context.mode = static_cast<ForwardContext::Mode>(mode);
        TensorView ranges = segment_count ? TensorView(const_cast<int32_t *>(segments), segment_count, 3, Type::I32, 0, -1)
                                          : TensorView::metadata(0, 3, Type::I32, 0, -1);
        l->layer->forward_segments(view_of(input), ranges, view_of(output), context);
    });
}
int b200q_linear_layer_normalized_forward(b200q_context *c, b200q_linear_layer *l, const b200q_tensor *input,
                                          const b200q_tensor *normalized, const b200q_tensor *output,
                                          const b200q_tensor *norm_weight, const b200q_tensor *norm_bias, float epsilon,
                                          const b200q_norm_fusion *fusion, const b200q_epilogue *epilogue,
                                          const b200q_row_scaled *quantized_output, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        ExecutionScope scope(context_of(c));
        if (!l || !l->layer) throw std::invalid_argument("null layer");
        if (!l->scratch) throw std::logic_error("layer was not prepared before execution");
        ops::Epilogue e = epilogue_of(epilogue);
        if (e.bias.data) throw std::invalid_argument("linear already owns its bias");
        l->layer->normalized_forward(*l->scratch, view_of(input), view_of(normalized), view_of(output), view_of(norm_weight),
                                     view_of(norm_bias), epsilon, fusion_of(fusion), e, nullptr,
                                     quantized_output ? scaled_of(quantized_output) : RowScaledView{});
    });
}
int b200q_linear_layer_weight(b200q_linear_layer *l, b200q_row_scaled *weight, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        if (!l || !l->layer || !weight) throw std::invalid_argument("null layer");
        auto w = l->layer->weight();
        auto put = [](const TensorView &v) { return b200q_tensor{v.data, v.rows, v.cols, v.stride, int32_t(v.type), v.device}; };
        *weight = {put(w.values), put(w.scales), w.group_size, w.rotation_size};
    });
}
int b200q_inject_wait_expiry(int32_t extra_bytes, int64_t limit_cycles, char *error, size_t capacity) {
    return guarded(error, capacity, [&] { quant_linear_inject_wait_expiry(extra_bytes, limit_cycles); });
}
int b200q_status(b200q_context *c, int32_t *status, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        auto &gpu = context_of(c);
        ExecutionScope scope(gpu);
        int value = gpu.quantization->status();
        if (status) *status = value;
    });
}
int b200q_multiprocessors(b200q_context *c) { return c && c->gpu ? c->gpu->multiprocessors : 0; }
int32_t b200q_row_capacity(int32_t rows, uint32_t bins_per_octave) {
    try {
        return row_capacity(rows, bins_per_octave);
    } catch (...) {
        return -1;
    }
}
int b200q_plan_path(int32_t rows, int32_t channels, int32_t reduction, int32_t activation_group, int32_t weight_group,
                    int32_t format, int32_t multiprocessors, size_t workspace_bytes, b200q_path *chosen,
                    size_t *workspace_needed, char *error, size_t capacity) {
    return guarded(error, capacity, [&] {
        if (rows < 1 || channels < 1 || reduction < 1 || reduction % 16 || channels % 16)
            throw std::invalid_argument("quantized GEMM unsupported shape");
        KernelProblem problem{rows, channels, reduction, activation_group, weight_group};
        LinearPath path = select_tcgen05_path(problem, type_of(format), multiprocessors, workspace_bytes);
        put_path(chosen, path);
        if (workspace_needed) *workspace_needed = quant_linear_workspace_bytes(path, problem);
    });
}
int b200q_candidates(int32_t rows, int32_t channels, int32_t reduction, int32_t activation_group, int32_t weight_group,
                     int32_t format, b200q_path *paths, int32_t capacity, char *error, size_t error_capacity) {
    int count = -1;
    guarded(error, error_capacity, [&] {
        auto found = quant_linear_candidates({rows, channels, reduction, activation_group, weight_group}, {}, type_of(format));
        for (size_t i = 0; i < found.size() && int(i) < capacity; ++i) put_path(paths ? paths + i : nullptr, found[i]);
        count = int(found.size());
    });
    return count;
}
double b200q_path_cost(int32_t rows, int32_t channels, int32_t reduction, int32_t activation_group, int32_t weight_group,
                       int32_t format, const b200q_path *path, int32_t multiprocessors, int32_t gemm_only, char *error,
                       size_t error_capacity) {
    double cost = -1;
    guarded(error, error_capacity, [&] {
        if (!path) throw std::invalid_argument("null path");
        KernelProblem problem{rows, channels, reduction, activation_group, weight_group};
        LinearPath p{static_cast<LinearKind>(path->kind), path->tokens, path->channels, path->splits};
        const ChipModel chip = ChipModel::b200(multiprocessors);
        cost = gemm_only ? linear_cost(problem, p, type_of(format), chip)
                         : linear_pipeline_cost(problem, p, type_of(format), chip, {}, true);
    });
    return cost;
}
}
