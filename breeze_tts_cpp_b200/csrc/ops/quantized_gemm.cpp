#include "ops/quantized_gemm.h"
#include "kernels/quant_dispatch.h"
#include "kernels/sequence_pointwise.h"
#include "ops/epilogue.h"
#include "ops/quantization_policy.h"
#include "ops/sequence.h"
#include <map>
#include <tuple>

namespace tts {
namespace {
using PlanKey = std::tuple<int, int, int, Type, int, int>;
struct Plan {
    LinearPath path;
    int rows, channels, reduction;
    Type output_type;
    QuantizationGroups groups;
};
// reference: src/ops/cuda/quantization.cpp:94-102
void check_linear(Type format, const RowScaledView &input, const RowScaledView &weight, const TensorView &output,
                  int device) {
    input.validate();
    weight.validate();
    if (input.values.type != format || weight.values.type != format ||
        input.rotation_size != weight.rotation_size || input.values.cols != weight.values.cols ||
        input.values.rows != output.rows || weight.values.rows != output.cols ||
        (output.type != Type::BF16 && output.type != Type::F16) || !output.dense())
        throw std::invalid_argument("quantized linear dimensions/type mismatch");
    for (const TensorView *v : {&input.values, &input.scales, &weight.values, &weight.scales, &output})
        if (v->device != device) throw std::invalid_argument("quantized linear operand is on another device");
}
} // namespace

struct QuantizedGemm::Impl {
    cudaStream_t stream;
    Type format;
    Buffer &workspace;
    int multiprocessors = 0;
    bool sealed = false;
    std::map<PlanKey, Plan> plans;
    // TMA descriptors of the weight matrices announced before seal(), looked up by pointer at run time
    // (a few tree steps; weights that were never announced get their descriptor built per launch).
    std::map<const void *, WeightMaps> weight_maps;
    ChipModel chip;
    SelectionStats stats;

    const Plan *find(int rows, int channels, int reduction, Type type, int input_group, int weight_group) const {
        auto it = plans.find(PlanKey{row_capacity(rows), channels, reduction, type, input_group, weight_group});
        return it == plans.end() ? nullptr : &it->second;
    }
    void run(const Plan &plan, const RowScaledView &input, const RowScaledView &weight, const TensorView &output,
             const ops::Epilogue *finish) {
        const auto known = weight_maps.find(weight.values.data);
        launch_quant_linear(plan.path,
                            {output.rows, plan.channels, plan.reduction, plan.groups.activation, plan.groups.weight},
                            input.values.data, input.scales.ptr<float>(), weight.values.data,
                            weight.scales.ptr<float>(), output.data, workspace.data(), workspace.size(), stream,
                            format, plan.output_type, finish, known == weight_maps.end() ? nullptr : &known->second);
    }
};

QuantizedGemm::QuantizedGemm(cudaStream_t stream, void *, Buffer &workspace, Type format)
    : impl(new Impl{stream, format, workspace}) {
    if (format != Type::FP8 && format != Type::I8) throw std::invalid_argument("unsupported quantized storage type");
    quant_linear_initialize(workspace.device());
    cudaDeviceProp p{};
    if (cudaGetDeviceProperties(&p, workspace.device()) != cudaSuccess)
        throw std::runtime_error("cudaGetDeviceProperties failed");
    impl->multiprocessors = p.multiProcessorCount;
    impl->chip = ChipModel::b200(p.multiProcessorCount);
    quant_linear_reset_workspace(workspace.data(), workspace.size(), stream);
}
QuantizedGemm::~QuantizedGemm() = default;
void QuantizedGemm::seal() { impl->sealed = true; }
QuantCacheStats QuantizedGemm::cache_stats() const {
    QuantCacheStats s;
    s.selection = impl->stats;
    s.selection.entries = impl->plans.size();
    s.prepared_plans = impl->plans.size();
    return s;
}
void QuantizedGemm::prepare(int rows, int channels, int reduction, Type output_type, QuantizationGroups groups) {
    if (output_type != Type::BF16 && output_type != Type::F16)
        throw std::invalid_argument("quantized GEMM output must be F16 or BF16");
    if (rows < 1 || channels < 1 || reduction < 1 || reduction % 16 || channels % 16)
        throw std::invalid_argument("quantized GEMM unsupported shape");
    if (impl->format == Type::I8 && reduction > INT32_MAX / (128 * 128))
        throw std::invalid_argument("INT8 reduction can overflow INT32");
    rows = row_capacity(rows);
    PlanKey key{rows, channels, reduction, output_type, groups.activation, groups.weight};
    if (impl->plans.count(key)) {
        ++impl->stats.hits;
        return;
    }
    if (impl->sealed) throw std::logic_error("prepared resource missing after initialization");
    KernelProblem problem{rows, channels, reduction, groups.activation, groups.weight};
    Plan plan{select_linear(problem, KernelLimits{false, 0, impl->workspace.size()}, impl->format, impl->chip), rows,
              channels, reduction, output_type, groups};
    if (quant_linear_workspace_bytes(plan.path, problem) > impl->workspace.size())
        throw std::invalid_argument("quantized GEMM workspace too small for this shape");
    ++impl->stats.searches;
    impl->plans.emplace(key, plan);
}
void QuantizedGemm::prepare_weight(TensorView values) {
    if (!values.data || (values.type != Type::I8 && values.type != Type::FP8) || !values.dense()) return;
    if (impl->weight_maps.count(values.data)) return;
    if (impl->sealed) throw std::logic_error("prepared resource missing after initialization");
    impl->weight_maps.emplace(values.data, quant_linear_weight_maps(values.data, values.rows, values.cols));
}
void QuantizedGemm::prepare_finish(int rows, int channels, int reduction, Type output_type,
                                   const ops::Epilogue &finish, QuantizationGroups groups) {
    if (!ops::fusable(finish)) return;
    if (!impl->find(rows, channels, reduction, output_type, groups.activation, groups.weight))
        throw std::logic_error("quantized finish requires a prepared projection");
}
void QuantizedGemm::linear(RowScaledView input, RowScaledView weight, TensorView output) {
    check_linear(impl->format, input, weight, output, impl->workspace.device());
    const Plan *plan = impl->find(output.rows, output.cols, input.values.cols, output.type, input.group_size,
                                  weight.group_size);
    if (!plan) throw std::logic_error("quantized GEMM shape was not prepared before execution");
    impl->run(*plan, input, weight, output, nullptr);
}
bool QuantizedGemm::linear_finish(RowScaledView input, RowScaledView weight, TensorView output,
                                  const ops::Epilogue &finish) {
    if (!ops::fusable(finish)) return false;
    check_linear(impl->format, input, weight, output, impl->workspace.device());
    const Plan *plan = impl->find(output.rows, output.cols, input.values.cols, output.type, input.group_size,
                                  weight.group_size);
    if (!plan) return false;
    impl->run(*plan, input, weight, output, &finish);
    return true;
}
// reference: QuantizedGemm::normalized_linear (src/ops/cuda/quantization.cpp:479-494) in front of
// normalized_quantized_linear (src/ops/kernels/sequence/sequence_norm.cu:518-575): every condition
// under which that kernel declines returns false here too.
bool QuantizedGemm::normalized_linear(TensorView x, TensorView normalized, TensorView norm_weight, TensorView norm_bias,
                                      float epsilon, const ops::NormFusion &f, RowScaledView weight, TensorView output,
                                      const ops::Epilogue &e, RowScaledView encoded, const QkvProjectionOutput *writeback) {
    if (writeback || e.packed || e.condition_sources || e.output_rows || weight.group_size || encoded.group_size ||
        weight.rotation_size || encoded.rotation_size)
        return false;
    weight.validate();
    const int n = weight.values.rows, k = weight.values.cols;
    if (weight.values.type != impl->format || !x.data || !weight.values.data || !weight.scales.data || !output.data ||
        x.rows < 1 || x.rows > 65535 || n < 1 || k < 4 || k % 4 || reinterpret_cast<uintptr_t>(weight.values.data) % 4 ||
        k > 512 || x.cols != k || (x.type != Type::F16 && x.type != Type::BF16) || output.type != x.type ||
        output.rows != x.rows || output.cols != n || f.source_rows ||
        (normalized.data && (normalized.rows != x.rows || normalized.cols != k || normalized.type != x.type)) ||
        (e.activation != ops::Activation::Identity && e.activation != ops::Activation::Relu) || e.residual.data ||
        e.residual_f32.data || e.gate.data || e.condition.data || e.raw.data || e.residual_rows || e.input_repeat != 1 ||
        e.value_scale != 1 || e.output_scale != 1 || !(epsilon > 0))
        return false;
    for (const TensorView &source : {x, f.residual, f.projection_bias, f.gate, f.scale, f.shift, norm_weight, norm_bias,
                                     weight.values, weight.scales, e.bias})
        if (normalized.overlaps(source) || output.overlaps(source) || f.raw.overlaps(source)) return false;
    if (normalized.overlaps(output) || f.raw.overlaps(output) || f.raw.overlaps(normalized)) return false;
    auto vector_of = [&](const TensorView &v) { return !v.data || (v.type == x.type && v.numel() == size_t(k)); };
    auto rows_of = [&](const TensorView &v) { return !v.data || (v.type == x.type && v.rows == x.rows && v.cols == k); };
    if (!vector_of(norm_weight) || !vector_of(norm_bias) || !vector_of(f.projection_bias) || !rows_of(f.residual) ||
        !rows_of(f.raw) || f.rows_per_sequence < 1 || x.rows % f.rows_per_sequence)
        throw std::invalid_argument("sequence operation shape/type mismatch");
    for (const TensorView *v : {&f.gate, &f.shift, &f.scale})
        if (v->data && (v->type != x.type || v->cols != k || (v->rows != 1 && v->rows != x.rows / f.rows_per_sequence)))
            throw std::invalid_argument("invalid normalization modulation");
    if (e.bias.data && (e.bias.type != x.type || e.bias.numel() != size_t(n)))
        throw std::invalid_argument("sequence operation shape/type mismatch");
    if (e.rows_per_sequence < 1 || x.rows % e.rows_per_sequence || e.valid_rows_per_sequence < 0 ||
        e.valid_rows_per_sequence > e.rows_per_sequence)
        throw std::invalid_argument("invalid epilogue sequence length");
    if (encoded.values.data || encoded.scales.data) {
        encoded.validate();
        if (encoded.values.type != weight.values.type || encoded.values.rows != x.rows || encoded.values.cols != k)
            throw std::invalid_argument("normalized projection quantized output mismatch");
        for (const TensorView &source : {x, normalized, norm_weight, norm_bias, f.residual, f.projection_bias, f.raw, f.gate,
                                         f.shift, f.scale, weight.values, weight.scales, output, e.bias})
            if (encoded.values.overlaps(source) || encoded.scales.overlaps(source))
                throw std::invalid_argument("quantized output overlaps sequence storage");
    }
    launch_normalized_quantized_linear(x, normalized, norm_weight, norm_bias, epsilon, f, weight, output, e, encoded,
                                       impl->stream);
    return true;
}
LinearPath QuantizedGemm::planned_path(int rows, int channels, int reduction, Type output_type,
                                       QuantizationGroups groups) const {
    const Plan *plan = impl->find(rows, channels, reduction, output_type, groups.activation, groups.weight);
    if (!plan) throw std::logic_error("quantized GEMM shape was not prepared before execution");
    return plan->path;
}
int QuantizedGemm::status() const { return quant_linear_status(impl->workspace.data(), impl->stream); }
} // namespace tts
