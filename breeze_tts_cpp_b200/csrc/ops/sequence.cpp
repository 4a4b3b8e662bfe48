// Host side of the row-wise operators: argument validation in the reference's terms, then the launch.
// The checks restate the reference's (src/ops/kernels/sequence/sequence_internal.cuh:140-219,
// sequence_pointwise.cu:283-326, sequence_norm.cu:371-428); error texts are kept so callers that match
// on them keep working.
#include "ops/sequence.h"
#include "kernels/sequence_pointwise.h"
#include "ops/context.h"
#include <cmath>
#include <initializer_list>

namespace tts::ops {
namespace {
void same_shape(const TensorView &v, TensorShape target, Type type, bool vector = false) {
    if (!v.data) return;
    const bool shape_ok = vector ? v.numel() == size_t(target.cols) : v.rows == target.rows && v.cols == target.cols;
    if (v.type != type || !shape_ok) throw std::invalid_argument("sequence operation shape/type mismatch");
}
void check_row_output(const TensorView &out) {
    if (!out.data || !out.rows || !out.cols || (out.type != Type::BF16 && out.type != Type::F16))
        throw std::invalid_argument("sequence operation requires nonempty F16/BF16 output");
}
void reject_indirect(const Epilogue &e, const char *what) {
    if (e.packed || e.condition_sources || e.output_rows) throw std::invalid_argument(what);
}
void check_epilogue(const Epilogue &e, TensorShape out, Type type) {
    same_shape(e.bias, out, type, true);
    if (e.residual_rows) {
        if (!e.residual.data || e.residual.type != type || e.residual.cols != out.cols)
            throw std::invalid_argument("invalid indexed residual");
    } else {
        same_shape(e.residual, out, type);
    }
    same_shape(e.raw, out, type);
    if (e.residual_f32.data) throw std::invalid_argument("the fp32 residual exists only inside the GEMM epilogue");
    if (e.rows_per_sequence < 1 || out.rows % e.rows_per_sequence || e.valid_rows_per_sequence < 0 ||
        e.valid_rows_per_sequence > e.rows_per_sequence)
        throw std::invalid_argument("invalid epilogue sequence length");
    const int sequences = out.rows / e.rows_per_sequence;
    for (const TensorView *v : {&e.gate, &e.condition})
        if (v->data && (v->type != type || v->cols != out.cols || (v->rows != 1 && v->rows != sequences)))
            throw std::invalid_argument(v == &e.gate ? "invalid epilogue gate" : "invalid epilogue condition");
}
TensorShape check_quantized_output(const TensorView &x, const RowScaledView &q, const TensorView &retained) {
    q.validate();
    if (q.rotation_size && !q.group_size) throw std::invalid_argument("rotated sequence fusion requires group scales");
    if (!q.values.data || !q.scales.data || q.values.rows < 1 || q.values.cols < 1 ||
        (x.type != Type::F16 && x.type != Type::BF16))
        throw std::invalid_argument("quantized sequence output requires F16/BF16 input");
    if (retained.data) {
        check_row_output(retained);
        same_shape(retained, TensorShape(q.values), x.type);
    }
    if (q.values.overlaps(q.scales)) throw std::invalid_argument("quantized values/scales overlap");
    return TensorShape(q.values);
}
void check_quantized_aliases(const RowScaledView &q, std::initializer_list<TensorView> sources) {
    for (const auto &source : sources)
        if (q.values.overlaps(source) || q.scales.overlaps(source))
            throw std::invalid_argument("quantized output overlaps sequence storage");
}
// A row kernel may overwrite an input row once it has consumed it; broadcast, indexed, repeated or
// partially overlapping rows cannot be updated in place.
void check_row_alias(const TensorView &output, const TensorView &source, bool same_rows) {
    if (output.overlaps(source) && (!same_rows || output.data != source.data || output.rows != source.rows ||
                                    output.cols != source.cols || output.ld() != source.ld()))
        throw std::invalid_argument("quantized sequence output has unsafe row alias");
}
void check_retained_raw(const TensorView &retained, const TensorView &raw, std::initializer_list<TensorView> broadcast) {
    if (retained.overlaps(raw)) throw std::invalid_argument("raw and retained sequence outputs overlap");
    for (const auto &source : broadcast) {
        check_row_alias(retained, source, false);
        check_row_alias(raw, source, false);
    }
}
void check_norm_shape(const TensorView &x, TensorShape y, Type type, const void *retained, const TensorView &w,
                      const TensorView &bias, float eps, const NormFusion &f) {
    same_shape(w, y, type, true);
    same_shape(bias, y, type, true);
    if (f.source_rows) {
        if (x.type != type || x.cols != y.cols || x.data == retained || f.gate.data || f.shift.data || f.scale.data)
            throw std::invalid_argument("invalid indexed normalization");
    } else {
        same_shape(x, y, type);
    }
    same_shape(f.residual, TensorShape(x), x.type);
    same_shape(f.projection_bias, y, type, true);
    same_shape(f.raw, y, type);
    if (f.rows_per_sequence < 1 || y.rows % f.rows_per_sequence)
        throw std::invalid_argument("invalid normalization sequence length");
    for (const TensorView *v : {&f.gate, &f.shift, &f.scale})
        if (v->data && (v->type != type || v->cols != y.cols || (v->rows != 1 && v->rows != y.rows / f.rows_per_sequence)))
            throw std::invalid_argument("invalid normalization modulation");
    if (!x.data || !(eps > 0) || !std::isfinite(eps)) throw std::invalid_argument("invalid layer normalization");
}
} // namespace

void pointwise(TensorView x, TensorView y, const Epilogue &e) {
    auto &gpu = execution_context(y, {x, e.bias, e.residual, e.gate, e.condition, e.raw});
    reject_indirect(e, "the finishing pass does not accept indirect epilogue addressing");
    check_row_output(y);
    check_epilogue(e, TensorShape(y), y.type);
    if (!x.data || e.input_repeat < 1 || x.type != y.type || x.cols != y.cols ||
        int64_t(x.rows) * e.input_repeat != y.rows || (e.input_repeat > 1 && x.data == y.data))
        throw std::invalid_argument("invalid pointwise input/repetition");
    launch_pointwise(x, y, e, gpu.stream);
}

TensorShape validate_pointwise_quantize(TensorView x, RowScaledView q, const Epilogue &e, TensorView retained) {
    reject_indirect(e, "quantized pointwise does not accept indirect epilogue addressing");
    const TensorShape shape = check_quantized_output(x, q, retained);
    check_epilogue(e, shape, x.type);
    if (!x.data || e.input_repeat < 1 || x.cols != shape.cols || int64_t(x.rows) * e.input_repeat != shape.rows ||
        (e.input_repeat > 1 && x.data == retained.data))
        throw std::invalid_argument("invalid quantized pointwise input/repetition");
    check_quantized_aliases(q, {x, retained, e.bias, e.residual, e.raw, e.gate, e.condition});
    check_retained_raw(retained, e.raw, {e.bias, e.gate, e.condition});
    for (const TensorView &output : {retained, e.raw}) {
        check_row_alias(output, x, e.input_repeat == 1);
        check_row_alias(output, e.residual, !e.residual_rows);
    }
    return shape;
}

void pointwise_quantize(TensorView x, RowScaledView q, const Epilogue &e, TensorView retained, int multiprocessors) {
    auto &gpu = execution_context(x, {q.values, q.scales, retained, e.bias, e.residual, e.gate, e.condition, e.raw});
    validate_pointwise_quantize(x, q, e, retained);
    launch_pointwise_quantize(x, q, e, retained, multiprocessors > 0 ? multiprocessors : gpu.multiprocessors, gpu.stream);
}

void layer_norm_quantize(TensorView x, RowScaledView q, TensorView w, TensorView bias, float eps, const NormFusion &f,
                         TensorView retained) {
    auto &gpu = execution_context(x, {q.values, q.scales, w, bias, retained, f.residual, f.projection_bias, f.raw, f.gate,
                                      f.shift, f.scale});
    const TensorShape shape = check_quantized_output(x, q, retained);
    check_norm_shape(x, shape, x.type, retained.data, w, bias, eps, f);
    check_quantized_aliases(q, {x, retained, w, bias, f.residual, f.projection_bias, f.raw, f.gate, f.shift, f.scale});
    check_retained_raw(retained, f.raw, {w, bias, f.projection_bias, f.gate, f.shift, f.scale});
    for (const TensorView &output : {retained, f.raw}) {
        check_row_alias(output, x, !f.source_rows);
        check_row_alias(output, f.residual, !f.source_rows);
    }
    launch_layer_norm_quantize(x, q, w, bias, eps, f, retained, gpu.stream);
}
} // namespace tts::ops
