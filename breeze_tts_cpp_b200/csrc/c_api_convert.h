// POD structs of the C ABI -> the C++ value types of the library. Shared by every extern "C" source.
#pragma once
#include "b200q.h"
#include "core/quantization.h"
#include "ops/epilogue.h"
#include "ops/sequence.h"

namespace tts::capi {
inline Type type_of(int code) {
    if (code < 0 || code > int(Type::F64)) throw std::invalid_argument("invalid type code");
    return static_cast<Type>(code);
}
inline TensorView view_of(const b200q_tensor *t) {
    if (!t || !t->data) return {};
    return TensorView(t->data, t->rows, t->cols, type_of(t->type), t->stride, t->device);
}
inline RowScaledView scaled_of(const b200q_row_scaled *r) {
    if (!r) throw std::invalid_argument("null row-scaled view");
    RowScaledView v;
    v.values = view_of(&r->values);
    v.scales = view_of(&r->scales);
    v.group_size = r->group_size;
    v.rotation_size = r->rotation_size;
    return v;
}
inline ops::Epilogue epilogue_of(const b200q_epilogue *e) {
    ops::Epilogue out;
    if (!e) return out;
    out.bias = view_of(&e->bias);
    out.residual = view_of(&e->residual);
    out.residual_f32 = view_of(&e->residual_f32);
    out.value_scale = e->value_scale;
    out.output_scale = e->output_scale;
    out.residual_scale = e->residual_scale;
    out.alpha = e->alpha;
    if (e->activation < 0 || e->activation > int(ops::Activation::Sigmoid)) throw std::invalid_argument("invalid activation");
    out.activation = static_cast<ops::Activation>(e->activation);
    out.gate = view_of(&e->gate);
    out.condition = view_of(&e->condition);
    out.raw = view_of(&e->raw);
    out.rows_per_sequence = e->rows_per_sequence ? e->rows_per_sequence : 1;
    out.valid_rows_per_sequence = e->valid_rows_per_sequence;
    out.input_repeat = e->input_repeat ? e->input_repeat : 1;
    out.residual_rows = e->residual_rows;
    return out;
}
inline ops::NormFusion fusion_of(const b200q_norm_fusion *f) {
    ops::NormFusion out;
    if (!f) return out;
    out.residual = view_of(&f->residual);
    out.projection_bias = view_of(&f->projection_bias);
    out.raw = view_of(&f->raw);
    out.gate = view_of(&f->gate);
    out.shift = view_of(&f->shift);
    out.scale = view_of(&f->scale);
    out.rows_per_sequence = f->rows_per_sequence ? f->rows_per_sequence : 1;
    out.source_rows = f->source_rows;
    return out;
}
} // namespace tts::capi
