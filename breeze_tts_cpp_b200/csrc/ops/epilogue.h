// What may follow a projection inside the same pass: bias, gate, residual, condition, activation.
// Field names and meaning follow the reference's `ops::Epilogue` (src/ops/sequence.h:8-27) and
// `ops::Activation` (src/ops/activation.h:4) so callers build it the same way. `residual_f32` is
// the one addition: an fp32 residual stream added before the first rounding, which the synthetic
// decode workload uses.
#pragma once
#include "core/tensor.h"

namespace tts::ops {
enum class Activation { Identity, Relu, LeakyRelu, Silu, Gelu, GeluTanh, Mish, Tanh, Sigmoid };

struct Epilogue {
    TensorView bias, residual;
    float value_scale = 1;
    float output_scale = 1;
    float residual_scale = 1;
    Activation activation = Activation::Identity;
    float alpha = .1f;
    TensorView raw;       // optional pre-activation copy
    TensorView gate;      // per-sequence multiplicative gate
    TensorView condition; // per-sequence additive condition
    int rows_per_sequence = 1;
    int valid_rows_per_sequence = 0;
    int input_repeat = 1;
    const int *residual_rows = nullptr; // index into residual rows; negative entries contribute zero
    // Indirect addressing of the reference's packed-sequence consumers. No operator of this library
    // takes them: they are kept so that an Epilogue is built the same way, and rejected when set.
    const struct SequenceLayout *packed = nullptr;
    const void *const *condition_sources = nullptr;
    void *const *output_rows = nullptr;
    TensorView residual_f32; // extension: fp32 [rows, channels], added in fp32 before rounding
};

// True when the GEMM's own epilogue can apply the whole description (no second pass needed).
inline bool fusable(const Epilogue &e) {
    return !e.raw.data && !e.gate.data && !e.condition.data && !e.valid_rows_per_sequence &&
           e.input_repeat == 1 && !e.residual_rows && e.activation != Activation::Mish && !e.packed &&
           !e.condition_sources && !e.output_rows;
}
// True when nothing at all follows the projection.
inline bool plain(const Epilogue &e) {
    return !e.bias.data && !e.residual.data && !e.residual_f32.data && !e.gate.data && !e.condition.data &&
           !e.raw.data && e.activation == Activation::Identity && e.value_scale == 1 && e.output_scale == 1 &&
           !e.valid_rows_per_sequence && !e.packed && !e.condition_sources && !e.output_rows;
}
} // namespace tts::ops
