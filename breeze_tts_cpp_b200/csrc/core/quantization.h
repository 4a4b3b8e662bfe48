// Quantized-operand contract shared by the producers (quantize kernels) and the consumer (GEMM).
// Same names and meaning as the reference so its layers can hold these views unchanged
// (reference: include/tts/quantization.h:6-29, src/core/quantization.h:6-49,
//  src/core/kernel_problem.h:4-23, src/ops/kernels/quant/kernel_config.h:5-9,
//  src/core/row_capacity.h:10-19).
#pragma once
#include "core/tensor.h"
#include <algorithm>
#include <string>

namespace tts {
enum class Quantization { None, FP8, INT8, GroupINT8, GroupFP8 };

inline const char *quantization_name(Quantization q) {
    static const char *names[] = {"none", "fp8", "int8", "group_int8", "group_fp8"};
    int i = int(q);
    if (i < 0 || i > 4) throw std::invalid_argument("invalid quantization mode");
    return names[i];
}
inline Quantization quantization_from_string(const std::string &s) {
    if (s.empty()) return Quantization::None;
    for (int i = 1; i <= 4; ++i)
        if (s == quantization_name(Quantization(i))) return Quantization(i);
    throw std::invalid_argument("quantization must be int8, fp8, group_int8 or group_fp8");
}
inline Type quantized_type(Quantization q) {
    if (q == Quantization::FP8 || q == Quantization::GroupFP8) return Type::FP8;
    if (q == Quantization::INT8 || q == Quantization::GroupINT8) return Type::I8;
    throw std::invalid_argument("BF16 has no quantized storage type");
}
inline const char *quantized_name(Type t) { return t == Type::I8 ? "INT8" : "FP8"; }

// K-group widths of activations and weights plus the Hadamard block; all zero = per-row scales.
struct QuantizationGroups {
    int activation = 0, weight = 0, rotation = 0;
};
inline QuantizationGroups quantization_groups(Quantization q) {
    if (q == Quantization::GroupINT8 || q == Quantization::GroupFP8) return {128, 128, 128};
    return {};
}
// Per-row scales are [rows,1]; K-group scales are group-major [ceil(K/g), rows] (rows contiguous).
inline TensorShape quantization_scale_shape(int rows, int columns, int group) {
    return group ? TensorShape{(columns + group - 1) / group, rows} : TensorShape{rows, 1};
}

// One-byte values [rows,K] row-major plus fp32 scales. `rotation_size` records that the producer
// applied the matched sign-flip + 128-point Hadamard transform along K; the GEMM only checks
// that both operands agree.
struct RowScaledView {
    TensorView values, scales;
    int group_size = 0, rotation_size = 0;
    int groups() const { return group_size ? (values.cols + group_size - 1) / group_size : 1; }
    void validate() const {
        bool type_ok = values.type == Type::FP8 || values.type == Type::I8;
        bool rotation_ok = !rotation_size || (rotation_size == 128 && values.cols % 128 == 0);
        bool group_ok = !group_size || group_size == 32 || group_size == 64 || group_size == 128;
        bool scale_ok = scales.type == Type::F32 && scales.dense() &&
                        scales.numel() == size_t(values.rows) * groups() &&
                        (!group_size || (scales.rows == groups() && scales.cols == values.rows));
        if (!type_ok || !values.dense() || !rotation_ok || !group_ok || !scale_ok ||
            values.device != scales.device)
            throw std::invalid_argument("invalid row-scaled quantized tensor");
    }
};

// GEMM problem: rows = tokens (M), channels = N, reduction = K; group widths 0 = per-row scales.
struct KernelProblem {
    int rows, channels, reduction;
    int input_group = 0, weight_group = 0;
};
struct KernelResources {
    int registers = 0, resident_ctas = 0;
};
struct SelectionStats {
    size_t entries = 0, hits = 0, searches = 0;
};

// The reference's five kinds keep their values; Tcgen05 is the one value this build adds.
// tokens = token-tile (MMA N when weights are the 128-row operand), channels = channel tile,
// splits = split-K factor.
enum class LinearKind { Lt, Gemv, Sm80, Hopper, Grouped, Tcgen05 };
struct LinearPath {
    LinearKind kind = LinearKind::Lt;
    int tokens = 1, channels = 0, splits = 1;
};

// Logarithmic row classes: plans are keyed by the class, not by the exact token count.
inline int row_capacity(int rows, unsigned bins_per_octave = 8) {
    if (rows < 1 || !bins_per_octave) throw std::invalid_argument("invalid row capacity class");
    int64_t pow2 = 1;
    while (pow2 < rows) pow2 <<= 1;
    int64_t step = std::max<int64_t>(1, pow2 / (2ll * bins_per_octave));
    int64_t cap = (int64_t(rows) + step - 1) / step * step;
    return int(std::min<int64_t>(cap, std::numeric_limits<int>::max()));
}
} // namespace tts
