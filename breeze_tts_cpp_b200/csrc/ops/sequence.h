// Row-wise operators around the quantized projections: the separate finishing pass, the
// finish-and-quantize pass, LayerNorm fused with quantization, and the fused norm + quantize +
// projection for narrow models. Names and arguments follow the reference
// (src/ops/sequence.h:29-41,51-63; src/ops/kernels/sequence/norm_projection.h) so layers call them
// unchanged; the operands are borrowed views on the bound device.
#pragma once
#include "core/quantization.h"
#include "ops/epilogue.h"

namespace tts::ops {
// y = finish(x): bias, gate, residual, condition, raw copy, masking, activation in one pass.
void pointwise(TensorView x, TensorView y, const Epilogue & = {});
// Quantizes the storage-rounded finished rows in the same pass. `retained` optionally keeps the 16-bit
// result; `raw` keeps its pre-activation meaning. Pass the SM count to spread short K-group batches.
void pointwise_quantize(TensorView x, RowScaledView quantized, const Epilogue & = {}, TensorView retained = {},
                        int multiprocessors = 0);
TensorShape validate_pointwise_quantize(TensorView x, RowScaledView quantized, const Epilogue & = {},
                                        TensorView retained = {});

// Residual and projection bias are added before normalization; `raw` keeps that sum for the next
// residual branch. gate / shift / scale are per-sequence modulations ([1, C] or [sequences, C]).
struct NormFusion {
    TensorView residual, projection_bias, raw, gate, shift, scale;
    int rows_per_sequence = 1;
    const int *source_rows = nullptr;
};
// LayerNorm of each row, then quantization of the storage-rounded result; `retained` optionally keeps
// the normalized 16-bit rows.
void layer_norm_quantize(TensorView x, RowScaledView quantized, TensorView weight, TensorView bias, float eps,
                         const NormFusion & = {}, TensorView retained = {});
} // namespace tts::ops
