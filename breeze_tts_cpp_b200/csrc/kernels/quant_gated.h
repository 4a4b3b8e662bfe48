// act(gate) * up + quantize in one pass; feeds the down projection.
// Same calls as the reference's (src/ops/kernels/quant/quant_gated.h:6-8).
#pragma once
#include "core/quantization.h"
#include <cuda_runtime_api.h>
namespace tts {
bool quant_gated_supports_clusters(int device);
void launch_quantized_gated(TensorView input, RowScaledView output, int kind, cudaStream_t stream,
                            int multiprocessors, bool clusters);
} // namespace tts
