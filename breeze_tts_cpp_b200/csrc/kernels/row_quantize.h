// Launcher of the fused per-token quantize(+rotate)(+K-group) kernel.
// Same call as the reference's `launch_row_quantize(TensorView, RowScaledView, cudaStream_t)`
// (src/ops/kernels/quant/row_quantize.h:6); the optional SM count only steers how short batches
// are spread over the machine in K-group mode.
#pragma once
#include "core/quantization.h"
#include <cuda_runtime_api.h>

namespace tts {
void launch_row_quantize(TensorView source, RowScaledView destination, cudaStream_t stream,
                         int multiprocessors = 0);
} // namespace tts
