// The execution resources the quantized ops read: device, stream, GEMM workspace, SM count and the
// plan cache. A minimal counterpart of the reference's `CudaContext`
// (src/runtime/cuda_context.h:13-35) and its thread-local binding `ExecutionScope` /
// `execution_context()` (src/ops/cuda/execution_context.h:9-29): ops are free functions that look
// up the context bound to the calling thread and refuse operands that live on another device.
#pragma once
#include "core/buffer.h"
#include "core/quantization.h"
#include "ops/quantized_gemm.h"
#include <initializer_list>
#include <memory>

namespace tts {
struct CudaContext {
    const int device;
    const cudaStream_t stream;
    Buffer gemm_workspace;
    int multiprocessors = 0, sm_major = 0, sm_minor = 0;
    bool quant_gated_clusters = false, plans_sealed = false;
    Quantization mode;
    std::unique_ptr<QuantizedGemm> quantization;
    // workspace == nullptr allocates the reference's 8 MiB (src/runtime/cuda_context.cpp:61);
    // otherwise the caller's memory is borrowed and must outlive the context.
    CudaContext(int device, Quantization mode, cudaStream_t stream = nullptr, void *workspace = nullptr,
                size_t workspace_bytes = 0);
    CudaContext(const CudaContext &) = delete;
};
class ExecutionScope {
    CudaContext *previous_;

  public:
    explicit ExecutionScope(CudaContext &);
    ~ExecutionScope();
    ExecutionScope(const ExecutionScope &) = delete;
};
CudaContext &execution_context(const TensorView &anchor, std::initializer_list<TensorView> others = {});
CudaContext &execution_context(int device);
} // namespace tts
