#include "ops/context.h"
#include "kernels/quant_dispatch.h"
#include <string>

namespace tts {
namespace {
thread_local CudaContext *active_context = nullptr;
constexpr size_t kDefaultWorkspace = 8u << 20;
Buffer make_workspace(int device, void *pointer, size_t bytes) {
    if (cudaSetDevice(device) != cudaSuccess) throw std::runtime_error("cudaSetDevice failed");
    return pointer ? Buffer::borrow(pointer, bytes, device) : Buffer(bytes ? bytes : kDefaultWorkspace);
}
} // namespace

CudaContext::CudaContext(int ordinal, Quantization requested, cudaStream_t s, void *workspace, size_t bytes)
    : device(ordinal), stream(s), gemm_workspace(make_workspace(ordinal, workspace, bytes)), mode(requested) {
    cudaDeviceProp p{};
    if (cudaGetDeviceProperties(&p, device) != cudaSuccess) throw std::runtime_error("cudaGetDeviceProperties failed");
    multiprocessors = p.multiProcessorCount;
    sm_major = p.major;
    sm_minor = p.minor;
    int clusters = 0;
    cudaDeviceGetAttribute(&clusters, cudaDevAttrClusterLaunch, device);
    quant_gated_clusters = clusters != 0;
    if (mode != Quantization::None)
        quantization = std::make_unique<QuantizedGemm>(stream, nullptr, gemm_workspace, quantized_type(mode));
}

ExecutionScope::ExecutionScope(CudaContext &context) : previous_(active_context) {
    active_context = &context;
    if (cudaSetDevice(context.device) != cudaSuccess) throw std::runtime_error("cudaSetDevice failed");
}
ExecutionScope::~ExecutionScope() { active_context = previous_; }

CudaContext &execution_context(int device) {
    if (!active_context) throw std::logic_error("no execution context is bound to this thread");
    if (active_context->device != device)
        throw std::invalid_argument("tensor device " + std::to_string(device) + " is not the bound device");
    return *active_context;
}
CudaContext &execution_context(const TensorView &anchor, std::initializer_list<TensorView> others) {
    CudaContext &context = execution_context(anchor.device);
    for (const auto &v : others)
        if (v.data && v.device != anchor.device) throw std::invalid_argument("operands are on different devices");
    return context;
}
} // namespace tts
