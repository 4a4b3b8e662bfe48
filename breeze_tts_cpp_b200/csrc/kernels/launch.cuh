// Launch helper shared by every kernel of the path: all of them are launched with the
// programmatic-stream-serialization attribute, so a kernel's prologue may overlap the tail of the
// kernel before it in the stream. The contract each kernel keeps in return:
//   * it executes `pdl_launch_dependents()` early, and
//   * it executes `pdl_wait_upstream()` before its first read of data a previous kernel may have
//     written and before its first global write.
// Because every kernel waits for its predecessor to finish before it finishes itself, ordering
// stays transitive along the whole chain. Outside such a launch both instructions do nothing.
#pragma once
#include <cuda_runtime.h>
#include <stdexcept>
#include <string>

namespace tts::b200 {
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait_upstream() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <class... Params, class... Args>
void launch_pdl(const char *what, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                Args... args) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    cudaError_t status = cudaLaunchKernelEx(&config, kernel, Params(args)...);
    if (status != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(status));
}
} // namespace tts::b200
