// b200q_quant_linear_static: the quantized GEMM for callers that must not allocate device memory.
//
// Who needs it: an engine that has sealed its memory pools before serving (the reference freezes
// every plan and buffer at `seal()` and treats any later allocation as a bug), code that runs
// inside a region where cudaMalloc is not permitted, or a host that hands this library a stream but
// no workspace. The regular entry points take their scratch from a context that allocates (or
// borrows) a workspace; this one keeps the GEMM's scratch — the 32 KiB header holding the device
// status word — in a file-scope device array that every GPU loading the library carries until exit.
//
// Rules that follow from sharing one array:
//   * every call on a device uses the same scratch and finds the previous call's contents there;
//     the status word is cleared on the stream before each launch, so read it (b200q_static_status,
//     which allocates nothing either) before the next call if you want to know about this one;
//   * two calls that overlap on the GPU (different streams, no ordering) race on it;
//   * the first call on a device performs the one-time set-up (kernel attributes, the array's
//     device address) and should therefore be made before any stream capture begins;
//   * problems whose scratch need exceeds the array are rejected, nothing is allocated instead.
#include "b200q.h"
#include "c_api_convert.h"
#include "kernels/quant_dispatch.h"
#include "ops/epilogue.h"
#include <cstdio>
#include <exception>
#include <mutex>
#include <stdexcept>
#include <string>

namespace {
using namespace tts;
constexpr size_t kStaticScratchBytes = 32768; // 32 KiB, the stated maximum (the GEMM's status header)

static __device__ __align__(256) unsigned char static_scratch[kStaticScratchBytes];

// Host code may not use `static_scratch` as a pointer: on the host the name is only a handle.
// The device address is looked up once per device, with that device current; the SM count the
// planner needs is cached under the same lock.
struct DeviceScratch {
    void *address = nullptr;
    int multiprocessors = 0;
};
DeviceScratch scratch_of(int device) {
    static std::mutex guard;
    static DeviceScratch known[64];
    if (device < 0 || device >= 64) throw std::invalid_argument("device ordinal out of range");
    std::lock_guard<std::mutex> lock(guard);
    if (!known[device].address) {
        int current = -1;
        if (cudaGetDevice(&current) != cudaSuccess || current != device)
            throw std::logic_error("the target device must be current during set-up");
        quant_linear_initialize(device);
        void *pointer = nullptr;
        cudaError_t status = cudaGetSymbolAddress(&pointer, static_scratch);
        if (status != cudaSuccess || !pointer)
            throw std::runtime_error(std::string("cudaGetSymbolAddress(static_scratch): ") + cudaGetErrorString(status));
        status = cudaMemset(pointer, 0, kStaticScratchBytes);
        if (status != cudaSuccess)
            throw std::runtime_error(std::string("clearing the static scratch: ") + cudaGetErrorString(status));
        int count = 0;
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count < 1)
            throw std::runtime_error("cudaDeviceGetAttribute(multiprocessor count) failed");
        known[device].multiprocessors = count;
        known[device].address = pointer;
    }
    return known[device];
}
// Makes `device` current for the duration of a call and puts the caller's device back afterwards.
class DeviceScope {
    int previous_ = -1;

  public:
    explicit DeviceScope(int device) {
        if (cudaGetDevice(&previous_) != cudaSuccess) previous_ = -1;
        if (previous_ != device && cudaSetDevice(device) != cudaSuccess) throw std::runtime_error("cudaSetDevice failed");
        if (previous_ == device) previous_ = -1;
    }
    ~DeviceScope() {
        if (previous_ >= 0) cudaSetDevice(previous_);
    }
};

} // namespace

extern "C" int b200q_quant_linear_static(int32_t device, void *stream, const b200q_path *path,
                                         const b200q_row_scaled *input, const b200q_row_scaled *weight,
                                         const b200q_tensor *output, const b200q_epilogue *epilogue, char *error,
                                         size_t error_capacity) {
    try {
        if (!output) throw std::invalid_argument("null output");
        DeviceScope current(device);
        const DeviceScratch on_device = scratch_of(device);
        void *scratch = on_device.address;
        RowScaledView x = capi::scaled_of(input), w = capi::scaled_of(weight);
        TensorView y = capi::view_of(output);
        x.validate();
        w.validate();
        if (x.values.type != w.values.type || x.values.cols != w.values.cols || x.rotation_size != w.rotation_size ||
            !y.data || y.rows != x.values.rows || y.cols != w.values.rows || !y.dense())
            throw std::invalid_argument("quantized linear dimensions/type mismatch");
        for (const TensorView *v : {&x.values, &x.scales, &w.values, &w.scales, &y})
            if (v->device != device) throw std::invalid_argument("operand is not on the requested device");
        KernelProblem problem{y.rows, y.cols, x.values.cols, x.group_size, w.group_size};
        LinearPath chosen = path ? LinearPath{static_cast<LinearKind>(path->kind), path->tokens, path->channels, path->splits}
                                 : select_tcgen05_path(problem, x.values.type, on_device.multiprocessors, kStaticScratchBytes);
        const size_t need = quant_linear_workspace_bytes(chosen, problem);
        if (need > kStaticScratchBytes)
            throw std::invalid_argument("this problem needs " + std::to_string(need) + " bytes of scratch; the built-in scratch holds " +
                                        std::to_string(kStaticScratchBytes) + " and this entry point never allocates");
        const ops::Epilogue finish = capi::epilogue_of(epilogue);
        auto s = static_cast<cudaStream_t>(stream);
        // The shared array still holds whatever the previous call left; the GEMM expects its header
        // (status word included) to start at zero, so clear it on the stream ahead of the launch.
        if (cudaMemsetAsync(scratch, 0, need, s) != cudaSuccess) throw std::runtime_error("clearing the scratch header failed");
        launch_quant_linear(chosen, problem, x.values.data, x.scales.ptr<float>(), w.values.data, w.scales.ptr<float>(), y.data,
                            scratch, kStaticScratchBytes, s, x.values.type, y.type, epilogue ? &finish : nullptr);
        if (error && error_capacity) error[0] = 0;
        return 0;
    } catch (const std::exception &e) {
        if (error && error_capacity) std::snprintf(error, error_capacity, "%s", e.what());
    } catch (...) {
        if (error && error_capacity) std::snprintf(error, error_capacity, "unknown error");
    }
    return -1;
}

extern "C" int b200q_static_status(int32_t device, void *stream, int32_t *status, char *error, size_t error_capacity) {
    try {
        if (!status) throw std::invalid_argument("null status");
        DeviceScope current(device);
        const DeviceScratch on_device = scratch_of(device);
        *status = quant_linear_status(on_device.address, static_cast<cudaStream_t>(stream));
        if (error && error_capacity) error[0] = 0;
        return 0;
    } catch (const std::exception &e) {
        if (error && error_capacity) std::snprintf(error, error_capacity, "%s", e.what());
    } catch (...) {
        if (error && error_capacity) std::snprintf(error, error_capacity, "unknown error");
    }
    return -1;
}
