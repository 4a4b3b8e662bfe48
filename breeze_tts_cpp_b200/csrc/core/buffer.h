// Device byte storage for the few buffers the path owns itself (GEMM workspace, activation
// scratch). Either owns a cudaMalloc allocation or borrows caller memory (C ABI callers hand in
// their own workspace). Plays the role of the reference's `Buffer` (src/core/buffer.h:4) for the
// members this path touches: data(), size(), device(), view().
#pragma once
#include "core/tensor.h"
#include <cuda_runtime_api.h>
#include <string>
#include <utility>

namespace tts {
class Buffer {
    void *data_ = nullptr;
    size_t size_ = 0;
    int device_ = -1;
    bool owned_ = false;

  public:
    Buffer() = default;
    explicit Buffer(size_t bytes) : size_(bytes), owned_(true) {
        if (cudaGetDevice(&device_) != cudaSuccess) throw std::runtime_error("no CUDA device for Buffer");
        if (bytes) {
            cudaError_t status = cudaMalloc(&data_, bytes);
            if (status != cudaSuccess)
                throw std::runtime_error(std::string("cudaMalloc: ") + cudaGetErrorString(status));
        }
    }
    static Buffer borrow(void *pointer, size_t bytes, int device) {
        Buffer b;
        b.data_ = pointer; b.size_ = bytes; b.device_ = device; b.owned_ = false;
        return b;
    }
    Buffer(Buffer &&o) noexcept { *this = std::move(o); }
    Buffer &operator=(Buffer &&o) noexcept {
        if (this != &o) {
            release();
            data_ = o.data_; size_ = o.size_; device_ = o.device_; owned_ = o.owned_;
            o.data_ = nullptr; o.size_ = 0; o.owned_ = false;
        }
        return *this;
    }
    Buffer(const Buffer &) = delete;
    Buffer &operator=(const Buffer &) = delete;
    ~Buffer() { release(); }
    void *data() const { return data_; }
    size_t size() const { return size_; }
    int device() const { return device_; }
    TensorView view(int rows, int cols, Type type, size_t byte_offset = 0) const {
        if (byte_offset > size_ || size_t(rows) * cols * bytes(type) > size_ - byte_offset)
            throw std::out_of_range("buffer view exceeds storage");
        return TensorView(static_cast<char *>(data_) + byte_offset, rows, cols, type, 0, device_);
    }

  private:
    void release() {
        if (owned_ && data_) cudaFree(data_);
        data_ = nullptr;
    }
};
} // namespace tts
