// Metadata-only tensor views for the quantized-linear path. No CUDA, no allocation.
// Mirrors the reference's value types so call sites read the same
// (reference: src/core/tensor.h:8-119 — Type, TensorShape, TensorView).
#pragma once
#include <cstddef>
#include <cstdint>
#include <limits>
#include <stdexcept>

namespace tts {
// Enumerator order is part of the boundary: the C ABI passes these as integers.
enum class Type { BF16, F32, I32, FP8, I8, F16, I16, I64, F64 };

inline size_t bytes(Type t) {
    switch (t) {
    case Type::FP8: case Type::I8: return 1;
    case Type::BF16: case Type::F16: case Type::I16: return 2;
    case Type::I64: case Type::F64: return 8;
    default: return 4;
    }
}

struct TensorShape {
    int rows = 0, cols = 0;
    TensorShape() = default;
    TensorShape(int r, int c) : rows(r), cols(c) {
        if (r < 0 || c < 0) throw std::invalid_argument("negative tensor dimension");
    }
    size_t numel() const { return size_t(rows) * size_t(cols); }
};

// A borrowed 2-D view: rows × cols with the inner axis dense and an optional row stride
// (in elements; 0 = dense). `device` is the CUDA ordinal, -1 for host/metadata.
struct TensorView : TensorShape {
    void *data = nullptr;
    Type type = Type::BF16;
    int stride = 0;
    int device = -1;

    TensorView() = default;
    TensorView(void *pointer, int r, int c, Type t = Type::BF16, int leading = 0, int ordinal = -1)
        : TensorShape(r, c), data(pointer), type(t), stride(leading), device(ordinal) {
        check_layout();
        if (numel() && !pointer) throw std::invalid_argument("invalid tensor pointer/stride");
    }
    static TensorView metadata(int r, int c, Type t, int leading = 0, int ordinal = -1) {
        TensorView v;
        static_cast<TensorShape &>(v) = TensorShape(r, c);
        v.type = t; v.stride = leading; v.device = ordinal;
        v.check_layout();
        return v;
    }
    int ld() const { return stride ? stride : cols; }
    bool dense() const { return rows <= 1 || ld() == cols; }
    size_t size() const { return numel() * bytes(type); }
    size_t span_elements() const { return rows && cols ? size_t(rows - 1) * ld() + cols : 0; }
    size_t span_bytes() const { return span_elements() * bytes(type); }
    bool overlaps(const TensorView &o) const {
        if (!data || !o.data) return false;
        auto a = reinterpret_cast<uintptr_t>(data), b = reinterpret_cast<uintptr_t>(o.data);
        return a < b + o.span_bytes() && b < a + span_bytes();
    }
    TensorView slice(int row, int n = 1) const {
        if (row < 0 || n < 0 || row > rows || n > rows - row) throw std::out_of_range("tensor row slice");
        return alias(at(size_t(row) * ld()), n, cols, stride);
    }
    TensorView columns(int first, int count) const {
        if (first < 0 || count < 0 || first > cols || count > cols - first)
            throw std::out_of_range("tensor column slice");
        return alias(at(size_t(first)), rows, count, ld());
    }
    template <class T> T *ptr() const { return static_cast<T *>(data); }

  private:
    void check_layout() const {
        if (stride < 0 || (stride && stride < cols)) throw std::invalid_argument("invalid tensor stride");
        if (span_elements() > std::numeric_limits<size_t>::max() / bytes(type))
            throw std::overflow_error("tensor byte size overflow");
    }
    TensorView alias(void *p, int r, int c, int leading) const {
        TensorView v = metadata(r, c, type, leading, device);
        v.data = p;
        return v;
    }
    void *at(size_t elements) const {
        return data ? static_cast<char *>(data) + elements * bytes(type) : nullptr;
    }
};
} // namespace tts
