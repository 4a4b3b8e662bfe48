// The part of the reference's `ForwardContext` (src/core/forward_context.h:57-110) that a layer
// reads: the phase it is called in and the row bounds of the run. Plan and Capture launch nothing
// from a layer; Prepare makes plans (and may allocate); Execute runs kernels and allocates nothing.
// Scratch outputs come from a caller-provided arena instead of the engine's tensor allocator.
#pragma once
#include "core/buffer.h"

namespace tts {
struct ForwardContext {
    enum Mode { Plan, Prepare, Capture, Execute } mode = Execute;
    int max_batch, max_time, max_rows;
    Buffer *arena = nullptr; // optional scratch for layer outputs requested through tensor()
    size_t arena_used = 0;
    ForwardContext(int batches, int time, int rows) : max_batch(batches), max_time(time), max_rows(rows) {}
    // A [rows, cols] scratch tensor carved from the arena (256-byte aligned, never freed individually).
    TensorView tensor(TensorShape shape, Type type) {
        if (!arena) throw std::logic_error("forward context has no scratch arena");
        const size_t bytes_needed = (shape.numel() * bytes(type) + 255) / 256 * 256;
        if (arena_used + bytes_needed > arena->size()) throw std::runtime_error("forward scratch arena exhausted");
        TensorView view = arena->view(shape.rows, shape.cols, type, arena_used);
        arena_used += bytes_needed;
        return view;
    }
};
} // namespace tts
