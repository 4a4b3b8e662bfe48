// Tile geometry of the tcgen05 GEMM family and the shared-memory budget of one launch shape. Host
// and device code share these numbers; the planner uses them to list only shapes that fit.
#pragma once
#include <algorithm>
#include <cstddef>

namespace tts::b200 {
constexpr int kBlockChannels = 128; // MMA M: weight rows per tile
constexpr int kBlockK = 128;        // bytes of K per pipeline stage (one 128B-swizzled TMA box)
constexpr int kMaxStages = 12;
constexpr int kRowsPerPass = 16;    // token rows the epilogue warps finish per pass (16 threads x 8 channels per row)
constexpr int kMaxSplits = 8;       // portable thread-block cluster size
constexpr int kPrefillTokens = 256; // token tile of the persistent per-row kernels
constexpr int kGroupedTokens = 128; // token tile of the persistent K-group kernel
constexpr size_t kSmemBudget = 224 * 1024; // dynamic part per CTA: all but 3 KiB of the SM, which is what the static barriers and a co-resident quantizer CTA of the next launch need

struct LaunchShape {
    bool fits = false;
    int stages = 0, owned_passes = 0;
    size_t tile_region = 0, smem = 0;
};
// K groups per 128-byte K block (1, 2 or 4 for group widths 128, 64, 32): the narrower of the two
// operands' widths decides, an operand without K groups counts as 128.
inline int group_units(int input_group, int weight_group) {
    const int narrow = std::min(input_group ? input_group : kBlockK, weight_group ? weight_group : kBlockK);
    return kBlockK / std::max(32, narrow);
}
// Shared memory of one CTA of the weight-streaming kernel: alignment slack + pipeline stages
// (unsplit: later the transposed [token][channel] tile of 4-byte partials) + split-K slots the
// cluster peers push into + the K-group scales of the CTA's K range, one pair per group.
inline LaunchShape launch_shape(int bn, bool grouped, int kb_per_split, int splits, int units = 1) {
    const size_t stage = size_t(kBlockChannels + bn) * kBlockK;
    const size_t transposed = splits == 1 ? size_t(bn) * kBlockChannels * sizeof(float) : 0;
    const int passes = (bn + kRowsPerPass - 1) / kRowsPerPass;
    const int owned = splits > 1 ? (passes + splits - 1) / splits : 0;
    const size_t reduce = size_t(splits > 1 ? splits : 0) * owned * kRowsPerPass * kBlockChannels * sizeof(float);
    const size_t scales = grouped ? size_t(kb_per_split) * units * (bn + kBlockChannels) * sizeof(float) : 0;
    const size_t fixed = 1024 + reduce + scales;
    LaunchShape shape;
    if (fixed + std::max(2 * stage, transposed) > kSmemBudget) return shape;
    // As many stages as fit (capped by the K blocks of one CTA): the ring is what gets prefetched
    // while the upstream kernel is still running. Measured on the decode chain, deep rings with one
    // CTA per SM beat half-size rings with two co-resident CTAs.
    int stages = int((kSmemBudget - fixed) / stage);
    stages = std::max(2, std::min({stages, kMaxStages, std::max(2, kb_per_split)}));
    shape.fits = true;
    shape.stages = stages;
    shape.owned_passes = owned;
    shape.tile_region = std::max(size_t(stages) * stage, transposed);
    shape.smem = fixed + shape.tile_region;
    return shape;
}
} // namespace tts::b200
