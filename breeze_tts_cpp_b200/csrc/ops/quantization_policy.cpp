#include "ops/quantization_policy.h"
#include "kernels/quant_linear_geometry.h"
#include <cmath>
#include <limits>
#include <stdexcept>

namespace tts {
using namespace b200;

// Figures measured on a B200 at 1965 MHz: 6.55 TB/s copy bandwidth; one SM pulls about 85 GB/s
// through TMA when it streams alone, about 60 GB/s inside a chain of launches; one `tcgen05.mma` stream per SM adds up to about 4.5 POP/s; a dependent launch costs
// about 4 us that do not scale with bytes (launch boundary, arrival of the first activation tile,
// accumulator drain and store).
ChipModel ChipModel::b200(int multiprocessors) {
    ChipModel chip;
    chip.sms = multiprocessors > 0 ? multiprocessors : 148;
    chip.memory_bytes_per_us = 6.55e6;
    chip.tensor_ops_per_us = 4.5e9 * chip.sms / 148.;
    chip.scalar_ops_per_us = 128. * 2 * 1965 * chip.sms;
    chip.kernel_us = 4.0;
    chip.warp_tensor_ops_per_us = chip.tensor_ops_per_us / chip.sms;
    chip.warp_instructions_per_us = 4. * 1965;
    chip.cache_bytes = size_t(126) << 20;
    chip.cache_bytes_per_us = 60e3 * chip.sms; // per SM while the next launch of a chain prefetches too (85 GB/s alone)
    return chip;
}

std::string path_name(const LinearPath &p) {
    static const char *kinds[] = {"cublaslt", "gemv", "sm80", "hopper", "grouped", "tcgen05"};
    const int kind = int(p.kind);
    if (kind < 0 || kind > 5) throw std::invalid_argument("invalid linear path kind");
    if (p.kind == LinearKind::Lt) return kinds[0];
    if (p.kind == LinearKind::Gemv)
        return "gemv_tokens" + std::to_string(p.tokens) + "_split" + std::to_string(p.splits);
    return std::string(kinds[kind]) + "_channels" + std::to_string(p.channels) + "_tokens" + std::to_string(p.tokens) +
           "_split" + std::to_string(p.splits);
}

namespace {
bool grouped(const KernelProblem &p) { return p.input_group || p.weight_group; }
int blocks(int size, int tile) { return (size + tile - 1) / tile; }
// Which kernel the launcher picks for a path (mirrors launch_quant_linear's dispatch).
bool persistent_per_row(const KernelProblem &p, const LinearPath &path) {
    return !grouped(p) && path.tokens == kPrefillTokens && path.splits == 1;
}
bool persistent_grouped(const KernelProblem &p, const LinearPath &path, int sms) {
    return p.input_group == kBlockK && p.weight_group == kBlockK && path.tokens == kGroupedTokens &&
           path.splits == 1 && p.rows % 4 == 0 &&
           int64_t(blocks(p.channels, kBlockChannels)) * blocks(p.rows, kGroupedTokens) >= int64_t(sms) * 2 / 3;
}
} // namespace

std::vector<LinearPath> quant_linear_candidates(KernelProblem p, KernelLimits limits, Type format) {
    if (format != Type::FP8 && format != Type::I8) throw std::invalid_argument("unsupported quantized storage type");
    std::vector<LinearPath> paths;
    if (p.rows < 1 || p.channels < 1 || p.reduction < 1 || p.reduction % 16) return paths;
    const bool group = grouped(p);
    const int kb_total = blocks(p.reduction, kBlockK);
    int cover = 16;
    while (cover < (group ? kGroupedTokens : kPrefillTokens) && cover < p.rows) cover *= 2;
    std::vector<int> token_tiles{cover};
    if (group && cover == kGroupedTokens) token_tiles.push_back(64); // the split-K kernel's widest K-group tile below 128
    for (int tokens : token_tiles)
        for (int splits = 1; splits <= std::min(kb_total, kMaxSplits); ++splits) {
            const LaunchShape shape = launch_shape(tokens, group, blocks(kb_total, splits), splits,
                                                   group_units(p.input_group, p.weight_group));
            if (!shape.fits || (limits.shared_bytes && shape.smem > limits.shared_bytes)) continue;
            paths.push_back({LinearKind::Tcgen05, tokens, kBlockChannels, splits});
        }
    return paths;
}

double linear_cost(KernelProblem p, LinearPath path, Type, const ChipModel &chip) {
    if (path.kind != LinearKind::Tcgen05) return std::numeric_limits<double>::infinity();
    const int sms = std::max(1, chip.sms);
    const int kb_total = blocks(p.reduction, kBlockK);
    const double ops = 2.0 * p.rows * double(p.channels) * p.reduction;
    if (persistent_per_row(p, path)) {
        // CTA pairs over 256x256 tiles (one CTA per 128x256 tile when N < 256); the tensor pipe
        // sustains about two thirds of its issue rate, the last wave may be partly empty.
        const bool pair = p.channels >= 2 * kBlockChannels;
        const double tiles = double(blocks(p.channels, pair ? 2 * kBlockChannels : kBlockChannels)) * blocks(p.rows, kPrefillTokens);
        const double workers = pair ? sms / 2 : sms;
        const double waves = std::ceil(tiles / workers);
        return chip.kernel_us + ops * (waves * workers / tiles) / (0.65 * chip.tensor_ops_per_us);
    }
    if (persistent_grouped(p, path, sms)) {
        // Bound by the fp32 rescale of every K128 partial tile on the CUDA cores.
        const double tiles = double(blocks(p.channels, kBlockChannels)) * blocks(p.rows, kGroupedTokens);
        const double waves = std::ceil(tiles / sms);
        return chip.kernel_us + ops * (waves * sms / tiles) / (0.3 * chip.tensor_ops_per_us);
    }
    // Weight-streaming kernel, as it runs inside a decoder chain: the launch starts under programmatic
    // dependent launch while its quantizer still runs, so by the time the activations exist the ring
    // already holds `stages` K blocks of weights. What is left on the critical path is
    //   * the K blocks that did not fit the ring, at what one SM can pull or its share of HBM;
    //   * the MMAs, which cost a fixed ~0.12 us per K block up to 64 tokens (four instructions of at
    //     least 48 tensor-pipe cycles each, however few tokens), more for wider tiles;
    //   * the split-K exchange, about 0.3 us per CTA of the cluster at 64 tokens (less for narrower tiles); clusters of seven and eight lose
    //     about 6 us more (their CTAs are placed late and miss the weight prefetch);
    //   * the epilogue, about 0.4 us per 16-token pass a CTA finishes;
    //   * a crowding term: the more SMs a launch holds, the fewer the next launch of the chain finds
    //     free to start its own prefetch early; uneven K splits cost a little as well.
    // Calibrated on the decoder layer's four shapes at 8 to 64 rows, timed inside the chain.
    const int splits = std::max(1, path.splits), per_split = blocks(kb_total, splits);
    const LaunchShape shape = launch_shape(path.tokens, grouped(p), per_split, splits, group_units(p.input_group, p.weight_group));
    if (!shape.fits) return std::numeric_limits<double>::infinity();
    const double stage_bytes = double(kBlockChannels + path.tokens) * kBlockK;
    const int64_t ctas = int64_t(blocks(p.channels, kBlockChannels)) * blocks(p.rows, path.tokens) * splits;
    // Small tiles leave room for two CTAs per SM; clusters are placed whole.
    const int resident = (!grouped(p) && path.tokens <= 64 && shape.smem <= 108 * 1024) ? 2 : 1;
    const int64_t slots = std::max<int64_t>(splits, int64_t(sms) * resident / splits * splits);
    const double waves = double((ctas + slots - 1) / slots);
    const double per_sm = chip.cache_bytes_per_us > 0 ? chip.cache_bytes_per_us / sms : 60e3;
    const int exposed_blocks = std::max(0, per_split - shape.stages);
    const double exposed = exposed_blocks * stage_bytes *
                           std::max(1.0 / per_sm, double(std::min(ctas, slots)) / (0.84 * chip.memory_bytes_per_us));
    const double mma_block = path.tokens <= 64 ? 0.12 : path.tokens <= 128 ? 0.16 : 0.29;
    const double compute = std::max(per_split * mma_block, exposed + mma_block) * (grouped(p) ? 1.5 : 1.0);
    const double exchange = splits > 1 ? (0.15 + 0.15 * path.tokens / 64.0) * splits + (kb_total % splits ? 0.15 : 0.0) + (splits > 6 ? 6.0 : 0.0) : 0.0;
    const int passes = blocks(std::min(p.rows, path.tokens), kRowsPerPass);
    const double epilogue = 0.4 * (splits > 1 ? blocks(passes, splits) : passes);
    const double crowding = 0.01 * double(std::max<int64_t>(0, std::min(ctas, slots) - 64));
    // Later waves see a cold ring: they stream all of their K blocks.
    const double later_wave = per_split * stage_bytes * std::max(1.0 / per_sm, double(slots) / (0.84 * chip.memory_bytes_per_us)) +
                              exchange + epilogue;
    return chip.kernel_us + compute + exchange + epilogue + crowding + (waves - 1.0) * later_wave;
}

double linear_pipeline_cost(KernelProblem p, LinearPath path, Type format, const ChipModel &chip, LinearFinishWork finish,
                            bool fused, LibraryWork, KernelResources) {
    // Row quantizer: one launch, 2 bytes read and 1 written per activation element.
    const double quantize = chip.kernel_us / 2 + (3.0 * p.rows * p.reduction + 4.0 * p.rows) / chip.memory_bytes_per_us;
    const double gemm = linear_cost(p, path, format, chip);
    if (fused) return quantize + gemm; // the epilogue chain rides in the GEMM's own epilogue
    // A separate finishing pass reads and writes every output element once more.
    const double elements = double(p.rows) * p.channels;
    const double pass = chip.kernel_us / 2 + 4.0 * elements / chip.memory_bytes_per_us +
                        elements * finish.instructions_per_output / (32. * chip.warp_instructions_per_us * chip.sms);
    return quantize + gemm + pass;
}

LinearPath select_linear(KernelProblem p, KernelLimits limits, Type format, const ChipModel &chip, bool, LibraryWork) {
    double best = std::numeric_limits<double>::infinity();
    LinearPath selected;
    for (const LinearPath &path : quant_linear_candidates(p, limits, format)) {
        const double cost = linear_cost(p, path, format, chip);
        if (cost < best - 1e-9) { // ties keep the earlier (narrower split) candidate
            best = cost;
            selected = path;
        }
    }
    if (!std::isfinite(best)) throw std::invalid_argument("no supported quantized GEMM implementation");
    return selected;
}
} // namespace tts
