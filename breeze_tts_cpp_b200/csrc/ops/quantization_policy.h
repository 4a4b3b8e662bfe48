// Planner of the quantized GEMM: enumerates the launch shapes the tcgen05 kernels can run for a
// problem and ranks them with an analytic cost model. CPU only, no CUDA calls. Names, argument
// lists and result types follow the reference planner (src/ops/cuda/quantization_policy.h:9-33) so
// `QuantizedGemm` and any other caller keep their call sites; every path this build returns has
// kind `LinearKind::Tcgen05`.
#pragma once
#include "core/quantization.h"
#include <string>
#include <vector>

namespace tts {
// Planning inputs that describe the GPU. Field names as in the reference; `b200()` fills them with
// what was measured on a B200 (148 SMs, 1965 MHz) instead of the reference's per-architecture table.
struct ChipModel {
    int sms = 1;
    double memory_bytes_per_us = 1;      // sustained HBM read rate
    double tensor_ops_per_us = 1;        // dense 8-bit multiply-add rate of the whole chip (2 ops per MAC)
    double scalar_ops_per_us = 1;
    double kernel_us = 1;                // fixed cost of one dependent launch: boundary, first tile, epilogue
    double warp_tensor_ops_per_us = 0;
    double warp_instructions_per_us = 1;
    size_t cache_bytes = 0;
    double cache_bytes_per_us = 0;       // what all SMs together can pull through L2
    static ChipModel b200(int multiprocessors = 148);
};
struct KernelLimits {
    bool hopper = false; // accepted for signature compatibility; never true on sm_100
    size_t shared_bytes = 0, workspace_bytes = 0;
};
struct LinearFinishWork {
    double instructions_per_output = 0;
};
struct LibraryWork {
    double effective_waves = 0;
    unsigned kernel_launches = 2;
};

// Every launch shape the kernels accept for this problem: token tile = the smallest power of two in
// [16, 256] covering the rows (128 at most for K-group scales, where 64 is listed too because it
// splits K), channel tile 128, split-K 1..8 as far as K blocks and shared memory allow.
std::vector<LinearPath> quant_linear_candidates(KernelProblem, KernelLimits, Type format = Type::FP8);
std::string path_name(const LinearPath &);
// Estimated microseconds of quantize + GEMM (+ a separate finishing pass when `fused` is false).
double linear_pipeline_cost(KernelProblem, LinearPath, Type, const ChipModel &, LinearFinishWork, bool fused,
                            LibraryWork = {}, KernelResources = {});
// Estimated microseconds of the GEMM launch alone.
double linear_cost(KernelProblem, LinearPath, Type, const ChipModel &);
LinearPath select_linear(KernelProblem, KernelLimits, Type, const ChipModel &, bool library_compatible = true,
                         LibraryWork = {});
} // namespace tts
