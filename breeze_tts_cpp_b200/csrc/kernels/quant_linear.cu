// Host side of the sm_100a quantized GEMM: tensor-map construction, tile/split selection and the
// launch. Drop-in for the reference launchers `launch_quant_linear` and `grouped_quant_gemm`
// (src/ops/kernels/quant/quant_dispatch.cu:194-234, quant_grouped.cu:221-239).
#include "kernels/quant_dispatch.h"
#include "kernels/quant_linear_sm100.cuh"
#include "kernels/quant_prefill_sm100.cuh"
#include "kernels/quant_prefill_pair_sm100.cuh"
#include "kernels/quant_prefill_grouped_sm100.cuh"
#include "ops/epilogue.h"
#include "ops/quantization_policy.h"
#include <atomic>
#include <cudaTypedefs.h>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

namespace tts {
namespace {
using namespace b200;

void check(cudaError_t status, const char *what) {
    if (status != cudaSuccess)
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(status));
}

PFN_cuTensorMapEncodeTiled_v12000 encode_tiled() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
        void *entry = nullptr;
        cudaDriverEntryPointQueryResult result{};
        check(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result),
              "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
        if (!entry || result != cudaDriverEntryPointSuccess)
            throw std::runtime_error("cuTensorMapEncodeTiled is unavailable in this driver");
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(entry);
    }();
    return fn;
}

// Tensor maps are returned by value (128 bytes, encoded on the host without a driver round trip):
// the launch copies them into the kernel's parameters, so nothing has to outlive the call.
// Row-major one-byte matrix [rows, k]; box = 128 bytes of K by `box_rows` rows, 128B swizzle,
// out-of-range rows/columns read as zero (so ragged M, N and K tails need no special code).
CUtensorMap operand_map(const void *base, int rows, int k, int box_rows, bool weights) {
    if (reinterpret_cast<uintptr_t>(base) % 16 || k % 16)
        throw std::invalid_argument("quantized operand must be 16-byte aligned with K a multiple of 16");
    CUtensorMap map;
    cuuint64_t dims[2] = {cuuint64_t(k), cuuint64_t(rows)};
    cuuint64_t strides[1] = {cuuint64_t(k)};
    cuuint32_t box[2] = {cuuint32_t(kBlockK), cuuint32_t(box_rows)};
    cuuint32_t element_strides[2] = {1, 1};
    CUresult status = encode_tiled()(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims,
                                     strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                     CU_TENSOR_MAP_SWIZZLE_128B,
                                     weights ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS)
        throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(int(status)));
    return map;
}

// Group-major fp32 scales [K/128, rows]: box = 128 consecutive rows of one K group, no swizzle,
// rows past the end read as zero.
CUtensorMap scale_map(const float *base, int rows, int groups) {
    if (reinterpret_cast<uintptr_t>(base) % 16 || rows % 4)
        throw std::invalid_argument("K-group scales must be 16-byte aligned with a row count that is a multiple of 4");
    CUtensorMap map;
    cuuint64_t dims[2] = {cuuint64_t(rows), cuuint64_t(groups)};
    cuuint64_t strides[1] = {cuuint64_t(rows) * 4};
    cuuint32_t box[2] = {cuuint32_t(kGroupedTokens), 1};
    cuuint32_t element_strides[2] = {1, 1};
    CUresult status = encode_tiled()(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides,
                                     box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (status != CUDA_SUCCESS)
        throw std::runtime_error("cuTensorMapEncodeTiled (scales) failed with code " + std::to_string(int(status)));
    return map;
}

// Split-K launches group the `splits` CTAs of one output tile into a thread-block cluster (1,1,splits).
template <Type F, bool Grouped, int BN>
void launch_instance(const CUtensorMap &map_w, const CUtensorMap &map_x, const GemmArgs &args, dim3 grid,
                     size_t smem, cudaStream_t stream) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = dim3(kGemmThreads);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    unsigned count = 0;
    // Programmatic dependent launch: the prologue and the weight prefetch may overlap the upstream
    // kernel; the kernel itself waits before touching anything upstream produces.
    attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[count].val.programmaticStreamSerializationAllowed = 1;
    ++count;
    if (args.splits > 1) {
        attributes[count].id = cudaLaunchAttributeClusterDimension;
        attributes[count].val.clusterDim.x = 1;
        attributes[count].val.clusterDim.y = 1;
        attributes[count].val.clusterDim.z = unsigned(args.splits);
        ++count;
    }
    config.attrs = attributes;
    config.numAttrs = count;
    check(cudaLaunchKernelEx(&config, w8a8_tcgen05_gemm<F, Grouped, BN>, map_w, map_x, args), "quantized GEMM launch");
}
template <Type F, bool Grouped>
void launch_tokens(int bn, const CUtensorMap &map_w, const CUtensorMap &map_x, const GemmArgs &args, dim3 grid,
                   size_t smem, cudaStream_t stream) {
    switch (bn) {
    case 16: launch_instance<F, Grouped, 16>(map_w, map_x, args, grid, smem, stream); break;
    case 32: launch_instance<F, Grouped, 32>(map_w, map_x, args, grid, smem, stream); break;
    case 64: launch_instance<F, Grouped, 64>(map_w, map_x, args, grid, smem, stream); break;
    case 128: launch_instance<F, Grouped, 128>(map_w, map_x, args, grid, smem, stream); break;
    case 256:
        if constexpr (!Grouped) { launch_instance<F, false, 256>(map_w, map_x, args, grid, smem, stream); break; }
        [[fallthrough]];
    default: throw std::invalid_argument("unsupported token tile for the tcgen05 GEMM");
    }
}

template <Type F, bool Grouped, int BN> void raise_limit() {
    check(cudaFuncSetAttribute(w8a8_tcgen05_gemm<F, Grouped, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               int(kSmemBudget)),
          "cudaFuncSetAttribute(shared memory)");
}
constexpr size_t kPrefillSmem = 1024 + size_t(kPrefillStages) * (kBlockChannels + kPrefillTokens) * kBlockK + kPrefillPatchBytes;
int multiprocessor_count() {
    static std::atomic<int> cached[64];
    int device = 0;
    check(cudaGetDevice(&device), "cudaGetDevice");
    if (device < 0 || device >= 64) return 148;
    int count = cached[device].load(std::memory_order_relaxed);
    if (!count) {
        check(cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device), "cudaDeviceGetAttribute");
        cached[device].store(count, std::memory_order_relaxed);
    }
    return count;
}
template <Type F>
void launch_prefill(const CUtensorMap &map_w, const CUtensorMap &map_x, const PrefillArgs &args, cudaStream_t stream) {
    const int tiles = ((args.n + kBlockChannels - 1) / kBlockChannels) * ((args.m + kPrefillTokens - 1) / kPrefillTokens);
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(unsigned(std::min(tiles, multiprocessor_count())));
    config.blockDim = dim3(kGemmThreads);
    config.dynamicSmemBytes = kPrefillSmem;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    check(cudaLaunchKernelEx(&config, w8a8_tcgen05_prefill<F>, map_w, map_x, args), "quantized prefill GEMM launch");
}

constexpr size_t kPairSmem = 1024 + size_t(kPairStages) * (kBlockChannels + kPrefillTokens / 2) * kBlockK + kPrefillPatchBytes;
// CTA pairs: one cluster of two per 256-channel x 256-token tile, persistent over the tiles.
template <Type F>
void launch_prefill_pair(const CUtensorMap &map_w, const CUtensorMap &map_x, const PrefillArgs &args, cudaStream_t stream) {
    const int tiles = ((args.n + 2 * kBlockChannels - 1) / (2 * kBlockChannels)) * ((args.m + kPrefillTokens - 1) / kPrefillTokens);
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(2u * unsigned(std::min(tiles, multiprocessor_count() / 2)));
    config.blockDim = dim3(kGemmThreads);
    config.dynamicSmemBytes = kPairSmem;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    // Up to 4096 output channels the tile runs with the tokens as MMA rows (epilogue straight from registers).
    if (args.n <= 4096)
        check(cudaLaunchKernelEx(&config, w8a8_tcgen05_prefill_pair<F, true>, map_w, map_x, args), "quantized pair GEMM launch");
    else
        check(cudaLaunchKernelEx(&config, w8a8_tcgen05_prefill_pair<F, false>, map_w, map_x, args), "quantized pair GEMM launch");
}

// Persistent K-group kernel: one CTA per multiprocessor over 128x128 tiles.
template <Type F>
void launch_prefill_grouped(const CUtensorMap &map_w, const CUtensorMap &map_x, const CUtensorMap &map_sw,
                            const CUtensorMap &map_sx, const PrefillArgs &args, cudaStream_t stream) {
    const int tiles = ((args.n + kBlockChannels - 1) / kBlockChannels) * ((args.m + kGroupedTokens - 1) / kGroupedTokens);
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(unsigned(std::min(tiles, multiprocessor_count())));
    config.blockDim = dim3(kGroupedThreads);
    config.dynamicSmemBytes = kGroupedSmem;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    check(cudaLaunchKernelEx(&config, w8a8_tcgen05_prefill_grouped<F>, map_w, map_x, map_sw, map_sx, args),
          "quantized K-group prefill GEMM launch");
}

template <Type F> void raise_limits() {
    check(cudaFuncSetAttribute(w8a8_tcgen05_prefill_grouped<F>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kGroupedSmem)),
          "cudaFuncSetAttribute(shared memory)");
    check(cudaFuncSetAttribute(w8a8_tcgen05_prefill_pair<F>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kPairSmem)),
          "cudaFuncSetAttribute(shared memory)");
    check(cudaFuncSetAttribute(w8a8_tcgen05_prefill_pair<F, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kPairSmem)),
          "cudaFuncSetAttribute(shared memory)");
    check(cudaFuncSetAttribute(w8a8_tcgen05_prefill<F>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kPrefillSmem)),
          "cudaFuncSetAttribute(shared memory)");
    raise_limit<F, false, 16>(); raise_limit<F, false, 32>(); raise_limit<F, false, 64>();
    raise_limit<F, false, 128>(); raise_limit<F, false, 256>();
    raise_limit<F, true, 16>(); raise_limit<F, true, 32>(); raise_limit<F, true, 64>(); raise_limit<F, true, 128>();
}
} // namespace

void quant_linear_initialize(int device) {
    static std::mutex guard;
    static std::map<int, bool> done;
    std::lock_guard<std::mutex> lock(guard);
    if (done[device]) return;
    int current = 0;
    check(cudaGetDevice(&current), "cudaGetDevice");
    check(cudaSetDevice(device), "cudaSetDevice");
    cudaDeviceProp p{};
    check(cudaGetDeviceProperties(&p, device), "cudaGetDeviceProperties");
    if (p.major != 10)
        throw std::runtime_error("this library only carries sm_100a kernels; device is sm_" +
                                 std::to_string(p.major) + std::to_string(p.minor));
    raise_limits<Type::I8>();
    raise_limits<Type::FP8>();
    encode_tiled();
    check(cudaSetDevice(current), "cudaSetDevice");
    done[device] = true;
}

void quant_linear_reset_workspace(void *workspace, size_t bytes, cudaStream_t stream) {
    if (!workspace || bytes < kWorkspaceHeader) throw std::invalid_argument("GEMM workspace is smaller than its header");
    check(cudaMemsetAsync(workspace, 0, kWorkspaceHeader, stream), "cudaMemsetAsync(workspace header)");
}

int quant_linear_status(const void *workspace, cudaStream_t stream) {
    int status = 0;
    check(cudaMemcpyAsync(&status, static_cast<const char *>(workspace) + kStatusOffset, sizeof(int),
                          cudaMemcpyDeviceToHost, stream),
          "cudaMemcpyAsync(status)");
    check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    return status;
}

// Split-K partials live in shared memory, so every path needs only the status header.
size_t quant_linear_workspace_bytes(LinearPath, KernelProblem) { return kWorkspaceHeader; }

namespace {
struct WaitExpiry {
    int extra_bytes = 0;
    long long limit_cycles = 0;
};
thread_local WaitExpiry pending_expiry;
} // namespace
void quant_linear_inject_wait_expiry(int extra_bytes, long long limit_cycles) {
    if (extra_bytes < 0 || extra_bytes > 1024 || limit_cycles < 0) throw std::invalid_argument("invalid wait-expiry injection");
    pending_expiry = {extra_bytes, limit_cycles};
}

LinearPath select_tcgen05_path(KernelProblem p, Type format, int sms, size_t workspace_bytes) {
    return select_linear(p, KernelLimits{false, 0, workspace_bytes}, format, ChipModel::b200(sms));
}

WeightMaps quant_linear_weight_maps(const void *weights, int channels, int reduction) {
    WeightMaps maps;
    maps.values = operand_map(weights, channels, reduction, kBlockChannels, true);
    maps.weights = weights;
    maps.channels = channels;
    maps.reduction = reduction;
    return maps;
}

void launch_quant_linear(LinearPath config, KernelProblem shape, const void *input, const float *xs,
                         const void *weights, const float *ws, void *y, void *workspace, size_t bytes,
                         cudaStream_t stream, Type format, Type output_type, const ops::Epilogue *finish,
                         const WeightMaps *prepared) {
    const bool grouped = shape.input_group || shape.weight_group;
    if (output_type != Type::BF16 && output_type != Type::F16 &&
        !(output_type == Type::I32 && format == Type::I8 && !grouped && !finish))
        throw std::invalid_argument("quantized GEMM output must be F16 or BF16");
    if (format != Type::I8 && format != Type::FP8) throw std::invalid_argument("unsupported quantized storage type");
    if (config.kind != LinearKind::Tcgen05)
        throw std::invalid_argument("this build executes LinearKind::Tcgen05 paths only");
    if (shape.rows < 1 || shape.channels < 1 || shape.reduction < 1 || shape.reduction % 16 || shape.channels % 16)
        throw std::invalid_argument("quantized GEMM unsupported shape");
    if (format == Type::I8 && shape.reduction > INT32_MAX / (128 * 128))
        throw std::invalid_argument("INT8 reduction can overflow INT32");
    for (int group : {shape.input_group, shape.weight_group})
        if (group && group != 32 && group != 64 && group != 128)
            throw std::invalid_argument("unsupported GEMM quantization group size");
    if (!input || !xs || !weights || !ws || !y) throw std::invalid_argument("quantized GEMM null operand");
    const int kb_total = (shape.reduction + kBlockK - 1) / kBlockK;
    const int bn = config.tokens, splits = config.splits;
    if (config.channels != kBlockChannels || splits < 1 || splits > kb_total || splits > kMaxSplits)
        throw std::invalid_argument("invalid tcgen05 tile or split (splits form a cluster of at most 8 CTAs)");
    const int n_tiles = (shape.channels + kBlockChannels - 1) / kBlockChannels, m_tiles = (shape.rows + bn - 1) / bn;
    if (m_tiles > 65535 || splits > 65535) throw std::invalid_argument("quantized GEMM grid exceeds capacity");
    if (!workspace || bytes < kWorkspaceHeader) throw std::invalid_argument("quantized GEMM workspace missing");

    GemmArgs args{};
    args.m = shape.rows; args.n = shape.channels; args.k = shape.reduction;
    args.sx = xs; args.sw = ws; args.out = y; args.out_type = int(output_type);
    args.input_group = shape.input_group; args.weight_group = shape.weight_group;
    args.splits = splits;
    args.status = reinterpret_cast<int *>(static_cast<char *>(workspace) + kStatusOffset);
    auto aligned16 = [](const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    bool vector_io = aligned16(y) && shape.channels % 8 == 0;
    if (finish) {
        const auto &e = *finish;
        if (!ops::fusable(e)) throw std::invalid_argument("unsupported quantized native Finish path");
        auto same_type = [&](const TensorView &v) { return !v.data || v.type == output_type; };
        if (!same_type(e.bias) || !same_type(e.residual) ||
            (e.bias.data && e.bias.numel() != size_t(shape.channels)) ||
            (e.residual.data && (e.residual.rows != shape.rows || e.residual.cols != shape.channels)) ||
            (e.residual_f32.data && (e.residual_f32.type != Type::F32 || !e.residual_f32.dense() ||
                                     e.residual_f32.rows != shape.rows || e.residual_f32.cols != shape.channels)))
            throw std::invalid_argument("quantized linear finish operand mismatch");
        args.ep.bias = e.bias.data;
        args.ep.residual = e.residual.data;
        args.ep.residual_ld = e.residual.data ? e.residual.ld() : 0;
        args.ep.residual_f32 = e.residual_f32.ptr<const float>();
        args.ep.value_scale = e.value_scale; args.ep.residual_scale = e.residual_scale;
        args.ep.output_scale = e.output_scale; args.ep.alpha = e.alpha;
        args.ep.activation = int(e.activation);
        args.ep.chain = e.bias.data || e.residual.data || e.value_scale != 1.f || e.output_scale != 1.f ||
                        e.activation != ops::Activation::Identity;
        vector_io = vector_io && aligned16(e.residual_f32.data);
    }
    args.vector_io = vector_io;
    // The weight map is the caller's prepared one when it describes these weights, else built here.
    CUtensorMap local_w;
    const bool reuse = prepared && prepared->weights == weights && prepared->channels == shape.channels &&
                       prepared->reduction == shape.reduction;
    if (!reuse) local_w = operand_map(weights, shape.channels, shape.reduction, kBlockChannels, true);
    const CUtensorMap &map_w = reuse ? prepared->values : local_w;
    // Compute-bound shapes with a plain epilogue take the persistent, double-buffered kernels:
    // CTA pairs (each CTA loads half of the token tile) when there are at least two channel tiles.
    if (!grouped && bn == kPrefillTokens && splits == 1 && !args.ep.chain && output_type != Type::I32 && args.vector_io) {
        PrefillArgs prefill{args.m, args.n, args.k, xs, ws, y, int(output_type), args.ep.residual_f32, args.status};
        if (shape.channels >= 2 * kBlockChannels) {
            const CUtensorMap map_half = operand_map(input, shape.rows, shape.reduction, kPrefillTokens / 2, false);
            if (format == Type::I8) launch_prefill_pair<Type::I8>(map_w, map_half, prefill, stream);
            else launch_prefill_pair<Type::FP8>(map_w, map_half, prefill, stream);
            return;
        }
        const CUtensorMap map_x = operand_map(input, shape.rows, shape.reduction, bn, false);
        if (format == Type::I8) launch_prefill<Type::I8>(map_w, map_x, prefill, stream);
        else launch_prefill<Type::FP8>(map_w, map_x, prefill, stream);
        return;
    }
    // Compute-bound K-group shapes (both operands grouped by 128, enough 128x128 tiles to fill most of
    // the GPU, plain epilogue, no split) take the persistent K-group kernel.
    if (grouped && shape.input_group == kBlockK && shape.weight_group == kBlockK && bn == kGroupedTokens && splits == 1 &&
        !args.ep.chain && args.vector_io && shape.rows % 4 == 0 &&
        int64_t(n_tiles) * ((shape.rows + kGroupedTokens - 1) / kGroupedTokens) >= int64_t(multiprocessor_count()) * 2 / 3) {
        PrefillArgs prefill{args.m, args.n, args.k, xs, ws, y, int(output_type), args.ep.residual_f32, args.status};
        const CUtensorMap map_x = operand_map(input, shape.rows, shape.reduction, kGroupedTokens, false);
        const CUtensorMap map_sw = scale_map(ws, shape.channels, kb_total);
        const CUtensorMap map_sx = scale_map(xs, shape.rows, kb_total);
        if (format == Type::I8) launch_prefill_grouped<Type::I8>(map_w, map_x, map_sw, map_sx, prefill, stream);
        else launch_prefill_grouped<Type::FP8>(map_w, map_x, map_sw, map_sx, prefill, stream);
        return;
    }
    const CUtensorMap map_x = operand_map(input, shape.rows, shape.reduction, bn, false);
    LaunchShape launch = launch_shape(bn, grouped, (kb_total + splits - 1) / splits, splits,
                                      group_units(shape.input_group, shape.weight_group));
    if (!launch.fits)
        throw std::invalid_argument("quantized GEMM: this tile/split combination exceeds shared memory; use more splits");
    // A K-group CTA allocates all 512 columns of tensor memory, so two of them must never share a
    // multiprocessor (the second allocation would wait for the first CTA, and with split-K clusters
    // two such waits can form a cycle): ask for more than half of the shared memory.
    if (grouped) launch.smem = std::max(launch.smem, size_t(120) * 1024);
    args.expiry_extra_bytes = pending_expiry.extra_bytes; // one-shot, only the weight-streaming kernel honours it
    args.wait_limit_cycles = pending_expiry.limit_cycles;
    pending_expiry = {};
    args.stages = launch.stages;
    args.tile_region = int(launch.tile_region);
    args.owned_passes = launch.owned_passes;
    dim3 grid(n_tiles, m_tiles, splits);
    if (format == Type::I8) {
        if (grouped) launch_tokens<Type::I8, true>(bn, map_w, map_x, args, grid, launch.smem, stream);
        else launch_tokens<Type::I8, false>(bn, map_w, map_x, args, grid, launch.smem, stream);
    } else {
        if (grouped) launch_tokens<Type::FP8, true>(bn, map_w, map_x, args, grid, launch.smem, stream);
        else launch_tokens<Type::FP8, false>(bn, map_w, map_x, args, grid, launch.smem, stream);
    }
}

void grouped_quant_gemm(KernelProblem problem, const void *input, const float *input_scales,
                        const void *weights, const float *weight_scales, void *output, cudaStream_t stream,
                        Type format, Type output_type, int tokens, int splits, void *workspace,
                        size_t workspace_bytes) {
    if (!problem.input_group && !problem.weight_group)
        throw std::invalid_argument("group scales require a grouped GEMM implementation");
    launch_quant_linear({LinearKind::Tcgen05, tokens, kBlockChannels, splits}, problem, input, input_scales, weights,
                        weight_scales, output, workspace, workspace_bytes, stream, format, output_type, nullptr);
}

KernelResources quant_linear_finish_resources(LinearPath, Type, Type) { return {}; }
} // namespace tts
