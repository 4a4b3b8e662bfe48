/* b200q — C ABI of the B200-native quantized linear path of breeze_tts_cpp.
 *
 * The reference engine exposes quantization only as the `quantization` string of tts_create
 * (include/tts/tts.h:68-73); its quantized ops are internal C++ free functions. This header is the
 * op-granular doorway a maintainer (or a test, or a non-C++ caller) binds instead of those
 * internal functions. Every entry point cites the reference interface it stands in for.
 *
 * Conventions (same as the reference's bindings/c_api.cpp:25-40): every call returns 0 on success
 * and -1 on failure, copying a message into `error` (capacity `error_capacity`, may be NULL).
 * All device pointers are borrowed; nothing here allocates at call time except the *_create calls.
 * Weights and weight scales must be complete on the device (stream-synchronized, or ordered by an
 * ordinary stream dependency) before the first GEMM that reads them is enqueued: the GEMM kernels
 * prefetch weight tiles and weight scales ahead of their wait on the preceding kernel.
 * Type codes are the integer values of the reference's tts::Type (src/core/tensor.h:8):
 * BF16=0 F32=1 I32=2 FP8=3 I8=4 F16=5.
 */
#ifndef B200Q_H
#define B200Q_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum { B200Q_BF16 = 0, B200Q_F32 = 1, B200Q_I32 = 2, B200Q_FP8 = 3, B200Q_I8 = 4, B200Q_F16 = 5 };

/* reference: tts::TensorView (src/core/tensor.h:27-119). stride in elements, 0 = dense. */
typedef struct b200q_tensor {
    void *data;
    int32_t rows, cols, stride, type, device;
} b200q_tensor;

/* reference: tts::RowScaledView (src/core/quantization.h:33-49). scales are [rows] fp32, or
 * group-major [ceil(cols/group_size), rows] when group_size != 0. */
typedef struct b200q_row_scaled {
    b200q_tensor values, scales;
    int32_t group_size, rotation_size;
} b200q_row_scaled;

/* reference: tts::ops::Epilogue (src/ops/sequence.h:8-27), plus the fp32 residual of the synthetic
 * decode workload. activation uses ops::Activation codes (src/ops/activation.h:4): 0 identity, 1 relu,
 * 2 leaky relu, 3 silu, 4 gelu, 5 gelu-tanh, 6 mish, 7 tanh, 8 sigmoid. gate and condition are
 * [1, N] or [sequences, N]; raw receives the pre-activation value; rows past
 * valid_rows_per_sequence inside each sequence of rows_per_sequence rows are zeroed (0 = no masking);
 * residual_rows (device int32 per output row, negative = no residual) indexes the residual rows;
 * input_repeat > 1 reads input row r / input_repeat (finishing passes only). Zero-initialise the
 * struct and set value_scale = output_scale = residual_scale = 1, rows_per_sequence = input_repeat = 1.
 * bias, residual, residual_f32, the scales and activations 0-5,7,8 ride inside the GEMM; everything
 * else runs as a separate finishing pass, as in the reference (src/ops/linear.cpp:76-82). */
typedef struct b200q_epilogue {
    b200q_tensor bias, residual, residual_f32;
    float value_scale, output_scale, residual_scale, alpha;
    int32_t activation;
    b200q_tensor gate, condition, raw;
    int32_t rows_per_sequence, valid_rows_per_sequence, input_repeat;
    const int32_t *residual_rows;
} b200q_epilogue;

/* reference: tts::ops::NormFusion (src/ops/sequence.h:53-57): what is added to a row before
 * LayerNorm (projection bias, gate, residual; raw keeps that sum) and the per-sequence modulation
 * applied after it (scale, shift). source_rows (device int32 per output row) gathers input rows. */
typedef struct b200q_norm_fusion {
    b200q_tensor residual, projection_bias, raw, gate, shift, scale;
    int32_t rows_per_sequence;
    const int32_t *source_rows;
} b200q_norm_fusion;

/* reference: tts::LinearPath (src/ops/kernels/quant/kernel_config.h:5-9). kind 5 = tcgen05. */
typedef struct b200q_path {
    int32_t kind, tokens, channels, splits;
} b200q_path;

typedef struct b200q_context b200q_context;

/* "b200q <version>; quantization=int8,fp8,group_int8,group_fp8" — reference: tts_version(). */
const char *b200q_version(void);

/* reference: CudaContext + QuantizedGemm construction (src/runtime/cuda_context.cpp:45-80).
 * `quantization` is one of the reference's mode strings. `stream` is a cudaStream_t (NULL = default
 * stream). `workspace` NULL lets the context own 8 MiB; otherwise it borrows the caller's memory,
 * whose first 32 KiB it zeroes once. One-time device set-up happens here, so create the context
 * before any stream capture. */
int b200q_context_create(int32_t device, void *stream, void *workspace, size_t workspace_bytes,
                         const char *quantization, b200q_context **out, char *error, size_t error_capacity);
void b200q_context_destroy(b200q_context *);

/* reference: ops::quantize_rows / launch_row_quantize (src/ops/storage.h:12,
 * src/ops/kernels/quant/row_quantize.h:6). source is BF16 or F16. */
int b200q_row_quantize(b200q_context *, const b200q_tensor *source, const b200q_row_scaled *destination,
                       char *error, size_t error_capacity);

/* reference: ops::quantized_norm / launch_quantized_norm (src/ops/basic.h:33-34,
 * src/ops/kernels/quant/quant_norm.h:5-7). update, update_scale may have data == NULL. */
int b200q_quantized_norm(b200q_context *, const b200q_tensor *residual, const b200q_tensor *update,
                         const b200q_tensor *weight, const b200q_row_scaled *output, float epsilon,
                         int32_t gemma, const b200q_tensor *update_scale, char *error, size_t error_capacity);

/* reference: ops::quantized_gated / launch_quantized_gated (src/ops/basic.h:35,
 * src/ops/kernels/quant/quant_gated.h:7-8). input is [rows, 2*K]; kind 0 SiLU, 1 tanh-GELU. */
int b200q_quantized_gated(b200q_context *, const b200q_tensor *input, const b200q_row_scaled *output,
                          int32_t kind, char *error, size_t error_capacity);

/* reference: ops::prepare_quantized / QuantizedGemm::prepare (src/ops/basic.h:25-26,
 * src/ops/cuda/quantization.h:27-28). Plans are keyed by the row-capacity class of `rows`. */
int b200q_prepare(b200q_context *, int32_t rows, int32_t output_channels, int32_t input_channels,
                  int32_t output_type, int32_t activation_group, int32_t weight_group, b200q_path *chosen,
                  char *error, size_t error_capacity);
/* reference: the weight argument of ops::prepare_quantized (src/ops/basic.h:25-26). Builds the TMA
 * descriptor of a quantized weight matrix once, before b200q_seal, so that launches on that weight
 * need not encode it. Optional: weights that were never announced still work. */
int b200q_prepare_weight(b200q_context *, const b200q_row_scaled *weight, char *error, size_t error_capacity);
/* reference: QuantizedGemm::seal / ops::seal (src/ops/cuda/quantization.h:24). */
int b200q_seal(b200q_context *, char *error, size_t error_capacity);

/* reference: ops::matmul(RowScaledView, RowScaledView, TensorView) / QuantizedGemm::linear and
 * linear_finish (src/ops/basic.h:11, src/ops/cuda/quantization.h:31-33). epilogue may be NULL. */
int b200q_linear(b200q_context *, const b200q_row_scaled *input, const b200q_row_scaled *weight,
                 const b200q_tensor *output, const b200q_epilogue *epilogue, char *error, size_t error_capacity);

/* reference: launch_quant_linear (src/ops/kernels/quant/quant_dispatch.h:11-15) with an explicit
 * path, bypassing the plan cache. output type I32 returns the raw INT32 accumulators
 * (per-row INT8 only, no epilogue). */
int b200q_quant_linear(b200q_context *, const b200q_path *path, const b200q_row_scaled *input,
                       const b200q_row_scaled *weight, const b200q_tensor *output, const b200q_epilogue *epilogue,
                       char *error, size_t error_capacity);
/* The path the planner would choose for a problem (reference: select_linear,
 * src/ops/cuda/quantization_policy.h:32-33). */
int b200q_select_path(b200q_context *, int32_t rows, int32_t output_channels, int32_t input_channels,
                      int32_t activation_group, int32_t weight_group, b200q_path *chosen, char *error,
                      size_t error_capacity);

/* reference: ops::linear with a dense activation (src/ops/linear.h:11-14): quantize `input` into
 * `scratch`, run the GEMM with the epilogue fused where it can be and as a finishing pass where it
 * cannot; with `quantized_output` (may be NULL) the finished rows are also quantized for the next
 * projection. */
int b200q_linear_forward(b200q_context *, const b200q_tensor *input, const b200q_row_scaled *weight,
                         const b200q_row_scaled *scratch, const b200q_tensor *output,
                         const b200q_epilogue *epilogue, const b200q_row_scaled *quantized_output, char *error,
                         size_t error_capacity);

/* reference: ops::pointwise (src/ops/sequence.h:35): y = finish(x) as a pass of its own; x may be y. */
int b200q_pointwise(b200q_context *, const b200q_tensor *x, const b200q_tensor *y, const b200q_epilogue *epilogue,
                    char *error, size_t error_capacity);
/* reference: ops::pointwise_quantize (src/ops/sequence.h:36-41): finish(x), rounded to x's type,
 * optionally kept in `retained` (may be NULL), quantized in the same pass. */
int b200q_pointwise_quantize(b200q_context *, const b200q_tensor *x, const b200q_row_scaled *quantized,
                             const b200q_epilogue *epilogue, const b200q_tensor *retained, char *error,
                             size_t error_capacity);
/* reference: ops::layer_norm_quantize (src/ops/sequence.h:60-63). weight, bias, fusion, retained may
 * be NULL / have data == NULL. Rows of up to 8192 columns. */
int b200q_layer_norm_quantize(b200q_context *, const b200q_tensor *x, const b200q_row_scaled *quantized,
                              const b200q_tensor *weight, const b200q_tensor *bias, float epsilon,
                              const b200q_norm_fusion *fusion, const b200q_tensor *retained, char *error,
                              size_t error_capacity);
/* reference: ops::normalized_linear over a quantized weight (src/ops/linear.h:15-18): LayerNorm +
 * quantize + projection + bias/ReLU in one launch when K <= 512 with per-row scales. *taken = 0 means
 * the fused kernel declined (nothing was launched) and the caller runs the two-step path. */
int b200q_normalized_linear(b200q_context *, const b200q_tensor *input, const b200q_row_scaled *weight,
                            const b200q_tensor *bias, const b200q_tensor *normalized, const b200q_tensor *output,
                            const b200q_tensor *norm_weight, const b200q_tensor *norm_bias, float epsilon,
                            const b200q_norm_fusion *fusion, const b200q_epilogue *epilogue,
                            const b200q_row_scaled *quantized_output, int32_t *taken, char *error, size_t error_capacity);

/* ---- Linear layer object --------------------------------------------------------------------
 * reference: tts::Linear (src/layers/linear.h:11-76) over a quantized weight, with the load-time
 * step of Weights::quantized (src/io/weights.cpp:80-87,133-154): `parts` are `part_count` 16-bit
 * [N_i, K] matrices fused by rows (Q,K,V -> QKV; gate,up -> gate_up) and quantized on the device
 * into storage the layer owns, in the context's mode. bias may be NULL or have data == NULL. */
typedef struct b200q_linear_layer b200q_linear_layer;
int b200q_linear_layer_create(b200q_context *, const b200q_tensor *parts, int32_t part_count, const b200q_tensor *bias,
                              b200q_linear_layer **out, char *error, size_t error_capacity);
void b200q_linear_layer_destroy(b200q_linear_layer *);
/* reference: Linear::prepare_range (src/layers/linear.cpp:132-148): plans for every row class up to
 * max_rows, and the layer's activation scratch (QuantizationWorkspace) sized for max_rows. */
int b200q_linear_layer_prepare(b200q_context *, b200q_linear_layer *, int32_t max_rows, char *error, size_t error_capacity);
/* reference: Linear::forward(workspace, input, output, epilogue, quantized_output)
 * (src/layers/linear.h:66-68). quantized_output may be NULL. */
int b200q_linear_layer_forward(b200q_context *, b200q_linear_layer *, const b200q_tensor *input, const b200q_tensor *output,
                               const b200q_epilogue *epilogue, const b200q_row_scaled *quantized_output, char *error,
                               size_t error_capacity);
/* reference: Linear::forward(input, output, ForwardContext &, finish) and its phase switch
 * (src/layers/linear.cpp:49-76): mode 0 Plan and 2 Capture launch nothing, 1 Prepare plans every row
 * class up to max_rows and sizes the layer's activation scratch (before b200q_seal), 3 Execute runs
 * quantize -> GEMM -> epilogue and allocates nothing. */
int b200q_linear_layer_apply(b200q_context *, b200q_linear_layer *, int32_t mode, int32_t max_rows, const b200q_tensor *input,
                             const b200q_tensor *output, const b200q_epilogue *epilogue, char *error, size_t error_capacity);
/* reference: Linear::forward_segments (src/layers/linear.cpp:89-121). `segments` is a HOST array of
 * segment_count triples (first input row, row count, first output row). Same modes as above. */
int b200q_linear_layer_forward_segments(b200q_context *, b200q_linear_layer *, int32_t mode, int32_t max_rows,
                                        const b200q_tensor *input, const int32_t *segments, int32_t segment_count,
                                        const b200q_tensor *output, char *error, size_t error_capacity);
/* reference: Linear::normalized_forward with a workspace (src/layers/linear.cpp:195-214): LayerNorm of
 * the input fused with the projection (one launch when K <= 512 with per-row scales, else LayerNorm +
 * quantize followed by the GEMM). normalized, norm_bias, fusion, epilogue, quantized_output may be NULL.
 * The layer must have been prepared (b200q_linear_layer_prepare) for at least input->rows rows. */
int b200q_linear_layer_normalized_forward(b200q_context *, b200q_linear_layer *, const b200q_tensor *input,
                                          const b200q_tensor *normalized, const b200q_tensor *output,
                                          const b200q_tensor *norm_weight, const b200q_tensor *norm_bias, float epsilon,
                                          const b200q_norm_fusion *fusion, const b200q_epilogue *epilogue,
                                          const b200q_row_scaled *quantized_output, char *error, size_t error_capacity);
/* The layer's quantized weight view (borrowed; valid while the layer lives). */
int b200q_linear_layer_weight(b200q_linear_layer *, b200q_row_scaled *weight, char *error, size_t error_capacity);

/* No counterpart in the reference. The same GEMM as b200q_quant_linear for callers that cannot
 * allocate device memory (an engine whose pools are sealed, a region where cudaMalloc is not
 * allowed, a host that provides a stream but no workspace): needs no context and no workspace, its
 * 32 KiB of scratch is a device array built into the library. `path` NULL lets the planner choose.
 * Limits: one array per GPU shared by every call, so calls that overlap on the GPU race and each call
 * finds the previous call's contents (the status word is cleared per call: read it with
 * b200q_static_status before the next call); the caller's current device is left unchanged; problems needing more
 * than 32 KiB of scratch are rejected; the first call on a device does one-time set-up and should
 * come before any stream capture. */
int b200q_quant_linear_static(int32_t device, void *stream, const b200q_path *path, const b200q_row_scaled *input,
                              const b200q_row_scaled *weight, const b200q_tensor *output,
                              const b200q_epilogue *epilogue, char *error, size_t error_capacity);

/* No counterpart in the reference. Status word of the built-in scratch that
 * b200q_quant_linear_static uses on `device`: waits for `stream`, then returns 0 = clean, nonzero = a
 * bounded device-side wait gave up during the last static call (its output is invalid). Allocates
 * nothing. Each static call clears the word before it launches, so ask before the next call. */
int b200q_static_status(int32_t device, void *stream, int32_t *status, char *error, size_t error_capacity);

/* No counterpart in the reference. Exercises the failure path without faulting the GPU: the next
 * GEMM this thread launches through b200q_quant_linear (weight-streaming kernel, i.e. a token tile
 * below 256 or a split) expects `extra_bytes` (1..1024) more on its first weight barrier than the
 * copy delivers and gives up every device-side wait after `limit_cycles` SM cycles; it then leaves
 * through its normal teardown, writes no output and sets the status word. One-shot. */
int b200q_inject_wait_expiry(int32_t extra_bytes, int64_t limit_cycles, char *error, size_t error_capacity);

/* Blocks until the context's stream is idle and returns the device status word through `status`:
 * 0 = clean; nonzero = a bounded device-side wait gave up (results are invalid). */
int b200q_status(b200q_context *, int32_t *status, char *error, size_t error_capacity);
int b200q_multiprocessors(b200q_context *);

/* Host-only helpers (no GPU needed). Row-capacity class of a token count — reference:
 * row_capacity (src/core/row_capacity.h:10-19); returns -1 for invalid input. */
int32_t b200q_row_capacity(int32_t rows, uint32_t bins_per_octave);
/* The planner's choice without a context: pure function of the problem, the SM count and the
 * workspace size. format is B200Q_I8 or B200Q_FP8. */
int b200q_plan_path(int32_t rows, int32_t output_channels, int32_t input_channels, int32_t activation_group,
                    int32_t weight_group, int32_t format, int32_t multiprocessors, size_t workspace_bytes,
                    b200q_path *chosen, size_t *workspace_needed, char *error, size_t error_capacity);

/* The launch shapes the kernels accept for a problem — reference: quant_linear_candidates
 * (src/ops/cuda/quantization_policy.h:27-28). Writes up to `capacity` paths and returns how many
 * exist (which may exceed `capacity`), or -1 on error. Host only. */
int b200q_candidates(int32_t rows, int32_t output_channels, int32_t input_channels, int32_t activation_group,
                     int32_t weight_group, int32_t format, b200q_path *paths, int32_t capacity, char *error,
                     size_t error_capacity);
/* The planner's estimate, in microseconds, of one GEMM launch with `path` (fused == 0: plus the row
 * quantizer before it and a separate finishing pass after it) — reference: linear_pipeline_cost
 * (src/ops/cuda/quantization_policy.h:30-31). Host only; a negative value reports an error. */
double b200q_path_cost(int32_t rows, int32_t output_channels, int32_t input_channels, int32_t activation_group,
                       int32_t weight_group, int32_t format, const b200q_path *path, int32_t multiprocessors,
                       int32_t gemm_only, char *error, size_t error_capacity);

#ifdef __cplusplus
}
#endif
#endif
