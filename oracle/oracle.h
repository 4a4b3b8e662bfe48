/* TEST INFRASTRUCTURE ONLY — the CPU oracle of the quantized-linear path.
 *
 * A scalar restatement, in plain loops, of the arithmetic the reference's CUDA kernels perform.
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg may load it; the product
 * library never does.
 *
 * Pinned by outputs of the reference itself: the reference ships no tests, golden vectors or
 * known-answer fixtures for this path, so (1) the reference's own kernels are built from its sources
 * into oracle/_ref/libttsref.so and run beside this oracle on the same inputs (GPU tests), (2) their
 * outputs are stored beside the oracle's in the fixtures under tests/golden/ (`ref_*` keys, written by
 * tests/golden/make_golden.py --reference) and checked on the CPU, and (3) hand-derived known
 * answers in tests/test_oracle.py cover the scalar rules.
 *
 * Types are passed as the integer values of the reference's `tts::Type`
 * (src/core/tensor.h:8): BF16=0, F32=1, I32=2, FP8=3, I8=4, F16=5.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* Scalar conversions (round to nearest even). */
uint16_t oracle_f32_to_bf16(float x);
float oracle_bf16_to_f32(uint16_t x);
float oracle_f16_to_f32(uint16_t x);
uint8_t oracle_fp8_e4m3_encode(float x);       /* own software encoder, saturating to +-448 */
float oracle_fp8_e4m3_decode(uint8_t x);
uint8_t oracle_fp8_e4m3_encode_toolkit(float x); /* the CUDA toolkit's host conversion, for pinning */
uint8_t oracle_int8_encode(float x);           /* clamp +-127, round half even */
float oracle_scale(float amax, int format);    /* amax==0 ? 1 : max(amax/range, FLT_MIN) */
float oracle_rotation_sign(uint32_t column);

/* In-place sign flip + 128-point Hadamard + 2^-3.5 on one aligned block starting at `column`. */
void oracle_rotate128(float *block, int column);

/* Stage 1 / stage-3 producer. source: 16-bit [rows, cols] with row stride `stride` elements.
 * scales: [rows] when group==0, else group-major [ceil(cols/group), rows]. */
void oracle_row_quantize(const uint16_t *source, int source_type, int rows, int cols, int stride,
                         uint8_t *values, float *scales, int format, int group, int rotation);

/* Exact INT32 accumulators acc[m,n] = sum_k xq[m,k]*wq[n,k]. */
void oracle_int8_accumulate(const int8_t *xq, const int8_t *wq, int m, int n, int k, int32_t *acc);

/* Epilogue description for oracle_quant_linear. All pointers optional (NULL = absent). */
typedef struct {
    const uint16_t *bias;        /* [n], output dtype */
    const uint16_t *residual;    /* [m,n], output dtype: reference chain, rounded after the GEMM store */
    const float *residual_f32;   /* [m,n]: synthetic variant, added in fp32 before the single rounding */
    float value_scale, residual_scale, output_scale;
    int activation;              /* reference ops::Activation: 0 identity, 1 relu, 2 leaky relu, 3 silu, 4 gelu (erf),
                                    5 gelu-tanh, 6 mish, 7 tanh, 8 sigmoid */
    float alpha;                 /* negative slope of the leaky relu */
} oracle_epilogue;

/* Stage 2 / stage 3 GEMM + dequant. Output bf16 (type 0) or f16 (type 5) [m,n]; `exact` (optional)
 * receives the fp32 value before the last rounding. Per-row scales when both groups are 0,
 * otherwise K-group scales in group-major layout. `threads` >= 1 host threads split the channels. */
void oracle_quant_linear(const uint8_t *xq, const float *sx, const uint8_t *wq, const float *sw, int m,
                         int n, int k, int input_group, int weight_group, int format, int output_type,
                         uint16_t *output, float *exact, const oracle_epilogue *epilogue, int threads);

/* RMSNorm + quantize given the producer's rounding points; see oracle.cpp for what is and is not
 * reproducible on a CPU. residual is updated in place when update != NULL. */
void oracle_quantized_norm(uint16_t *residual, const uint16_t *update, const uint16_t *weight,
                           const uint16_t *update_scale, int rows, int cols, int type, float epsilon,
                           int gemma, uint16_t *normalized, uint8_t *values, float *scales, int format,
                           int group, int rotation);
/* act(gate)*up on [rows, 2*width] then quantize. kind 0 = SiLU, 1 = tanh-GELU. */
void oracle_quantized_gated(const uint16_t *input, int rows, int width, int type, int kind,
                            uint16_t *activated, uint8_t *values, float *scales, int format, int group,
                            int rotation);

/* The epilogue chain of the row-wise operators (reference ops::Epilogue, src/ops/sequence.h:8-27). Operands are dense
 * [rows, cols] arrays of the storage type; an operand with one row broadcasts. */
typedef struct {
    const uint16_t *bias;            /* [cols] */
    const uint16_t *gate;            /* [gate_rows, cols], indexed by sequence */
    const uint16_t *residual;        /* [residual_rows, cols] */
    const uint16_t *condition;       /* [condition_rows, cols], indexed by sequence */
    uint16_t *raw;                   /* [rows, cols]: receives the value before the activation */
    const int32_t *residual_index;   /* [rows]: row of `residual` each output row adds (-1 = none) */
    int gate_rows, residual_rows, condition_rows;
    int rows_per_sequence, valid_rows_per_sequence, input_repeat;
    float value_scale, residual_scale, output_scale, alpha;
    int activation;
} oracle_finish;
/* y[r] = finish(x[r / input_repeat]). */
void oracle_pointwise(const uint16_t *x, int x_rows, int rows, int cols, int type, const oracle_finish *finish, uint16_t *y);
/* finish, round to storage (kept in `retained` when given), then quantize the row. */
void oracle_pointwise_quantize(const uint16_t *x, int x_rows, int rows, int cols, int type, const oracle_finish *finish,
                               uint16_t *retained, uint8_t *values, float *scales, int format, int group, int rotation);

/* LayerNorm with the reference's row fusion (reference ops::NormFusion, src/ops/sequence.h:29-37). */
typedef struct {
    const uint16_t *weight, *bias;           /* [cols] */
    const uint16_t *projection_bias;         /* [cols], added to the input first */
    const uint16_t *residual;                /* [residual_rows, cols] */
    const uint16_t *gate, *scale, *shift;    /* [*_rows, cols], indexed by sequence */
    int residual_rows, gate_rows, scale_rows, shift_rows;
    int rows_per_sequence;
    const int32_t *source_rows;              /* [rows]: gathers input rows (layer_norm_quantize only) */
    float eps;
} oracle_norm;
void oracle_layer_norm_quantize(const uint16_t *x, int x_rows, int rows, int cols, int type, const oracle_norm *norm,
                                uint16_t *normalized, uint16_t *raw, uint8_t *values, float *scales, int format, int group,
                                int rotation);
/* LayerNorm + per-row quantize + projection by wq[channels, cols] (per-channel scales sw) + finish, K <= 512. */
void oracle_normalized_linear(const uint16_t *x, int rows, int cols, int type, const oracle_norm *norm, const uint8_t *wq,
                              const float *sw, int channels, int format, const oracle_finish *finish, uint16_t *out,
                              uint8_t *encoded, float *encoded_scales, uint16_t *normalized, uint16_t *raw);

/* Timed scalar host-core baseline: quantize + GEMM + dequant of one linear, `threads` threads.
 * Only the first `n_slice` channels are computed (n_slice == n for the whole matrix).
 * Returns seconds. */
double oracle_time_linear(const uint16_t *x, const uint8_t *wq, const float *sw, int m, int n, int k,
                          int n_slice, int format, int group, int rotation, uint16_t *output,
                          const float *residual_f32, int threads);
int oracle_hardware_threads(void);
#ifdef __cplusplus
}
#endif
