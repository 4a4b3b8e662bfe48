"""The row-wise operators around the quantized projections — the separate finishing pass, finish +
quantize, LayerNorm + quantize, and the fused norm + quantize + projection — against the reference's
own kernels on identical inputs (src/ops/kernels/sequence/sequence_pointwise.cu,
sequence_norm.cu, built into oracle/_ref).

Bar: bytes, scales and every 16-bit side output identical to the reference kernels' for every activation
(the transcendental ones are evaluated by the same device instruction sequences in both builds) and for
epilogue scales that are not powers of two (the reference build contracts its scale-and-add).
"""
import ctypes as C

import numpy as np
import pytest
import torch

from tests.oracle_binding import BF16, F16, FP8, I8, ref_epilogue, ref_fusion, ref_view

pytestmark = pytest.mark.gpu
DTYPES = {BF16: torch.bfloat16, F16: torch.float16}


def randn(rows, cols, seed, dtype, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(rows, cols, generator=g, device="cuda") * scale).to(dtype)


def bits(t):
    return t.contiguous().view(torch.int16 if t.element_size() == 2 else torch.uint8)


def steps_apart(a, b, dtype):
    """Largest distance in units of the storage type's spacing at the larger magnitude."""
    mantissa = 8 if dtype == torch.bfloat16 else 11
    a, b = a.double(), b.double()
    spacing = torch.maximum(a.abs(), b.abs()).clamp_min(1e-30).log2().floor().exp2() * 2.0 ** (1 - mantissa)
    return float(((a - b).abs() / spacing).max())


def quantized(rows, cols, fmt, group=0, rotation=0):
    from breeze_tts_cpp_b200 import ops
    return ops.RowScaledView.empty(rows, cols, fmt, group, rotation)


def ctx_mode(fmt, group):
    return ("group_" if group else "") + ("fp8" if fmt == FP8 else "int8")


def epilogue_case(rows, cols, dtype, seed, activation, what):
    """Keyword arguments understood both by ops._epilogue and by ref_epilogue."""
    sequences = rows // 4 if rows % 4 == 0 else 1
    kw = dict(activation=activation, alpha=0.25)
    if "bias" in what:
        kw["bias"] = randn(1, cols, seed + 1, dtype, 0.5)
    if "gate" in what:
        kw["gate"] = randn(sequences, cols, seed + 2, dtype)
        kw["rows_per_sequence"] = rows // sequences
    if "condition" in what:
        kw["condition"] = randn(1, cols, seed + 3, dtype)
        kw.setdefault("rows_per_sequence", rows // sequences)
    if "residual" in what:
        kw["residual"] = randn(rows, cols, seed + 4, dtype)
        kw.update(value_scale=0.5, residual_scale=2.0)
    if "indexed" in what:
        kw["residual"] = randn(5, cols, seed + 4, dtype)
        g = torch.Generator(device="cuda").manual_seed(seed)
        kw["residual_rows"] = torch.randint(-1, 5, (rows,), generator=g, device="cuda", dtype=torch.int32)
    if "mask" in what:
        kw.update(rows_per_sequence=rows // sequences, valid_rows_per_sequence=max(1, rows // sequences - 1))
    if "scale" in what:
        kw["output_scale"] = 0.25
    if "odd" in what:  # scales whose products round: a fused multiply-add anywhere in the chain would show
        kw.update(value_scale=0.7, residual_scale=1.3, output_scale=0.9)
    return kw


POINTWISE = [(16, 512, 0, "bias"), (64, 2048, 1, "bias gate residual raw"), (12, 776, 2, "bias condition mask raw scale"),
             (20, 4096, 1, "indexed gate"), (8, 100, 0, "bias residual"), (32, 1024, 6, "bias gate"), (32, 1024, 3, "bias scale"),
             (16, 640, 4, "residual"), (16, 640, 5, "bias"), (16, 640, 7, "condition"), (16, 640, 8, "bias raw"),
             (64, 2048, 0, "bias residual odd"), (24, 1000, 1, "bias gate residual raw odd"), (20, 512, 2, "indexed odd"),
             (64, 4096, 3, "bias odd"), (64, 4096, 4, "bias odd"), (64, 4096, 5, "bias residual odd"), (64, 4096, 6, "bias odd"),
             (64, 4096, 7, "bias odd"), (64, 4096, 8, "bias residual odd")]


@pytest.mark.parametrize("type_code", [BF16, F16])
@pytest.mark.parametrize("rows,cols,activation,what", POINTWISE)
def test_finishing_pass_matches_reference(reference_kernels, ctx_factory, type_code, rows, cols, activation, what):
    dtype = DTYPES[type_code]
    ctx = ctx_factory("int8")
    x = randn(rows, cols, 10 * rows + cols, dtype)
    kw = epilogue_case(rows, cols, dtype, rows + cols, activation, what)
    mine, theirs = torch.empty_like(x), torch.empty_like(x)
    raw_mine = torch.zeros_like(x) if "raw" in what else None
    raw_theirs = torch.zeros_like(x) if "raw" in what else None
    ctx.pointwise(x, mine, raw=raw_mine, **kw)
    ep = ref_epilogue(raw=raw_theirs, **kw)
    rc = reference_kernels.ttsref_pointwise(C.byref(ref_view(x)), C.byref(ref_view(theirs)), type_code, C.byref(ep), None)
    assert rc == 0, reference_kernels.ttsref_last_error()
    torch.cuda.synchronize()
    if raw_mine is not None:
        assert torch.equal(bits(raw_mine), bits(raw_theirs))
    assert torch.equal(bits(mine), bits(theirs))
    # in place
    again = x.clone()
    ctx.pointwise(again, again, raw=raw_mine, **kw)
    assert torch.equal(bits(again), bits(mine))


def test_finishing_pass_repeats_input_rows(reference_kernels, ctx_factory):
    ctx = ctx_factory("int8")
    x = randn(6, 256, 3, torch.bfloat16)
    bias = randn(1, 256, 4, torch.bfloat16)
    mine, theirs = torch.empty(18, 256, dtype=torch.bfloat16, device="cuda"), torch.empty(18, 256, dtype=torch.bfloat16, device="cuda")
    ctx.pointwise(x, mine, bias=bias, input_repeat=3, activation=1)
    ep = ref_epilogue(bias=bias, input_repeat=3, activation=1)
    assert reference_kernels.ttsref_pointwise(C.byref(ref_view(x)), C.byref(ref_view(theirs)), BF16, C.byref(ep), None) == 0
    torch.cuda.synchronize()
    assert torch.equal(bits(mine), bits(theirs))


QUANTIZE = [(16, 512, I8, 0, 0), (64, 2048, I8, 0, 0), (7, 3000, FP8, 0, 0), (64, 6144, I8, 0, 0), (5, 9000, I8, 0, 0),
            (3, 12288, FP8, 0, 0), (16, 2048, I8, 128, 128), (64, 6144, FP8, 128, 128), (9, 1024, I8, 128, 0),
            (12, 768, I8, 64, 0), (12, 768, FP8, 32, 0), (200, 4096, I8, 128, 128)]


@pytest.mark.parametrize("type_code", [BF16, F16])
@pytest.mark.parametrize("rows,cols,fmt,group,rotation", QUANTIZE)
@pytest.mark.parametrize("activation,what", [(1, "bias gate residual raw"), (0, "bias mask scale"), (3, "bias"),
                                             (0, "bias residual odd")])
def test_finish_and_quantize_matches_reference(reference_kernels, ctx_factory, type_code, rows, cols, fmt, group, rotation,
                                               activation, what):
    dtype = DTYPES[type_code]
    ctx = ctx_factory(ctx_mode(fmt, group))
    x = randn(rows, cols, rows + cols + fmt, dtype, 2.0)
    kw = epilogue_case(rows, cols, dtype, rows * 3 + cols, activation, what)
    mine, theirs = quantized(rows, cols, fmt, group, rotation), quantized(rows, cols, fmt, group, rotation)
    kept_mine, kept_theirs = torch.zeros_like(x), torch.zeros_like(x)
    raw_mine = torch.zeros_like(x) if "raw" in what else None
    raw_theirs = torch.zeros_like(x) if "raw" in what else None
    ctx.pointwise_quantize(x, mine, retained=kept_mine, raw=raw_mine, **kw)
    ep = ref_epilogue(raw=raw_theirs, **kw)
    rc = reference_kernels.ttsref_pointwise_quantize(C.byref(ref_view(x)), type_code, theirs.values.data_ptr(),
                                                     theirs.scales.data_ptr(), rows, cols, fmt, group, rotation, C.byref(ep),
                                                     C.byref(ref_view(kept_theirs)), 148, None)
    assert rc == 0, reference_kernels.ttsref_last_error()
    torch.cuda.synchronize()
    if raw_mine is not None:
        assert torch.equal(bits(raw_mine), bits(raw_theirs))
    assert torch.equal(bits(kept_mine), bits(kept_theirs))
    assert torch.equal(mine.scales.view(torch.int32), theirs.scales.view(torch.int32))
    assert torch.equal(mine.values, theirs.values)


def test_finish_and_quantize_rejects_bad_requests(ctx_factory):
    from breeze_tts_cpp_b200 import B200QError
    ctx = ctx_factory("int8")
    x = randn(8, 256, 1, torch.bfloat16)
    with pytest.raises(B200QError):  # rotation needs K-group scales (reference: sequence_internal.cuh:179-180)
        ctx.pointwise_quantize(x, quantized(8, 256, I8, 0, 128))
    with pytest.raises(B200QError):  # raw and retained may not overlap
        ctx.pointwise_quantize(x, quantized(8, 256, I8), retained=x, raw=x)
    with pytest.raises(B200QError):  # gate with the wrong number of sequences
        ctx.pointwise_quantize(x, quantized(8, 256, I8), gate=randn(3, 256, 2, torch.bfloat16), rows_per_sequence=4)


NORM = [(16, 256, I8, 0, 0, "weight bias"), (64, 768, I8, 0, 0, "weight bias residual raw"), (33, 1024, FP8, 0, 0, "weight"),
        (12, 2048, I8, 0, 0, "weight bias projection gate shift scale raw"), (8, 4096, I8, 0, 0, "weight bias"),
        (16, 1024, I8, 128, 128, "weight bias residual"), (16, 512, FP8, 128, 128, "weight bias"), (10, 1000, I8, 0, 0, "bias"),
        (16, 1536, FP8, 64, 0, "weight"), (16, 1024, I8, 0, 0, "weight bias gather")]


@pytest.mark.parametrize("type_code", [BF16, F16])
@pytest.mark.parametrize("rows,cols,fmt,group,rotation,what", NORM)
def test_layer_norm_quantize_matches_reference(reference_kernels, ctx_factory, type_code, rows, cols, fmt, group, rotation, what):
    dtype = DTYPES[type_code]
    ctx = ctx_factory(ctx_mode(fmt, group))
    x = randn(rows, cols, rows + cols, dtype, 1.5) + 0.25
    weight = randn(1, cols, 2, dtype, 0.2) + 1 if "weight" in what else None
    bias = randn(1, cols, 3, dtype, 0.3) if "bias" in what else None
    sequences = rows // 4 if rows % 4 == 0 else 1
    fusion = {}
    if "residual" in what:
        fusion["residual"] = randn(rows, cols, 4, dtype)
    if "projection" in what:
        fusion["projection_bias"] = randn(1, cols, 5, dtype, 0.5)
    for i, name in enumerate(("gate", "shift", "scale")):
        if name in what:
            fusion[name] = randn(sequences, cols, 6 + i, dtype, 0.5)
            fusion["rows_per_sequence"] = rows // sequences
    out_rows = rows
    if "gather" in what:
        out_rows = rows + 4
        g = torch.Generator(device="cuda").manual_seed(1)
        fusion["source_rows"] = torch.randint(-1, rows + 1, (out_rows,), generator=g, device="cuda", dtype=torch.int32)
    mine, theirs = quantized(out_rows, cols, fmt, group, rotation), quantized(out_rows, cols, fmt, group, rotation)
    kept_mine = torch.zeros(out_rows, cols, dtype=dtype, device="cuda")
    kept_theirs = torch.zeros_like(kept_mine)
    raw_mine = torch.zeros_like(kept_mine) if "raw" in what else None
    raw_theirs = torch.zeros_like(kept_mine) if "raw" in what else None
    ctx.layer_norm_quantize(x, mine, weight, bias, 1e-5, retained=kept_mine, raw=raw_mine, **fusion)
    fu = ref_fusion(raw=raw_theirs, **fusion)
    rc = reference_kernels.ttsref_layer_norm_quantize(C.byref(ref_view(x)), type_code, theirs.values.data_ptr(),
                                                      theirs.scales.data_ptr(), out_rows, cols, fmt, group, rotation,
                                                      C.byref(ref_view(weight)), C.byref(ref_view(bias)), 1e-5, C.byref(fu),
                                                      C.byref(ref_view(kept_theirs)), None)
    assert rc == 0, reference_kernels.ttsref_last_error()
    torch.cuda.synchronize()
    assert ctx.status() == 0
    if raw_mine is not None:
        assert torch.equal(bits(raw_mine), bits(raw_theirs))
    assert torch.equal(bits(kept_mine), bits(kept_theirs))  # NaN rows of a bad gather index included: same bits
    assert torch.equal(mine.scales.view(torch.int32), theirs.scales.view(torch.int32))
    assert torch.equal(mine.values, theirs.values)


PROJECT = [(16, 512, 1536, I8), (64, 256, 64, I8), (5, 384, 100, I8), (16, 512, 1536, FP8), (33, 128, 520, FP8), (1, 512, 512, I8)]


@pytest.mark.parametrize("type_code", [BF16, F16])
@pytest.mark.parametrize("rows,k,n,fmt", PROJECT)
@pytest.mark.parametrize("what", ["weight bias", "weight bias residual raw relu outbias"])
def test_fused_norm_projection_matches_reference(reference_kernels, ctx_factory, type_code, rows, k, n, fmt, what):
    from breeze_tts_cpp_b200 import ops
    dtype = DTYPES[type_code]
    ctx = ctx_factory(ctx_mode(fmt, 0))
    x = randn(rows, k, rows + k + n, dtype, 1.5)
    w16 = randn(n, k, 3, dtype, 0.05)
    wv = ctx.quantize_rows(w16, ops.RowScaledView.empty(n, k, fmt))
    norm_weight, norm_bias = randn(1, k, 4, dtype, 0.2) + 1, randn(1, k, 5, dtype, 0.3)
    fusion, epilogue = {}, {}
    raw_mine = raw_theirs = None
    if "residual" in what:
        fusion["residual"] = randn(rows, k, 6, dtype)
    if "raw" in what:
        raw_mine, raw_theirs = torch.zeros_like(x), torch.zeros_like(x)
    out_bias = randn(1, n, 7, dtype, 0.5) if "outbias" in what else None
    if "relu" in what:
        epilogue["activation"] = 1
    mine, theirs = torch.empty(rows, n, dtype=dtype, device="cuda"), torch.empty(rows, n, dtype=dtype, device="cuda")
    normalized_mine, normalized_theirs = torch.zeros_like(x), torch.zeros_like(x)
    taken = ctx.normalized_linear(x, wv, mine, norm_weight, norm_bias, 1e-5, bias=out_bias, normalized=normalized_mine,
                                  fusion=dict(raw=raw_mine, **fusion), **epilogue)
    assert taken and ctx.status() == 0
    ep = ref_epilogue(bias=out_bias, **epilogue)
    fu = ref_fusion(raw=raw_theirs, **fusion)
    encoded = ops.RowScaledView.empty(rows, k, fmt)
    rc = reference_kernels.ttsref_normalized_quantized_linear(
        C.byref(ref_view(x)), type_code, C.byref(ref_view(normalized_theirs)), C.byref(ref_view(norm_weight)),
        C.byref(ref_view(norm_bias)), 1e-5, C.byref(fu), wv.values.data_ptr(), wv.scales.data_ptr(), n, k, fmt,
        C.byref(ref_view(theirs)), C.byref(ep), encoded.values.data_ptr(), encoded.scales.data_ptr(), None)
    assert rc == 1, reference_kernels.ttsref_last_error()
    torch.cuda.synchronize()
    if raw_mine is not None:
        assert torch.equal(bits(raw_mine), bits(raw_theirs))
    assert torch.equal(bits(normalized_mine), bits(normalized_theirs))
    assert torch.equal(bits(mine), bits(theirs))
    # the row-level quantization inside the fused kernel equals LayerNorm + quantize as a pass of its own
    separate = ctx.layer_norm_quantize(x, ops.RowScaledView.empty(rows, k, fmt), norm_weight, norm_bias, 1e-5, **fusion)
    assert torch.equal(separate.values, encoded.values) and torch.equal(separate.scales.view(-1), encoded.scales.view(-1))


def test_fused_norm_projection_declines_what_the_reference_declines(ctx_factory):
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory("int8")
    x = randn(4, 1024, 1, torch.bfloat16)
    wv = ctx.quantize_rows(randn(64, 1024, 2, torch.bfloat16, 0.05), ops.RowScaledView.empty(64, 1024, I8))
    out = torch.empty(4, 64, dtype=torch.bfloat16, device="cuda")
    assert not ctx.normalized_linear(x, wv, out, randn(1, 1024, 3, torch.bfloat16))               # K > 512
    x = randn(4, 256, 1, torch.bfloat16)
    wv = ctx.quantize_rows(randn(64, 256, 2, torch.bfloat16, 0.05), ops.RowScaledView.empty(64, 256, I8))
    assert not ctx.normalized_linear(x, wv, out, randn(1, 256, 3, torch.bfloat16), activation=3)   # only identity / ReLU
    assert ctx.normalized_linear(x, wv, out, randn(1, 256, 3, torch.bfloat16), activation=1)


@pytest.mark.parametrize("mode,fmt,group", [("int8", I8, 0), ("group_fp8", FP8, 128)])
@pytest.mark.parametrize("requantize", [False, True])
def test_linear_with_an_epilogue_the_gemm_cannot_fuse(reference_kernels, ctx_factory, mode, fmt, group, requantize):
    """ops::linear with a per-sequence gate, a condition, a raw copy and tail masking: GEMM, then the
    finishing pass (fused with re-quantization when asked), equal to the same GEMM followed by the
    reference's finishing kernels."""
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory(mode)
    rows, k, n = 24, 1024, 768
    dtype = torch.bfloat16
    x = randn(rows, k, 1, dtype)
    wv = ctx.quantize_rows(randn(n, k, 2, dtype, 0.05), ops.RowScaledView.empty(n, k, fmt, group, group))
    bias = randn(1, n, 3, dtype, 0.5)
    kw = dict(gate=randn(rows // 4, n, 4, dtype), condition=randn(1, n, 5, dtype), rows_per_sequence=4,
              valid_rows_per_sequence=3, activation=6 if not requantize else 1)
    ctx.prepare_quantized(rows, n, k)
    scratch = ops.RowScaledView.empty(rows, k, fmt, group, group)
    out, raw = torch.empty(rows, n, dtype=dtype, device="cuda"), torch.zeros(rows, n, dtype=dtype, device="cuda")
    requantized = ops.RowScaledView.empty(rows, n, fmt, group, group) if requantize else None
    ctx.linear(x, wv, scratch, out, bias=bias, raw=raw, quantized_output=requantized, **kw)
    assert ctx.status() == 0
    plain = torch.empty_like(out)
    ctx.matmul(scratch, wv, plain)  # the projection alone
    raw_theirs = torch.zeros_like(raw)
    ep = ref_epilogue(bias=bias, raw=raw_theirs, **kw)
    if requantize:
        theirs = ops.RowScaledView.empty(rows, n, fmt, group, group)
        rc = reference_kernels.ttsref_pointwise_quantize(C.byref(ref_view(plain)), BF16, theirs.values.data_ptr(),
                                                         theirs.scales.data_ptr(), rows, n, fmt, group, group, C.byref(ep),
                                                         C.byref(ref_view(None)), 148, None)
        assert rc == 0, reference_kernels.ttsref_last_error()
        torch.cuda.synchronize()
        assert torch.equal(requantized.values, theirs.values)
        assert torch.equal(requantized.scales.view(torch.int32), theirs.scales.view(torch.int32))
    else:
        finished = torch.empty_like(plain)
        rc = reference_kernels.ttsref_pointwise(C.byref(ref_view(plain)), C.byref(ref_view(finished)), BF16, C.byref(ep), None)
        assert rc == 0, reference_kernels.ttsref_last_error()
        torch.cuda.synchronize()
        assert steps_apart(out, finished, dtype) <= 2
    assert torch.equal(bits(raw), bits(raw_theirs))


# ---------------------------------------------------------------------------------------------------------
# The same operators against the CPU oracle (oracle/oracle.cpp restates Finish::apply, the finish-and-
# quantize pass, LayerNorm + quantize and the fused norm + quantize + projection in scalar loops).
# Bars: exact arithmetic chains bit for bit; LayerNorm within one storage step / one quantization step (the
# device's rsqrtf is approximate, the oracle's 1/sqrt is not); transcendental activations within two steps.
def host16(t):
    return None if t is None else t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def host_kwargs(kw):
    out = {}
    for key, value in kw.items():
        if torch.is_tensor(value):
            out[key] = value.cpu().numpy().astype(np.int32) if value.dtype == torch.int32 else host16(value)
        else:
            out[key] = value
    return out


def from16(bits16, dtype):
    return torch.from_numpy(bits16.view(np.int16)).view(dtype).double()


def decoded(values, fmt, oracle):
    raw = values.cpu().numpy() if torch.is_tensor(values) else values
    if fmt == I8:
        return raw.view(np.int8).astype(np.float64)
    table = np.array([oracle.lib.oracle_fp8_e4m3_decode(q) for q in range(256)], dtype=np.float64)
    return table[raw]


def assert_within_one_quantization_step(oracle, fmt, group, mine, want_values, want_scales):
    """Dequantized rows agree to one step of the format at that magnitude (plus one storage step of the scale)."""
    rows, cols = want_values.shape
    def expand(scales):
        s = scales.cpu().numpy() if torch.is_tensor(scales) else scales
        return np.repeat(s.reshape(-1, rows).T, group, axis=1)[:, :cols] if group else s.reshape(rows, 1) * np.ones((1, cols))
    a, b = decoded(mine.values, fmt, oracle), decoded(want_values, fmt, oracle)
    sa, sb = expand(mine.scales).astype(np.float64), expand(want_scales).astype(np.float64)
    step = np.maximum(sa, sb) * (1.0 if fmt == I8 else np.maximum(np.maximum(np.abs(a), np.abs(b)) * 2.0 ** -3, 2.0 ** -9))
    assert np.all(np.abs(a * sa - b * sb) <= 1.01 * step + np.abs(b * sb) * 2.0 ** -7)


@pytest.mark.parametrize("type_code", [BF16, F16])
@pytest.mark.parametrize("rows,cols,activation,what", POINTWISE)
def test_finishing_pass_matches_oracle(oracle, ctx_factory, type_code, rows, cols, activation, what):
    dtype = DTYPES[type_code]
    ctx = ctx_factory("int8")
    x = randn(rows, cols, 10 * rows + cols, dtype)
    kw = epilogue_case(rows, cols, dtype, rows + cols, activation, what)
    mine = torch.empty_like(x)
    raw_mine = torch.zeros_like(x) if "raw" in what else None
    ctx.pointwise(x, mine, raw=raw_mine, **kw)
    torch.cuda.synchronize()
    want, want_raw = oracle.pointwise(host16(x), type_code, raw="raw" in what, **host_kwargs(kw))
    if raw_mine is not None:
        assert np.array_equal(host16(raw_mine), want_raw)
    if activation in (0, 1, 2):
        assert np.array_equal(host16(mine), want)
    else:
        # libm on the host, device intrinsics (and the hardware's approximate tanh) on the GPU: two storage steps, or
        # 2e-3 absolute where the activation's value is tiny next to its argument
        got, expect = mine.double().cpu(), from16(want, dtype)
        mantissa = 8 if dtype == torch.bfloat16 else 11
        spacing = torch.maximum(got.abs(), expect.abs()).clamp_min(1e-30).log2().floor().exp2() * 2.0 ** (1 - mantissa)
        assert bool(((got - expect).abs() <= 2 * spacing + 2e-3).all())


@pytest.mark.parametrize("type_code", [BF16, F16])
@pytest.mark.parametrize("rows,cols,fmt,group,rotation", [(16, 512, I8, 0, 0), (7, 3000, FP8, 0, 0), (5, 9000, I8, 0, 0),
                                                          (16, 2048, I8, 128, 128), (12, 768, FP8, 32, 0), (9, 1024, FP8, 128, 128)])
@pytest.mark.parametrize("activation,what", [(1, "bias gate residual raw"), (0, "bias mask scale"), (2, "bias residual odd")])
def test_finish_and_quantize_matches_oracle(oracle, ctx_factory, type_code, rows, cols, fmt, group, rotation, activation, what):
    dtype = DTYPES[type_code]
    ctx = ctx_factory(ctx_mode(fmt, group))
    x = randn(rows, cols, rows + cols + fmt, dtype, 2.0)
    kw = epilogue_case(rows, cols, dtype, rows * 3 + cols, activation, what)
    mine = quantized(rows, cols, fmt, group, rotation)
    kept, raw_mine = torch.zeros_like(x), (torch.zeros_like(x) if "raw" in what else None)
    ctx.pointwise_quantize(x, mine, retained=kept, raw=raw_mine, **kw)
    torch.cuda.synchronize()
    want_kept, want_raw, values, scales = oracle.pointwise_quantize(host16(x), fmt, group, rotation, type_code, raw="raw" in what,
                                                                    **host_kwargs(kw))
    if raw_mine is not None:
        assert np.array_equal(host16(raw_mine), want_raw)
    assert np.array_equal(host16(kept), want_kept)
    assert np.array_equal(mine.scales.cpu().numpy().reshape(scales.shape).view(np.uint32), scales.view(np.uint32))
    assert np.array_equal(mine.values.cpu().numpy(), values)


@pytest.mark.parametrize("type_code", [BF16, F16])
@pytest.mark.parametrize("rows,cols,fmt,group,rotation,what", [case for case in NORM if "gather" not in case[5]])
def test_layer_norm_quantize_matches_oracle(oracle, ctx_factory, type_code, rows, cols, fmt, group, rotation, what):
    dtype = DTYPES[type_code]
    ctx = ctx_factory(ctx_mode(fmt, group))
    x = randn(rows, cols, rows + cols, dtype, 1.5) + 0.25
    weight = randn(1, cols, 2, dtype, 0.2) + 1 if "weight" in what else None
    bias = randn(1, cols, 3, dtype, 0.3) if "bias" in what else None
    sequences = rows // 4 if rows % 4 == 0 else 1
    fusion = {}
    if "residual" in what:
        fusion["residual"] = randn(rows, cols, 4, dtype)
    if "projection" in what:
        fusion["projection_bias"] = randn(1, cols, 5, dtype, 0.5)
    for i, name in enumerate(("gate", "shift", "scale")):
        if name in what:
            fusion[name] = randn(sequences, cols, 6 + i, dtype, 0.5)
            fusion["rows_per_sequence"] = rows // sequences
    mine = quantized(rows, cols, fmt, group, rotation)
    kept, raw_mine = torch.zeros_like(x), torch.zeros_like(x)
    ctx.layer_norm_quantize(x, mine, weight, bias, 1e-5, retained=kept, raw=raw_mine, **fusion)
    torch.cuda.synchronize()
    normalized, raw, values, scales = oracle.layer_norm_quantize(host16(x), host16(weight), host16(bias), 1e-5, fmt, group,
                                                                 rotation, type_code, **host_kwargs(fusion))
    assert np.array_equal(host16(raw_mine), raw)            # the value that is normalized: exact arithmetic
    assert steps_apart(kept.cpu(), from16(normalized, dtype), dtype) <= 1
    if not rotation:
        assert_within_one_quantization_step(oracle, fmt, group, mine, values, scales)


@pytest.mark.parametrize("type_code", [BF16, F16])
@pytest.mark.parametrize("rows,k,n,fmt", [(16, 512, 256, I8), (5, 384, 100, I8), (16, 512, 192, FP8), (33, 128, 72, FP8)])
def test_fused_norm_projection_matches_oracle(oracle, ctx_factory, type_code, rows, k, n, fmt):
    from breeze_tts_cpp_b200 import ops
    dtype = DTYPES[type_code]
    ctx = ctx_factory(ctx_mode(fmt, 0))
    x = randn(rows, k, rows + k + n, dtype, 1.5)
    wv = ctx.quantize_rows(randn(n, k, 3, dtype, 0.05), ops.RowScaledView.empty(n, k, fmt))
    norm_weight, norm_bias = randn(1, k, 4, dtype, 0.2) + 1, randn(1, k, 5, dtype, 0.3)
    residual, out_bias = randn(rows, k, 6, dtype), randn(1, n, 7, dtype, 0.5)
    mine = torch.empty(rows, n, dtype=dtype, device="cuda")
    assert ctx.normalized_linear(x, wv, mine, norm_weight, norm_bias, 1e-5, bias=out_bias, fusion=dict(residual=residual),
                                 activation=1)
    torch.cuda.synchronize()
    want, *_ = oracle.normalized_linear(host16(x), host16(norm_weight), host16(norm_bias), 1e-5, wv.values.cpu().numpy(),
                                        wv.scales.cpu().numpy().ravel(), fmt, type_code, fusion=dict(residual=host16(residual)),
                                        bias=host16(out_bias), activation=1)
    got, expect = mine.double().cpu().numpy(), from16(want, dtype).numpy()
    floor = 1e-2 * np.sqrt(np.mean(expect ** 2)) + 1e-30
    assert float(np.max(np.abs(got - expect) / np.maximum(np.abs(expect), floor))) < 2e-2
