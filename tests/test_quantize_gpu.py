"""Stage 1 / stage-3 producer on the GPU: bytes and scales must equal the CPU oracle bit for bit
(INT8 and FP8 alike — the encode is deterministic), and equal the reference's own kernels."""
import numpy as np
import pytest
import torch

from tests import synth
from tests.oracle_binding import BF16, F16, FP8, I8

pytestmark = pytest.mark.gpu

MODES = [  # (mode string for the context, format, group, rotation)
    ("int8", I8, 0, 0), ("fp8", FP8, 0, 0), ("group_int8", I8, 128, 128), ("group_fp8", FP8, 128, 128),
    ("int8", I8, 0, 128), ("int8", I8, 128, 0), ("int8", I8, 64, 0), ("fp8", FP8, 32, 0),
]
SHAPES = [(1, 128), (3, 256), (16, 2048), (17, 6144), (64, 2048), (5, 8192), (2, 12288), (130, 384)]


def _to_torch_bf16(x16: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(x16.view(np.int16)).cuda().view(torch.bfloat16)


@pytest.mark.parametrize("mode,fmt,group,rotation", MODES)
@pytest.mark.parametrize("rows,cols", SHAPES)
def test_row_quantize_matches_oracle(oracle, ctx_factory, mode, fmt, group, rotation, rows, cols):
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory(mode)
    x16 = oracle.to_bf16(synth.activations(rows, cols, seed=rows * 131 + cols))
    want_q, want_s = oracle.row_quantize(x16, fmt, group, rotation)
    out = ops.RowScaledView.empty(rows, cols, fmt, group, rotation)
    ctx.quantize_rows(_to_torch_bf16(x16), out)
    torch.cuda.synchronize()
    assert np.array_equal(out.values.cpu().numpy(), want_q)
    assert np.array_equal(out.scales.cpu().numpy().reshape(want_s.shape).view(np.uint32), want_s.view(np.uint32))


def test_edge_rows(oracle, ctx_factory):
    """All-zero rows get scale 1; exact ties round to even; +-max maps to +-127."""
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory("int8")
    x = np.zeros((4, 256), dtype=np.float32)
    x[1, :8] = [127, -127, 0.5, 1.5, 2.5, -0.5, -1.5, 126.5]
    x[2, :4] = [1e-30, -1e-30, 0, 0]
    x[3, :] = np.linspace(-3, 3, 256)
    x16 = oracle.to_bf16(x)
    want_q, want_s = oracle.row_quantize(x16, I8)
    out = ops.RowScaledView.empty(4, 256, I8)
    ctx.quantize_rows(_to_torch_bf16(x16), out)
    got_q, got_s = out.values.cpu().numpy(), out.scales.cpu().numpy().ravel()
    assert got_s[0] == 1.0 and not got_q[0].any()
    assert np.array_equal(got_q, want_q) and np.array_equal(got_s, want_s)
    assert list(got_q[1, :8].view(np.int8)) == [127, -127, 0, 2, 2, 0, -2, 126]


def test_strided_and_f16_sources(oracle, ctx_factory):
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory("int8")
    rows, cols, stride = 6, 2048, 4096
    wide = synth.activations(rows, stride, seed=5)
    x16 = oracle.to_bf16(wide)
    want_q, want_s = oracle.row_quantize(np.ascontiguousarray(x16[:, :cols]), I8)
    source = _to_torch_bf16(x16)[:, :cols]
    out = ops.RowScaledView.empty(rows, cols, I8)
    ctx.quantize_rows(source, out)
    assert np.array_equal(out.values.cpu().numpy(), want_q)
    assert np.array_equal(out.scales.cpu().numpy().ravel(), want_s)
    # unaligned column offset -> element-wise loads
    source = _to_torch_bf16(x16)[:, 3:3 + cols]
    want_q, want_s = oracle.row_quantize(np.ascontiguousarray(x16[:, 3:3 + cols]), I8)
    ctx.quantize_rows(source, out)
    assert np.array_equal(out.values.cpu().numpy(), want_q)
    # f16 source
    half = wide[:, :cols].astype(np.float16)
    want_q, want_s = oracle.row_quantize(half.view(np.uint16), I8, src_type=F16)
    ctx.quantize_rows(torch.from_numpy(half).cuda(), out)
    assert np.array_equal(out.values.cpu().numpy(), want_q)
    assert np.array_equal(out.scales.cpu().numpy().ravel(), want_s)


def test_rejects_bad_arguments(ctx_factory):
    from breeze_tts_cpp_b200 import B200QError, ops
    ctx = ctx_factory("int8")
    x = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(B200QError):
        ctx.quantize_rows(x, ops.RowScaledView.empty(4, 128, I8))
    with pytest.raises(B200QError):
        ctx.quantize_rows(x.float(), ops.RowScaledView.empty(4, 256, I8))
    bad = ops.RowScaledView.empty(4, 256, I8, group=0, rotation=128)
    bad.rotation_size = 64
    with pytest.raises(B200QError):
        ctx.quantize_rows(x, bad)


@pytest.mark.parametrize("fmt,group,rotation", [(I8, 0, 0), (FP8, 0, 0), (I8, 128, 128), (FP8, 128, 128), (I8, 0, 128)])
@pytest.mark.parametrize("rows,cols", [(16, 2048), (7, 6144), (64, 4096)])
def test_row_quantize_matches_reference_kernels(reference_kernels, ctx_factory, oracle, fmt, group, rotation, rows, cols):
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory("int8" if fmt == I8 else "fp8")
    x = _to_torch_bf16(oracle.to_bf16(synth.activations(rows, cols, seed=99 + rows, student_t=3.0)))
    mine = ops.RowScaledView.empty(rows, cols, fmt, group, rotation)
    theirs = ops.RowScaledView.empty(rows, cols, fmt, group, rotation)
    ctx.quantize_rows(x, mine)
    rc = reference_kernels.ttsref_row_quantize(x.data_ptr(), rows, cols, 0, BF16, theirs.values.data_ptr(),
                                               theirs.scales.data_ptr(), fmt, group, rotation, None)
    assert rc == 0, reference_kernels.ttsref_last_error()
    torch.cuda.synchronize()
    assert torch.equal(mine.values, theirs.values)
    assert torch.equal(mine.scales.view(torch.int32), theirs.scales.view(torch.int32))


@pytest.mark.parametrize("fmt", [I8, FP8])
@pytest.mark.parametrize("rows,cols,stride,type_code", [(8192, 2048, 0, BF16), (1500, 520, 0, BF16), (2000, 4096, 0, F16),
                                                        (1300, 1024, 2048, BF16), (1187, 8, 0, BF16), (4096, 4104, 0, BF16)])
def test_long_batches_take_the_warp_per_row_kernel(reference_kernels, ctx_factory, fmt, rows, cols, stride, type_code):
    """Thousands of rows with one scale per row (the prefill quantizer): bytes and scales identical to the
    reference's row quantizer, strided sources and both 16-bit types included; the last shape is one column
    packet too wide for the warp-per-row kernel and takes the CTA-per-row one."""
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory("int8" if fmt == I8 else "fp8")
    dtype = torch.bfloat16 if type_code == BF16 else torch.float16
    g = torch.Generator(device="cuda").manual_seed(rows + cols)
    wide = (torch.randn(rows, stride or cols, generator=g, device="cuda") * 3).to(dtype)
    wide[5] = 0  # an all-zero row: scale 1
    x = wide[:, :cols]
    mine, theirs = ops.RowScaledView.empty(rows, cols, fmt), ops.RowScaledView.empty(rows, cols, fmt)
    ctx.quantize_rows(x, mine)
    rc = reference_kernels.ttsref_row_quantize(x.data_ptr(), rows, cols, stride, type_code, theirs.values.data_ptr(),
                                               theirs.scales.data_ptr(), fmt, 0, 0, None)
    assert rc == 0, reference_kernels.ttsref_last_error()
    torch.cuda.synchronize()
    assert torch.equal(mine.scales.view(torch.int32), theirs.scales.view(torch.int32))
    assert torch.equal(mine.values, theirs.values)
    assert float(mine.scales[5]) == 1.0
