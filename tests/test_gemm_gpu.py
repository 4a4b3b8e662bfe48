"""Stage 2 / stage 3 GEMM on the GPU against the CPU oracle and the reference's own kernels.

Bars: INT8 per-row — INT32 accumulators and bf16 outputs bit-exact; K-group INT8 and all FP8 —
bf16 outputs within 1e-2 (INT8) / 2e-2 (FP8) relative of the oracle's dequantized result, with
relative error |a-b| / max(|b|, eps * rms(b)), eps = 1e-2."""
import numpy as np
import pytest
import torch

from tests import synth
from tests.oracle_binding import BF16, FP8, I8

pytestmark = pytest.mark.gpu
TCGEN05 = 5
EPS = 1e-2


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    want = want.astype(np.float64)
    floor = EPS * np.sqrt(np.mean(want ** 2)) + 1e-30
    return float(np.max(np.abs(got.astype(np.float64) - want) / np.maximum(np.abs(want), floor)))


def bf16_tensor(x16: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(x16.view(np.int16)).cuda().view(torch.bfloat16)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def make_operands(oracle, m, n, k, fmt, group, rotation, seed, student_t=None):
    from breeze_tts_cpp_b200 import ops
    x16 = oracle.to_bf16(synth.activations(m, k, seed, student_t=student_t))
    w16 = oracle.to_bf16(synth.weights(n, k, seed + 1))
    xq, sx = oracle.row_quantize(x16, fmt, group, rotation)
    wq, sw = oracle.row_quantize(w16, fmt, group, rotation)
    xv = ops.RowScaledView(torch.from_numpy(xq).cuda(), torch.from_numpy(sx).cuda().reshape(-1, m) if group else
                           torch.from_numpy(sx).cuda().reshape(m, 1), fmt, group, rotation)
    wv = ops.RowScaledView(torch.from_numpy(wq).cuda(), torch.from_numpy(sw).cuda().reshape(-1, n) if group else
                           torch.from_numpy(sw).cuda().reshape(n, 1), fmt, group, rotation)
    return (xq, sx, wq, sw), (xv, wv)


INT8_CASES = [  # m, n, k, tokens tile, splits
    (16, 128, 128, 16, 1), (16, 256, 256, 16, 1), (1, 2048, 2048, 16, 1), (3, 64, 2048, 16, 4),
    (16, 2048, 2048, 16, 8), (17, 2048, 2048, 32, 2), (64, 4096, 2048, 64, 4), (16, 2048, 6144, 16, 8), (64, 2048, 6144, 64, 7),
    (4, 12288, 2048, 16, 1), (100, 2048, 2048, 128, 3), (300, 384, 1024, 256, 1), (16, 2048, 2064, 16, 2),
]


@pytest.mark.parametrize("m,n,k,tokens,splits", INT8_CASES)
def test_int8_accumulators_and_outputs_bit_exact(oracle, ctx_factory, m, n, k, tokens, splits):
    ctx = ctx_factory("int8")
    (xq, sx, wq, sw), (xv, wv) = make_operands(oracle, m, n, k, I8, 0, 0, seed=m + n + k)
    path = (TCGEN05, tokens, 128, splits)
    raw = torch.empty(m, n, dtype=torch.int32, device="cuda")
    ctx.quant_linear(path, xv, wv, raw)
    want_acc = oracle.int8_accumulate(xq.view(np.int8), wq.view(np.int8))
    assert ctx.status() == 0
    assert np.array_equal(raw.cpu().numpy(), want_acc)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.quant_linear(path, xv, wv, out)
    want, _ = oracle.quant_linear(xq, sx, wq, sw, I8)
    assert ctx.status() == 0
    assert np.array_equal(bf16_bits(out), want)


@pytest.mark.parametrize("m,n,k", [(16, 2048, 2048), (1, 4096, 2048), (64, 2048, 6144), (4, 12288, 2048), (2048, 2048, 2048)])
def test_planned_int8_linear_with_fp32_residual(oracle, ctx_factory, m, n, k):
    """The prepared-plan path (whatever tile/split the planner picks) with the decode epilogue."""
    ctx = ctx_factory("int8")
    (xq, sx, wq, sw), (xv, wv) = make_operands(oracle, m, n, k, I8, 0, 0, seed=7 * m + k)
    residual = synth.activations(m, n, seed=3, outlier_columns=0)
    ctx.prepare_quantized(m, n, k)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.matmul(xv, wv, out, residual_f32=torch.from_numpy(residual).cuda())
    want, _ = oracle.quant_linear(xq, sx, wq, sw, I8, residual_f32=residual)
    assert ctx.status() == 0
    assert np.array_equal(bf16_bits(out), want)


@pytest.mark.parametrize("m,n,k,tokens,splits", [(16, 256, 256, 16, 1), (16, 2048, 2048, 16, 4), (64, 2048, 6144, 64, 6),
                                                 (130, 4096, 2048, 256, 1), (2048, 2048, 2048, 256, 1)])
def test_fp8_per_row(oracle, ctx_factory, m, n, k, tokens, splits):
    ctx = ctx_factory("fp8")
    (xq, sx, wq, sw), (xv, wv) = make_operands(oracle, m, n, k, FP8, 0, 0, seed=m + k)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.quant_linear((TCGEN05, tokens, 128, splits), xv, wv, out)
    _, exact = oracle.quant_linear(xq, sx, wq, sw, FP8)
    assert ctx.status() == 0
    assert rel_err(out.float().cpu().numpy(), exact) < 2e-2


@pytest.mark.parametrize("mode,fmt,tol", [("group_int8", I8, 1e-2), ("group_fp8", FP8, 2e-2)])
@pytest.mark.parametrize("m,n,k,tokens,splits", [(16, 256, 256, 16, 1), (16, 2048, 6144, 16, 1), (16, 2048, 6144, 16, 8),
                                                 (5, 2048, 6144, 16, 3), (64, 2048, 2048, 64, 2), (200, 2048, 6144, 128, 1)])
def test_k_group_gemm(oracle, ctx_factory, mode, fmt, tol, m, n, k, tokens, splits):
    ctx = ctx_factory(mode)
    (xq, sx, wq, sw), (xv, wv) = make_operands(oracle, m, n, k, fmt, 128, 128, seed=m + k, student_t=3.0)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.quant_linear((TCGEN05, tokens, 128, splits), xv, wv, out)
    want16, exact = oracle.quant_linear(xq, sx, wq, sw, fmt, 128, 128)
    assert ctx.status() == 0
    assert rel_err(out.float().cpu().numpy(), exact) < tol
    if fmt == I8 and splits == 1:  # exact integer partials accumulated in K order: bit for bit
        assert np.array_equal(bf16_bits(out), want16)


@pytest.mark.parametrize("mode,fmt,tol", [("group_int8", I8, 1e-2), ("group_fp8", FP8, 2e-2)])
@pytest.mark.parametrize("m,n,k,residual", [(1300, 1152, 512, False), (2048, 2048, 384, True), (1540, 1168, 256, True),
                                            (1300, 1152, 128, True), (1302, 1152, 256, False)])  # one K block; M % 4 != 0 -> generic kernel
def test_k_group_prefill_kernel(oracle, ctx_factory, mode, fmt, tol, m, n, k, residual):
    """Enough 128x128 tiles to fill the GPU: the persistent K-group kernel (ragged M and N tiles, several
    tiles per CTA, optional fp32 residual), against the oracle and against the generic split-K kernel."""
    ctx = ctx_factory(mode)
    (xq, sx, wq, sw), (xv, wv) = make_operands(oracle, m, n, k, fmt, 128, 128, seed=m + k, student_t=3.0)
    skip = synth.activations(m, n, seed=3, outlier_columns=0) if residual else None
    kw = {"residual_f32": torch.from_numpy(skip).cuda()} if residual else {}
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.quant_linear((TCGEN05, 128, 128, 1), xv, wv, out, **kw)      # tile count >= 2/3 of the SMs: persistent kernel
    other = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.quant_linear((TCGEN05, 64, 128, 1), xv, wv, other, **kw)     # 64-token tiles: the generic kernel
    _, exact = oracle.quant_linear(xq, sx, wq, sw, fmt, 128, 128, residual_f32=skip)
    assert ctx.status() == 0
    assert rel_err(out.float().cpu().numpy(), exact) < tol
    assert rel_err(out.float().cpu().numpy(), other.float().cpu().numpy().astype(np.float64)) < tol


def test_fused_epilogue_chain(oracle, ctx_factory):
    """bias + same-dtype residual + ReLU with the reference's rounding points."""
    ctx = ctx_factory("int8")
    m, n, k = 16, 512, 1024
    (xq, sx, wq, sw), (xv, wv) = make_operands(oracle, m, n, k, I8, 0, 0, seed=11)
    bias16 = oracle.to_bf16(synth.weights(1, n, 5, std=0.5))
    res16 = oracle.to_bf16(synth.activations(m, n, 6, outlier_columns=0))
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.quant_linear((TCGEN05, 16, 128, 2), xv, wv, out, bias=bf16_tensor(bias16), residual=bf16_tensor(res16),
                     activation=1)
    want, _ = oracle.quant_linear(xq, sx, wq, sw, I8, bias=bias16.ravel(), residual=res16, activation=1)
    assert np.array_equal(bf16_bits(out), want)


@pytest.mark.parametrize("activation", [0, 1, 2, 3, 4, 5, 7, 8])
def test_fused_epilogue_chain_with_rounding_scales(oracle, reference_kernels, ctx_factory, activation):
    """Value, residual and output scales that are not powers of two: the reference's finishing pass contracts
    value_scale*v + residual_scale*skip into one product and a fused multiply-add. The GEMM's fused chain and the
    reference's GEMM followed by its finishing pass must give the same bf16 bits for every activation the chain
    fuses; the oracle (libm activations) too where the activation is exact arithmetic."""
    import ctypes as C
    from tests.oracle_binding import ref_epilogue, ref_view
    ctx = ctx_factory("int8")
    m, n, k = 64, 768, 1024
    (xq, sx, wq, sw), (xv, wv) = make_operands(oracle, m, n, k, I8, 0, 0, seed=17)
    bias16 = oracle.to_bf16(synth.weights(1, n, 5, std=0.5))
    res16 = oracle.to_bf16(synth.activations(m, n, 6, outlier_columns=0))
    scales = dict(value_scale=0.7, residual_scale=1.3, output_scale=0.9)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.quant_linear((TCGEN05, 64, 128, 2), xv, wv, out, bias=bf16_tensor(bias16), residual=bf16_tensor(res16),
                     activation=activation, alpha=0.2, **scales)
    assert ctx.status() == 0
    if activation in (0, 1, 2):
        want, _ = oracle.quant_linear(xq, sx, wq, sw, I8, bias=bias16.ravel(), residual=res16, activation=activation, alpha=0.2,
                                      **scales)
        assert np.array_equal(bf16_bits(out), want)
    plain = torch.empty_like(out)
    workspace = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    rc = reference_kernels.ttsref_quant_linear(2, 16, 64, 1, m, n, k, 0, 0, xv.values.data_ptr(), xv.scales.data_ptr(),
                                               wv.values.data_ptr(), wv.scales.data_ptr(), plain.data_ptr(),
                                               workspace.data_ptr(), workspace.numel(), None, I8, BF16)
    assert rc == 0, reference_kernels.ttsref_last_error()
    theirs = torch.empty_like(out)
    ep = ref_epilogue(bias=bf16_tensor(bias16), residual=bf16_tensor(res16), activation=activation, alpha=0.2, **scales)
    rc = reference_kernels.ttsref_pointwise(C.byref(ref_view(plain)), C.byref(ref_view(theirs)), BF16, C.byref(ep), None)
    assert rc == 0, reference_kernels.ttsref_last_error()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), theirs.view(torch.int16))


@pytest.mark.parametrize("activation", [1, 2, 3, 4, 5, 7, 8])  # relu, leaky relu, silu, gelu, gelu-tanh, tanh, sigmoid
@pytest.mark.parametrize("m,tokens,splits", [(16, 16, 2), (100, 128, 1)])
def test_fused_activations(oracle, ctx_factory, activation, m, tokens, splits):
    """Every activation the fused epilogue accepts, with bias, output scale and the leaky slope, against the
    oracle. The device uses expf / erff / tanhf where the oracle uses libm, so all but ReLU and leaky ReLU are
    compared to within two bf16 steps of the value instead of bit for bit."""
    ctx = ctx_factory("int8")
    n, k = 384, 512
    (xq, sx, wq, sw), (xv, wv) = make_operands(oracle, m, n, k, I8, 0, 0, seed=13 + activation)
    bias16 = oracle.to_bf16(synth.weights(1, n, 5, std=0.5))
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.quant_linear((TCGEN05, tokens, 128, splits), xv, wv, out, bias=bf16_tensor(bias16), activation=activation,
                     output_scale=0.5, alpha=0.2)
    want, _ = oracle.quant_linear(xq, sx, wq, sw, I8, bias=bias16.ravel(), activation=activation, output_scale=0.5,
                                  alpha=0.2)
    assert ctx.status() == 0
    if activation in (1, 2):
        assert np.array_equal(bf16_bits(out), want)
    else:
        expect = (want.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        got = out.float().cpu().numpy().astype(np.float64)
        assert np.all(np.abs(got - expect) <= 2.0 ** -7 * np.abs(expect) + 1e-6)


def test_rejects_unprepared_and_mismatched(ctx_factory, oracle):
    from breeze_tts_cpp_b200 import B200QError
    ctx = ctx_factory("int8")
    _, (xv, wv) = make_operands(oracle, 8, 144, 272, I8, 0, 0, seed=1)
    out = torch.empty(8, 144, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(B200QError):
        ctx.matmul(xv, wv, out)  # never prepared
    with pytest.raises(B200QError):
        ctx.quant_linear((TCGEN05, 16, 128, 1), xv, wv, torch.empty(8, 160, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(B200QError):
        ctx.quant_linear((2, 16, 64, 1), xv, wv, out)  # a reference kind this build does not execute


@pytest.mark.parametrize("m,n,k", [(16, 2048, 2048), (64, 4096, 2048), (4, 2048, 6144)])
def test_int8_matches_reference_kernels(reference_kernels, ctx_factory, oracle, m, n, k):
    """Same quantized operands through the reference's CUTLASS SM80 GEMM and through this library:
    identical bf16 bits (both compute D((acc*sx)*sw) from exact INT32 sums)."""
    ctx = ctx_factory("int8")
    _, (xv, wv) = make_operands(oracle, m, n, k, I8, 0, 0, seed=m * k)
    mine = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    theirs = torch.empty_like(mine)
    ctx.prepare_quantized(m, n, k)
    ctx.matmul(xv, wv, mine)
    workspace = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    rc = reference_kernels.ttsref_quant_linear(2, 16, 64, 1, m, n, k, 0, 0, xv.values.data_ptr(), xv.scales.data_ptr(),
                                               wv.values.data_ptr(), wv.scales.data_ptr(), theirs.data_ptr(),
                                               workspace.data_ptr(), workspace.numel(), None, I8, BF16)
    assert rc == 0, reference_kernels.ttsref_last_error()
    torch.cuda.synchronize()
    assert torch.equal(mine.view(torch.int16), theirs.view(torch.int16))


@pytest.mark.parametrize("fmt,tol", [(I8, 1e-2), (FP8, 2e-2)])
def test_k_group_matches_reference_kernels(reference_kernels, ctx_factory, oracle, fmt, tol):
    m, n, k = 16, 2048, 6144
    ctx = ctx_factory("group_int8" if fmt == I8 else "group_fp8")
    _, (xv, wv) = make_operands(oracle, m, n, k, fmt, 128, 128, seed=21, student_t=3.0)
    mine = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    theirs = torch.empty_like(mine)
    ctx.prepare_quantized(m, n, k)
    ctx.matmul(xv, wv, mine)
    workspace = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    rc = reference_kernels.ttsref_quant_linear(4, 16, 64, 1, m, n, k, 128, 128, xv.values.data_ptr(),
                                               xv.scales.data_ptr(), wv.values.data_ptr(), wv.scales.data_ptr(),
                                               theirs.data_ptr(), workspace.data_ptr(), workspace.numel(), None, fmt, BF16)
    assert rc == 0, reference_kernels.ttsref_last_error()
    torch.cuda.synchronize()
    assert rel_err(mine.float().cpu().numpy(), theirs.float().cpu().numpy()) < tol


def test_bounded_wait_expires_into_the_status_word(oracle):
    """The failure path, made on the host: one barrier is armed for a byte more than its (fully completing)
    copy delivers and the wait limit is cut to about a millisecond, so the kernel gives up, leaves through its
    normal teardown, stores nothing and raises the status word. Nothing faults and nothing stays in flight: the
    next launch on the same context computes the right answer."""
    from breeze_tts_cpp_b200 import _lib, ops
    ctx = ops.Context("int8", device=0)
    m, n, k = 16, 256, 512
    (xq, sx, wq, sw), (xv, wv) = make_operands(oracle, m, n, k, I8, 0, 0, seed=5)
    out = torch.full((m, n), 3.0, dtype=torch.bfloat16, device="cuda")
    assert ctx.status() == 0
    _lib.call("b200q_inject_wait_expiry", 1, 2_000_000)
    ctx.quant_linear((TCGEN05, 16, 128, 1), xv, wv, out)
    assert ctx.status() != 0
    assert float(out.float().min()) == 3.0 and float(out.float().max()) == 3.0  # no row was stored
    ctx.close()
    ctx = ops.Context("int8", device=0)  # a fresh workspace header; the injection was one-shot
    ctx.quant_linear((TCGEN05, 16, 128, 1), xv, wv, out)
    want, _ = oracle.quant_linear(xq, sx, wq, sw, I8)
    assert ctx.status() == 0 and np.array_equal(bf16_bits(out), want)
    ctx.close()


NARROW_GROUPS = [  # m, n, k, activation group, weight group, token tile, splits
    (16, 256, 512, 32, 32, 16, 1), (5, 384, 768, 64, 64, 16, 3), (64, 512, 2048, 128, 32, 64, 2), (100, 256, 1024, 64, 128, 128, 1),
    (16, 2048, 6144, 32, 32, 16, 4), (8, 144, 160, 32, 32, 16, 1), (33, 640, 1536, 64, 32, 64, 4), (16, 256, 1024, 0, 64, 16, 2),
]


@pytest.mark.parametrize("fmt,tol", [(I8, 1e-2), (FP8, 2e-2)])
@pytest.mark.parametrize("m,n,k,gx,gw,tokens,splits", NARROW_GROUPS)
def test_k_groups_of_32_and_64(oracle, reference_kernels, ctx_factory, fmt, tol, m, n, k, gx, gw, tokens, splits):
    """Every RowScaledView group width the reference executes (32, 64, 128; the two operands may differ, the
    narrower one is the accumulation unit — reference: quant_grouped.cu:185-199), against the oracle and the
    reference's grouped kernel."""
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory("group_int8" if fmt == I8 else "group_fp8")
    x16 = oracle.to_bf16(synth.activations(m, k, m + k, student_t=3.0))
    w16 = oracle.to_bf16(synth.weights(n, k, m + k + 1))
    xq, sx = oracle.row_quantize(x16, fmt, gx, 0)
    wq, sw = oracle.row_quantize(w16, fmt, gw, 0)
    scales = lambda s, rows, g: torch.from_numpy(s).cuda().reshape(-1, rows) if g else torch.from_numpy(s).cuda().reshape(rows, 1)
    xv = ops.RowScaledView(torch.from_numpy(xq).cuda(), scales(sx, m, gx), fmt, gx, 0)
    wv = ops.RowScaledView(torch.from_numpy(wq).cuda(), scales(sw, n, gw), fmt, gw, 0)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.quant_linear((TCGEN05, tokens, 128, splits), xv, wv, out)
    _, exact = oracle.quant_linear(xq, sx, wq, sw, fmt, gx, gw)
    assert ctx.status() == 0
    assert rel_err(out.float().cpu().numpy(), exact) < tol
    planned = torch.empty_like(out)
    ctx.prepare_quantized(m, n, k, groups=(gx, gw))
    ctx.matmul(xv, wv, planned)
    assert ctx.status() == 0 and rel_err(planned.float().cpu().numpy(), exact) < tol
    if gx and k % 128 == 0:  # the reference kernel wants group scales on the activations and whole K128 stages
        theirs = torch.empty_like(out)
        workspace = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
        rc = reference_kernels.ttsref_quant_linear(4, 16, 64, 1, m, n, k, gx, gw, xv.values.data_ptr(), xv.scales.data_ptr(),
                                                   wv.values.data_ptr(), wv.scales.data_ptr(), theirs.data_ptr(),
                                                   workspace.data_ptr(), workspace.numel(), None, fmt, BF16)
        assert rc == 0, reference_kernels.ttsref_last_error()
        torch.cuda.synchronize()
        assert rel_err(out.float().cpu().numpy(), theirs.float().cpu().numpy()) < tol
        if fmt == I8 and splits == 1:  # same accumulation order as the reference's grouped kernel: same bits
            assert torch.equal(out.view(torch.int16), theirs.view(torch.int16))
