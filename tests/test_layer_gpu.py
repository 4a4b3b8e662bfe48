"""The Linear layer object through the C ABI: load-time fused weight quantization, plans for every
row class, dense-activation forward with bias / epilogue, re-quantized output for the next layer."""
import numpy as np
import pytest
import torch

from tests import synth
from tests.oracle_binding import FP8, I8

pytestmark = pytest.mark.gpu


def dev16(oracle, x):
    x16 = oracle.to_bf16(x)
    return x16, torch.from_numpy(x16.view(np.int16)).cuda().view(torch.bfloat16)


def bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def test_fused_qkv_layer_int8_bit_exact(oracle, ctx_factory):
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory("int8")
    k, parts_rows = 1024, (512, 256, 256)
    host, dev = zip(*[dev16(oracle, synth.weights(r, k, 40 + i)) for i, r in enumerate(parts_rows)])
    b16, bias = dev16(oracle, synth.weights(1, sum(parts_rows), 9, std=0.3))
    layer = ops.Linear(ctx, list(dev), bias=bias, max_rows=40)
    w16 = np.concatenate(host, axis=0)
    wq, sw = oracle.row_quantize(w16, I8)
    for rows in (1, 7, 33, 40):  # several row-capacity classes, one plan each
        x16, x = dev16(oracle, synth.activations(rows, k, seed=rows))
        out = layer.forward(x, activation=1)
        xq, sx = oracle.row_quantize(x16, I8)
        want, _ = oracle.quant_linear(xq, sx, wq, sw, I8, bias=b16.ravel(), activation=1)
        assert ctx.status() == 0
        assert np.array_equal(bits(out), want), rows
    with pytest.raises(Exception):
        layer.forward(torch.zeros(41, k, dtype=torch.bfloat16, device="cuda"))  # beyond the prepared workspace
    layer.close()


@pytest.mark.parametrize("mode,fmt,tol", [("group_int8", I8, 1e-2), ("group_fp8", FP8, 2e-2), ("fp8", FP8, 2e-2)])
def test_fused_gate_up_layer_other_modes(oracle, ctx_factory, mode, fmt, tol):
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory(mode)
    k, n_half, rows = 768, 384, 16
    group, rotation = (128, 128) if mode.startswith("group") else (0, 0)
    host, dev = zip(*[dev16(oracle, synth.weights(n_half, k, 60 + i)) for i in range(2)])
    layer = ops.Linear(ctx, list(dev), max_rows=rows)
    x16, x = dev16(oracle, synth.activations(rows, k, seed=3, student_t=3.0))
    out = layer.forward(x)
    wq, sw = oracle.row_quantize(np.concatenate(host, axis=0), fmt, group, rotation)
    xq, sx = oracle.row_quantize(x16, fmt, group, rotation)
    _, exact = oracle.quant_linear(xq, sx, wq, sw, fmt, group, group)
    got = out.float().cpu().numpy().astype(np.float64)
    floor = 1e-2 * np.sqrt(np.mean(exact.astype(np.float64) ** 2))
    assert ctx.status() == 0
    assert np.max(np.abs(got - exact) / np.maximum(np.abs(exact), floor)) < tol
    layer.close()


def test_layer_requantizes_output_for_next_layer(oracle, ctx_factory):
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory("int8")
    k, n, rows = 512, 256, 8
    _, w = dev16(oracle, synth.weights(n, k, 5))
    layer = ops.Linear(ctx, [w], max_rows=rows)
    _, x = dev16(oracle, synth.activations(rows, k, seed=8))
    nxt = ops.RowScaledView.empty(rows, n, I8)
    out = layer.forward(x, quantized_output=nxt)
    want_q, want_s = oracle.row_quantize(bits(out), I8)
    assert np.array_equal(nxt.values.cpu().numpy(), want_q) and np.array_equal(nxt.scales.cpu().numpy().ravel(), want_s)
    layer.close()


def test_phase_switch_plan_prepare_execute(ctx_factory, oracle):
    """reference: Linear::apply_context (src/layers/linear.cpp:64-76): Plan and Capture launch nothing, Prepare
    plans and sizes the scratch, Execute runs; Execute beyond the prepared rows fails instead of allocating."""
    from breeze_tts_cpp_b200 import B200QError, ops
    ctx = ops.Context("int8", device=0)  # a fresh context: its plans are not sealed yet
    k, n = 512, 384
    _, w = dev16(oracle, synth.weights(n, k, 5))
    b16, bias = dev16(oracle, synth.weights(1, n, 6, std=0.3))
    layer = ops.Linear(ctx, [w], bias=bias, max_rows=1)
    x16, x = dev16(oracle, synth.activations(24, k, seed=8))
    out = torch.full((24, n), 7.0, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(B200QError):
        layer.apply(ops.Linear.EXECUTE, 24, x, out)       # never prepared for 24 rows
    for mode in (ops.Linear.PLAN, ops.Linear.CAPTURE):
        layer.apply(mode, 24, x, out)
        assert float(out.float().min()) == 7.0            # nothing ran
    layer.apply(ops.Linear.PREPARE, 24, x, out, activation=1)
    assert float(out.float().min()) == 7.0
    ctx.seal()
    layer.apply(ops.Linear.EXECUTE, 24, x, out, activation=1)
    wq, sw = oracle.row_quantize(bits(w), I8)
    xq, sx = oracle.row_quantize(x16, I8)
    want, _ = oracle.quant_linear(xq, sx, wq, sw, I8, bias=b16.ravel(), activation=1)
    assert ctx.status() == 0 and np.array_equal(bits(out), want)
    # segments: scatter two row ranges of the input to other rows of the output
    scattered = torch.zeros(24, n, dtype=torch.bfloat16, device="cuda")
    layer.forward_segments(ops.Linear.EXECUTE, 24, x, [(0, 8, 16), (8, 16, 0)], scattered)
    plain = torch.empty(24, n, dtype=torch.bfloat16, device="cuda")
    layer.forward_segments(ops.Linear.EXECUTE, 24, x, [], plain)
    assert torch.equal(scattered[16:24], plain[0:8]) and torch.equal(scattered[0:16], plain[8:24])
    layer.close()
    ctx.close()


@pytest.mark.parametrize("k,fused", [(512, True), (1024, False)])
def test_normalized_forward_fused_and_two_step_agree(ctx_factory, oracle, k, fused):
    """reference: Linear::normalized_forward (src/layers/linear.cpp:195-214). For K <= 512 one launch does
    LayerNorm + quantize + projection; beyond that LayerNorm + quantize is followed by the GEMM. Both give
    the result of running the two steps by hand."""
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory("int8")
    n, rows = 256, 12
    _, w = dev16(oracle, synth.weights(n, k, 5))
    _, bias = dev16(oracle, synth.weights(1, n, 6, std=0.3))
    layer = ops.Linear(ctx, [w], bias=bias, max_rows=rows)
    _, x = dev16(oracle, synth.activations(rows, k, seed=8))
    _, gamma = dev16(oracle, 1.0 + synth.weights(1, k, 7, std=0.2))
    _, beta = dev16(oracle, synth.weights(1, k, 8, std=0.2))
    out = torch.empty(rows, n, dtype=torch.bfloat16, device="cuda")
    normalized = torch.zeros(rows, k, dtype=torch.bfloat16, device="cuda")
    layer.normalized_forward(x, out, gamma, beta, 1e-5, normalized=normalized, activation=1)
    assert ctx.status() == 0
    by_hand_q = ctx.layer_norm_quantize(x, ops.RowScaledView.empty(rows, k, I8), gamma, beta, 1e-5)
    weight = layer.weight()
    wv = ops.RowScaledView(torch.empty(0), torch.empty(0), I8)
    wv.c = lambda: weight  # the layer's own quantized weight view
    ctx.prepare_quantized(rows, n, k)
    by_hand = torch.empty_like(out)
    ctx.matmul(by_hand_q, wv, by_hand, bias=bias, activation=1)
    if fused:  # the fused kernel multiplies (acc * sw) * sx, the GEMM (acc * sx) * sw: at most one bf16 step apart
        a, b = out.double(), by_hand.double()
        assert float(((a - b).abs() / torch.maximum(a.abs(), b.abs()).clamp_min(1e-6)).max()) <= 2.0 ** -7
    else:
        assert torch.equal(out.view(torch.int16), by_hand.view(torch.int16))
    assert float(normalized.float().abs().max()) > 0
    layer.close()
