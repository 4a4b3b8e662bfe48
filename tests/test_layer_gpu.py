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
