"""Seeded random shapes through the planned path: quantizer and GEMM against the CPU oracle.

The fixed cases elsewhere pin the interesting corners; this sweep walks the space between them
(row counts on both sides of every tile size, ragged channel counts, K that is not a multiple of
the 128-byte block, all four modes, optional fp32 residual) so that a planner or tile-edge slip
shows up as a wrong number rather than going unnoticed.
"""
import numpy as np
import pytest
import torch

from tests import synth
from tests.oracle_binding import FP8, I8

pytestmark = pytest.mark.gpu

MODES = ["int8", "fp8", "group_int8", "group_fp8"]
ROWS = [1, 2, 3, 5, 8, 15, 16, 17, 31, 33, 63, 64, 65, 100, 127, 128, 129, 200, 255, 256, 257, 300, 520]


def rel_err(got, want):
    want = want.astype(np.float64)
    floor = 1e-2 * np.sqrt(np.mean(want ** 2)) + 1e-30
    return float(np.max(np.abs(got.astype(np.float64) - want) / np.maximum(np.abs(want), floor)))


def cases(count, seed):
    rng = np.random.default_rng(seed)
    out = []
    for case in range(count):
        mode = MODES[case % 4]
        group = 128 if mode.startswith("group") else 0
        m = int(rng.choice(ROWS))
        n = int(rng.integers(1, 80)) * 16
        k = int(rng.integers(1, 24)) * 128 if group else int(rng.integers(1, 160)) * 16
        out.append((case, mode, m, n, k, bool(rng.integers(0, 2))))
    return out


@pytest.mark.parametrize("case,mode,m,n,k,residual", cases(32, seed=20240607))
def test_random_linear(oracle, ctx_factory, case, mode, m, n, k, residual):
    from breeze_tts_cpp_b200 import ops
    ctx = ctx_factory(mode)
    fmt = FP8 if mode.endswith("fp8") else I8
    group = 128 if mode.startswith("group") else 0
    x16 = oracle.to_bf16(synth.activations(m, k, case, student_t=3.0 if group else None))
    w16 = oracle.to_bf16(synth.weights(n, k, case + 1))
    x = torch.from_numpy(x16.view(np.int16)).cuda().view(torch.bfloat16)
    xq, sx = oracle.row_quantize(x16, fmt, group, group)
    wq, sw = oracle.row_quantize(w16, fmt, group, group)
    # stage 1: the device quantizer reproduces the oracle's bytes and scales (FP8: up to the sign of zero)
    device_x = ctx.quantize_rows(x, ops.RowScaledView.empty(m, k, fmt, group, group))
    assert np.array_equal(device_x.scales.cpu().numpy().ravel().view(np.uint32), sx.ravel().view(np.uint32))
    differs = device_x.values.cpu().numpy() != xq
    if fmt == FP8:
        differs &= ((device_x.values.cpu().numpy() | xq) & 0x7F) != 0
    assert not differs.any()
    # stages 2-3: the planned GEMM over the oracle's operands
    scales = (lambda s, rows: torch.from_numpy(s).cuda().reshape(-1, rows) if group else torch.from_numpy(s).cuda().reshape(rows, 1))
    xv = ops.RowScaledView(torch.from_numpy(xq).cuda(), scales(sx, m), fmt, group, group)
    wv = ops.RowScaledView(torch.from_numpy(wq).cuda(), scales(sw, n), fmt, group, group)
    skip = synth.activations(m, n, seed=3, outlier_columns=0) if residual else None
    ctx.prepare_quantized(m, n, k)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.matmul(xv, wv, out, **({"residual_f32": torch.from_numpy(skip).cuda()} if residual else {}))
    want, exact = oracle.quant_linear(xq, sx, wq, sw, fmt, group, group, residual_f32=skip)
    assert ctx.status() == 0
    if fmt == I8 and not group:
        assert np.array_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), want)
    else:
        assert rel_err(out.float().cpu().numpy(), exact) < (2e-2 if fmt == FP8 else 1e-2)
