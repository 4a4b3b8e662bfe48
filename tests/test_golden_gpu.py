"""The committed golden fixtures (made by tests/golden/make_golden.py) replayed on the GPU."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.oracle_binding import FP8, I8

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
MODE = {(I8, 0): "int8", (FP8, 0): "fp8", (I8, 128): "group_int8", (FP8, 128): "group_fp8"}


@pytest.mark.parametrize("case", json.loads((GOLDEN / "index.json").read_text())["cases"], ids=lambda c: c["file"])
def test_golden_case(ctx_factory, case):
    from breeze_tts_cpp_b200 import ops
    data = np.load(GOLDEN / case["file"])
    fmt, group, rotation, m, n, k = (case[key] for key in ("format", "group", "rotation", "m", "n", "k"))
    ctx = ctx_factory(MODE[(fmt, group)])
    dev = lambda a: torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    xv = ctx.quantize_rows(dev(data["x16"]), ops.RowScaledView.empty(m, k, fmt, group, rotation))
    wv = ctx.quantize_rows(dev(data["w16"]), ops.RowScaledView.empty(n, k, fmt, group, rotation))
    assert np.array_equal(xv.values.cpu().numpy(), data["xq"]) and np.array_equal(wv.values.cpu().numpy(), data["wq"])
    assert np.array_equal(xv.scales.cpu().numpy().reshape(data["sx"].shape), data["sx"])
    assert np.array_equal(wv.scales.cpu().numpy().reshape(data["sw"].shape), data["sw"])
    # the reference kernels' own bytes and scales, recorded in the fixture
    assert np.array_equal(xv.scales.cpu().numpy().reshape(data["ref_sx"].shape), data["ref_sx"])
    differs = xv.values.cpu().numpy() != data["ref_xq"]
    if fmt == FP8:
        differs &= ((xv.values.cpu().numpy() | data["ref_xq"]) & 0x7F) != 0
    assert not differs.any()
    ctx.prepare_quantized(m, n, k)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.matmul(xv, wv, out)
    got = out.view(torch.int16).cpu().numpy().view(np.uint16)
    if fmt == I8 and not group:
        assert np.array_equal(got, data["ref_out16"])  # the reference CUTLASS kernel's bits
    want = data["out16"]
    if fmt == I8 and not group:
        assert np.array_equal(got, want)
        raw = torch.empty(m, n, dtype=torch.int32, device="cuda")
        ctx.quant_linear(ctx.select_path(m, n, k), xv, wv, raw)
        assert np.array_equal(raw.cpu().numpy(), data["acc"])
    else:
        to_f = lambda b: (b.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        g, w = to_f(got), to_f(want)
        floor = 1e-2 * np.sqrt(np.mean(w ** 2))
        tol = 1e-2 if fmt == I8 else 2e-2
        assert np.max(np.abs(g - w) / np.maximum(np.abs(w), floor)) < tol + 2 ** -8  # + one bf16 rounding of the oracle
