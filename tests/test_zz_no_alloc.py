"""The allocation-free entry point. Some hosts of this library cannot allocate device memory when
they call it — an engine that sealed its pools before serving, or code running where cudaMalloc is
off limits — so `b200q_quant_linear_static` keeps the GEMM's scratch in a device array built into the
library. This test drives it through the C ABI, twice in a row on the shared scratch, and requires
the same bits as the regular entry point. It is collected last so a failure here cannot hide others."""
import ctypes as C

import numpy as np
import pytest
import torch

from tests import synth
from tests.oracle_binding import I8

pytestmark = pytest.mark.gpu
TCGEN05 = 5


def operands(oracle, m, n, k, seed):
    from breeze_tts_cpp_b200 import ops
    x16 = oracle.to_bf16(synth.activations(m, k, seed))
    w16 = oracle.to_bf16(synth.weights(n, k, seed + 1))
    xq, sx = oracle.row_quantize(x16, I8)
    wq, sw = oracle.row_quantize(w16, I8)
    xv = ops.RowScaledView(torch.from_numpy(xq).cuda(), torch.from_numpy(sx).cuda().reshape(m, 1), I8)
    wv = ops.RowScaledView(torch.from_numpy(wq).cuda(), torch.from_numpy(sw).cuda().reshape(n, 1), I8)
    return xv, wv


@pytest.mark.parametrize("m,n,k,splits", [(16, 2048, 2048, 4), (64, 512, 6144, 1)])
def test_static_entry_matches_regular_entry_twice(oracle, ctx_factory, m, n, k, splits):
    from breeze_tts_cpp_b200 import _lib, ops
    from breeze_tts_cpp_b200._lib import Path_
    ctx = ctx_factory("int8")
    path = (TCGEN05, 16 if m <= 16 else 64, 128, splits)
    residual = torch.from_numpy(synth.activations(m, n, 5, outlier_columns=0)).cuda()
    for call in range(2):  # the second call reuses the scratch the first one left behind
        xv, wv = operands(oracle, m, n, k, seed=10 * call + m)
        want = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
        ctx.quant_linear(path, xv, wv, want, residual_f32=residual)
        got = torch.zeros_like(want)
        ep = ops._epilogue(residual_f32=residual)
        _lib.call("b200q_quant_linear_static", 0, None, C.byref(Path_(*path)), C.byref(xv.c()), C.byref(wv.c()),
                  C.byref(ops._tensor(got)), C.byref(ep))
        status = C.c_int32(-1)
        _lib.call("b200q_static_status", 0, None, C.byref(status))  # waits for the stream, allocates nothing
        assert status.value == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}"
    # planner-chosen path (path == NULL) gives the same bits as well
    got2 = torch.zeros_like(want)
    _lib.call("b200q_quant_linear_static", 0, None, None, C.byref(xv.c()), C.byref(wv.c()), C.byref(ops._tensor(got2)),
              C.byref(ep))
    torch.cuda.synchronize()
    assert torch.equal(got2.view(torch.int16), want.view(torch.int16))


def test_static_entry_rejects_bad_arguments():
    from breeze_tts_cpp_b200 import B200QError, _lib, ops
    xv = ops.RowScaledView.empty(4, 256, I8)
    wv = ops.RowScaledView.empty(32, 128, I8)  # K mismatch
    out = torch.empty(4, 32, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(B200QError):
        _lib.call("b200q_quant_linear_static", 0, None, None, C.byref(xv.c()), C.byref(wv.c()), C.byref(ops._tensor(out)), None)
