"""Parity at the benchmark's own sizes, where every persistent CTA (or CTA pair) of the compute-bound
kernels walks several tiles: accumulator hand-over, ring wrap-around and barrier parities of the
second and later tiles all produce checked numbers here.

Checkers:
  * INT8 per-row: the reference's CUTLASS SM80 kernel (exact INT32 sums, same scale order) — bf16
    bits must be identical; with the fp32 residual, a plain PyTorch restatement
    bf16((float(acc) * sx) * sw + residual) over torch._int_mm's exact INT32 sums — identical bits.
  * FP8 per-row and K-group modes: the CPU oracle on a slice of the output (first, last and two
    seeded channels of every channel tile, all token rows), tolerance 2e-2 (FP8) / 1e-2 (INT8)
    relative with floor 1e-2 * rms; the whole output against an fp64 PyTorch product within the
    same tolerance; K-group also against the reference's grouped kernel.
Operands are quantized on the device by this library's quantizer, whose bytes are pinned to the
oracle and to the reference kernels elsewhere in the suite.
"""
import numpy as np
import pytest
import torch

from tests.oracle_binding import BF16, FP8, I8

pytestmark = pytest.mark.gpu
TCGEN05, SM80, GEMV, GROUPED = 5, 2, 1, 4
LAYER = {"qkv": (2048, 4096), "o": (2048, 2048), "gate_up": (2048, 12288), "down": (6144, 2048)}  # K, N


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    want = want.astype(np.float64)
    floor = 1e-2 * np.sqrt(np.mean(want ** 2)) + 1e-30
    return float(np.max(np.abs(got.astype(np.float64) - want) / np.maximum(np.abs(want), floor)))


def rel_err_torch(got: torch.Tensor, want: torch.Tensor) -> float:
    floor = 1e-2 * want.pow(2).mean().sqrt() + 1e-30
    return float(((got.double() - want).abs() / torch.maximum(want.abs(), floor)).max())


def synth_device(rows, cols, seed, student_t=False, std=1.0, outliers=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, cols, generator=g, device="cuda")
    if student_t:  # Student-t with 3 degrees of freedom: normal / sqrt(chi2_3 / 3)
        chi = torch.randn(3, rows, cols, generator=g, device="cuda").pow(2).sum(0)
        x = x / (chi / 3).sqrt()
    if outliers:
        columns = torch.randperm(cols, generator=g, device="cuda")[:max(1, round(cols * 0.005))]
        x[:, columns] *= 20.0
    return (x * std).to(torch.bfloat16)


def quantized_operands(ctx, m, k, n, fmt, group, seed, student_t=False):
    from breeze_tts_cpp_b200 import ops
    x = synth_device(m, k, seed, student_t)
    w = synth_device(n, k, seed + 1, std=0.02, outliers=False)
    xv = ctx.quantize_rows(x, ops.RowScaledView.empty(m, k, fmt, group, group))
    wv = ctx.quantize_rows(w, ops.RowScaledView.empty(n, k, fmt, group, group))
    return xv, wv


def tiles_per_worker(m, n, tile_m, tile_n, workers):
    tiles = -(-m // tile_m) * -(-n // tile_n)
    return tiles / min(tiles, workers)


def channel_slice(n, tile, seed):
    """First, last and two seeded channels of every `tile`-channel tile."""
    rng = np.random.default_rng(seed)
    picked = []
    for first in range(0, n, tile):
        width = min(tile, n - first)
        picked += [first, first + width - 1] + [first + int(c) for c in rng.integers(0, width, 2)]
    return np.unique(np.array(picked))


def decode(values: torch.Tensor, fmt: int) -> torch.Tensor:
    if fmt == I8:
        return values.view(torch.int8).double()
    return values.view(torch.float8_e4m3fn).double()


def exact_product(xv, wv, fmt, group):
    """fp64 restatement of the whole output on the device (a checker, never the product path)."""
    x, w = decode(xv.values, fmt), decode(wv.values, fmt)
    if not group:
        return (x @ w.T) * xv.scales.double().reshape(-1, 1) * wv.scales.double().reshape(1, -1)
    m, k = x.shape
    n = w.shape[0]
    out = torch.zeros(m, n, dtype=torch.float64, device="cuda")
    for g in range(k // group):
        block = x[:, g * group:(g + 1) * group] @ w[:, g * group:(g + 1) * group].T
        out += block * xv.scales[g].double().reshape(-1, 1) * wv.scales[g].double().reshape(1, -1)
    return out


def oracle_slice(oracle, xv, wv, fmt, group, channels, rows=None, residual=None):
    xq, wq = xv.values.cpu().numpy(), wv.values[torch.from_numpy(channels).cuda()].cpu().numpy()
    sx, sw = xv.scales.cpu().numpy(), wv.scales.cpu().numpy()
    if rows is not None:
        xq = xq[rows]
    if group:
        sw = np.ascontiguousarray(sw[:, channels])
        sx = np.ascontiguousarray(sx[:, rows]) if rows is not None else sx
    else:
        sw = np.ascontiguousarray(sw.reshape(-1)[channels])
        sx = sx.reshape(-1)[rows] if rows is not None else sx.reshape(-1)
    skip = None
    if residual is not None:
        skip = residual[:, torch.from_numpy(channels).cuda()].cpu().numpy()
        skip = np.ascontiguousarray(skip[rows] if rows is not None else skip)
    return oracle.quant_linear(np.ascontiguousarray(xq), np.ascontiguousarray(sx), np.ascontiguousarray(wq), sw, fmt,
                               group, group, residual_f32=skip, threads=16)


def reference_gemm(lib, path, xv, wv, m, n, k, fmt, group=0, out_type=BF16, dtype=torch.bfloat16):
    out = torch.empty(m, n, dtype=dtype, device="cuda")
    workspace = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    rc = lib.ttsref_quant_linear(*path, m, n, k, group, group, xv.values.data_ptr(), xv.scales.data_ptr(),
                                 wv.values.data_ptr(), wv.scales.data_ptr(), out.data_ptr(), workspace.data_ptr(),
                                 workspace.numel(), None, fmt, out_type)
    assert rc == 0, lib.ttsref_last_error()
    torch.cuda.synchronize()
    return out


# ------------------------------------------------------------------------------------------------ INT8 per-row
INT8_PREFILL = [(8192, name) for name in LAYER] + [(2048, "gate_up"), (2048, "qkv")]


@pytest.mark.parametrize("m,shape", INT8_PREFILL)
def test_int8_prefill_bits_match_reference_kernel(reference_kernels, ctx_factory, m, shape):
    k, n = LAYER[shape]
    ctx = ctx_factory("int8")
    xv, wv = quantized_operands(ctx, m, k, n, I8, 0, seed=m + n)
    path = ctx.prepare_quantized(m, n, k)
    assert path[1] == 256 and path[3] == 1, "expected the persistent 256-token path"
    if m == 8192 or shape == "gate_up":
        assert tiles_per_worker(m, n, 256, 256, ctx.multiprocessors // 2) >= 3
    mine = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.matmul(xv, wv, mine)
    assert ctx.status() == 0
    theirs = reference_gemm(reference_kernels, (SM80, 128, 128, 1), xv, wv, m, n, k, I8)
    assert torch.equal(mine.view(torch.int16), theirs.view(torch.int16))
    # with the fp32 residual of the decode workload (the reference has no such epilogue)
    residual = torch.randn(m, n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    ctx.matmul(xv, wv, mine, residual_f32=residual)
    assert ctx.status() == 0
    acc = torch._int_mm(xv.values.view(torch.int8), wv.values.view(torch.int8).T)
    want = ((acc.float() * xv.scales.reshape(-1, 1)) * wv.scales.reshape(1, -1) + residual).to(torch.bfloat16)
    assert torch.equal(mine.view(torch.int16), want.view(torch.int16))


def test_int8_single_cta_prefill_kernel_many_tiles(reference_kernels, ctx_factory):
    """N < 256 takes the one-CTA persistent kernel; 2 channel tiles x 223 token tiles on 148 CTAs."""
    m, n, k = 57000, 192, 512
    ctx = ctx_factory("int8")
    assert tiles_per_worker(m, n, 256, 128, ctx.multiprocessors) >= 3
    xv, wv = quantized_operands(ctx, m, k, n, I8, 0, seed=77)
    mine = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.quant_linear((TCGEN05, 256, 128, 1), xv, wv, mine)
    assert ctx.status() == 0
    theirs = reference_gemm(reference_kernels, (SM80, 128, 64, 1), xv, wv, m, n, k, I8)
    assert torch.equal(mine.view(torch.int16), theirs.view(torch.int16))


# ------------------------------------------------------------------------------------------------ FP8 per-row
@pytest.mark.parametrize("m,shape", [(8192, name) for name in LAYER] + [(2048, name) for name in LAYER])
def test_fp8_prefill_against_oracle_slice_and_fp64(oracle, ctx_factory, m, shape):
    k, n = LAYER[shape]
    ctx = ctx_factory("fp8")
    xv, wv = quantized_operands(ctx, m, k, n, FP8, 0, seed=m + n + 1)
    path = ctx.prepare_quantized(m, n, k)
    assert path[1] == 256 and path[3] == 1
    if m == 8192:
        assert tiles_per_worker(m, n, 256, 256, ctx.multiprocessors // 2) >= 3
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.matmul(xv, wv, out)
    assert ctx.status() == 0
    assert rel_err_torch(out, exact_product(xv, wv, FP8, 0)) < 2e-2
    channels = channel_slice(n, 256, seed=n)
    _, exact = oracle_slice(oracle, xv, wv, FP8, 0, channels)
    got = out[:, torch.from_numpy(channels).cuda()].float().cpu().numpy()
    assert rel_err(got, exact) < 2e-2


@pytest.mark.parametrize("m,tokens", [(1, 1), (2, 2), (4, 4)])
@pytest.mark.parametrize("shape", ["qkv", "down"])
def test_fp8_small_m_matches_reference_gemv(reference_kernels, ctx_factory, m, tokens, shape):
    """The reference's only runnable FP8 per-channel path on this GPU is its scalar GEMV
    (src/ops/kernels/quant/quant_dispatch.cu:12-130)."""
    k, n = LAYER[shape]
    ctx = ctx_factory("fp8")
    xv, wv = quantized_operands(ctx, m, k, n, FP8, 0, seed=31 * m + n)
    ctx.prepare_quantized(m, n, k)
    mine = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.matmul(xv, wv, mine)
    assert ctx.status() == 0
    theirs = reference_gemm(reference_kernels, (GEMV, tokens, 8, 1), xv, wv, m, n, k, FP8)
    assert rel_err(mine.float().cpu().numpy(), theirs.float().cpu().numpy()) < 2e-2


# ------------------------------------------------------------------------------------------------ K-group modes
@pytest.mark.parametrize("mode,fmt,tol", [("group_int8", I8, 1e-2), ("group_fp8", FP8, 2e-2)])
@pytest.mark.parametrize("residual", [False, True])
def test_k_group_down_projection_m4096(oracle, reference_kernels, ctx_factory, mode, fmt, tol, residual):
    """BASELINE config 4: M=4096, K=6144, N=2048 through the persistent K-group kernel (48 K blocks per
    tile, 512 tiles on 148 CTAs: every ring and accumulator wraps many times)."""
    m, (k, n) = 4096, LAYER["down"]
    ctx = ctx_factory(mode)
    assert tiles_per_worker(m, n, 128, 128, ctx.multiprocessors) >= 3
    xv, wv = quantized_operands(ctx, m, k, n, fmt, 128, seed=4096 + fmt, student_t=True)
    path = ctx.prepare_quantized(m, n, k)
    assert path[1] == 128, "expected the persistent K-group path"
    skip = torch.randn(m, n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(9)) if residual else None
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.matmul(xv, wv, out, **({"residual_f32": skip} if residual else {}))
    assert ctx.status() == 0
    whole = exact_product(xv, wv, fmt, 128)
    assert rel_err_torch(out, whole + skip.double() if residual else whole) < tol
    channels = channel_slice(n, 128, seed=3)
    rows = np.unique(np.concatenate([np.arange(0, m, 128), np.arange(127, m, 128),
                                     np.random.default_rng(1).integers(0, m, 64)]))
    want16, exact = oracle_slice(oracle, xv, wv, fmt, 128, channels, rows=rows, residual=skip)
    picked = out[torch.from_numpy(rows).cuda()][:, torch.from_numpy(channels).cuda()]
    assert rel_err(picked.float().cpu().numpy(), exact) < tol
    if fmt == I8:  # exact integer partials, one fused multiply-add per K group in K order: the same bits everywhere
        assert np.array_equal(picked.contiguous().view(torch.int16).cpu().numpy().view(np.uint16), want16)
    if not residual:
        theirs = reference_gemm(reference_kernels, (GROUPED, 64, 64, 1), xv, wv, m, n, k, fmt, group=128)
        assert rel_err(out.float().cpu().numpy(), theirs.float().cpu().numpy()) < tol
        if fmt == I8:
            assert torch.equal(out.view(torch.int16), theirs.view(torch.int16))


# ------------------------------------------------------------------------------------------------ smaller holes
@pytest.mark.parametrize("m,n,k,path", [(16, 2048, 2048, (SM80, 16, 64, 1)), (64, 4096, 2048, (SM80, 64, 128, 2)),
                                        (300, 640, 1024, (SM80, 128, 64, 1))])
def test_oracle_matches_reference_gemm_directly(oracle, reference_kernels, ctx_factory, m, n, k, path):
    """Pins the CPU oracle to the reference's GEMM without this library's GEMM in between."""
    ctx = ctx_factory("int8")
    xv, wv = quantized_operands(ctx, m, k, n, I8, 0, seed=m * n)
    theirs = reference_gemm(reference_kernels, path, xv, wv, m, n, k, I8)
    want, _ = oracle.quant_linear(xv.values.cpu().numpy(), xv.scales.cpu().numpy().reshape(-1),
                                  wv.values.cpu().numpy(), wv.scales.cpu().numpy().reshape(-1), I8)
    assert np.array_equal(theirs.view(torch.int16).cpu().numpy().view(np.uint16), want)


@pytest.mark.parametrize("mode,fmt,group", [("int8", I8, 0), ("fp8", FP8, 0), ("group_int8", I8, 128), ("group_fp8", FP8, 128)])
@pytest.mark.parametrize("m,tokens,splits", [(16, 16, 2), (2048, None, 1)])
def test_f16_outputs(oracle, reference_kernels, ctx_factory, mode, fmt, group, m, tokens, splits):
    """Type::F16 outputs of every mode, decode tile and persistent kernels, against the oracle (and bit
    for bit against the reference CUTLASS kernel for INT8 per-row)."""
    from tests.oracle_binding import F16
    n, k = 1024, 1024
    ctx = ctx_factory(mode)
    xv, wv = quantized_operands(ctx, m, k, n, fmt, group, seed=m + fmt + group, student_t=bool(group))
    out = torch.empty(m, n, dtype=torch.float16, device="cuda")
    if tokens:
        ctx.quant_linear((TCGEN05, tokens, 128, splits), xv, wv, out)
    else:
        ctx.prepare_quantized(m, n, k, out_dtype=torch.float16)
        ctx.matmul(xv, wv, out)
    assert ctx.status() == 0
    if fmt == I8 and not group:
        theirs = reference_gemm(reference_kernels, (SM80, 16 if m == 16 else 128, 64, 1), xv, wv, m, n, k, I8,
                                out_type=F16, dtype=torch.float16)
        assert torch.equal(out.view(torch.int16), theirs.view(torch.int16))
    assert rel_err_torch(out, exact_product(xv, wv, fmt, group)) < (2e-2 if fmt == FP8 else 1e-2)
    rows = np.arange(0, m, max(1, m // 16))
    channels = channel_slice(n, 128, seed=1)
    want16, exact = oracle.quant_linear(np.ascontiguousarray(xv.values.cpu().numpy()[rows]),
                                        np.ascontiguousarray(xv.scales.cpu().numpy()[:, rows] if group else xv.scales.cpu().numpy().reshape(-1)[rows]),
                                        np.ascontiguousarray(wv.values.cpu().numpy()[channels]),
                                        np.ascontiguousarray(wv.scales.cpu().numpy()[:, channels] if group else wv.scales.cpu().numpy().reshape(-1)[channels]),
                                        fmt, group, group, out_type=F16)
    got = out[torch.from_numpy(rows).cuda()][:, torch.from_numpy(channels).cuda()]
    if fmt == I8 and not group:
        assert np.array_equal(got.contiguous().view(torch.int16).cpu().numpy().view(np.uint16), want16)
    else:
        assert rel_err(got.float().cpu().numpy(), exact) < (2e-2 if fmt == FP8 else 1e-2)


@pytest.mark.parametrize("mode,fmt,group,tol", [("fp8", FP8, 0, 2e-2), ("group_int8", I8, 128, 1e-2), ("group_fp8", FP8, 128, 2e-2)])
@pytest.mark.parametrize("m,tokens,splits", [(16, 16, 2), (128, 128, 4), (130, 64, 1)])
def test_fused_chain_other_modes(oracle, ctx_factory, mode, fmt, group, tol, m, tokens, splits):
    """bias + same-dtype residual + ReLU on the modes the bit-exact chain test does not cover. The error
    is measured against the magnitude of the terms that were added, so a sum that cancels to nearly
    zero is not held to a relative bound of its own size."""
    n, k = 496, 1280
    ctx = ctx_factory(mode)
    xv, wv = quantized_operands(ctx, m, k, n, fmt, group, seed=7 * m + fmt, student_t=bool(group))
    bias = synth_device(1, n, 3, std=0.5, outliers=False)
    skip = synth_device(m, n, 4, outliers=False)
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    ctx.quant_linear((TCGEN05, tokens, 128, splits), xv, wv, out, bias=bias, residual=skip, activation=1)
    assert ctx.status() == 0
    product = exact_product(xv, wv, fmt, group)
    want = torch.relu(product + bias.double() + skip.double())
    magnitude = product.abs() + bias.double().abs() + skip.double().abs()
    assert float(((out.double() - want).abs() / (tol * magnitude + 1e-6)).max()) < 1.0
    to_np = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
    sx = xv.scales.cpu().numpy() if group else xv.scales.cpu().numpy().reshape(-1)
    sw = wv.scales.cpu().numpy() if group else wv.scales.cpu().numpy().reshape(-1)
    want16, _ = oracle.quant_linear(xv.values.cpu().numpy(), sx, wv.values.cpu().numpy(), sw, fmt, group, group,
                                    bias=to_np(bias).ravel(), residual=to_np(skip), activation=1)
    oracle_value = torch.from_numpy((want16.astype(np.uint32) << 16).view(np.float32)).cuda().double()
    assert float(((out.double() - oracle_value).abs() / (tol * magnitude + 1e-6)).max()) < 1.0
