"""Pins of the CPU oracle. The reference ships no tests or golden vectors for this path, so the
pins are hand-derived known answers for every rule the oracle restates (each test names the
reference lines the rule comes from), algebraic properties, and the committed fixtures in
tests/golden/, which also hold the outputs of the reference's own kernels on the same inputs."""
import json
from pathlib import Path

import numpy as np
import pytest

from tests import synth
from tests.oracle_binding import BF16, F16, FP8, I8

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_int8_round_half_even_and_clamp(oracle):
    # reference: src/ops/kernels/quant/quant_format.cuh:37-47 — clamp to +-127, then ties to even; -128 never appears
    cases = {0.5: 0, 1.5: 2, 2.5: 2, -0.5: 0, -1.5: -2, -2.5: -2, 126.5: 126, 127.5: 127, -127.5: -127,
             1e9: 127, -1e9: -127, 0.49999997: 0, 126.50001: 127}
    for value, want in cases.items():
        assert np.int8(np.uint8(oracle.lib.oracle_int8_encode(value))) == want, value


def test_scale_rule(oracle):
    # reference: quant_format.cuh:62-64
    assert oracle.lib.oracle_scale(0.0, I8) == 1.0
    assert oracle.lib.oracle_scale(127.0, I8) == 1.0
    assert oracle.lib.oracle_scale(448.0, FP8) == 1.0
    assert oracle.lib.oracle_scale(1.0, I8) == np.float32(1.0) / np.float32(127.0)
    tiny = np.float32(1e-45)
    assert oracle.lib.oracle_scale(float(tiny), I8) == np.finfo(np.float32).tiny  # floor at FLT_MIN


def test_fp8_known_answers(oracle):
    # reference: quant_format.cuh:12-22 (cuda_fp8.h conversions): RN-even, saturate to 448, subnormals down to 2^-9
    enc, dec = oracle.lib.oracle_fp8_e4m3_encode, oracle.lib.oracle_fp8_e4m3_decode
    assert dec(enc(1.0625)) == 1.0 and dec(enc(1.1875)) == 1.25  # ties to even
    assert dec(enc(460.0)) == 448.0 and dec(enc(1e9)) == 448.0 and dec(enc(-1e9)) == -448.0
    assert enc(2.0 ** -10) == 0 and enc(2.0 ** -9) == 1 and enc(3 * 2.0 ** -10) == 2
    assert enc(0.0) == 0 and enc(-0.0) == 0x80
    assert dec(0x7E) == 448.0 and dec(0x08) == 2.0 ** -6 and dec(0x01) == 2.0 ** -9


def test_fp8_software_encoder_equals_toolkit_conversion(oracle):
    rng = np.random.default_rng(0)
    values = np.concatenate([rng.standard_normal(20000) * s for s in (1e-3, 0.05, 1, 30, 500)]).astype(np.float32)
    exact = np.array([oracle.lib.oracle_fp8_e4m3_decode(q) for q in range(256) if q & 0x7F != 0x7F], dtype=np.float32)
    mids = ((exact[:-1].astype(np.float64) + exact[1:]) / 2).astype(np.float32)  # exact ties between neighbours
    for v in np.concatenate([values, exact, mids, np.nextafter(mids, 1e9), np.nextafter(mids, -1e9)]):
        assert oracle.lib.oracle_fp8_e4m3_encode(float(v)) == oracle.lib.oracle_fp8_e4m3_encode_toolkit(float(v)), v


def test_fp8_decode_encode_round_trip(oracle):
    for q in range(256):
        if q & 0x7F == 0x7F:
            continue
        assert oracle.lib.oracle_fp8_e4m3_encode(oracle.lib.oracle_fp8_e4m3_decode(q)) == q


def test_bf16_and_f16_conversions(oracle):
    assert oracle.lib.oracle_f32_to_bf16(1.0) == 0x3F80
    assert oracle.lib.oracle_f32_to_bf16(float(np.float32(1.00390625))) == 0x3F80  # tie -> even
    assert oracle.lib.oracle_f32_to_bf16(float(np.float32(1.01171875))) == 0x3F82  # tie -> even (up)
    rng = np.random.default_rng(1)
    x = (rng.standard_normal(4096) * 3).astype(np.float32)
    assert np.array_equal(oracle.to_bf16(x), np.array([oracle.lib.oracle_f32_to_bf16(float(v)) for v in x], dtype=np.uint16))
    halves = rng.integers(0, 0x7C00, 4096, dtype=np.uint16)
    want = halves.view(np.float16).astype(np.float32)
    got = np.array([oracle.lib.oracle_f16_to_f32(int(h)) for h in halves], dtype=np.float32)
    assert np.array_equal(got, want)


def test_rotation_sign_hash(oracle):
    # reference: src/ops/kernels/quant/quant_device.cuh:100-104 — 32-bit wraparound integer hash of the column
    def sign(j):
        h = (j * 0x45D9F3B) & 0xFFFFFFFF
        h = ((h ^ (h >> 16)) * 0x45D9F3B) & 0xFFFFFFFF
        return 1.0 if (h ^ (h >> 16)) & 1 else -1.0
    for j in list(range(300)) + [6143, 65535, 2 ** 31 - 1]:
        assert oracle.lib.oracle_rotation_sign(j) == sign(j)


def _rotate(oracle, v, column=0):
    buf = np.ascontiguousarray(v, dtype=np.float32).copy()
    oracle.lib.oracle_rotate128(buf.ctypes.data, column)
    return buf


def test_rotation_is_signed_sylvester_hadamard(oracle):
    # reference: quant_device.cuh:96-125. The butterfly network equals H128 (Sylvester order) / sqrt(128) applied to D x.
    h = np.array([[1.0]])
    while h.shape[0] < 128:
        h = np.block([[h, h], [h, -h]])
    rng = np.random.default_rng(2)
    x = rng.integers(-8, 9, 128).astype(np.float32)  # small integers: every butterfly sum is exact
    signs = np.array([oracle.lib.oracle_rotation_sign(256 + j) for j in range(128)], dtype=np.float32)
    want = ((h @ (x * signs).astype(np.float64)) * 0.08838834764831845).astype(np.float32)
    assert np.array_equal(_rotate(oracle, x, 256), (h @ (x * signs)).astype(np.float32) * np.float32(0.08838834764831845))
    assert np.allclose(_rotate(oracle, x, 256), want, rtol=1e-6)


def test_rotation_preserves_norm_and_dot_product(oracle):
    rng = np.random.default_rng(3)
    x, w = rng.standard_normal(128).astype(np.float32), rng.standard_normal(128).astype(np.float32)
    rx, rw = _rotate(oracle, x, 384), _rotate(oracle, w, 384)
    assert abs(np.linalg.norm(rx) - np.linalg.norm(x)) < 1e-4 * np.linalg.norm(x)
    assert abs(float(rx @ rw) - float(x @ w)) < 1e-4 * np.linalg.norm(x) * np.linalg.norm(w)


def test_unsigned_transform_twice_is_identity(oracle):
    # With all signs equal the matrix is symmetric orthogonal: applying it twice returns the input.
    rng = np.random.default_rng(4)
    x = rng.standard_normal(128).astype(np.float32)
    signs = np.array([oracle.lib.oracle_rotation_sign(j) for j in range(128)], dtype=np.float32)
    once = _rotate(oracle, x * signs, 0)          # D cancels: H/sqrt(128) x
    twice = _rotate(oracle, once * signs, 0)
    assert np.allclose(twice, x, atol=1e-5)


def test_row_quantize_layouts(oracle):
    x = synth.activations(5, 384, seed=9)
    x16 = oracle.to_bf16(x)
    xf = oracle.from_bf16(x16)
    q, s = oracle.row_quantize(x16, I8)
    assert s.shape == (5,) and np.array_equal(s, np.abs(xf).max(axis=1) / np.float32(127))
    assert np.abs(q.view(np.int8).astype(np.int32)).max() == 127
    qg, sg = oracle.row_quantize(x16, I8, group=128)
    assert sg.shape == (3, 5)  # group-major: [K/128, rows]
    for g in range(3):
        assert np.array_equal(sg[g], np.abs(xf[:, g * 128:(g + 1) * 128]).max(axis=1) / np.float32(127))
    # ragged tail group (reference: quant_device.cuh:63-88 handles columns - column remaining)
    q2, s2 = oracle.row_quantize(np.ascontiguousarray(x16[:, :200]), I8, group=128)
    assert s2.shape == (2, 5) and np.array_equal(s2[1], np.abs(xf[:, 128:200]).max(axis=1) / np.float32(127))
    zeros = np.zeros((2, 128), dtype=np.uint16)
    qz, sz = oracle.row_quantize(zeros, FP8, group=128, rotation=128)
    assert not (qz & 0x7F).any() and np.all(sz == 1.0)  # -0.0 keeps its sign bit, as on the GPU


def test_dequantized_linear_tracks_float_matmul(oracle):
    m, n, k = 8, 96, 512
    x16, w16 = oracle.to_bf16(synth.activations(m, k, 1, outlier_columns=0)), oracle.to_bf16(synth.weights(n, k, 2))
    truth = oracle.from_bf16(x16).astype(np.float64) @ oracle.from_bf16(w16).astype(np.float64).T
    for fmt, group, rotation, tol in ((I8, 0, 0, 0.03), (FP8, 0, 0, 0.08), (I8, 128, 128, 0.03), (FP8, 128, 128, 0.08)):
        xq, sx = oracle.row_quantize(x16, fmt, group, rotation)
        wq, sw = oracle.row_quantize(w16, fmt, group, rotation)
        _, exact = oracle.quant_linear(xq, sx, wq, sw, fmt, group, group, threads=2)
        assert np.abs(exact - truth).max() < tol * np.abs(truth).max(), (fmt, group)


def test_int8_accumulators_are_exact_integers(oracle):
    rng = np.random.default_rng(5)
    xq = rng.integers(-127, 128, (4, 256), dtype=np.int8)
    wq = rng.integers(-127, 128, (32, 256), dtype=np.int8)
    want = xq.astype(np.int64) @ wq.astype(np.int64).T
    assert np.array_equal(oracle.int8_accumulate(xq, wq), want.astype(np.int32))
    ones = np.full((1, 6144), 127, dtype=np.int8)
    assert oracle.int8_accumulate(ones, ones)[0, 0] == 6144 * 127 * 127  # the largest sum the path can see


def test_epilogue_rounding_chain(oracle):
    # reference: src/ops/kernels/sequence/sequence_internal.cuh:52-74 — every step rounds to the storage type
    xq = np.full((1, 16), 3, dtype=np.uint8)
    wq = np.full((16, 16), 5, dtype=np.uint8)
    sx, sw = np.array([0.5], dtype=np.float32), np.full(16, 0.25, dtype=np.float32)
    base = 16 * 15 * 0.5 * 0.25  # 30
    bias = oracle.to_bf16(np.full(16, 0.0078125, dtype=np.float32))  # 2^-7: lost when added to 30 in bf16
    out, _ = oracle.quant_linear(xq, sx, wq, sw, I8, bias=bias)
    assert np.all(oracle.from_bf16(out) == base)
    res = np.full((1, 16), -100.0, dtype=np.float32)
    out, _ = oracle.quant_linear(xq, sx, wq, sw, I8, residual_f32=res, activation=1)
    assert np.all(oracle.from_bf16(out) == 0.0)  # relu(30 - 100)


def test_golden_fixtures(oracle):
    """Fixtures made by tests/golden/make_golden.py from this oracle on seeded inputs: they freeze the
    oracle's answers so that a later change to it cannot drift unnoticed."""
    index = json.loads((GOLDEN / "index.json").read_text())
    assert index["cases"], "no golden cases"
    for case in index["cases"]:
        data = np.load(GOLDEN / case["file"])
        fmt, group, rotation = case["format"], case["group"], case["rotation"]
        q, s = oracle.row_quantize(data["x16"], fmt, group, rotation)
        assert np.array_equal(q, data["xq"]) and np.array_equal(s.view(np.uint32), data["sx"].view(np.uint32)), case
        wq, sw = oracle.row_quantize(data["w16"], fmt, group, rotation)
        assert np.array_equal(wq, data["wq"]) and np.array_equal(sw.view(np.uint32), data["sw"].view(np.uint32)), case
        out, _ = oracle.quant_linear(q, s, wq, sw, fmt, group, group, threads=2)
        assert np.array_equal(out, data["out16"]), case
        if fmt == I8 and not group:
            assert np.array_equal(oracle.int8_accumulate(q.view(np.int8), wq.view(np.int8)), data["acc"]), case


def test_producers_keep_reference_rounding_points(oracle):
    # reference: quant_norm.cu:14-123 and quant_gated.cu:18-85
    rng = np.random.default_rng(6)
    x16 = oracle.to_bf16(rng.standard_normal((3, 256)).astype(np.float32))
    w16 = oracle.to_bf16((1 + 0.1 * rng.standard_normal(256)).astype(np.float32))
    _, normalized, q, s = oracle.quantized_norm(x16, None, w16, I8, 1e-6)
    xf, wf = oracle.from_bf16(x16), oracle.from_bf16(w16)
    approx = xf / np.sqrt((xf.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + 1e-6) * wf
    assert np.abs(oracle.from_bf16(normalized) - approx).max() < 0.03
    q2, s2 = oracle.row_quantize(normalized, I8)
    assert np.array_equal(q, q2) and np.array_equal(s, s2)  # the tail is the plain row quantizer
    gu16 = oracle.to_bf16(rng.standard_normal((2, 512)).astype(np.float32))
    act, q, s = oracle.quantized_gated(gu16, I8, kind=0)
    g, u = oracle.from_bf16(gu16[:, :256]), oracle.from_bf16(gu16[:, 256:])
    assert np.abs(oracle.from_bf16(act) - g / (1 + np.exp(-g)) * u).max() < 0.03


def _bf16(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def test_oracle_against_reference_held_fixtures(oracle):
    """The `ref_*` arrays of the fixtures are outputs of the REFERENCE's kernels (row quantizer, CUTLASS SM80 /
    GEMV / grouped GEMM) recorded on a B200 by tests/golden/make_golden.py --reference. INT8: bytes, scales and
    bf16 GEMM bits equal the oracle's; FP8 bytes equal up to the sign of zero; FP8 and K-group GEMM outputs
    within 2e-2 / 1e-2 relative (floor 1e-2 * rms) of the oracle's exact result."""
    index = json.loads((GOLDEN / "index.json").read_text())
    assert index.get("reference_held"), "fixtures were generated without the reference kernels"
    for case in index["cases"]:
        data = np.load(GOLDEN / case["file"])
        fmt, group, rotation = case["format"], case["group"], case["rotation"]
        for tag, source in (("x", "x16"), ("w", "w16")):
            q, s = oracle.row_quantize(data[source], fmt, group, rotation)
            theirs_q, theirs_s = data[f"ref_{tag}q"], data[f"ref_s{tag}"]
            assert np.array_equal(s.ravel().view(np.uint32), theirs_s.ravel().view(np.uint32)), (case, tag)
            differs = q != theirs_q
            if fmt == FP8:
                differs &= ((q | theirs_q) & 0x7F) != 0
            assert not differs.any(), (case, tag)
        out, exact = oracle.quant_linear(data["ref_xq"], data["ref_sx"], data["ref_wq"], data["ref_sw"], fmt, group, group,
                                         threads=2)
        if fmt == I8 and not group:
            assert np.array_equal(out, data["ref_out16"]), case
        else:
            want = exact.astype(np.float64)
            floor = 1e-2 * np.sqrt(np.mean(want ** 2))
            error = np.max(np.abs(_bf16(data["ref_out16"]) - want) / np.maximum(np.abs(want), floor))
            assert error < (2e-2 if fmt == FP8 else 1e-2) + 2.0 ** -8, (case, error)


def test_oracle_producers_against_reference_held_fixtures(oracle):
    """Residual + RMSNorm + quantize and SiLU-gate + quantize as the reference's kernels computed them. The residual
    written back is exact bf16 arithmetic and must match bit for bit; the quantized rows depend on the GPU's
    approximate rsqrt / exp, which a CPU cannot reproduce bit for bit, so bytes may differ by one step on a small
    fraction of elements and scales by a few ulps."""
    index = json.loads((GOLDEN / "index.json").read_text())
    for case in index["producers"]:
        data = np.load(GOLDEN / case["file"])
        fmt, group, rotation = case["format"], case["group"], case["rotation"]
        residual, _, q, s = oracle.quantized_norm(data["residual16"], data["update16"], data["weight16"].ravel(), fmt, 1e-6,
                                                  group=group, rotation=rotation)
        assert np.array_equal(residual, data["ref_norm_residual"]), case
        _, gq, gs = oracle.quantized_gated(data["gate_up16"], fmt, kind=0, group=group, rotation=rotation)
        for mine_q, mine_s, theirs_q, theirs_s in ((q, s, data["ref_norm_q"], data["ref_norm_s"]),
                                                   (gq, gs, data["ref_gated_q"], data["ref_gated_s"])):
            assert np.allclose(mine_s.ravel(), theirs_s.ravel(), rtol=2e-2), case
            if fmt == I8:
                step = np.abs(mine_q.view(np.int8).astype(np.int32) - theirs_q.view(np.int8).astype(np.int32))
                assert step.max() <= 1 + (1 if rotation else 0) and (step > 0).mean() < 0.05, (case, step.max(), (step > 0).mean())
            else:
                decode = np.array([oracle.lib.oracle_fp8_e4m3_decode(v) for v in range(256)], dtype=np.float64)
                a, b = decode[mine_q], decode[theirs_q]
                close = np.abs(a - b) <= 0.13 * np.maximum(np.abs(a), np.abs(b)) + 2.0 ** -9  # one e4m3 step
                assert close.mean() > 0.999 and (mine_q != theirs_q).mean() < 0.05, case


def test_finish_chain_known_answers(oracle):
    # reference: Finish::apply, src/ops/kernels/sequence/sequence_internal.cuh:52-74
    x = oracle.to_bf16(np.array([[30.0, -2.0, 1.0, 1.0]], dtype=np.float32))
    bias = oracle.to_bf16(np.array([[0.0078125, 0.5, 0.0, 0.0]], dtype=np.float32))  # 2^-7 vanishes next to 30 in bf16
    y, raw = oracle.pointwise(x, bias=bias, activation=1, raw=True)
    assert oracle.from_bf16(y).tolist() == [[30.0, 0.0, 1.0, 1.0]]
    assert oracle.from_bf16(raw).tolist() == [[30.0, -1.5, 1.0, 1.0]]      # raw holds the value before the activation
    # a residual row index past the end poisons the row, -1 adds nothing (sequence_internal.cuh:63-66)
    res = oracle.to_bf16(np.ones((2, 4), dtype=np.float32))
    y, _ = oracle.pointwise(np.repeat(x, 3, axis=0), residual=res, residual_rows=np.array([1, -1, 2]))
    out = oracle.from_bf16(y)
    assert out[0].tolist() == [31.0, -1.0, 2.0, 2.0] and out[1].tolist() == [30.0, -2.0, 1.0, 1.0] and np.isnan(out[2]).all()
    # rows past valid_rows_per_sequence are zeroed, the gate is per sequence, input rows repeat
    gate = oracle.to_bf16(np.array([[2.0] * 4, [0.5] * 4], dtype=np.float32))
    y, _ = oracle.pointwise(x, gate=gate, rows_per_sequence=2, valid_rows_per_sequence=1, input_repeat=4)
    out = oracle.from_bf16(y)
    assert out[0].tolist() == [60.0, -4.0, 2.0, 2.0] and not out[1].any() and out[2].tolist() == [15.0, -1.0, 0.5, 0.5]
    # value_scale * v + residual_scale * skip is one rounded product and a fused multiply-add (the reference's
    # finishing pass is built with contraction): 0.7f*3 + fl(1.3f*7) differs from fl(0.7f*3) + fl(1.3f*7) in fp32
    v, r = np.float32(-0.9296875), np.float32(1.53125)
    one = oracle.to_bf16(np.array([[v]], dtype=np.float32))
    y, _ = oracle.pointwise(one, residual=oracle.to_bf16(np.array([[r]], dtype=np.float32)), value_scale=0.7, residual_scale=1.3)
    assert float(oracle.from_bf16(y)[0, 0]) == 1.3359375  # separate roundings would give 1.34375


def test_oracle_sequence_operators_against_reference_held_fixtures(oracle):
    """Finishing pass, finish + quantize, LayerNorm + quantize and the fused norm + quantize + projection: the oracle's
    answers are frozen in the fixtures and compared with what the REFERENCE's kernels produced on the same inputs (`ref_*`,
    recorded on a B200). The finishing chain (ReLU, scales that are not powers of two) is exact arithmetic: bit for bit.
    LayerNorm goes through the GPU's approximate rsqrt: normalized values within one bf16 step, bytes within one
    quantization step, projection outputs within 2e-2 relative (floor 1e-2 * rms)."""
    from tests.golden.make_golden import sequence_oracle
    index = json.loads((GOLDEN / "index.json").read_text())
    assert index.get("sequence"), "no sequence fixtures"
    decode = np.array([oracle.lib.oracle_fp8_e4m3_decode(v) for v in range(256)], dtype=np.float64)
    for case in index["sequence"]:
        data = np.load(GOLDEN / case["file"])
        fmt, group, rotation = case["format"], case["group"], case["rotation"]
        mine = sequence_oracle(oracle, data, fmt, group, rotation)
        for key, value in mine.items():  # the oracle has not drifted from what was frozen
            assert np.array_equal(np.asarray(value).view(np.uint8), data[key].view(np.uint8)), (case, key)
        for key in ("pw_y", "pw_raw", "pwq_retained", "pwq_values", "ln_raw"):
            assert np.array_equal(mine[key], data["ref_" + key]), (case, key)
        assert np.array_equal(mine["pwq_scales"].ravel().view(np.uint32), data["ref_pwq_scales"].ravel().view(np.uint32)), case
        a, b = _bf16(mine["ln_normalized"]), _bf16(data["ref_ln_normalized"])
        assert np.all(np.abs(a - b) <= 2.0 ** -7 * np.maximum(np.abs(a), np.abs(b))), case
        assert np.allclose(mine["ln_scales"].ravel(), data["ref_ln_scales"].ravel(), rtol=2e-2), case
        if fmt == I8:
            step = np.abs(mine["ln_values"].view(np.int8).astype(np.int32) - data["ref_ln_values"].view(np.int8).astype(np.int32))
            assert step.max() <= 1 + (1 if rotation else 0), (case, step.max())
        else:
            qa, qb = decode[mine["ln_values"]], decode[data["ref_ln_values"]]
            close = np.abs(qa - qb) <= 0.13 * np.maximum(np.abs(qa), np.abs(qb)) + 2.0 ** -9
            assert close.mean() > 0.999, case
        if not group:
            want, got = _bf16(mine["nl_out"]), _bf16(data["ref_nl_out"])
            floor = 1e-2 * np.sqrt(np.mean(want ** 2))
            assert np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)) < 2e-2, case
