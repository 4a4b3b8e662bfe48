"""Generates the golden fixtures in this folder on seeded synthetic inputs.

    python -m tests.golden.make_golden [--reference] [--out DIR]

The reference project holds no golden vectors for this path. Every fixture freezes the CPU oracle's
answers (bytes, scales, INT32 accumulators, bf16 outputs) for a small case of each mode; with
`--reference` (needs a CUDA device and oracle/_ref/libttsref.so, the reference's own kernels built from
its sources) the outputs of the REFERENCE kernels on the same inputs are stored beside them under
`ref_*` keys: its row quantizer's bytes and scales for both operands, its GEMM's bf16 output (CUTLASS
SM80 kernel for INT8, scalar GEMV for FP8, grouped kernel for the K-group modes), and its fused
producers' outputs (residual + RMSNorm + quantize; SiLU gate + quantize), and the outputs of its row-wise
operators (finishing pass, finish + quantize, LayerNorm + quantize, fused norm + quantize + projection).
The fixtures then pin the oracle to the reference without the reference tree or a GPU at test time.
"""
import argparse
import ctypes as C
import json
from pathlib import Path

import numpy as np

from tests import oracle_binding, synth
from tests.oracle_binding import BF16, FP8, I8

HERE = Path(__file__).resolve().parent
CASES = [  # name, format, group, rotation, m, n, k, student-t dof, reference GEMM path
    ("int8_m16_k2048_n256", I8, 0, 0, 16, 256, 2048, None, (2, 16, 64, 1)),
    ("fp8_m8_k1024_n128", FP8, 0, 0, 8, 128, 1024, None, (1, 4, 8, 1)),
    ("group_int8_m16_k768_n128", I8, 128, 128, 16, 128, 768, 3.0, (4, 16, 64, 1)),
    ("group_fp8_m5_k512_n144", FP8, 128, 128, 5, 144, 512, 3.0, (4, 16, 64, 1)),
]
SEQUENCE = [("sequence_int8_r8_c512", I8, 0, 0, 8, 512, 64), ("sequence_group_fp8_r8_c512", FP8, 128, 128, 8, 512, 64),
            ("sequence_fp8_r8_c384", FP8, 0, 0, 8, 384, 72)]
FINISH = dict(value_scale=0.7, residual_scale=1.3, output_scale=0.9, activation=1, rows_per_sequence=4)
PRODUCERS = [("producers_int8_r8_k512", I8, 0, 0, 8, 512), ("producers_group_fp8_r8_k512", FP8, 128, 128, 8, 512)]


def reference_outputs(lib, torch, fmt, group, rotation, x16, w16, path):
    dev = lambda a: torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    m, k = x16.shape
    n = w16.shape[0]
    out = {}
    views = {}
    for tag, source, rows in (("x", x16, m), ("w", w16, n)):
        values = torch.empty(rows, k, dtype=torch.uint8, device="cuda")
        scales = torch.empty(((k + group - 1) // group, rows) if group else (rows,), dtype=torch.float32, device="cuda")
        held = dev(source)
        rc = lib.ttsref_row_quantize(held.data_ptr(), rows, k, 0, BF16, values.data_ptr(), scales.data_ptr(), fmt, group,
                                     rotation, None)
        assert rc == 0, lib.ttsref_last_error()
        views[tag] = (values, scales)
        out[f"ref_{tag}q"], out[f"ref_s{tag}"] = values.cpu().numpy(), scales.cpu().numpy()
    y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    workspace = torch.zeros(8 << 20, dtype=torch.uint8, device="cuda")
    rc = lib.ttsref_quant_linear(*path, m, n, k, group, group, views["x"][0].data_ptr(), views["x"][1].data_ptr(),
                                 views["w"][0].data_ptr(), views["w"][1].data_ptr(), y.data_ptr(), workspace.data_ptr(),
                                 workspace.numel(), None, fmt, BF16)
    assert rc == 0, lib.ttsref_last_error()
    torch.cuda.synchronize()
    out["ref_out16"] = y.view(torch.int16).cpu().numpy().view(np.uint16)
    return out


def reference_producers(lib, torch, fmt, group, rotation, residual16, update16, weight16, gate_up16):
    dev = lambda a: torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    rows, cols = residual16.shape
    shape = ((cols + group - 1) // group, rows) if group else (rows,)
    out = {}
    residual = dev(residual16).clone()
    values = torch.empty(rows, cols, dtype=torch.uint8, device="cuda")
    scales = torch.empty(shape, dtype=torch.float32, device="cuda")
    update, weight = dev(update16), dev(weight16)
    rc = lib.ttsref_quantized_norm(residual.data_ptr(), update.data_ptr(), weight.data_ptr(), None, rows, cols, BF16,
                                   values.data_ptr(), scales.data_ptr(), fmt, group, rotation, 1e-6, 0, None)
    assert rc == 0, lib.ttsref_last_error()
    torch.cuda.synchronize()
    out.update(ref_norm_q=values.cpu().numpy(), ref_norm_s=scales.cpu().numpy(),
               ref_norm_residual=residual.view(torch.int16).cpu().numpy().view(np.uint16))
    gate_up = dev(gate_up16)
    rc = lib.ttsref_quantized_gated(gate_up.data_ptr(), rows, cols, BF16, values.data_ptr(), scales.data_ptr(), fmt, group,
                                    rotation, 0, 148, 1, None)
    assert rc == 0, lib.ttsref_last_error()
    torch.cuda.synchronize()
    out.update(ref_gated_q=values.cpu().numpy(), ref_gated_s=scales.cpu().numpy())
    return out


def sequence_inputs(oracle, name, fmt, group, rotation, rows, cols, channels):
    seed = len(name)
    a = dict(x16=oracle.to_bf16(synth.activations(rows, cols, seed, outlier_columns=4)),
             bias16=oracle.to_bf16(synth.weights(1, cols, seed + 1, std=0.5)),
             gate16=oracle.to_bf16(1.0 + synth.weights(rows // 4, cols, seed + 2, std=0.3)),
             residual16=oracle.to_bf16(synth.activations(rows, cols, seed + 3, outlier_columns=0)),
             norm_weight16=oracle.to_bf16(1.0 + synth.weights(1, cols, seed + 4, std=0.1)),
             norm_bias16=oracle.to_bf16(synth.weights(1, cols, seed + 5, std=0.2)),
             out_bias16=oracle.to_bf16(synth.weights(1, channels, seed + 6, std=0.5)))
    a["wq"], a["sw"] = oracle.row_quantize(oracle.to_bf16(synth.weights(channels, cols, seed + 7)), fmt)
    return a


def sequence_oracle(oracle, a, fmt, group, rotation):
    """The oracle's answers for one sequence fixture (also what tests/test_oracle.py recomputes)."""
    finish = dict(bias=a["bias16"], gate=a["gate16"], residual=a["residual16"], **FINISH)
    out = {}
    out["pw_y"], out["pw_raw"] = oracle.pointwise(a["x16"], BF16, raw=True, **finish)
    out["pwq_retained"], _, out["pwq_values"], out["pwq_scales"] = oracle.pointwise_quantize(a["x16"], fmt, group, rotation, BF16,
                                                                                          **finish)
    out["ln_normalized"], out["ln_raw"], out["ln_values"], out["ln_scales"] = oracle.layer_norm_quantize(
        a["x16"], a["norm_weight16"], a["norm_bias16"], 1e-5, fmt, group, rotation, BF16, residual=a["residual16"])
    if not group:
        out["nl_out"], out["nl_encoded"], out["nl_scales"], _, _ = oracle.normalized_linear(
            a["x16"], a["norm_weight16"], a["norm_bias16"], 1e-5, a["wq"], a["sw"], fmt, BF16,
            fusion=dict(residual=a["residual16"]), bias=a["out_bias16"], activation=1)
    return out


def reference_sequence(lib, torch, a, fmt, group, rotation):
    from tests.oracle_binding import ref_epilogue, ref_fusion, ref_view
    dev = lambda b: torch.from_numpy(b.view(np.int16)).cuda().view(torch.bfloat16)
    bits = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)
    x, bias, gate, residual = dev(a["x16"]), dev(a["bias16"]), dev(a["gate16"]), dev(a["residual16"])
    rows, cols = x.shape
    shape = ((cols + group - 1) // group, rows) if group else (rows,)
    out = {}
    y, raw = torch.empty_like(x), torch.zeros_like(x)
    ep = ref_epilogue(bias=bias, gate=gate, residual=residual, raw=raw, **FINISH)
    assert lib.ttsref_pointwise(C.byref(ref_view(x)), C.byref(ref_view(y)), BF16, C.byref(ep), None) == 0, lib.ttsref_last_error()
    torch.cuda.synchronize()
    out.update(ref_pw_y=bits(y), ref_pw_raw=bits(raw))
    values = torch.empty(rows, cols, dtype=torch.uint8, device="cuda")
    scales = torch.empty(shape, dtype=torch.float32, device="cuda")
    kept = torch.zeros_like(x)
    ep = ref_epilogue(bias=bias, gate=gate, residual=residual, **FINISH)
    rc = lib.ttsref_pointwise_quantize(C.byref(ref_view(x)), BF16, values.data_ptr(), scales.data_ptr(), rows, cols, fmt, group,
                                       rotation, C.byref(ep), C.byref(ref_view(kept)), 148, None)
    assert rc == 0, lib.ttsref_last_error()
    torch.cuda.synchronize()
    out.update(ref_pwq_retained=bits(kept), ref_pwq_values=values.cpu().numpy(), ref_pwq_scales=scales.cpu().numpy())
    weight, norm_bias = dev(a["norm_weight16"]), dev(a["norm_bias16"])
    raw, kept = torch.zeros_like(x), torch.zeros_like(x)
    fu = ref_fusion(residual=residual, raw=raw)
    rc = lib.ttsref_layer_norm_quantize(C.byref(ref_view(x)), BF16, values.data_ptr(), scales.data_ptr(), rows, cols, fmt, group,
                                        rotation, C.byref(ref_view(weight)), C.byref(ref_view(norm_bias)), 1e-5, C.byref(fu),
                                        C.byref(ref_view(kept)), None)
    assert rc == 0, lib.ttsref_last_error()
    torch.cuda.synchronize()
    out.update(ref_ln_normalized=bits(kept), ref_ln_raw=bits(raw), ref_ln_values=values.cpu().numpy(),
               ref_ln_scales=scales.cpu().numpy())
    if not group:
        channels = a["wq"].shape[0]
        wq, sw = torch.from_numpy(a["wq"]).cuda(), torch.from_numpy(a["sw"]).cuda()
        result = torch.empty(rows, channels, dtype=torch.bfloat16, device="cuda")
        encoded = torch.empty(rows, cols, dtype=torch.uint8, device="cuda")
        encoded_scales = torch.empty(rows, dtype=torch.float32, device="cuda")
        normalized = torch.zeros_like(x)
        ep = ref_epilogue(bias=dev(a["out_bias16"]), activation=1)
        fu = ref_fusion(residual=residual)
        rc = lib.ttsref_normalized_quantized_linear(
            C.byref(ref_view(x)), BF16, C.byref(ref_view(normalized)), C.byref(ref_view(weight)), C.byref(ref_view(norm_bias)), 1e-5,
            C.byref(fu), wq.data_ptr(), sw.data_ptr(), channels, cols, fmt, C.byref(ref_view(result)), C.byref(ep),
            encoded.data_ptr(), encoded_scales.data_ptr(), None)
        assert rc == 1, lib.ttsref_last_error()
        torch.cuda.synchronize()
        out.update(ref_nl_out=bits(result), ref_nl_encoded=encoded.cpu().numpy(), ref_nl_scales=encoded_scales.cpu().numpy())
    return out


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", action="store_true", help="also store the reference kernels' outputs (needs a GPU)")
    parser.add_argument("--out", default=str(HERE))
    args = parser.parse_args()
    target = Path(args.out)
    target.mkdir(parents=True, exist_ok=True)
    oracle = oracle_binding.load()
    lib = torch = None
    if args.reference:
        import torch
        lib = oracle_binding.load_reference()
        if lib is None or not torch.cuda.is_available():
            raise SystemExit("--reference needs a CUDA device and oracle/_ref/libttsref.so")
    index = {"generator": "tests/golden/make_golden.py", "reference_held": bool(lib), "cases": [], "producers": [],
             "sequence": []}
    for name, fmt, group, rotation, m, n, k, dof, path in CASES:
        x16 = oracle.to_bf16(synth.activations(m, k, seed=len(name), outlier_columns=8, student_t=dof))
        w16 = oracle.to_bf16(synth.weights(n, k, seed=len(name) + 100))
        xq, sx = oracle.row_quantize(x16, fmt, group, rotation)
        wq, sw = oracle.row_quantize(w16, fmt, group, rotation)
        out16, _ = oracle.quant_linear(xq, sx, wq, sw, fmt, group, group, threads=2)
        arrays = dict(x16=x16, w16=w16, xq=xq, sx=sx, wq=wq, sw=sw, out16=out16)
        if fmt == I8 and not group:
            arrays["acc"] = oracle.int8_accumulate(xq.view(np.int8), wq.view(np.int8))
        if lib:
            arrays.update(reference_outputs(lib, torch, fmt, group, rotation, x16, w16, path))
        np.savez_compressed(target / f"{name}.npz", **arrays)
        index["cases"].append(dict(file=f"{name}.npz", format=fmt, group=group, rotation=rotation, m=m, n=n, k=k,
                                   reference_path=list(path)))
    for name, fmt, group, rotation, rows, cols in PRODUCERS:
        residual16 = oracle.to_bf16(synth.activations(rows, cols, seed=len(name), outlier_columns=4))
        update16 = oracle.to_bf16(synth.activations(rows, cols, seed=len(name) + 1, outlier_columns=0))
        weight16 = oracle.to_bf16(1.0 + synth.weights(1, cols, seed=len(name) + 2, std=0.1))
        gate_up16 = oracle.to_bf16(synth.activations(rows, 2 * cols, seed=len(name) + 3, outlier_columns=0))
        arrays = dict(residual16=residual16, update16=update16, weight16=weight16, gate_up16=gate_up16)
        if lib:
            arrays.update(reference_producers(lib, torch, fmt, group, rotation, residual16, update16, weight16, gate_up16))
        np.savez_compressed(target / f"{name}.npz", **arrays)
        index["producers"].append(dict(file=f"{name}.npz", format=fmt, group=group, rotation=rotation, rows=rows, cols=cols))
    for name, fmt, group, rotation, rows, cols, channels in SEQUENCE:
        arrays = sequence_inputs(oracle, name, fmt, group, rotation, rows, cols, channels)
        answers = sequence_oracle(oracle, arrays, fmt, group, rotation)
        if lib:
            answers.update(reference_sequence(lib, torch, arrays, fmt, group, rotation))
        np.savez_compressed(target / f"{name}.npz", **arrays, **answers)
        index["sequence"].append(dict(file=f"{name}.npz", format=fmt, group=group, rotation=rotation, rows=rows, cols=cols,
                                      channels=channels))
    (target / "index.json").write_text(json.dumps(index, indent=1))


if __name__ == "__main__":
    main()
