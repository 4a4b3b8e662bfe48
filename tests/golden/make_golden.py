"""Generates the golden fixtures in this folder on seeded synthetic inputs.

    python -m tests.golden.make_golden [--reference] [--out DIR]

The reference project holds no golden vectors for this path. Every fixture freezes the CPU oracle's
answers (bytes, scales, INT32 accumulators, bf16 outputs) for a small case of each mode; with
`--reference` (needs a CUDA device and oracle/_ref/libttsref.so, the reference's own kernels built from
its sources) the outputs of the REFERENCE kernels on the same inputs are stored beside them under
`ref_*` keys: its row quantizer's bytes and scales for both operands, its GEMM's bf16 output (CUTLASS
SM80 kernel for INT8, scalar GEMV for FP8, grouped kernel for the K-group modes), and its fused
producers' outputs (residual + RMSNorm + quantize; SiLU gate + quantize). The fixtures then pin the
oracle to the reference without the reference tree or a GPU at test time.
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
    index = {"generator": "tests/golden/make_golden.py", "reference_held": bool(lib), "cases": [], "producers": []}
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
    (target / "index.json").write_text(json.dumps(index, indent=1))


if __name__ == "__main__":
    main()
