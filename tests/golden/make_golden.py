"""Generates the golden fixtures in this folder from the CPU oracle on seeded synthetic inputs.

    python -m tests.golden.make_golden

The reference project holds no golden vectors for this path; these fixtures freeze the oracle's own
answers (bytes, scales, INT32 accumulators, bf16 outputs) for small cases of each mode so they can
be compared on the GPU box, where neither the reference tree nor a rebuild of the oracle is needed
to read them."""
import json
from pathlib import Path

import numpy as np

from tests import oracle_binding, synth
from tests.oracle_binding import FP8, I8

HERE = Path(__file__).resolve().parent
CASES = [  # name, format, group, rotation, m, n, k, student-t dof
    ("int8_m16_k2048_n256", I8, 0, 0, 16, 256, 2048, None),
    ("fp8_m8_k1024_n128", FP8, 0, 0, 8, 128, 1024, None),
    ("group_int8_m16_k768_n128", I8, 128, 128, 16, 128, 768, 3.0),
    ("group_fp8_m5_k512_n144", FP8, 128, 128, 5, 144, 512, 3.0),
]


def main():
    oracle = oracle_binding.load()
    index = {"generator": "tests/golden/make_golden.py", "cases": []}
    for name, fmt, group, rotation, m, n, k, dof in CASES:
        x16 = oracle.to_bf16(synth.activations(m, k, seed=len(name), outlier_columns=8, student_t=dof))
        w16 = oracle.to_bf16(synth.weights(n, k, seed=len(name) + 100))
        xq, sx = oracle.row_quantize(x16, fmt, group, rotation)
        wq, sw = oracle.row_quantize(w16, fmt, group, rotation)
        out16, _ = oracle.quant_linear(xq, sx, wq, sw, fmt, group, group, threads=2)
        arrays = dict(x16=x16, w16=w16, xq=xq, sx=sx, wq=wq, sw=sw, out16=out16)
        if fmt == I8 and not group:
            arrays["acc"] = oracle.int8_accumulate(xq.view(np.int8), wq.view(np.int8))
        np.savez_compressed(HERE / f"{name}.npz", **arrays)
        index["cases"].append(dict(file=f"{name}.npz", format=fmt, group=group, rotation=rotation, m=m, n=n, k=k))
    (HERE / "index.json").write_text(json.dumps(index, indent=1))


if __name__ == "__main__":
    main()
