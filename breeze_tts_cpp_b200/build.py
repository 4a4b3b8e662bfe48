"""Builds libb200q.so (the CUDA kernels + C++ host layer + C ABI) in-tree for sm_100a.

Run as `python -m breeze_tts_cpp_b200.build`. Objects are rebuilt only when a source or header
is newer; the producers are compiled with --fmad=false like the reference's own producers
(reference: CMakeLists.txt:94-105), the GEMM with default contraction.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
INCLUDE = HERE.parent / "include"
OBJ = HERE / "build"
LIB = HERE / "libb200q.so"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

# (source, extra flags)
SOURCES = [
    ("kernels/row_quantize.cu", ["--fmad=false"]),
    ("kernels/quant_norm.cu", ["--fmad=false"]),
    ("kernels/quant_gated.cu", ["--fmad=false"]),
    ("kernels/quant_linear.cu", []),
    ("kernels/quant_linear_static.cu", []),
    ("ops/quantized_gemm.cpp", []),
    ("ops/quantization_policy.cpp", []),
    ("ops/context.cpp", []),
    ("ops/ops.cpp", []),
    ("ops/sequence.cpp", []),
    ("kernels/sequence_pointwise.cu", ["--fmad=false"]),
    ("kernels/sequence_norm.cu", ["--fmad=false"]),
    ("layers/linear.cpp", []),
    ("c_api.cpp", []),
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libb200q.so")
    return found


def _newest_header() -> float:
    stamps = [p.stat().st_mtime for p in list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.cuh")) + list(INCLUDE.glob("*.h"))]
    return max(stamps) if stamps else 0.0


def _compile(nvcc: str, source: str, flags: list[str], header_stamp: float, verbose: bool) -> Path:
    src = CSRC / source
    obj = OBJ / (source.replace("/", "_") + ".o")
    if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, header_stamp):
        return obj
    cmd = [nvcc, "-std=c++17", "-O3", *ARCH, "-lineinfo", "-Xcompiler", "-fPIC", f"-I{CSRC}", f"-I{INCLUDE}",
           *flags, *os.environ.get("B200Q_NVCC_FLAGS", "").split(), "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode:
        raise RuntimeError(f"nvcc failed on {source}:\n{done.stdout}\n{done.stderr}")
    return obj


def build(verbose: bool = False, force: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    sources = [(s, f) for s, f in SOURCES if (CSRC / s).exists()]
    if force:
        for o in OBJ.glob("*.o"):
            o.unlink()
    stamp = _newest_header()
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objects = list(pool.map(lambda sf: _compile(nvcc, sf[0], sf[1], stamp, verbose), sources))
    if LIB.exists() and all(LIB.stat().st_mtime >= o.stat().st_mtime for o in objects):
        return LIB
    cmd = [nvcc, "-shared", *ARCH, "-o", str(LIB), *map(str, objects), "-lcudart"]
    if verbose:
        print(" ".join(cmd), flush=True)
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode:
        raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv))
