"""The C-ABI library loads without a GPU, exports every symbol include/b200q.h declares, and its
host-only logic (row classes, planner, argument checks) behaves like the reference's."""
import ctypes as C
import re
from pathlib import Path

import pytest

from breeze_tts_cpp_b200 import _lib
from breeze_tts_cpp_b200._lib import FP8, I8, Path_

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    header = (ROOT / "include" / "b200q.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b(b200q_[a-z0-9_]+)\s*\(", header)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/b200q.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert b"quantization=int8,fp8,group_int8,group_fp8" in lib.b200q_version()


def test_row_capacity_classes():
    # reference: src/core/row_capacity.h:10-19 — 8 bins per octave, so padding stays <= 12.5 %
    lib = _lib.load()
    assert [lib.b200q_row_capacity(r, 8) for r in (1, 2, 3, 15, 16, 17, 33, 64, 65, 100, 2048, 2049)] == \
           [1, 2, 3, 15, 16, 18, 36, 64, 72, 104, 2048, 2304]
    for rows in range(1, 3000, 7):
        cap = lib.b200q_row_capacity(rows, 8)
        assert rows <= cap <= rows * 1.125 + 1
    assert lib.b200q_row_capacity(0, 8) == -1 and lib.b200q_row_capacity(5, 0) == -1


def plan(rows, n, k, ga=0, gw=0, fmt=I8, sms=148, workspace=8 << 20):
    path, need = Path_(), C.c_size_t()
    _lib.call("b200q_plan_path", rows, n, k, ga, gw, fmt, sms, workspace, C.byref(path), C.byref(need))
    return (path.kind, path.tokens, path.channels, path.splits), need.value


def test_planner_spreads_decode_shapes_over_the_machine():
    for rows in (1, 4, 16, 64):
        for n, k in ((4096, 2048), (2048, 2048), (12288, 2048), (2048, 6144)):
            (kind, tokens, channels, splits), need = plan(rows, n, k)
            assert kind == 5 and channels == 128 and tokens >= min(rows, 16) and tokens in (16, 32, 64, 128, 256)
            ctas = (n // 128) * splits
            assert ctas >= 64, (rows, n, k, splits)           # memory-bound: many SMs stream weights
            assert splits <= k // 128 and need <= 8 << 20
    (_, tokens, _, splits), _ = plan(8192, 12288, 2048)
    assert tokens == 256 and splits == 1                      # compute-bound: big tiles, no split
    (_, tokens, _, _), _ = plan(4096, 2048, 6144, 128, 128)
    assert tokens == 128                                      # K-group epilogue keeps 128 tokens in registers


def test_planner_needs_only_the_status_header_and_rejects_bad_shapes():
    (_, _, _, splits), need = plan(64, 2048, 6144, workspace=32768)
    assert 1 <= splits <= 8 and need == 32768  # split-K partials stay in shared memory (cluster of <= 8 CTAs)
    with pytest.raises(_lib.B200QError):
        plan(16, 2048, 2040)       # K % 16 (reference: src/ops/cuda/quantization.cpp:210)
    with pytest.raises(_lib.B200QError):
        plan(0, 2048, 2048)


def test_context_creation_without_gpu_fails_loudly():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    handle = C.c_void_p()
    with pytest.raises(_lib.B200QError):
        _lib.call("b200q_context_create", 0, None, None, 0, b"int8", C.byref(handle))
    with pytest.raises(_lib.B200QError):
        _lib.call("b200q_context_create", 0, None, None, 0, b"int4", C.byref(handle))
