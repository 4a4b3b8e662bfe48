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


def candidates(rows, n, k, ga=0, gw=0, fmt=I8):
    paths = (Path_ * 64)()
    buf = C.create_string_buffer(256)
    count = _lib.load().b200q_candidates(rows, n, k, ga, gw, fmt, paths, 64, buf, len(buf))
    assert count >= 0, buf.value
    return [(p.kind, p.tokens, p.channels, p.splits) for p in paths[:count]]


def cost(rows, n, k, path, ga=0, gw=0, fmt=I8, gemm_only=1):
    buf = C.create_string_buffer(256)
    value = _lib.load().b200q_path_cost(rows, n, k, ga, gw, fmt, C.byref(Path_(*path)), 148, gemm_only, buf, len(buf))
    assert value >= 0, buf.value
    return value


def test_candidate_enumeration_and_cost_ranking():
    """reference interface: quant_linear_candidates / linear_pipeline_cost / select_linear
    (src/ops/cuda/quantization_policy.h:27-33); here every candidate is a tcgen05 launch shape."""
    found = candidates(64, 2048, 6144)
    assert found == [(5, 64, 128, s) for s in range(1, 9)]              # split-K 1..8 = cluster sizes
    assert candidates(1, 2048, 256) == [(5, 16, 128, 1), (5, 16, 128, 2)]  # never more splits than K blocks
    assert {p[1] for p in candidates(8192, 4096, 2048)} == {256}
    assert {p[1] for p in candidates(4096, 2048, 6144, 128, 128)} == {128, 64}
    assert candidates(16, 2048, 2040) == []                              # K % 16
    for rows, n, k, ga in ((64, 2048, 6144, 0), (16, 12288, 2048, 0), (4096, 2048, 6144, 128), (300, 640, 1024, 0)):
        options = candidates(rows, n, k, ga, ga)
        best = min(options, key=lambda p: (cost(rows, n, k, p, ga, ga), p[3]))
        chosen, _ = plan(rows, n, k, ga, ga)
        assert chosen == best                                            # select_linear = cheapest candidate
        assert cost(rows, n, k, best, ga, ga, gemm_only=0) > cost(rows, n, k, best, ga, ga)
    # the persistent K-group kernel never splits K: asking for a split selects the split-K kernel instead
    assert plan(4096, 2048, 6144, 128, 128)[0] == (5, 128, 128, 1)


def test_decode_plans_match_the_measured_table():
    """Splits that were measured fastest on a B200, inside the decoder chain, at 64 rows (the benchmark's
    single-GPU row count) for the layer's four shapes; at fewer rows neighbouring splits are within a few
    percent of each other, so only their range is pinned."""
    want = {(2048, 4096): 2, (2048, 2048): 4, (2048, 12288): 1, (6144, 2048): 6}
    for (k, n), splits in want.items():
        assert plan(64, n, k)[0][3] == splits
    for rows in (1, 4, 8, 16, 32):
        assert plan(rows, 12288, 2048)[0][3] == 1
        assert plan(rows, 2048, 2048)[0][3] in (3, 4) and plan(rows, 2048, 6144)[0][3] in (4, 5, 6)
        assert plan(rows, 4096, 2048)[0][3] in (2, 3, 4)
