"""ctypes/numpy access to the CPU oracle (oracle/liboracle.so) and, where built, to the reference's
own CUDA kernels (oracle/_ref/libttsref.so). Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_SO = ROOT / "oracle" / "liboracle.so"
REF_SO = ROOT / "oracle" / "_ref" / "libttsref.so"
BF16, F32, I32, FP8, I8, F16 = 0, 1, 2, 3, 4, 5


class OracleEpilogue(C.Structure):
    _fields_ = [("bias", C.c_void_p), ("residual", C.c_void_p), ("residual_f32", C.c_void_p),
                ("value_scale", C.c_float), ("residual_scale", C.c_float), ("output_scale", C.c_float),
                ("activation", C.c_int), ("alpha", C.c_float)]


class OracleFinish(C.Structure):
    _fields_ = [("bias", C.c_void_p), ("gate", C.c_void_p), ("residual", C.c_void_p), ("condition", C.c_void_p),
                ("raw", C.c_void_p), ("residual_index", C.c_void_p), ("gate_rows", C.c_int), ("residual_rows", C.c_int),
                ("condition_rows", C.c_int), ("rows_per_sequence", C.c_int), ("valid_rows_per_sequence", C.c_int),
                ("input_repeat", C.c_int), ("value_scale", C.c_float), ("residual_scale", C.c_float),
                ("output_scale", C.c_float), ("alpha", C.c_float), ("activation", C.c_int)]


class OracleNorm(C.Structure):
    _fields_ = [("weight", C.c_void_p), ("bias", C.c_void_p), ("projection_bias", C.c_void_p), ("residual", C.c_void_p),
                ("gate", C.c_void_p), ("scale", C.c_void_p), ("shift", C.c_void_p), ("residual_rows", C.c_int),
                ("gate_rows", C.c_int), ("scale_rows", C.c_int), ("shift_rows", C.c_int), ("rows_per_sequence", C.c_int),
                ("source_rows", C.c_void_p), ("eps", C.c_float)]


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _rows2d(a):
    """(contiguous uint16 [rows, cols] array or None, rows)."""
    if a is None:
        return None, 0
    a = np.ascontiguousarray(a, dtype=np.uint16)
    if a.ndim == 1:
        a = a.reshape(1, -1)
    return a, a.shape[0]


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        lib.oracle_f32_to_bf16.restype = C.c_uint16
        lib.oracle_f32_to_bf16.argtypes = [C.c_float]
        lib.oracle_bf16_to_f32.restype = C.c_float
        lib.oracle_bf16_to_f32.argtypes = [C.c_uint16]
        lib.oracle_f16_to_f32.restype = C.c_float
        lib.oracle_f16_to_f32.argtypes = [C.c_uint16]
        for name in ("oracle_fp8_e4m3_encode", "oracle_fp8_e4m3_encode_toolkit", "oracle_int8_encode"):
            getattr(lib, name).restype = C.c_uint8
            getattr(lib, name).argtypes = [C.c_float]
        lib.oracle_fp8_e4m3_decode.restype = C.c_float
        lib.oracle_fp8_e4m3_decode.argtypes = [C.c_uint8]
        lib.oracle_scale.restype = C.c_float
        lib.oracle_scale.argtypes = [C.c_float, C.c_int]
        lib.oracle_rotation_sign.restype = C.c_float
        lib.oracle_rotation_sign.argtypes = [C.c_uint32]
        lib.oracle_rotate128.argtypes = [C.c_void_p, C.c_int]
        lib.oracle_row_quantize.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                            C.c_int, C.c_int, C.c_int]
        lib.oracle_int8_accumulate.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        lib.oracle_quant_linear.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                            C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                            C.POINTER(OracleEpilogue), C.c_int]
        lib.oracle_quantized_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                                              C.c_float, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                              C.c_int]
        lib.oracle_quantized_gated.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                               C.c_void_p, C.c_int, C.c_int, C.c_int]
        finish, norm = C.POINTER(OracleFinish), C.POINTER(OracleNorm)
        lib.oracle_pointwise.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, finish, C.c_void_p]
        lib.oracle_pointwise_quantize.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, finish, C.c_void_p, C.c_void_p,
                                                  C.c_void_p, C.c_int, C.c_int, C.c_int]
        lib.oracle_layer_norm_quantize.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, norm, C.c_void_p, C.c_void_p,
                                                   C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        lib.oracle_normalized_linear.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, norm, C.c_void_p, C.c_void_p, C.c_int,
                                                 C.c_int, finish, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        lib.oracle_time_linear.restype = C.c_double
        lib.oracle_time_linear.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                           C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int]
        lib.oracle_hardware_threads.restype = C.c_int

    # ---- helpers over numpy -------------------------------------------------------------------
    def to_bf16(self, x: np.ndarray) -> np.ndarray:
        """fp32 array -> bf16 bit patterns (uint16), round to nearest even."""
        u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
        rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
        return rounded.astype(np.uint16)

    @staticmethod
    def from_bf16(b: np.ndarray) -> np.ndarray:
        return (b.astype(np.uint32) << 16).view(np.float32)

    def row_quantize(self, src16: np.ndarray, fmt: int, group=0, rotation=0, src_type=BF16, stride=0):
        rows, cols = src16.shape if stride == 0 else (src16.shape[0], src16.shape[1])
        src16 = np.ascontiguousarray(src16)
        values = np.zeros((rows, cols), dtype=np.uint8)
        scales = np.zeros(((cols + group - 1) // group, rows) if group else (rows,), dtype=np.float32)
        self.lib.oracle_row_quantize(_ptr(src16), src_type, rows, cols, stride, _ptr(values), _ptr(scales), fmt, group,
                                     rotation)
        return values, scales

    def int8_accumulate(self, xq: np.ndarray, wq: np.ndarray) -> np.ndarray:
        m, k = xq.shape
        n = wq.shape[0]
        acc = np.zeros((m, n), dtype=np.int32)
        self.lib.oracle_int8_accumulate(_ptr(np.ascontiguousarray(xq)), _ptr(np.ascontiguousarray(wq)), m, n, k, _ptr(acc))
        return acc

    def quant_linear(self, xq, sx, wq, sw, fmt, group_x=0, group_w=0, out_type=BF16, bias=None, residual=None,
                     residual_f32=None, activation=0, value_scale=1.0, residual_scale=1.0, output_scale=1.0, alpha=0.1,
                     threads=8):
        m, k = xq.shape
        n = wq.shape[0]
        out = np.zeros((m, n), dtype=np.uint16)
        exact = np.zeros((m, n), dtype=np.float32)
        keep = [np.ascontiguousarray(a) if a is not None else None for a in (bias, residual, residual_f32)]
        ep = OracleEpilogue(_ptr(keep[0]), _ptr(keep[1]), _ptr(keep[2]), value_scale, residual_scale, output_scale,
                            activation, alpha)
        self.lib.oracle_quant_linear(_ptr(np.ascontiguousarray(xq)), _ptr(np.ascontiguousarray(sx)),
                                     _ptr(np.ascontiguousarray(wq)), _ptr(np.ascontiguousarray(sw)), m, n, k, group_x,
                                     group_w, fmt, out_type, _ptr(out), _ptr(exact), C.byref(ep), threads)
        return out, exact

    def quantized_norm(self, residual16, update16, weight16, fmt, eps, gemma=False, update_scale16=None, group=0,
                       rotation=0, type_=BF16):
        rows, cols = residual16.shape
        residual16 = np.ascontiguousarray(residual16).copy()
        normalized = np.zeros((rows, cols), dtype=np.uint16)
        values = np.zeros((rows, cols), dtype=np.uint8)
        scales = np.zeros(((cols + group - 1) // group, rows) if group else (rows,), dtype=np.float32)
        upd = np.ascontiguousarray(update16) if update16 is not None else None
        us = np.ascontiguousarray(update_scale16) if update_scale16 is not None else None
        self.lib.oracle_quantized_norm(_ptr(residual16), _ptr(upd), _ptr(np.ascontiguousarray(weight16)), _ptr(us), rows,
                                       cols, type_, eps, int(gemma), _ptr(normalized), _ptr(values), _ptr(scales), fmt,
                                       group, rotation)
        return residual16, normalized, values, scales

    def quantized_gated(self, input16, fmt, kind=0, group=0, rotation=0, type_=BF16):
        rows, two = input16.shape
        width = two // 2
        activated = np.zeros((rows, width), dtype=np.uint16)
        values = np.zeros((rows, width), dtype=np.uint8)
        scales = np.zeros(((width + group - 1) // group, rows) if group else (rows,), dtype=np.float32)
        self.lib.oracle_quantized_gated(_ptr(np.ascontiguousarray(input16)), rows, width, type_, kind, _ptr(activated),
                                        _ptr(values), _ptr(scales), fmt, group, rotation)
        return activated, values, scales


    # ---- the row-wise operators (16-bit operands as uint16 bit patterns) ------------------------------
    @staticmethod
    def _finish(rows, cols, keep, bias=None, gate=None, residual=None, condition=None, raw=False, residual_rows=None,
                rows_per_sequence=1, valid_rows_per_sequence=0, input_repeat=1, value_scale=1.0, residual_scale=1.0,
                output_scale=1.0, alpha=0.1, activation=0):
        bias, _ = _rows2d(bias)
        gate, gate_rows = _rows2d(gate)
        residual, res_rows = _rows2d(residual)
        condition, condition_rows = _rows2d(condition)
        raw_out = np.zeros((rows, cols), dtype=np.uint16) if raw else None
        index = np.ascontiguousarray(residual_rows, dtype=np.int32) if residual_rows is not None else None
        keep.extend([bias, gate, residual, condition, raw_out, index])
        return OracleFinish(_ptr(bias), _ptr(gate), _ptr(residual), _ptr(condition), _ptr(raw_out), _ptr(index), gate_rows,
                            res_rows, condition_rows, rows_per_sequence, valid_rows_per_sequence, input_repeat, value_scale,
                            residual_scale, output_scale, alpha, activation), raw_out

    @staticmethod
    def _norm(keep, weight, bias, eps, residual=None, projection_bias=None, gate=None, shift=None, scale=None,
              rows_per_sequence=1, source_rows=None):
        weight, _ = _rows2d(weight)
        bias, _ = _rows2d(bias)
        projection_bias, _ = _rows2d(projection_bias)
        residual, residual_rows = _rows2d(residual)
        gate, gate_rows = _rows2d(gate)
        scale, scale_rows = _rows2d(scale)
        shift, shift_rows = _rows2d(shift)
        index = np.ascontiguousarray(source_rows, dtype=np.int32) if source_rows is not None else None
        keep.extend([weight, bias, projection_bias, residual, gate, scale, shift, index])
        return OracleNorm(_ptr(weight), _ptr(bias), _ptr(projection_bias), _ptr(residual), _ptr(gate), _ptr(scale), _ptr(shift),
                          residual_rows, gate_rows, scale_rows, shift_rows, rows_per_sequence, _ptr(index), eps)

    def pointwise(self, x16, type_=BF16, **finish):
        """-> (y, raw or None); output rows = input rows * input_repeat."""
        x16 = np.ascontiguousarray(x16, dtype=np.uint16)
        rows, cols = x16.shape[0] * finish.get("input_repeat", 1), x16.shape[1]
        keep = []
        f, raw = self._finish(rows, cols, keep, **finish)
        y = np.zeros((rows, cols), dtype=np.uint16)
        self.lib.oracle_pointwise(_ptr(x16), x16.shape[0], rows, cols, type_, C.byref(f), _ptr(y))
        return y, raw

    def pointwise_quantize(self, x16, fmt, group=0, rotation=0, type_=BF16, **finish):
        """-> (retained, raw or None, values, scales)."""
        x16 = np.ascontiguousarray(x16, dtype=np.uint16)
        rows, cols = x16.shape[0] * finish.get("input_repeat", 1), x16.shape[1]
        keep = []
        f, raw = self._finish(rows, cols, keep, **finish)
        retained = np.zeros((rows, cols), dtype=np.uint16)
        values = np.zeros((rows, cols), dtype=np.uint8)
        scales = np.zeros(((cols + group - 1) // group, rows) if group else (rows,), dtype=np.float32)
        self.lib.oracle_pointwise_quantize(_ptr(x16), x16.shape[0], rows, cols, type_, C.byref(f), _ptr(retained), _ptr(values),
                                           _ptr(scales), fmt, group, rotation)
        return retained, raw, values, scales

    def layer_norm_quantize(self, x16, weight16, bias16, eps, fmt, group=0, rotation=0, type_=BF16, **fusion):
        """-> (normalized, raw, values, scales)."""
        x16 = np.ascontiguousarray(x16, dtype=np.uint16)
        source = fusion.get("source_rows")
        rows, cols = (len(source) if source is not None else x16.shape[0]), x16.shape[1]
        keep = []
        n = self._norm(keep, weight16, bias16, eps, **fusion)
        normalized, raw = np.zeros((rows, cols), dtype=np.uint16), np.zeros((rows, cols), dtype=np.uint16)
        values = np.zeros((rows, cols), dtype=np.uint8)
        scales = np.zeros(((cols + group - 1) // group, rows) if group else (rows,), dtype=np.float32)
        self.lib.oracle_layer_norm_quantize(_ptr(x16), x16.shape[0], rows, cols, type_, C.byref(n), _ptr(normalized), _ptr(raw),
                                            _ptr(values), _ptr(scales), fmt, group, rotation)
        return normalized, raw, values, scales

    def normalized_linear(self, x16, weight16, bias16, eps, wq, sw, fmt, type_=BF16, fusion=None, **finish):
        """-> (out, encoded, encoded_scales, normalized, raw)."""
        x16 = np.ascontiguousarray(x16, dtype=np.uint16)
        rows, cols = x16.shape
        channels = wq.shape[0]
        keep = []
        n = self._norm(keep, weight16, bias16, eps, **(fusion or {}))
        f, _ = self._finish(rows, channels, keep, **finish)
        out = np.zeros((rows, channels), dtype=np.uint16)
        encoded, scales = np.zeros((rows, cols), dtype=np.uint8), np.zeros(rows, dtype=np.float32)
        normalized, raw = np.zeros((rows, cols), dtype=np.uint16), np.zeros((rows, cols), dtype=np.uint16)
        wq, sw = np.ascontiguousarray(wq, dtype=np.uint8), np.ascontiguousarray(sw, dtype=np.float32)
        self.lib.oracle_normalized_linear(_ptr(x16), rows, cols, type_, C.byref(n), _ptr(wq), _ptr(sw), channels, fmt, C.byref(f),
                                          _ptr(out), _ptr(encoded), _ptr(scales), _ptr(normalized), _ptr(raw))
        return out, encoded, scales, normalized, raw


def build_oracle():
    subprocess.run(["make", "-C", str(ROOT / "oracle"), "oracle"], check=True, capture_output=True)


def load() -> Oracle:
    if not ORACLE_SO.exists():
        build_oracle()
    return Oracle(C.CDLL(str(ORACLE_SO)))


class RefView(C.Structure):
    _fields_ = [("data", C.c_void_p), ("rows", C.c_int), ("cols", C.c_int), ("stride", C.c_int)]


class RefEpilogue(C.Structure):
    _fields_ = [("bias", RefView), ("residual", RefView), ("raw", RefView), ("gate", RefView), ("condition", RefView),
                ("value_scale", C.c_float), ("output_scale", C.c_float), ("residual_scale", C.c_float), ("alpha", C.c_float),
                ("activation", C.c_int), ("rows_per_sequence", C.c_int), ("valid_rows_per_sequence", C.c_int),
                ("input_repeat", C.c_int), ("residual_rows", C.c_void_p)]


class RefFusion(C.Structure):
    _fields_ = [("residual", RefView), ("projection_bias", RefView), ("raw", RefView), ("gate", RefView), ("shift", RefView),
                ("scale", RefView), ("rows_per_sequence", C.c_int), ("source_rows", C.c_void_p)]


def ref_view(t) -> RefView:
    """torch CUDA tensor (1-D or 2-D, dense inner axis) or None -> the shim's view struct."""
    if t is None:
        return RefView(None, 0, 0, 0)
    if t.dim() == 1:
        t = t.unsqueeze(0)
    stride = t.stride(0) if t.shape[0] > 1 and t.stride(0) != t.shape[1] else 0
    return RefView(t.data_ptr(), t.shape[0], t.shape[1], stride)


def ref_epilogue(bias=None, residual=None, raw=None, gate=None, condition=None, value_scale=1.0, output_scale=1.0,
                 residual_scale=1.0, alpha=0.1, activation=0, rows_per_sequence=1, valid_rows_per_sequence=0, input_repeat=1,
                 residual_rows=None) -> RefEpilogue:
    return RefEpilogue(ref_view(bias), ref_view(residual), ref_view(raw), ref_view(gate), ref_view(condition), value_scale,
                       output_scale, residual_scale, alpha, activation, rows_per_sequence, valid_rows_per_sequence,
                       input_repeat, residual_rows.data_ptr() if residual_rows is not None else None)


def ref_fusion(residual=None, projection_bias=None, raw=None, gate=None, shift=None, scale=None, rows_per_sequence=1,
               source_rows=None) -> RefFusion:
    return RefFusion(ref_view(residual), ref_view(projection_bias), ref_view(raw), ref_view(gate), ref_view(shift),
                     ref_view(scale), rows_per_sequence, source_rows.data_ptr() if source_rows is not None else None)


def load_reference():
    if not REF_SO.exists():
        return None
    lib = C.CDLL(str(REF_SO))
    lib.ttsref_last_error.restype = C.c_char_p
    lib.ttsref_row_quantize.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_int,
                                        C.c_int, C.c_int, C.c_void_p]
    lib.ttsref_quant_linear.argtypes = [C.c_int] * 9 + [C.c_void_p] * 6 + [C.c_size_t, C.c_void_p, C.c_int, C.c_int]
    lib.ttsref_quantized_norm.argtypes = [C.c_void_p] * 4 + [C.c_int] * 3 + [C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                                                             C.c_int, C.c_float, C.c_int, C.c_void_p]
    lib.ttsref_quantized_gated.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p] + [C.c_int] * 6 + [C.c_void_p]
    lib.ttsref_residual_add_f32.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    view, ep, fu = C.POINTER(RefView), C.POINTER(RefEpilogue), C.POINTER(RefFusion)
    lib.ttsref_pointwise.argtypes = [view, view, C.c_int, ep, C.c_void_p]
    lib.ttsref_pointwise_quantize.argtypes = [view, C.c_int, C.c_void_p, C.c_void_p] + [C.c_int] * 5 + [ep, view, C.c_int, C.c_void_p]
    lib.ttsref_layer_norm_quantize.argtypes = [view, C.c_int, C.c_void_p, C.c_void_p] + [C.c_int] * 5 + [view, view, C.c_float, fu,
                                                                                                    view, C.c_void_p]
    lib.ttsref_normalized_quantized_linear.argtypes = [view, C.c_int, view, view, view, C.c_float, fu, C.c_void_p, C.c_void_p,
                                                       C.c_int, C.c_int, C.c_int, view, ep, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ttsref_candidates.argtypes = [C.c_int] * 6 + [C.c_size_t, C.c_size_t, C.c_void_p, C.c_int]
    lib.ttsref_select.argtypes = [C.c_int] * 7 + [C.c_size_t, C.c_void_p, C.c_char_p, C.c_int]
    return lib
