"""ctypes binding of libb200q.so — the C ABI declared in include/b200q.h.

There is no fallback: if the shared library is missing or fails to load, importing the compute
functions raises. Nothing here computes; it only marshals pointers.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libb200q.so"

BF16, F32, I32, FP8, I8, F16 = 0, 1, 2, 3, 4, 5


class Tensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("rows", C.c_int32), ("cols", C.c_int32), ("stride", C.c_int32),
                ("type", C.c_int32), ("device", C.c_int32)]


class RowScaled(C.Structure):
    _fields_ = [("values", Tensor), ("scales", Tensor), ("group_size", C.c_int32), ("rotation_size", C.c_int32)]


class Epilogue(C.Structure):
    _fields_ = [("bias", Tensor), ("residual", Tensor), ("residual_f32", Tensor), ("value_scale", C.c_float),
                ("output_scale", C.c_float), ("residual_scale", C.c_float), ("alpha", C.c_float),
                ("activation", C.c_int32), ("gate", Tensor), ("condition", Tensor), ("raw", Tensor),
                ("rows_per_sequence", C.c_int32), ("valid_rows_per_sequence", C.c_int32), ("input_repeat", C.c_int32),
                ("residual_rows", C.c_void_p)]


class NormFusion(C.Structure):
    _fields_ = [("residual", Tensor), ("projection_bias", Tensor), ("raw", Tensor), ("gate", Tensor), ("shift", Tensor),
                ("scale", Tensor), ("rows_per_sequence", C.c_int32), ("source_rows", C.c_void_p)]


class Path_(C.Structure):
    _fields_ = [("kind", C.c_int32), ("tokens", C.c_int32), ("channels", C.c_int32), ("splits", C.c_int32)]


_ERR = (C.c_char_p, C.c_size_t)
_PT, _PR, _PE, _PP = C.POINTER(Tensor), C.POINTER(RowScaled), C.POINTER(Epilogue), C.POINTER(Path_)
_PF = C.POINTER(NormFusion)

# name -> (restype, argtypes); the single source of truth the symbol-export test checks against.
SIGNATURES = {
    "b200q_version": (C.c_char_p, ()),
    "b200q_context_create": (C.c_int, (C.c_int32, C.c_void_p, C.c_void_p, C.c_size_t, C.c_char_p,
                                       C.POINTER(C.c_void_p), *_ERR)),
    "b200q_context_destroy": (None, (C.c_void_p,)),
    "b200q_row_quantize": (C.c_int, (C.c_void_p, _PT, _PR, *_ERR)),
    "b200q_quantized_norm": (C.c_int, (C.c_void_p, _PT, _PT, _PT, _PR, C.c_float, C.c_int32, _PT, *_ERR)),
    "b200q_quantized_gated": (C.c_int, (C.c_void_p, _PT, _PR, C.c_int32, *_ERR)),
    "b200q_prepare": (C.c_int, (C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _PP, *_ERR)),
    "b200q_prepare_weight": (C.c_int, (C.c_void_p, _PR, *_ERR)),
    "b200q_seal": (C.c_int, (C.c_void_p, *_ERR)),
    "b200q_linear": (C.c_int, (C.c_void_p, _PR, _PR, _PT, _PE, *_ERR)),
    "b200q_quant_linear": (C.c_int, (C.c_void_p, _PP, _PR, _PR, _PT, _PE, *_ERR)),
    "b200q_select_path": (C.c_int, (C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _PP, *_ERR)),
    "b200q_linear_forward": (C.c_int, (C.c_void_p, _PT, _PR, _PR, _PT, _PE, _PR, *_ERR)),
    "b200q_pointwise": (C.c_int, (C.c_void_p, _PT, _PT, _PE, *_ERR)),
    "b200q_pointwise_quantize": (C.c_int, (C.c_void_p, _PT, _PR, _PE, _PT, *_ERR)),
    "b200q_layer_norm_quantize": (C.c_int, (C.c_void_p, _PT, _PR, _PT, _PT, C.c_float, _PF, _PT, *_ERR)),
    "b200q_normalized_linear": (C.c_int, (C.c_void_p, _PT, _PR, _PT, _PT, _PT, _PT, _PT, C.c_float, _PF, _PE, _PR,
                                          C.POINTER(C.c_int32), *_ERR)),
    "b200q_linear_layer_create": (C.c_int, (C.c_void_p, _PT, C.c_int32, _PT, C.POINTER(C.c_void_p), *_ERR)),
    "b200q_linear_layer_destroy": (None, (C.c_void_p,)),
    "b200q_linear_layer_prepare": (C.c_int, (C.c_void_p, C.c_void_p, C.c_int32, *_ERR)),
    "b200q_linear_layer_forward": (C.c_int, (C.c_void_p, C.c_void_p, _PT, _PT, _PE, _PR, *_ERR)),
    "b200q_linear_layer_apply": (C.c_int, (C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, _PT, _PT, _PE, *_ERR)),
    "b200q_linear_layer_forward_segments": (C.c_int, (C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, _PT,
                                                      C.POINTER(C.c_int32), C.c_int32, _PT, *_ERR)),
    "b200q_linear_layer_normalized_forward": (C.c_int, (C.c_void_p, C.c_void_p, _PT, _PT, _PT, _PT, _PT, C.c_float, _PF,
                                                        _PE, _PR, *_ERR)),
    "b200q_linear_layer_weight": (C.c_int, (C.c_void_p, _PR, *_ERR)),
    "b200q_quant_linear_static": (C.c_int, (C.c_int32, C.c_void_p, _PP, _PR, _PR, _PT, _PE, *_ERR)),
    "b200q_static_status": (C.c_int, (C.c_int32, C.c_void_p, C.POINTER(C.c_int32), *_ERR)),
    "b200q_inject_wait_expiry": (C.c_int, (C.c_int32, C.c_int64, *_ERR)),
    "b200q_status": (C.c_int, (C.c_void_p, C.POINTER(C.c_int32), *_ERR)),
    "b200q_multiprocessors": (C.c_int, (C.c_void_p,)),
    "b200q_row_capacity": (C.c_int32, (C.c_int32, C.c_uint32)),
    "b200q_candidates": (C.c_int, (C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _PP, C.c_int32, *_ERR)),
    "b200q_path_cost": (C.c_double, (C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, _PP, C.c_int32,
                                     C.c_int32, *_ERR)),
    "b200q_plan_path": (C.c_int, (C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                  C.c_size_t, _PP, C.POINTER(C.c_size_t), *_ERR)),
}

_lib = None


def load() -> C.CDLL:
    """Loads the library once; raises with the build command when it is absent."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m breeze_tts_cpp_b200.build` "
                               "(there is no CPU or PyTorch fallback)")
        lib = C.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = list(argtypes)
        _lib = lib
    return _lib


class B200QError(RuntimeError):
    pass


def call(name: str, *args):
    """Calls an int-returning entry point, appending the error buffer; raises B200QError on -1."""
    lib = load()
    buf = C.create_string_buffer(512)
    rc = getattr(lib, name)(*args, buf, len(buf))
    if rc != 0:
        raise B200QError(f"{name}: {buf.value.decode(errors='replace')}")
