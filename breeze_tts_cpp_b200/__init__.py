"""B200-native (sm_100a) quantized linear path of breeze_tts_cpp: fused quantize(+rotate) producers,
a tcgen05/TMEM/TMA W8A8 GEMM with a fused dequant epilogue, behind the reference's op interface."""
from . import _lib  # noqa: F401
from ._lib import BF16, F16, F32, FP8, I8, I32, B200QError  # noqa: F401

__all__ = ["_lib", "BF16", "F16", "F32", "FP8", "I8", "I32", "B200QError"]
