"""Host-side mirror of the reference's operator interface for the quantized linear path, over
torch CUDA tensors (torch is only the owner of device memory and streams here).

Names follow the reference: `quantize_rows`, `matmul`, `prepare_quantized`, `quantized_norm`,
`quantized_gated`, `linear` (src/ops/storage.h:12, src/ops/basic.h:11,25-26,33-35,
src/ops/linear.h:11-14) and `RowScaledView` (src/core/quantization.h:33-49). Every function ends in
a call through the C ABI of libb200q.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import BF16, F16, F32, FP8, I8, I32, Epilogue, NormFusion, Path_, RowScaled, Tensor

MODES = ("int8", "fp8", "group_int8", "group_fp8")
_TORCH_TYPES = {torch.bfloat16: BF16, torch.float16: F16, torch.float32: F32, torch.int32: I32,
                torch.int8: I8, torch.uint8: None}
RELU, LEAKY_RELU, SILU, GELU, GELU_TANH, TANH, SIGMOID = 1, 2, 3, 4, 5, 7, 8


def groups_of(mode: str) -> tuple[int, int, int]:
    """(activation group, weight group, rotation) — reference: quantization_groups, src/core/quantization.h:19-23."""
    return (128, 128, 128) if mode.startswith("group_") else (0, 0, 0)


def format_of(mode: str) -> int:
    return FP8 if mode.endswith("fp8") else I8


def _tensor(t: torch.Tensor | None, type_code: int | None = None) -> Tensor:
    if t is None:
        return Tensor(None, 0, 0, 0, 0, -1)
    if not t.is_cuda:
        raise ValueError("operands must live on a CUDA device")
    if t.dim() == 1:
        t = t.unsqueeze(0)
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("operands must be 2-D with a dense inner axis")
    code = type_code if type_code is not None else _TORCH_TYPES[t.dtype]
    stride = t.stride(0) if t.shape[0] > 1 and t.stride(0) != t.shape[1] else 0
    return Tensor(t.data_ptr(), t.shape[0], t.shape[1], stride, code, t.device.index)


@dataclass
class RowScaledView:
    """One-byte values [rows, K] + fp32 scales ([rows] or group-major [K/g, rows])."""
    values: torch.Tensor  # uint8 storage
    scales: torch.Tensor  # float32
    format: int           # I8 or FP8
    group_size: int = 0
    rotation_size: int = 0

    @staticmethod
    def empty(rows: int, cols: int, fmt: int, group: int = 0, rotation: int = 0, device="cuda") -> "RowScaledView":
        values = torch.empty(rows, cols, dtype=torch.uint8, device=device)
        shape = ((cols + group - 1) // group, rows) if group else (rows, 1)
        scales = torch.empty(shape, dtype=torch.float32, device=device)
        return RowScaledView(values, scales, fmt, group, rotation)

    def c(self) -> RowScaled:
        return RowScaled(_tensor(self.values, self.format), _tensor(self.scales, F32), self.group_size, self.rotation_size)

    def rows(self, first: int, count: int) -> "RowScaledView":
        """Leading-row view; only for per-row scales (K-group scales are row-minor)."""
        if self.group_size:
            raise ValueError("row slices of K-group scales are not contiguous")
        return RowScaledView(self.values[first:first + count], self.scales[first:first + count], self.format, 0,
                             self.rotation_size)


def _epilogue(bias=None, residual=None, residual_f32=None, activation=0, value_scale=1.0, output_scale=1.0,
              residual_scale=1.0, alpha=0.1, gate=None, condition=None, raw=None, rows_per_sequence=1,
              valid_rows_per_sequence=0, input_repeat=1, residual_rows=None) -> Epilogue:
    """reference: ops::Epilogue (src/ops/sequence.h:8-27); residual_rows is a device int32 tensor."""
    rows_ptr = C.c_void_p(residual_rows.data_ptr()) if residual_rows is not None else None
    return Epilogue(_tensor(bias), _tensor(residual), _tensor(residual_f32, F32), value_scale, output_scale,
                    residual_scale, alpha, activation, _tensor(gate), _tensor(condition), _tensor(raw), rows_per_sequence,
                    valid_rows_per_sequence, input_repeat, rows_ptr)


def _fusion(residual=None, projection_bias=None, raw=None, gate=None, shift=None, scale=None, rows_per_sequence=1,
            source_rows=None) -> NormFusion:
    """reference: ops::NormFusion (src/ops/sequence.h:53-57); source_rows is a device int32 tensor."""
    rows_ptr = C.c_void_p(source_rows.data_ptr()) if source_rows is not None else None
    return NormFusion(_tensor(residual), _tensor(projection_bias), _tensor(raw), _tensor(gate), _tensor(shift),
                      _tensor(scale), rows_per_sequence, rows_ptr)


class Context:
    """Device + stream + GEMM workspace + plan cache (reference: CudaContext, src/runtime/cuda_context.h:13-35)."""

    def __init__(self, mode: str = "int8", device: int = 0, stream: torch.cuda.Stream | None = None,
                 workspace_bytes: int = 8 << 20):
        if mode not in MODES:
            raise ValueError(f"quantization must be one of {MODES}")
        self.mode, self.device = mode, device
        self.format = format_of(mode)
        self.stream = stream
        self._workspace = torch.empty(workspace_bytes, dtype=torch.uint8, device=f"cuda:{device}")
        handle = C.c_void_p()
        stream_ptr = C.c_void_p(stream.cuda_stream) if stream is not None else None
        _lib.call("b200q_context_create", device, stream_ptr, C.c_void_p(self._workspace.data_ptr()), workspace_bytes,
                  mode.encode(), C.byref(handle))
        self._handle = handle
        self.multiprocessors = _lib.load().b200q_multiprocessors(handle)

    def close(self):
        if getattr(self, "_handle", None):
            _lib.load().b200q_context_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- producers
    def quantize_rows(self, x: torch.Tensor, out: RowScaledView) -> RowScaledView:
        _lib.call("b200q_row_quantize", self._handle, C.byref(_tensor(x)), C.byref(out.c()))
        return out

    def quantized_norm(self, residual, update, weight, out: RowScaledView, epsilon: float, gemma=False, update_scale=None):
        _lib.call("b200q_quantized_norm", self._handle, C.byref(_tensor(residual)), C.byref(_tensor(update)),
                  C.byref(_tensor(weight)), C.byref(out.c()), epsilon, int(gemma), C.byref(_tensor(update_scale)))
        return out

    def quantized_gated(self, x: torch.Tensor, out: RowScaledView, kind: int = 0) -> RowScaledView:
        _lib.call("b200q_quantized_gated", self._handle, C.byref(_tensor(x)), C.byref(out.c()), kind)
        return out

    # ---- GEMM
    def prepare_quantized(self, rows: int, channels: int, reduction: int, out_dtype=torch.bfloat16,
                          groups: tuple[int, int] | None = None, weight: RowScaledView | None = None) -> tuple[int, int, int, int]:
        ga, gw = groups if groups is not None else groups_of(self.mode)[:2]
        path = Path_()
        _lib.call("b200q_prepare", self._handle, rows, channels, reduction, _TORCH_TYPES[out_dtype], ga, gw, C.byref(path))
        if weight is not None:
            _lib.call("b200q_prepare_weight", self._handle, C.byref(weight.c()))
        return (path.kind, path.tokens, path.channels, path.splits)

    def select_path(self, rows, channels, reduction, groups=None):
        ga, gw = groups if groups is not None else groups_of(self.mode)[:2]
        path = Path_()
        _lib.call("b200q_select_path", self._handle, rows, channels, reduction, ga, gw, C.byref(path))
        return (path.kind, path.tokens, path.channels, path.splits)

    def seal(self):
        _lib.call("b200q_seal", self._handle)

    def matmul(self, x: RowScaledView, w: RowScaledView, out: torch.Tensor, **epilogue) -> torch.Tensor:
        ep = C.byref(_epilogue(**epilogue)) if epilogue else None
        _lib.call("b200q_linear", self._handle, C.byref(x.c()), C.byref(w.c()), C.byref(_tensor(out)), ep)
        return out

    def quant_linear(self, path, x: RowScaledView, w: RowScaledView, out: torch.Tensor, **epilogue) -> torch.Tensor:
        ep = C.byref(_epilogue(**epilogue)) if epilogue else None
        _lib.call("b200q_quant_linear", self._handle, C.byref(Path_(*path)), C.byref(x.c()), C.byref(w.c()),
                  C.byref(_tensor(out)), ep)
        return out

    def linear(self, x: torch.Tensor, w: RowScaledView, scratch: RowScaledView, out: torch.Tensor,
               quantized_output: RowScaledView | None = None, **epilogue):
        ep = C.byref(_epilogue(**epilogue)) if epilogue else None
        qo = C.byref(quantized_output.c()) if quantized_output is not None else None
        _lib.call("b200q_linear_forward", self._handle, C.byref(_tensor(x)), C.byref(w.c()), C.byref(scratch.c()),
                  C.byref(_tensor(out)), ep, qo)
        return out

    # ---- row-wise operators around the projections
    def pointwise(self, x: torch.Tensor, y: torch.Tensor, **epilogue) -> torch.Tensor:
        _lib.call("b200q_pointwise", self._handle, C.byref(_tensor(x)), C.byref(_tensor(y)), C.byref(_epilogue(**epilogue)))
        return y

    def pointwise_quantize(self, x: torch.Tensor, out: RowScaledView, retained: torch.Tensor | None = None,
                           **epilogue) -> RowScaledView:
        _lib.call("b200q_pointwise_quantize", self._handle, C.byref(_tensor(x)), C.byref(out.c()),
                  C.byref(_epilogue(**epilogue)), C.byref(_tensor(retained)))
        return out

    def layer_norm_quantize(self, x: torch.Tensor, out: RowScaledView, weight=None, bias=None, epsilon: float = 1e-5,
                            retained: torch.Tensor | None = None, **fusion) -> RowScaledView:
        _lib.call("b200q_layer_norm_quantize", self._handle, C.byref(_tensor(x)), C.byref(out.c()), C.byref(_tensor(weight)),
                  C.byref(_tensor(bias)), epsilon, C.byref(_fusion(**fusion)), C.byref(_tensor(retained)))
        return out

    def normalized_linear(self, x: torch.Tensor, w: RowScaledView, out: torch.Tensor, norm_weight=None, norm_bias=None,
                          epsilon: float = 1e-5, bias=None, normalized=None, fusion: dict | None = None,
                          quantized_output: RowScaledView | None = None, **epilogue) -> bool:
        """True when the fused kernel ran; False leaves the two-step path to the caller."""
        taken = C.c_int32(0)
        qo = C.byref(quantized_output.c()) if quantized_output is not None else None
        _lib.call("b200q_normalized_linear", self._handle, C.byref(_tensor(x)), C.byref(w.c()), C.byref(_tensor(bias)),
                  C.byref(_tensor(normalized)), C.byref(_tensor(out)), C.byref(_tensor(norm_weight)),
                  C.byref(_tensor(norm_bias)), epsilon, C.byref(_fusion(**(fusion or {}))), C.byref(_epilogue(**epilogue)),
                  qo, C.byref(taken))
        return bool(taken.value)

    def status(self) -> int:
        value = C.c_int32(0)
        _lib.call("b200q_status", self._handle, C.byref(value))
        return value.value


class Linear:
    """Quantized Linear layer (reference: tts::Linear, src/layers/linear.h:11-76): fuses the given 16-bit
    weight matrices by rows, quantizes them on the device at construction (the load-time step of
    Weights::quantized), and runs quantize -> GEMM -> fused epilogue per call."""

    def __init__(self, ctx: Context, parts: list[torch.Tensor], bias: torch.Tensor | None = None, max_rows: int = 64):
        self.ctx = ctx
        self._keep = (parts, bias)
        array = (Tensor * len(parts))(*[_tensor(p) for p in parts])
        handle = C.c_void_p()
        _lib.call("b200q_linear_layer_create", ctx._handle, array, len(parts), C.byref(_tensor(bias)), C.byref(handle))
        self._handle = handle
        self.out_features = sum(p.shape[0] for p in parts)
        self.in_features = parts[0].shape[1]
        _lib.call("b200q_linear_layer_prepare", ctx._handle, self._handle, max_rows)

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None, quantized_output: RowScaledView | None = None,
                **epilogue) -> torch.Tensor:
        if out is None:
            out = torch.empty(x.shape[0], self.out_features, dtype=x.dtype, device=x.device)
        ep = C.byref(_epilogue(**epilogue)) if epilogue else None
        qo = C.byref(quantized_output.c()) if quantized_output is not None else None
        _lib.call("b200q_linear_layer_forward", self.ctx._handle, self._handle, C.byref(_tensor(x)), C.byref(_tensor(out)), ep, qo)
        return out

    PLAN, PREPARE, CAPTURE, EXECUTE = 0, 1, 2, 3  # reference: ForwardContext::Mode (src/core/forward_context.h:58)

    def apply(self, mode: int, max_rows: int, x: torch.Tensor, out: torch.Tensor, **epilogue) -> torch.Tensor:
        """Phase-switched forward (reference: Linear::forward(input, output, ForwardContext &, finish))."""
        ep = C.byref(_epilogue(**epilogue)) if epilogue else None
        _lib.call("b200q_linear_layer_apply", self.ctx._handle, self._handle, mode, max_rows, C.byref(_tensor(x)),
                  C.byref(_tensor(out)), ep)
        return out

    def forward_segments(self, mode: int, max_rows: int, x: torch.Tensor, segments: list[tuple[int, int, int]],
                         out: torch.Tensor) -> torch.Tensor:
        flat = (C.c_int32 * (3 * len(segments)))(*[v for s in segments for v in s]) if segments else None
        _lib.call("b200q_linear_layer_forward_segments", self.ctx._handle, self._handle, mode, max_rows, C.byref(_tensor(x)),
                  flat, len(segments), C.byref(_tensor(out)))
        return out

    def normalized_forward(self, x: torch.Tensor, out: torch.Tensor, norm_weight=None, norm_bias=None, epsilon: float = 1e-5,
                           normalized=None, fusion: dict | None = None, quantized_output: RowScaledView | None = None,
                           **epilogue) -> torch.Tensor:
        ep = C.byref(_epilogue(**epilogue)) if epilogue else None
        qo = C.byref(quantized_output.c()) if quantized_output is not None else None
        _lib.call("b200q_linear_layer_normalized_forward", self.ctx._handle, self._handle, C.byref(_tensor(x)),
                  C.byref(_tensor(normalized)), C.byref(_tensor(out)), C.byref(_tensor(norm_weight)),
                  C.byref(_tensor(norm_bias)), epsilon, C.byref(_fusion(**(fusion or {}))), ep, qo)
        return out

    def weight(self) -> RowScaled:
        view = RowScaled()
        _lib.call("b200q_linear_layer_weight", self._handle, C.byref(view))
        return view

    def close(self):
        if getattr(self, "_handle", None):
            _lib.load().b200q_linear_layer_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
