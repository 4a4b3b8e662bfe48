#!/usr/bin/env python
"""Benchmark of the quantized linear hot path: one JSON line with the headline metric, the end-to-end
figure through host buffers, the roofline of the dominant kernel, a CPU baseline and one row per
benchmark configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200q|reference|reference-cpu]
    python bench.py --case <qkv|o|gate_up|down> <rows> [mode] [launches]     (one small case for a profiler)

Workload (`config.workload`): the quantized linears of a synthetic 28-layer decoder stack
(hidden 2048, fused QKV 4096, O 2048, fused gate+up 12288, down 6144->2048; INT8 W8A8 with
per-channel weight scales and dynamic per-token activation scales), 64 concurrent decode streams
sharded data-parallel over the GPUs (64/N rows per GPU), weights replicated. One step = one decode
step through the chain the reference decoder runs (src/layers/transformer/decoder.h:241-293): per
layer  residual-add + RMSNorm + quantize -> QKV GEMM -> row quantize (stands for the attention
output) -> O GEMM -> residual-add + RMSNorm + quantize -> gate/up GEMM -> SiLU-gate + quantize ->
down GEMM;  8 launches per layer, 224 per step, replayed as one CUDA graph. A step streams 1.41 GB
of distinct weights, far more than the 126 MB L2. Both arms (`--impl b200q`, `--impl reference`) run
the same chain; the reference arm uses only the reference's own kernels and plain torch tensors.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HIDDEN, QKV, FFN, LAYERS, STREAMS = 2048, 4096, 6144, 28, 64
SHAPES = {"qkv": (HIDDEN, QKV), "o": (HIDDEN, HIDDEN), "gate_up": (HIDDEN, 2 * FFN), "down": (FFN, HIDDEN)}  # name: (K, N)
SEED = 0x5EED
EPSILON = 1e-6
BF16, FP8, I8 = 0, 3, 4  # tts::Type codes
NOMINAL_HBM_GBS, NOMINAL_TENSOR_TOPS = 8000.0, 4500.0

# DRAM bytes (read + written) of one GEMM launch at M=64, from single-launch ncu captures of each of
# the four layer shapes (dram__bytes_read.sum + dram__bytes_write.sum). Other row counts scale them
# by the algorithmic bytes, which is what the traffic follows (weights dominate both).
NCU_DRAM_BYTES_M64 = {"qkv": 8_596_352, "o": 4_394_112, "gate_up": 25_406_720, "down": 13_044_992}  # the bf16 outputs stay in L2


# ------------------------------------------------------------------------------------------------
# algorithmic bytes / ops (per linear, per-channel modes): quantize 2MK read + MK+4M written;
# GEMM MK + NK + 4(M+N) read + 2MN written (+4MN when an fp32 residual is read); ops 2MNK.
def linear_bytes(m, k, n, residual=False, group=0, quantize=True):
    scales = 4 * (m + n) * (k // group if group else 1)
    gemm = m * k + n * k + scales + 2 * m * n + (4 * m * n if residual else 0)
    quant = (2 * m * k + m * k + 4 * m * (k // group if group else 1)) if quantize else 0
    return gemm + quant


def step_bytes(m, gemm_only=False):
    return LAYERS * sum(linear_bytes(m, k, n, quantize=not gemm_only) for k, n in SHAPES.values())


def step_ops(m):
    return LAYERS * sum(2 * m * k * n for k, n in SHAPES.values())


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data.get("bf16_tflops", 0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs (queries only)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc, self.index = None, gpu_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.samples = []
        if not self.proc:
            return
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9 and parts[1].replace(".", "").isdigit():
                self.samples.append(parts)

    def summary(self):
        if not getattr(self, "samples", None):
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = [float(s[1]) for s in self.samples]
        busy = [v for v in sm if v > 0.5 * max(sm)] or sm
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[5 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": float(self.samples[0][2]), "reasons": reasons,
                "samples": len(sm), "power_w_max": max(float(s[3]) for s in self.samples if s[3].replace(".", "").isdigit())}


# ------------------------------------------------------------------------------------------------
def synth_activations(torch, rows, cols, seed, device, outlier_fraction=0.005, student_t=False):
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32)
    if student_t:  # Student-t, 3 degrees of freedom
        x = x / (torch.randn(3, rows, cols, generator=g, device=device).pow(2).sum(0) / 3).sqrt()
    count = max(1, round(cols * outlier_fraction)) if outlier_fraction else 0
    if count:
        columns = torch.randperm(cols, generator=g, device=device)[:count]
        x[:, columns] *= 20.0
    return x


def synth_weight(torch, n, k, seed, device, std=0.02):
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(n, k, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


class Quantized:
    """One-byte values [rows, K] + fp32 scales, as plain torch tensors (both arms read these)."""

    def __init__(self, torch, rows, cols, device, group=0):
        self.values = torch.empty(rows, cols, dtype=torch.uint8, device=device)
        self.scales = torch.empty(((cols + group - 1) // group, rows) if group else (rows, 1), dtype=torch.float32, device=device)
        self.rows, self.cols, self.group = rows, cols, group


class Stack:
    """Weights (quantized once at load by the arm's own quantizer, like the reference's Weights::quantized),
    norm weights and activation buffers of the synthetic decoder."""

    def __init__(self, torch, arm, rows, device, layers=LAYERS):
        self.rows, self.layers = rows, layers
        self.weights = []
        for layer in range(layers):
            entry = {}
            for i, (name, (k, n)) in enumerate(SHAPES.items()):
                w = synth_weight(torch, n, k, SEED + 17 * layer + i, device)
                entry[name] = Quantized(torch, n, k, device)
                arm.quantize(w, entry[name])
            g = torch.Generator(device=device).manual_seed(SEED + 1000 + layer)
            for name in ("pre", "post"):
                entry[name] = (1.0 + 0.1 * torch.randn(1, HIDDEN, generator=g, device=device)).to(torch.bfloat16)
            self.weights.append(entry)
        torch.cuda.synchronize(device)
        self.x0 = synth_activations(torch, rows, HIDDEN, SEED - 1, device).to(torch.bfloat16)
        self.x = torch.empty_like(self.x0)                                            # residual stream
        self.u = torch.zeros(rows, HIDDEN, dtype=torch.bfloat16, device=device)      # branch output (O / down)
        self.qkv = torch.empty(rows, QKV, dtype=torch.bfloat16, device=device)
        self.gu = torch.empty(rows, 2 * FFN, dtype=torch.bfloat16, device=device)
        self.q_hidden = Quantized(torch, rows, HIDDEN, device)
        self.q_ffn = Quantized(torch, rows, FFN, device)


def decode_step(arm, stack, gemm_only=False):
    """The chain both arms run; `arm` supplies the kernels."""
    s = stack
    for index, layer in enumerate(s.weights):
        if not gemm_only:
            arm.norm(s.x, s.u if index else None, layer["pre"], s.q_hidden)
        arm.gemm("qkv", s.q_hidden, layer["qkv"], s.qkv)
        if not gemm_only:
            arm.quantize(s.qkv[:, :HIDDEN], s.q_hidden)
        arm.gemm("o", s.q_hidden, layer["o"], s.u)
        if not gemm_only:
            arm.norm(s.x, s.u, layer["post"], s.q_hidden)
        arm.gemm("gate_up", s.q_hidden, layer["gate_up"], s.gu)
        if not gemm_only:
            arm.gated(s.gu, s.q_ffn)
        arm.gemm("down", s.q_ffn, layer["down"], s.u)


LAUNCHES_PER_STEP = LAYERS * 8


# ------------------------------------------------------------------------------------------------ arms
class B200QArm:
    """This library through its C ABI (ctypes binding in breeze_tts_cpp_b200/ops.py)."""

    def __init__(self, torch, device, stream, rows):
        from breeze_tts_cpp_b200 import ops
        self.ops, self.torch = ops, torch
        self.ctx = ops.Context("int8", device=device.index, stream=stream, workspace_bytes=8 << 20)
        self.rows = rows

    def view(self, q):
        return self.ops.RowScaledView(q.values, q.scales, I8, q.group, q.group)

    def prepare(self, stack):
        for layer in stack.weights:
            for name, (k, n) in SHAPES.items():
                self.ctx.prepare_quantized(self.rows, n, k, weight=self.view(layer[name]))
        self.ctx.seal()

    def quantize(self, x, q):
        self.ctx.quantize_rows(x, self.view(q))

    def norm(self, x, update, weight, q):
        self.ctx.quantized_norm(x, update, weight, self.view(q), EPSILON)

    def gated(self, gu, q):
        self.ctx.quantized_gated(gu, self.view(q), 0)

    def gemm(self, name, q, w, out):
        self.ctx.matmul(self.view(q), self.view(w), out)

    def status(self):
        return self.ctx.status()


class ReferenceArm:
    """The reference's own CUDA kernels (built from its sources into oracle/_ref/libttsref.so) over plain torch
    tensors; nothing of this library is imported. The reference has no CPU implementation of this path; its stock
    code path on sm_100 is the CUTLASS SM80 GEMM / scalar GEMV chosen per shape, here by timing every candidate
    its planner enumerates."""

    def __init__(self, torch, device, stream, rows, lib):
        self.torch, self.lib, self.rows = torch, lib, rows
        self.sp = C.c_void_p(stream.cuda_stream)
        self.stream = stream
        self.workspace = torch.zeros(8 << 20, dtype=torch.uint8, device=device)
        self.sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.best = {}

    def check(self, rc):
        if rc != 0:
            raise RuntimeError(self.lib.ttsref_last_error().decode())

    def quantize(self, x, q):
        stride = x.stride(0) if x.stride(0) != x.shape[1] else 0
        self.check(self.lib.ttsref_row_quantize(x.data_ptr(), x.shape[0], x.shape[1], stride, BF16, q.values.data_ptr(),
                                                q.scales.data_ptr(), I8, 0, 0, self.sp))

    def norm(self, x, update, weight, q):
        self.check(self.lib.ttsref_quantized_norm(x.data_ptr(), update.data_ptr() if update is not None else None,
                                                  weight.data_ptr(), None, x.shape[0], x.shape[1], BF16, q.values.data_ptr(),
                                                  q.scales.data_ptr(), I8, 0, 0, EPSILON, 0, self.sp))

    def gated(self, gu, q):
        self.check(self.lib.ttsref_quantized_gated(gu.data_ptr(), gu.shape[0], gu.shape[1] // 2, BF16, q.values.data_ptr(),
                                                   q.scales.data_ptr(), I8, 0, 0, 0, self.sms, 1, self.sp))

    def gemm_path(self, path, q, w, out):
        self.check(self.lib.ttsref_quant_linear(path[0], path[1], path[2], path[3], q.rows, w.rows, w.cols, 0, 0,
                                                q.values.data_ptr(), q.scales.data_ptr(), w.values.data_ptr(),
                                                w.scales.data_ptr(), out.data_ptr(), self.workspace.data_ptr(),
                                                self.workspace.numel(), self.sp, I8, BF16))

    def gemm(self, name, q, w, out):
        self.gemm_path(self.best[name], q, w, out)

    def prepare(self, stack):
        """Best of the candidates the reference planner enumerates, per shape (a stronger baseline than its cost
        model's pick), timed over eight layers' distinct weights."""
        torch = self.torch
        buffers = {"qkv": stack.qkv, "o": stack.u, "gate_up": stack.gu, "down": stack.u}
        for name, (k, n) in SHAPES.items():
            cand = (C.c_int * (4 * 256))()
            count = self.lib.ttsref_candidates(self.rows, n, k, 0, 0, I8, 48 << 10, 8 << 20, cand, 256)
            q = stack.q_hidden if k == HIDDEN else stack.q_ffn
            q.values.random_(0, 255)
            q.scales.fill_(0.01)
            timings = []
            for c in range(min(count, 256)):
                path = tuple(cand[4 * c:4 * c + 4])
                try:
                    ws = [stack.weights[i][name] for i in range(min(LAYERS, 8))]
                    for w in ws:
                        self.gemm_path(path, q, w, buffers[name])
                    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record(self.stream)
                    for _ in range(2):
                        for w in ws:
                            self.gemm_path(path, q, w, buffers[name])
                    stop.record(self.stream)
                    stop.synchronize()
                    timings.append((start.elapsed_time(stop), path))
                except RuntimeError:
                    continue
            self.best[name] = min(timings)[1]

    def status(self):
        return 0


# ------------------------------------------------------------------------------------------------
def run_chain(args, torch, dist, rank, world, device, arm_factory):
    rows = STREAMS // world
    stream = torch.cuda.Stream(device=device)
    with torch.cuda.stream(stream):
        arm = arm_factory(stream, rows)
        stack = Stack(torch, arm, rows, device)
        arm.prepare(stack)
        stack.x.copy_(stack.x0)
        decode_step(arm, stack)  # eager once: lazy module loading, plans
        stream.synchronize()
        assert arm.status() == 0, "device status word set"
        # Three graphs: the step with its input reset on the device (value), the same step fed from and
        # read back to pinned host memory (e2e), and the GEMM launches alone (roofline).
        host_x = stack.x0.cpu().pin_memory()
        host_out = torch.empty(stack.rows, HIDDEN, dtype=torch.bfloat16).pin_memory()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            stack.x.copy_(stack.x0, non_blocking=True)
            decode_step(arm, stack)
        e2e_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(e2e_graph, stream=stream):
            stack.x.copy_(host_x, non_blocking=True)
            decode_step(arm, stack)
            host_out.copy_(stack.u, non_blocking=True)
        gemm_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gemm_graph, stream=stream):
            decode_step(arm, stack, gemm_only=True)
    result = time_steps(args, torch, dist, world, device, stream, stack, graph, e2e_graph, gemm_graph, host_x, host_out)
    assert arm.status() == 0, "device status word set during the timed region"
    return arm, stream, result


def time_steps(args, torch, dist, world, device, stream, stack, graph, e2e_graph, gemm_graph, host_x, host_out):
    """value: K graph replays with inputs resident (the graph resets the residual stream from a device copy);
    e2e: per step one graph that copies the step input from pinned host memory, runs the chain and copies the
    step result back to pinned host memory, then a stream sync; roofline: K replays of the GEMM launches alone."""

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(fn, steps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with torch.cuda.stream(stream):
            start.record(stream)
            for _ in range(steps):
                fn()
            stop.record(stream)
        stop.synchronize()
        barrier()
        return start.elapsed_time(stop)

    def resident_step():
        graph.replay()

    def e2e_step():
        e2e_graph.replay()
        stream.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            resident_step()
        stream.synchronize()
    with ClockSampler(device.index) as clocks:
        ms_value = timed(resident_step, args.steps)
    with torch.cuda.stream(stream):
        for _ in range(max(1, args.warmup // 2)):
            e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    if not bool(torch.isfinite(host_out.float()).all()) or float(host_out.float().abs().max()) == 0.0:
        raise SystemExit("bench: the step output read back to the host is not a finite, nonzero tensor")
    with torch.cuda.stream(stream):
        for _ in range(max(1, args.warmup // 2)):
            gemm_graph.replay()
    ms_gemm = timed(gemm_graph.replay, args.steps)
    return {"ms_value": ms_value, "ms_e2e": ms_e2e, "ms_gemm": ms_gemm, "clocks": clocks.summary(),
            "h2d": host_x.numel() * 2, "d2h": host_out.numel() * 2}


# ------------------------------------------------------------------------------------------------ per-configuration rows
def library_tensor_peaks(torch, device):
    """Dense 8-bit GEMM rate of the vendor library at 8192^3 on this GPU (best of 10): the measured denominator of
    the prefill rows. A library peak, not a reference path."""
    out = {}
    n = 8192
    ops = 2.0 * n ** 3

    def best(fn):
        fn()
        torch.cuda.synchronize(device)
        times = []
        for _ in range(10):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            stop.record()
            stop.synchronize()
            times.append(start.elapsed_time(stop))
        return ops / (min(times) * 1e-3) / 1e12

    try:
        a = torch.randint(-100, 100, (n, n), dtype=torch.int8, device=device)
        b = torch.randint(-100, 100, (n, n), dtype=torch.int8, device=device).t()
        out["int8_tops"] = round(best(lambda: torch._int_mm(a, b)), 1)
    except Exception as error:  # noqa: BLE001
        out["int8_tops"], out["int8_error"] = None, str(error)[:80]
    try:
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=device)
        out["fp8_tflops"] = round(best(lambda: torch._scaled_mm(a, b, one, one, out_dtype=torch.bfloat16)), 1)
    except Exception as error:  # noqa: BLE001
        out["fp8_tflops"], out["fp8_error"] = None, str(error)[:80]
    out["how"] = "torch._int_mm / torch._scaled_mm (cuBLASLt) 8192^3, best of 10, CUDA events: library peak, not a reference path"
    return out


def sustained_tensor_rates(torch, device, stream, seconds=1.5):
    """The same dense 8-bit GEMM rates held for `seconds` each instead of a burst, with the clocks seen meanwhile: at
    these rates a B200 runs into its 1000 W power cap and lowers the SM clock, for this library's prefill kernel and
    for the vendor library alike, so the burst figures of the `configs` rows and of `tensor_peaks` are upper ends."""
    from breeze_tts_cpp_b200 import ops
    k, n, m = SHAPES["gate_up"][0], SHAPES["gate_up"][1], 8192
    out = {"seconds": seconds, "shape": f"gate_up {k}->{n} at M={m} (this library); 8192^3 (vendor library)"}

    def hold(fn, sync, work):
        fn()
        sync()
        with ClockSampler(device.index) as clocks:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            calls, began = 0, time.time()
            while time.time() - began < seconds:
                for _ in range(10):
                    fn()
                calls += 10
                sync()
            stop.record(stream)
            stop.synchronize()
        seen = clocks.summary()
        return round(work * calls / (start.elapsed_time(stop) * 1e-3) / 1e12, 1), seen

    with torch.cuda.stream(stream):
        for mode, fmt, key in (("int8", I8, "int8_tops"), ("fp8", FP8, "fp8_tflops")):
            ctx = ops.Context(mode, device=device.index, stream=stream, workspace_bytes=8 << 20)
            ws = [ctx.quantize_rows(synth_weight(torch, n, k, SEED + c, device), ops.RowScaledView.empty(n, k, fmt, device=device))
                  for c in range(4)]
            xq = ctx.quantize_rows(synth_activations(torch, m, k, SEED, device).to(torch.bfloat16),
                                   ops.RowScaledView.empty(m, k, fmt, device=device))
            y = torch.empty(m, n, dtype=torch.bfloat16, device=device)
            ctx.prepare_quantized(m, n, k)
            for w in ws:
                ctx.matmul(xq, w, y)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for w in ws:
                    ctx.matmul(xq, w, y)
            rate, seen = hold(graph.replay, stream.synchronize, 2.0 * m * n * k * len(ws))
            out[key] = rate
            out[key.split("_")[0] + "_clocks"] = seen
            ok = ctx.status() == 0
            ctx.close()
            if not ok:
                out[key] = None
        side = 8192
        try:
            a = torch.randint(-100, 100, (side, side), dtype=torch.int8, device=device)
            b = torch.randint(-100, 100, (side, side), dtype=torch.int8, device=device).t()
            out["library_int8_tops"], out["library_int8_clocks"] = hold(lambda: torch._int_mm(a, b), stream.synchronize, 2.0 * side ** 3)
        except Exception as error:  # noqa: BLE001
            out["library_int8_tops"], out["library_int8_error"] = None, str(error)[:80]
        try:
            a = torch.randn(side, side, device=device).to(torch.float8_e4m3fn)
            b = torch.randn(side, side, device=device).to(torch.float8_e4m3fn).t()
            one = torch.ones((), device=device)
            out["library_fp8_tflops"], out["library_fp8_clocks"] = hold(
                lambda: torch._scaled_mm(a, b, one, one, out_dtype=torch.bfloat16), stream.synchronize, 2.0 * side ** 3)
        except Exception as error:  # noqa: BLE001
            out["library_fp8_tflops"], out["library_fp8_error"] = None, str(error)[:80]
    return out


def check_output(torch, fmt, group, xq, wq, out, residual):
    """Plain PyTorch restatement of the arithmetic on a slice of the output (a checker, never the product): INT8
    per-row must match bit for bit (exact INT32 sums, the same fp32 rounding chain), the other modes within
    2e-2 (FP8) / 1e-2 (INT8 K-group) relative with floor 1e-2 * rms."""
    m, n = out.shape
    g = torch.Generator(device="cpu").manual_seed(1)
    channels = torch.unique(torch.cat([torch.arange(0, n, 128), torch.arange(127, n, 128), torch.randint(0, n, (64,), generator=g)])).to(out.device)
    rows = torch.unique(torch.cat([torch.arange(0, m, 128), torch.arange(min(m, 127), m, 128), torch.randint(0, m, (64,), generator=g)])).to(out.device)
    got = out[rows][:, channels]
    skip = residual[rows][:, channels] if residual is not None else None
    xs, ws = xq.values[rows], wq.values[channels]
    if fmt == I8 and not group:
        pad = max(32, -(-rows.numel() // 8) * 8)
        a = torch.zeros(pad, xs.shape[1], dtype=torch.int8, device=out.device)
        a[:rows.numel()] = xs.view(torch.int8)
        pad_n = -(-channels.numel() // 8) * 8
        b = torch.zeros(pad_n, ws.shape[1], dtype=torch.int8, device=out.device)
        b[:channels.numel()] = ws.view(torch.int8)
        acc = torch._int_mm(a, b.t())[:rows.numel(), :channels.numel()]
        want = (acc.float() * xq.scales.reshape(-1, 1)[rows]) * wq.scales.reshape(1, -1)[:, channels]
        if skip is not None:
            want = want + skip
        return bool(torch.equal(want.to(torch.bfloat16).view(torch.int16), got.contiguous().view(torch.int16)))
    decode = (lambda t: t.view(torch.int8).double()) if fmt == I8 else (lambda t: t.view(torch.float8_e4m3fn).double())
    x, w = decode(xs), decode(ws)
    if group:
        want = torch.zeros(rows.numel(), channels.numel(), dtype=torch.float64, device=out.device)
        for block in range(x.shape[1] // group):
            part = x[:, block * group:(block + 1) * group] @ w[:, block * group:(block + 1) * group].T
            want += part * xq.scales[block][rows].double().reshape(-1, 1) * wq.scales[block][channels].double().reshape(1, -1)
    else:
        want = (x @ w.T) * xq.scales.reshape(-1, 1)[rows].double() * wq.scales.reshape(1, -1)[:, channels].double()
    if skip is not None:
        want = want + skip.double()
    floor = 1e-2 * want.pow(2).mean().sqrt() + 1e-30
    error = float(((got.double() - want).abs() / torch.maximum(want.abs(), floor)).max())
    return error < (2e-2 if fmt == FP8 else 1e-2)


def config_rows(torch, device, stream, peaks, tensor_peaks):
    """One row per shape of BASELINE configurations 1-4, each rotated over enough distinct weight copies to exceed
    L2. `us` times quantize + GEMM, `gemm_us` the GEMM launch alone (CUDA-graph replays); decode rows are held
    against the HBM roofline, prefill rows against the dense 8-bit tensor rate."""
    from breeze_tts_cpp_b200 import ops
    rows_out = []

    def measure(config, shape, mode, fmt, m, k, n, group, residual, bound, iters=20, student_t=False):
        ctx = ops.Context(mode, device=device.index, stream=stream, workspace_bytes=8 << 20)
        copies = max(2, min(24, (300 << 20) // (n * k)))
        with torch.cuda.stream(stream):
            ws = []
            for c in range(copies):
                w = synth_weight(torch, n, k, SEED + c, device)
                ws.append(ctx.quantize_rows(w, ops.RowScaledView.empty(n, k, fmt, group, group, device=device)))
            x = synth_activations(torch, m, k, SEED, device, student_t=student_t).to(torch.bfloat16)
            xq = ops.RowScaledView.empty(m, k, fmt, group, group, device=device)
            out = torch.empty(m, n, dtype=torch.bfloat16, device=device)
            res = torch.randn(m, n, device=device) if residual else None
            path = ctx.prepare_quantized(m, n, k)
            kw = {"residual_f32": res} if residual else {}
            ctx.quantize_rows(x, xq)
            ctx.matmul(xq, ws[-1], out, **kw)
            stream.synchronize()
            checked = check_output(torch, fmt, group, xq, ws[-1], out, res)

            def body(gemm_only):
                for w in ws:
                    if not gemm_only:
                        ctx.quantize_rows(x, xq)
                    ctx.matmul(xq, w, out, **kw)

            def timed(gemm_only):
                body(gemm_only)
                stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    body(gemm_only)
                g.replay()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = max(1, iters // copies)
                start.record(stream)
                for _ in range(reps):
                    g.replay()
                stop.record(stream)
                stop.synchronize()
                return start.elapsed_time(stop) * 1e3 / (reps * copies)

            us = timed(False)
            gemm_us = timed(True)
        status = ctx.status()
        ctx.close()
        nbytes = linear_bytes(m, k, n, residual, group)
        gemm_bytes = linear_bytes(m, k, n, residual, group, quantize=False)
        ops_count = 2.0 * m * n * k
        row = {"config": config, "shape": shape, "mode": mode, "m": m, "k": k, "n": n, "bound": bound,
               "algorithmic_bytes": nbytes, "ops": ops_count, "us": round(us, 2), "gemm_us": round(gemm_us, 2),
               "path": list(path), "checked": bool(checked and status == 0)}
        if bound == "hbm":
            row.update(gbs=round(nbytes / us / 1e3, 1), gemm_gbs=round(gemm_bytes / gemm_us / 1e3, 1),
                       frac_of_measured=round(nbytes / us / 1e3 / peaks["hbm_gbs"], 3),
                       gemm_frac_of_measured=round(gemm_bytes / gemm_us / 1e3 / peaks["hbm_gbs"], 3),
                       gemm_frac_of_nominal=round(gemm_bytes / gemm_us / 1e3 / NOMINAL_HBM_GBS, 3))
        else:
            library = tensor_peaks.get("fp8_tflops" if fmt == FP8 else "int8_tops")
            tops, gemm_tops = ops_count / us / 1e6, ops_count / gemm_us / 1e6
            row.update(tops=round(tops, 1), gemm_tops=round(gemm_tops, 1),
                       frac_of_measured=round(tops / library, 3) if library else None,
                       gemm_frac_of_measured=round(gemm_tops / library, 3) if library else None,
                       gemm_frac_of_nominal=round(gemm_tops / NOMINAL_TENSOR_TOPS, 3))
        return row

    rows_out.append(measure("c1", "o", "int8", I8, 16, HIDDEN, HIDDEN, 0, False, "hbm"))
    for m in (1, 4, 16, 64):
        for name, (k, n) in SHAPES.items():
            rows_out.append(measure("c2", name, "int8", I8, m, k, n, 0, True, "hbm"))
    for m in (2048, 8192):
        for name, (k, n) in SHAPES.items():
            rows_out.append(measure("c3", name, "fp8", FP8, m, k, n, 0, False, "tensor", iters=6))
    for name, (k, n) in SHAPES.items():  # the same prefill shapes in INT8 (the stack's own format)
        rows_out.append(measure("c3_int8", name, "int8", I8, 8192, k, n, 0, False, "tensor", iters=6))
    for mode, fmt in (("group_int8", I8), ("group_fp8", FP8)):
        rows_out.append(measure("c4", "down", mode, fmt, 16, FFN, HIDDEN, 128, False, "hbm", iters=8, student_t=True))
        rows_out.append(measure("c4", "down", mode, fmt, 4096, FFN, HIDDEN, 128, False, "tensor", iters=8, student_t=True))
    return rows_out


# ------------------------------------------------------------------------------------------------
def cpu_baseline(rows, max_seconds=20.0):
    """Scalar host-core port (the CPU oracle) on a bounded sample: one decoder layer's four linears."""
    import numpy as np
    from tests import oracle_binding
    oracle = oracle_binding.load()
    threads = oracle.lib.oracle_hardware_threads()
    rng = np.random.default_rng(SEED)
    total_bytes, total_s = 0, 0.0
    done = []
    for name, (k, n) in SHAPES.items():
        x16 = oracle.to_bf16(rng.standard_normal((rows, k)).astype(np.float32))
        wq = rng.integers(-127, 128, (n, k), dtype=np.int8).view(np.uint8)
        sw = np.full(n, 1e-3, dtype=np.float32)
        out = np.zeros((rows, n), dtype=np.uint16)
        seconds = oracle.lib.oracle_time_linear(x16.ctypes.data, wq.ctypes.data, sw.ctypes.data, rows, n, k, n, 4, 0, 0,
                                                out.ctypes.data, None, threads)
        total_s += seconds
        total_bytes += linear_bytes(rows, k, n)
        done.append(name)
        if total_s > max_seconds:
            break
    return {"value": round(total_bytes / total_s / 1e9, 4), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"one decoder layer ({'+'.join(done)}) at M={rows}: quantize+GEMM+dequant in {total_s:.2f} s"}


def run_reference_cpu(args):
    base = cpu_baseline(STREAMS)
    line = {"impl": "reference", "metric": "quantized_linear_algorithmic_GBps", "value": base["value"], "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": workload_config(STREAMS, 1),
            "cpu_baseline": base, "e2e": {"value": base["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def run_case(spec):
    """One small, self-ending case of a single quantized linear, meant to be run under a profiler:
    `--case <qkv|o|gate_up|down> <rows> [mode] [launches]` runs quantize + GEMM `launches` times (default 6) over
    enough distinct weight copies to exceed L2 (about 300 MB on the device in total), eagerly on one stream."""
    import torch
    from breeze_tts_cpp_b200 import ops
    name, rows = spec[0], int(spec[1])
    mode = spec[2] if len(spec) > 2 else "int8"
    launches = int(spec[3]) if len(spec) > 3 else 6
    k, n = SHAPES[name]
    fmt = ops.format_of(mode)
    group, _, rotation = ops.groups_of(mode)
    device = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=device)
    with torch.cuda.stream(stream):
        ctx = ops.Context(mode, device=0, stream=stream)
        copies = max(2, min(launches, (300 << 20) // (n * k)))
        weights = [ctx.quantize_rows(synth_weight(torch, n, k, SEED + c, device),
                                     ops.RowScaledView.empty(n, k, fmt, group, rotation, device=device)) for c in range(copies)]
        x = synth_activations(torch, rows, k, SEED, device, student_t=bool(group)).to(torch.bfloat16)
        xq = ops.RowScaledView.empty(rows, k, fmt, group, rotation, device=device)
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=device)
        path = ctx.prepare_quantized(rows, n, k)
        ctx.quantize_rows(x, xq)
        ctx.matmul(xq, weights[0], out)
        stream.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for i in range(launches):
            ctx.quantize_rows(x, xq)
            ctx.matmul(xq, weights[i % copies], out)
        stop.record(stream)
        stop.synchronize()
        status = ctx.status()
        ctx.close()
    print(f"{mode} {name} M={rows} K={k} N={n} path={path} avg {start.elapsed_time(stop) * 1e3 / launches:.2f} us per quantize+GEMM "
          f"(eager launches), status {status}")
    if status:
        raise SystemExit(1)


def workload_config(rows, world):
    return {"workload": "c5_decoder_stack28_int8_decode (per layer: residual+RMSNorm+quantize, QKV 2048->4096, row quantize, "
                        "O 2048->2048, residual+RMSNorm+quantize, gate+up 2048->12288, SiLU-gate+quantize, down 6144->2048)",
            "layers": LAYERS, "streams_total": STREAMS, "rows_per_gpu": rows, "parallelism": f"dp{world} (replicated weights, no collective)",
            "launches_per_step": LAUNCHES_PER_STEP,
            "l2": "inputs larger than L2: 1.41 GB of distinct weights per step vs 126 MB L2",
            "timing": "CUDA events on the launch stream, CUDA-graph replay; steps last about a millisecond, so the GPU stays at burst clocks"}


def dram_traffic_per_launch(rows):
    """Average DRAM bytes per GEMM launch of a step, from the per-shape ncu captures at M=64 scaled by the
    algorithmic bytes of the row count in use; None until every shape has a capture."""
    if any(v is None for v in NCU_DRAM_BYTES_M64.values()):
        return None
    total = 0.0
    for name, (k, n) in SHAPES.items():
        total += NCU_DRAM_BYTES_M64[name] * linear_bytes(rows, k, n, quantize=False) / linear_bytes(64, k, n, quantize=False)
    return int(total / len(SHAPES))


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="b200q", choices=["b200q", "reference", "reference-cpu"])
    parser.add_argument("--no-configs", action="store_true", help="skip the per-configuration rows (c1-c4)")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--case", nargs="+", metavar="ARG", help="profiling case: <qkv|o|gate_up|down> <rows> [mode] [launches]")
    args = parser.parse_args()
    args.warmup = max(3, args.warmup)
    if args.case:
        run_case(args.case)
        return

    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference-cpu":
        if rank == 0:
            run_reference_cpu(args)
        return
    import torch
    dist = None
    if not torch.cuda.is_available():
        if args.impl == "reference" and rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "no CUDA device: the reference's only implementation of this path is CUDA"}))
            return
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    if STREAMS % world:
        raise SystemExit("the 64 streams must divide over the GPUs")
    rows = STREAMS // world
    peaks = measured_peaks()

    if args.impl == "reference":
        from tests import oracle_binding
        lib = oracle_binding.load_reference()
        if lib is None:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libttsref.so (the reference's CUDA kernels) is not built"}))
            return
        arm, stream, result = run_chain(args, torch, dist, rank, world, device,
                                        lambda stream, r: ReferenceArm(torch, device, stream, r, lib))
    else:
        arm, stream, result = run_chain(args, torch, dist, rank, world, device,
                                        lambda stream, r: B200QArm(torch, device, stream, r))

    # whole-job numbers: work summed over ranks, time = the slowest rank
    from breeze_tts_cpp_b200.sharding import whole_job_rate  # pure Python; loads no native code
    seconds = {key: whole_job_rate(1.0, result[key] * 1e-3, dist, device)[2] for key in ("ms_value", "ms_e2e", "ms_gemm")}

    if rank == 0:
        total_bytes = step_bytes(rows) * world  # every GPU streams its own replica
        ms_step = seconds["ms_value"] * 1e3 / args.steps
        ms_e2e = seconds["ms_e2e"] * 1e3 / args.steps
        ms_gemm = seconds["ms_gemm"] * 1e3 / args.steps
        gemm_bytes = step_bytes(rows, gemm_only=True)
        achieved = gemm_bytes / (ms_gemm * 1e-3) / 1e9
        line = {
            "metric": "quantized_linear_algorithmic_GBps", "value": round(total_bytes / (ms_step * 1e-3) / 1e9, 2), "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": workload_config(rows, world),
            "tops": round(step_ops(rows) * world / (ms_step * 1e-3) / 1e12, 2),
            "tokens_per_s": round(STREAMS / (ms_step * 1e-3), 1),
            "e2e": {"value": round(total_bytes / (ms_e2e * 1e-3) / 1e9, 2), "unit": "GB/s", "ms_per_step": round(ms_e2e, 4),
                    "h2d_bytes_per_step": result["h2d"], "d2h_bytes_per_step": result["d2h"]},
            "roofline": {"bound": "hbm", "kernel": "w8a8 GEMM launches of one step (112 launches, 4 shapes)",
                         "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / peaks["hbm_gbs"], 4), "frac_of_nominal_8TBps": round(achieved / NOMINAL_HBM_GBS, 4),
                         "peak_source": peaks["source"], "avg_launch_us": round(ms_gemm * 1e3 / (LAYERS * 4), 3),
                         "algorithmic_bytes_per_launch": gemm_bytes // (LAYERS * 4),
                         "traffic": dram_traffic_per_launch(rows),
                         "traffic_source": "one-launch ncu captures of the four shapes at M=64, scaled by algorithmic bytes"},
            "clocks": result["clocks"],
        }
        if args.impl == "reference":
            line["impl"] = "reference"
            line["reference_paths"] = {k: list(v) for k, v in arm.best.items()}
            line["cpu_baseline"] = {"value": line["value"], "unit": "GB/s", "cores": 0, "kind": "reference",
                                    "sample": "the reference's own CUDA kernels on this GPU (it has no CPU implementation of the path)"}
            line["roofline"]["kernel"] = "reference GEMM launches of one step"
            line["roofline"]["traffic"] = None
        else:
            line["impl"] = "b200q"
            line["gpu_launches"] = LAUNCHES_PER_STEP * args.steps
            if world == 1 and not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_baseline(rows)
            if world == 1 and not args.no_configs:
                tensor_peaks = library_tensor_peaks(torch, device)
                line["tensor_peaks"] = tensor_peaks
                line["configs"] = config_rows(torch, device, stream, peaks, tensor_peaks)
                line["tensor_sustained"] = sustained_tensor_rates(torch, device, stream)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
