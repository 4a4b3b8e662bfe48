"""One small, self-ending case of a single quantized linear, meant to be run under a profiler.

    python -m breeze_tts_cpp_b200.profile_case <qkv|o|gate_up|down> <rows> [mode] [launches]

Runs quantize + GEMM `launches` times (default 6) over enough distinct weight copies to exceed L2
(about 300 MB on the device in total), eagerly on one stream, then prints the average time per pair.
"""
from __future__ import annotations

import sys

import torch

from . import ops

SHAPES = {"qkv": (2048, 4096), "o": (2048, 2048), "gate_up": (2048, 12288), "down": (6144, 2048)}  # name: (K, N)


def main(argv: list[str]) -> None:
    name, rows = argv[0], int(argv[1])
    mode = argv[2] if len(argv) > 2 else "int8"
    launches = int(argv[3]) if len(argv) > 3 else 6
    k, n = SHAPES[name]
    fmt = ops.format_of(mode)
    group, _, rotation = ops.groups_of(mode)
    device = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=device)
    with torch.cuda.stream(stream):
        ctx = ops.Context(mode, device=0, stream=stream)
        copies = max(2, min(launches, (300 << 20) // (n * k)))
        generator = torch.Generator(device=device).manual_seed(0x5EED)
        weights = []
        for _ in range(copies):
            w = (torch.randn(n, k, generator=generator, device=device) * 0.02).to(torch.bfloat16)
            weights.append(ctx.quantize_rows(w, ops.RowScaledView.empty(n, k, fmt, group, rotation, device=device)))
        x = torch.randn(rows, k, generator=generator, device=device).to(torch.bfloat16)
        xq = ops.RowScaledView.empty(rows, k, fmt, group, rotation, device=device)
        out = torch.empty(rows, n, dtype=torch.bfloat16, device=device)
        residual = torch.randn(rows, n, generator=generator, device=device) if name in ("o", "down") else None
        path = ctx.prepare_quantized(rows, n, k)
        kw = {"residual_f32": residual} if residual is not None else {}
        ctx.quantize_rows(x, xq)
        ctx.matmul(xq, weights[0], out, **kw)
        stream.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for i in range(launches):
            ctx.quantize_rows(x, xq)
            ctx.matmul(xq, weights[i % copies], out, **kw)
        stop.record(stream)
        stop.synchronize()
        status = ctx.status()
        ctx.close()
    print(f"{mode} {name} M={rows} K={k} N={n} path={path} avg {start.elapsed_time(stop) * 1e3 / launches:.2f} us per quantize+GEMM "
          f"(eager launches), status {status}")


if __name__ == "__main__":
    main(sys.argv[1:])
