"""Shape sweep of the conv and depthwise kernels: ``python -m flashim_b200.sweep [conv|dw|quant|heads|input|all]``.

Prints, as Markdown tables, the device time of each kernel over the shapes of BASELINE configs 3 and 4 (N = 4; conv
100x100x512, 200x200x256, 400x400x128, 800x800x64 with k = 3 and k = 1, plain and with the fused bias + GELU + MXFP8
requantisation epilogue; depthwise with each epilogue) with TFLOP/s, GB/s and the fraction of the measured peaks in
``MEASURED_PEAKS.json`` (fallback: 6650 GB/s, 1590 bf16 TFLOP/s; the fp8 / int8 tensor peak is taken as twice the bf16
figure). Each op is captured 20 times into a CUDA graph and the replay is timed with CUDA events, so the host's launch
cost is not in the numbers. Inputs are seeded synthetic tensors; nothing is checked here (the tests do that).
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

E4M3 = torch.float8_e4m3fn
BF16 = torch.bfloat16


def _peaks() -> tuple[float, float]:
    path = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if path.is_file():
        measured = json.loads(path.read_text())
        return float(measured["hbm_gbs"]), 2.0 * float(measured["bf16_tflops"])
    return 6650.0, 2.0 * 1590.0


def graph_time_ms(fn, count: int = 20, repeats: int = 3) -> float:
    """Device time of one call of ``fn`` (ms): ``count`` calls replayed from a CUDA graph, best of ``repeats``."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(count):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(repeats):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        best = min(best, start.elapsed_time(end) / count)
    return best


def conv_sweep() -> None:
    from flashim_b200 import check_status, ops
    from flashim_b200.quant import swizzle_scales

    hbm, tensor = _peaks()
    print("| shape (N=4) | k | epilogue | us | TFLOP/s | % tensor peak | GB/s | % HBM peak |")
    print("|---|---|---|---:|---:|---:|---:|---:|")
    n = 4
    for size, c in ((100, 512), (200, 256), (400, 128), (800, 64)):
        for k in (3, 1):
            x = torch.randn(n, size, size, c, device="cuda").to(E4M3)
            x_exponent = torch.zeros(c // 32, dtype=torch.int8, device="cuda")
            weight = (torch.randn(c, k * k * c, device="cuda") * 0.05).to(E4M3)
            weight_exponent = torch.zeros(c, k * k * c // 32, dtype=torch.int8, device="cuda")
            weight_scales = swizzle_scales(weight_exponent)
            bias = (torch.randn(c, device="cuda") * 0.02).to(BF16)
            out_exponent = torch.zeros(c // 32, dtype=torch.int8, device="cuda")
            plain = ops.mxfp8_conv2d.get("sm100")
            fused = ops.mxfp8_conv2d_fused.get("sm100")
            cases = (
                ("none -> bf16", 2, lambda: plain(x, x_exponent, weight, weight_exponent, None, k, k, 1, 1, k // 2, k // 2, 1, 1)),
                ("bias + GELU + MXFP8 requant", 1,
                 lambda: fused(x, x_exponent, weight, weight_scales, bias, k, k, 1, 1, k // 2, k // 2, 1, 1, act="gelu",
                               out_exponent=out_exponent)),
            )
            for name, out_bytes, fn in cases:
                ms = graph_time_ms(fn)
                flops = 2 * n * size * size * c * c * k * k
                moved = n * size * size * c * (1 + out_bytes) + c * k * k * c
                tf, gbs = flops / ms / 1e9, moved / ms / 1e6
                print(f"| {size}x{size}x{c} | {k} | {name} | {ms * 1e3:.1f} | {tf:.0f} | {100 * tf / tensor:.1f} | {gbs:.0f} | "
                      f"{100 * gbs / hbm:.1f} |", flush=True)
    check_status()


def depthwise_sweep() -> None:
    from flashim_b200 import check_status, ops

    hbm, _ = _peaks()
    print("| depthwise shape | epilogue | us | GB/s | % HBM peak |")
    print("|---|---|---:|---:|---:|")
    for n, size, c in ((4, 200, 256), (4, 400, 128), (4, 100, 512)):
        x = torch.randn(n, c, size, size, device="cuda", dtype=BF16).contiguous(memory_format=torch.channels_last)
        weight = (torch.randn(25, c, device="cuda") * 0.05).to(BF16)
        bias = torch.randn(c, device="cuda")
        scale = torch.tensor(0.03, device="cuda")
        dense, mx = ops.depthwise5x5_act.get("sm100"), ops.depthwise5x5_act_mxfp8.get("sm100")
        cases = (
            ("ReLU -> bf16", 2, lambda: dense(x, weight, bias, "relu")),
            ("GELU -> bf16", 2, lambda: dense(x, weight, bias, "gelu")),
            ("ReLU -> MXFP8 (reference op)", 1 + 1 / 32, lambda: ops.depthwise5x5_relu_mxfp8.get("sm100")(x, weight, bias)),
            ("GELU -> MXFP8", 1 + 1 / 32, lambda: mx(x, weight, bias, "gelu")),
            ("ReLU -> INT8 (reference op)", 1, lambda: ops.depthwise5x5_relu_int8.get("sm100")(x, weight, bias, scale)),
        )
        for name, out_bytes, fn in cases:
            ms = graph_time_ms(fn)
            moved = n * size * size * c * (2 + out_bytes)
            gbs = moved / ms / 1e6
            print(f"| {n}x{size}x{size}x{c} | {name} | {ms * 1e3:.1f} | {gbs:.0f} | {100 * gbs / hbm:.1f} |", flush=True)
    check_status()


def quantiser_sweep() -> None:
    """The standalone quantisers and the max-pool quantiser: one pass over HBM each."""
    from flashim_b200 import check_status, ops
    from flashim_b200.backends.sm100 import kernels

    hbm, _ = _peaks()
    print("| quantiser | input | us | GB/s | % HBM peak |")
    print("|---|---|---:|---:|---:|")
    for n, c, size in ((4, 256, 200), (4, 128, 400), (4, 512, 100)):
        nchw = torch.randn(n, c, size, size, device="cuda", dtype=BF16)
        nhwc = nchw.permute(0, 2, 3, 1).contiguous()
        exponent = torch.zeros(c // 32, dtype=torch.int8, device="cuda")
        scale = torch.tensor(0.03, device="cuda")
        view = nchw.permute(0, 2, 3, 1)
        elements = n * c * size * size
        cases = (
            ("static MXFP8, row-major", 3 * elements, lambda: ops.quantize_mxfp8.get("sm100")(nhwc, exponent)),
            ("static MXFP8, channels-first view", 3 * elements, lambda: ops.quantize_mxfp8.get("sm100")(view, exponent)),
            ("dynamic MXFP8, row-major", (3 + 1 / 32) * elements, lambda: ops.quantize_mxfp8_dynamic.get("sm100")(nhwc)),
            ("static INT8, row-major", 3 * elements, lambda: ops.quantize_int8.get("sm100")(nhwc, scale)),
            ("static INT8, channels-first view", 3 * elements, lambda: ops.quantize_int8.get("sm100")(view, scale)),
            ("MaxPool2d(2) -> INT8", 2.25 * elements, lambda: kernels.maxpool2_quantize_int8(nhwc, scale.reshape(1))),
        )
        for name, moved, fn in cases:
            ms = graph_time_ms(fn)
            gbs = moved / ms / 1e6
            print(f"| {name} | bf16 {n}x{size}x{size}x{c} | {ms * 1e3:.1f} | {gbs:.0f} | {100 * gbs / hbm:.1f} |", flush=True)
    check_status()


def heads_sweep() -> None:
    """RoMaV2 refiner heads on the three levels of the refiner pyramid (8 images)."""
    from flashim_b200 import check_status, ops

    hbm, _ = _peaks()
    print("| refiner heads input | us | GB/s | % HBM peak |")
    print("|---|---:|---:|---:|")
    for n, c, size in ((8, 512, 100), (8, 256, 200), (8, 128, 400)):
        z = torch.randn(n, c, size, size, device="cuda", dtype=BF16).contiguous(memory_format=torch.channels_last)
        weight, bias = torch.randn(6, c, device="cuda") * 0.1, torch.randn(6, device="cuda")
        prev_warp = torch.rand(n, size, size, 2, device="cuda")
        prev_conf = torch.randn(n, size, size, 4, device="cuda")
        ms = graph_time_ms(lambda: ops.romav2_refiner_heads.get("sm100")(z, weight, bias, prev_warp, prev_conf, 4.0))
        moved = n * size * size * (2 * c + 2 * (8 + 16))
        gbs = moved / ms / 1e6
        print(f"| bf16 {n}x{size}x{size}x{c} | {ms * 1e3:.1f} | {gbs:.0f} | {100 * gbs / hbm:.1f} |", flush=True)
    check_status()


def input_sweep() -> None:
    """RoMaV2 refiner input on the three refiner configurations (flashim/models/romav2/refiner.py:38-42), 8 images of a
    560 x 560 pair at strides 4 / 2 / 1; warps = identity + noise of about one pixel."""
    from flashim_b200 import check_status, ops

    print("| refiner input | us | algorithmic GB/s |")
    print("|---|---:|---:|")
    for n, size, p, e, radius in ((8, 140, 192, 79, 3), (8, 280, 48, 23, 1), (8, 560, 12, 8, -1)):
        f_a, f_b = torch.randn(n, size, size, p, device="cuda"), torch.randn(n, size, size, p, device="cuda")
        line = torch.linspace(-1, 1, size, device="cuda")
        gy, gx = torch.meshgrid(line, line, indexing="ij")
        warp = (torch.stack((gx, gy), -1)[None] + torch.randn(n, size, size, 2, device="cuda") * (2.0 / size)).contiguous()
        emb_w, emb_b = torch.randn(e, 2, device="cuda"), torch.randn(e, device="cuda")
        scale = torch.tensor([3.0, 2.0])
        ms = graph_time_ms(lambda: ops.romav2_refiner_input.get("sm100")(f_a, f_b, warp, emb_w, emb_b, scale, radius, 0))
        k = (2 * radius + 1) ** 2 if radius >= 0 else 0
        moved = n * size * size * (2 * p * 4 + 8 + (2 * p + e + k) * 2)
        print(f"| {n}x{size}x{size}, P={p}, E={e}, r={radius} | {ms * 1e3:.1f} | {moved / ms / 1e6:.0f} |", flush=True)
    check_status()


def main() -> None:
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    if not torch.cuda.is_available():
        raise SystemExit("the sweep needs a CUDA device: the sm_100a kernels have no CPU path")
    if which in ("conv", "all"):
        conv_sweep()
    if which in ("dw", "all"):
        print()
        depthwise_sweep()
    if which in ("quant", "all"):
        print()
        quantiser_sweep()
    if which in ("heads", "all"):
        print()
        heads_sweep()
    if which in ("input", "all"):
        print()
        input_sweep()


if __name__ == "__main__":
    main()
