#!/usr/bin/env python
"""Benchmark of the sm_100a conv path. One JSON line on stdout (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload stack|conv|dw|int8] [--impl reference]

Workloads (BASELINE.json configs; seeded synthetic inputs of the stated shapes and distributions):
  stack  config 5: synthetic refiner stack, 64 image pairs (128 direction-images) over the 3-level bf16 pyramid,
         batch-sharded over the N GPUs with no communication; metric pairs/s ("strong" scaling: 64 pairs in total).
  conv   config 3, H=W=100 C=512->512 3x3, N=4: bf16 -> static MXFP8 quantise -> conv + bias + GELU + MXFP8 requant;
         metric TFLOP/s (algorithmic 2*N*Ho*Wo*Cout*Cin*kh*kw); every GPU runs its own batch ("weak").
  int8   config 2: bf16 [2,100,100,256] -> INT8 quantise -> 256->256 3x3 conv + bias -> bf16; TOP/s.
  dw     config 4: depthwise 5x5 + bias + GELU, bf16 [4,200,200,256]; metric GB/s (algorithmic N*H*W*C*4 bytes).

A step is one pass of the workload over one batch. `value` is measured with inputs resident in HBM, `e2e` through the
public API with pinned host buffers (H2D of the step's inputs and D2H of its result inside the timed region). Inputs
rotate through buffers that together exceed the 126 MB L2, so no step finds its input cached.
`--impl reference` times the CPU oracle (the restatement of FlashIM's torch reference) on this host's cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ---- clocks ---------------------------------------------------------------------------------------------------------


class ClockSampler:
    """`nvidia-smi` clock / throttle-reason samples every 200 ms while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.proc = index, None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.report = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, maxes, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                maxes.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(names, parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        if clocks:
            busy = [c for c in clocks if c > 0.5 * max(clocks)] or clocks
            self.report = {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(maxes), "reasons": sorted(reasons),
                           "samples": len(clocks)}


# ---- workloads -----------------------------------------------------------------------------------------------------------


class Workload:
    name = metric = unit = dtype = ""
    scaling = "weak"
    launches_per_step = 0

    def __init__(self, device, rank: int, world: int) -> None:
        self.device, self.rank, self.world = device, rank, world
        self.i = 0

    def config(self) -> dict: ...
    def units_per_step(self) -> float: ...       # per rank, in `unit` numerator units
    def step(self) -> None: ...                  # device-resident inputs
    def step_e2e(self) -> None: ...              # pinned host inputs -> device -> result back on the host
    def e2e_bytes(self) -> tuple[int, int]: ...
    def roofline(self, steps: int) -> dict: ...
    def cpu_sample(self, budget_s: float) -> dict: ...


def _rotation(bytes_per_buffer: int) -> int:
    return max(2, -(-int(1.3 * L2_BYTES) // bytes_per_buffer))


def _time_launches(fn, count: int) -> float:
    """Average device time of one call of `fn` in ms: `count` calls are captured into a CUDA graph (so that the host's
    launch cost, 40-60 us per op from Python, is not in the figure for kernels shorter than that) and the replay is
    bracketed by CUDA events on the stream it runs on. `fn` should rotate over inputs larger than L2."""
    count = max(count, 10)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(count):
            fn()
    graph.replay()  # warm
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / count


class ConvWorkload(Workload):
    """BASELINE config 3 at its largest compute-bound shape: N=4, H=W=100, 512 -> 512, 3x3 pad 1."""

    name, metric, unit, dtype = "mxfp8-conv-100x100x512-k3", "mxfp8_conv_tflops", "TFLOP/s", "fp8_e4m3"
    launches_per_step = 2
    N, H, C, K = 4, 100, 512, 3

    def __init__(self, device, rank, world):
        super().__init__(device, rank, world)
        from flashim_b200 import ops
        from flashim_b200.quant import QuantizedWeight, scale_exponent_from_amax, swizzle_scales

        self.ops = ops
        g = torch.Generator().manual_seed(2 + rank)
        n, h, c, k = self.N, self.H, self.C, self.K
        weight = torch.empty(c, c, k, k)
        torch.nn.init.kaiming_normal_(weight, generator=g)
        packed = QuantizedWeight.from_conv(weight)
        self.weight = packed.values.to(device)
        self.weight_scales = swizzle_scales(packed.scale_exponent).to(device)
        self.bias = (torch.randn(c, generator=g) * 0.02).to(torch.bfloat16).to(device)
        count = _rotation(n * h * h * c * 2)
        self.host = [torch.randn(n, h, h, c, generator=g).to(torch.bfloat16).pin_memory() for _ in range(count)]
        self.inputs = [x.to(device) for x in self.host]
        amax = self.host[0].float().abs().reshape(-1, c // 32, 32).amax(dim=(0, 2))
        self.act_exponent = scale_exponent_from_amax(amax * 1.25).to(device)
        # output exponents calibrated on the kernel's own GELU output (one untimed run)
        dense = self._conv(self._quantize(self.inputs[0]), None)
        self.out_exponent = scale_exponent_from_amax(dense.float().abs().reshape(-1, c // 32, 32).amax(dim=(0, 2))).to(device)
        self.result_host = torch.empty((n, h, h, c), dtype=torch.uint8).pin_memory()
        self.staging = torch.empty_like(self.inputs[0])
        self.q0 = self._quantize(self.inputs[0])

    def _quantize(self, x):
        return self.ops.quantize_mxfp8(x, self.act_exponent).values

    def _conv(self, q, out_exponent):
        k = self.K
        return self.ops.mxfp8_conv2d_fused(q, self.act_exponent, self.weight, self.weight_scales, self.bias, k, k, 1, 1,
                                           k // 2, k // 2, 1, 1, act="gelu", out_exponent=out_exponent)

    def config(self):
        return {"workload": self.name, "batch": self.N, "height": self.H, "width": self.H, "cin": self.C, "cout": self.C,
                "kernel": self.K, "epilogue": "bias+gelu+mxfp8-requant", "input": "bf16, quantised in the step",
                "l2": f"{len(self.inputs)} rotating input buffers > L2"}

    def units_per_step(self):
        return 2.0 * self.N * self.H * self.H * self.C * self.C * self.K * self.K / 1e12

    def step(self):
        x = self.inputs[self.i % len(self.inputs)]
        self.i += 1
        self.last = self._conv(self._quantize(x), self.out_exponent)

    def step_e2e(self):
        self.staging.copy_(self.host[self.i % len(self.host)], non_blocking=True)
        self.i += 1
        out = self._conv(self._quantize(self.staging), self.out_exponent)
        self.result_host.copy_(out.view(torch.uint8), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def e2e_bytes(self):
        return self.staging.numel() * 2, self.result_host.numel()

    def roofline(self, steps):
        ms = _time_launches(lambda: self._conv(self.q0, self.out_exponent), max(steps, 10))
        peak, source = peaks()
        tensor_peak = 2.0 * peak["bf16_tflops"]
        achieved = self.units_per_step() / (ms * 1e-3)
        return {"bound": "tensor", "kernel": "conv_kernel<mxfp8>", "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s",
                "frac": achieved / tensor_peak, "traffic": _traffic(self.name), "launch_ms": ms,
                "peak_source": f"2 x bf16_tflops of {source} (fp8 dense rate is twice bf16)"}

    def cpu_sample(self, budget_s):
        return _cpu_conv_sample(self.H, self.C, self.K, budget_s)


class Int8Workload(ConvWorkload):
    """BASELINE config 2: INT8 [2,100,100,256] -> 256, 3x3 pad 1, bias, bf16 out."""

    name, metric, unit, dtype = "int8-conv-100x100x256-k3", "int8_conv_tops", "TOP/s", "int8"
    N, H, C, K = 2, 100, 256, 3

    def __init__(self, device, rank, world):
        Workload.__init__(self, device, rank, world)
        from flashim_b200 import ops
        from flashim_b200.quant.tensor import int8_weight_from_conv

        self.ops = ops
        g = torch.Generator().manual_seed(1 + rank)
        n, h, c, k = self.N, self.H, self.C, self.K
        weight = torch.empty(c, c, k, k)
        torch.nn.init.kaiming_normal_(weight, generator=g)
        wq, ws = int8_weight_from_conv(weight)
        self.weight, self.w_scale = wq.to(device), ws.to(device)
        self.bias = (torch.randn(c, generator=g) * 0.02).to(torch.bfloat16).to(device)
        count = _rotation(n * h * h * c * 2)
        self.host = [torch.randn(n, h, h, c, generator=g).to(torch.bfloat16).pin_memory() for _ in range(count)]
        self.inputs = [x.to(device) for x in self.host]
        self.a_scale = (self.host[0].float().abs().max() / 127).reshape(()).to(device)
        self.result_host = torch.empty((n, h, h, c), dtype=torch.bfloat16).pin_memory()
        self.staging = torch.empty_like(self.inputs[0])
        self.out_exponent = None
        self.q0 = self._quantize(self.inputs[0])

    def _quantize(self, x):
        return self.ops.quantize_int8(x, self.a_scale).values

    def _conv(self, q, _=None):
        k = self.K
        return self.ops.int8_conv2d(q, self.weight, self.a_scale, self.w_scale, self.bias, k, k, 1, 1, k // 2, k // 2, 1, 1)

    def config(self):
        cfg = super().config()
        cfg.update(epilogue="scales+bias->bf16", input="bf16, quantised in the step")
        return cfg

    def step_e2e(self):
        self.staging.copy_(self.host[self.i % len(self.host)], non_blocking=True)
        self.i += 1
        out = self._conv(self._quantize(self.staging))
        self.result_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def e2e_bytes(self):
        return self.staging.numel() * 2, self.result_host.numel() * 2

    def roofline(self, steps):
        r = super().roofline(steps)
        r.update(kernel="conv_kernel<int8>", unit="TOP/s")
        return r

    def cpu_sample(self, budget_s):
        import oracle

        torch.manual_seed(1)
        x = torch.randint(-127, 128, (1, self.H, self.H, self.C), dtype=torch.int8)
        w = torch.randint(-127, 128, (self.C, self.K * self.K * self.C), dtype=torch.int8)
        args = (x, w, torch.tensor(0.01), torch.rand(self.C) * 0.01, None, self.K, self.K, 1, 1, 1, 1, 1, 1)
        ops_per_call = 2.0 * self.H * self.H * self.C * self.C * self.K * self.K / 1e12
        return _cpu_loop(lambda: oracle.int8_conv2d(*args), ops_per_call, budget_s, "TOP/s",
                         f"1 of {self.N} images of the workload per call")


class DepthwiseWorkload(Workload):
    """BASELINE config 4: depthwise 5x5 + bias + GELU on bf16 [4,200,200,256] -> bf16."""

    name, metric, unit, dtype = "depthwise5x5-gelu-4x200x200x256", "depthwise_gbs", "GB/s", "f32"
    launches_per_step = 1
    N, H, C = 4, 200, 256

    def __init__(self, device, rank, world):
        super().__init__(device, rank, world)
        from flashim_b200 import ops

        self.ops = ops
        g = torch.Generator().manual_seed(3 + rank)
        n, h, c = self.N, self.H, self.C
        count = _rotation(n * h * h * c * 2)
        self.host = [torch.randn(n, h, h, c, generator=g).to(torch.bfloat16).pin_memory() for _ in range(count)]
        self.inputs = [x.to(device) for x in self.host]
        self.weight = (torch.randn(25, c, generator=g) * 0.05).to(torch.bfloat16).to(device)
        self.bias = torch.randn(c, generator=g).to(device)
        self.staging = torch.empty_like(self.inputs[0])
        self.result_host = torch.empty((n, h, h, c), dtype=torch.bfloat16).pin_memory()

    def _run(self, x):
        return self.ops.depthwise5x5_act(x.permute(0, 3, 1, 2), self.weight, self.bias, "gelu")

    def config(self):
        return {"workload": self.name, "batch": self.N, "height": self.H, "width": self.H, "channels": self.C,
                "epilogue": "bias+gelu->bf16", "l2": f"{len(self.inputs)} rotating input buffers > L2"}

    def units_per_step(self):
        return self.N * self.H * self.H * self.C * 4 / 1e9

    def step(self):
        self.last = self._run(self.inputs[self.i % len(self.inputs)])
        self.i += 1

    def step_e2e(self):
        self.staging.copy_(self.host[self.i % len(self.host)], non_blocking=True)
        self.i += 1
        self.result_host.copy_(self._run(self.staging), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def e2e_bytes(self):
        return self.staging.numel() * 2, self.result_host.numel() * 2

    def roofline(self, steps):
        state = {"i": 0}

        def launch():
            self._run(self.inputs[state["i"] % len(self.inputs)])
            state["i"] += 1

        ms = _time_launches(launch, max(steps, 10))
        peak, source = peaks()
        achieved = self.units_per_step() / (ms * 1e-3)
        return {"bound": "hbm", "kernel": "dw5x5_kernel<bf16>", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peak["hbm_gbs"], "traffic": _traffic(self.name), "launch_ms": ms,
                "peak_source": f"hbm_gbs of {source}"}

    def cpu_sample(self, budget_s):
        import oracle

        g = torch.Generator().manual_seed(3)
        x = torch.randn(1, self.C, self.H, self.H, generator=g).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        w = (torch.randn(25, self.C, generator=g) * 0.05).to(torch.bfloat16)
        b = torch.randn(self.C, generator=g)
        return _cpu_loop(lambda: oracle.depthwise5x5_act_ext(x, w, b, "gelu"), self.H * self.H * self.C * 4 / 1e9, budget_s,
                         "GB/s", f"1 of {self.N} images of the workload per call")


class StackWorkload(Workload):
    """BASELINE config 5: 64 pairs (128 direction-images) through the refiner stack, sharded by pairs over the ranks."""

    name, metric, unit, dtype = "refiner-stack-64-pairs", "refiner_stack_pairs_per_s", "pairs/s", "fp8_e4m3"
    scaling = "strong"
    PAIRS = 64

    def __init__(self, device, rank, world):
        super().__init__(device, rank, world)
        import flashim_b200
        from flashim_b200.refiner import LEVELS

        # graph replay: the stack is 2304 launches per step, whose host cost would otherwise bound the step
        self.model = flashim_b200.load("refiner-stack", "fp8", device=device, engine="cuda-graph")
        from flashim_b200.sharding import shard_pairs

        _, per_rank = shard_pairs(self.PAIRS, rank, world)
        self.pairs = per_rank
        images = 2 * per_rank
        g = torch.Generator().manual_seed(4 + rank)
        self.levels = LEVELS
        # the pyramid of this rank's images: device copy for `value`, pinned host copy for `e2e`
        self.host = [torch.randn(images, s, s, c, generator=g, dtype=torch.float32).to(torch.bfloat16) for s, c in LEVELS] \
            if images <= 16 else None
        if self.host is None:  # large shards: generate per level on the device (same distribution), keep a host mirror
            dg = torch.Generator(device=device).manual_seed(4 + rank)
            self.inputs = [torch.randn(images, s, s, c, generator=dg, device=device, dtype=torch.bfloat16) for s, c in LEVELS]
            self.host = [x.cpu().pin_memory() for x in self.inputs]
        else:
            self.host = [x.pin_memory() for x in self.host]
            self.inputs = [x.to(device) for x in self.host]
        # the graph's own input buffers hold the resident inputs (`value`) and receive the host copies (`e2e`)
        self.inputs = self.staging = self.model.static_inputs(self.inputs)
        self.result_host = [torch.empty((images, s, s, 32), dtype=torch.bfloat16).pin_memory() for s, _ in LEVELS]
        blocks = len(self.model.levels[0].blocks)
        self.launches_per_step = sum(-(-images // self.model.chunk) * (4 + 3 * blocks) for _ in LEVELS)

    def config(self):
        return {"workload": self.name, "pairs": self.PAIRS, "images": 2 * self.PAIRS,
                "pyramid": [[2 * self.PAIRS, s, s, c] for s, c in self.levels], "blocks": 4, "preset": "fp8",
                "parallelism": f"batch-sharded x{self.world}, no collectives",
                "l2": "per-rank pyramid (>= 1.1 GB) exceeds L2"}

    def units_per_step(self):
        return float(self.pairs)

    def step(self):
        self.last = self.model(self.inputs)

    def step_e2e(self):
        # pinned host pyramid -> device -> stack -> pinned host outputs, chunk by chunk with copies and compute overlapped
        self.model.forward_host(self.host, self.result_host)

    def e2e_bytes(self):
        return sum(x.numel() * 2 for x in self.staging), sum(x.numel() * 2 for x in self.result_host)

    def roofline(self, steps):
        # dominant kernel of the stack by device time (38 % in the ncu launch list): the depthwise 5x5 + GELU -> MXFP8
        # producer, timed on its largest level (400 x 400 x 128, one chunk of images)
        from flashim_b200 import ops

        block = self.model.levels[-1].blocks[0]
        size, c = self.levels[-1]
        n = min(self.model.chunk, self.inputs[-1].shape[0])
        x = self.inputs[-1][:n].permute(0, 3, 1, 2)
        ms = _time_launches(lambda: ops.depthwise5x5_act_mxfp8(x, block.dw_weight, block.dw_bias, "gelu"), max(steps, 10))
        algorithmic = n * size * size * c * (2 + 1 + 1 / 32)  # bf16 in, E4M3 + E8M0 out
        peak, source = peaks()
        achieved = algorithmic / 1e9 / (ms * 1e-3)
        return {"bound": "hbm", "kernel": "dw5x5_kernel<mxfp8, gelu> 400x400x128", "achieved": achieved,
                "peak": peak["hbm_gbs"], "unit": "GB/s", "frac": achieved / peak["hbm_gbs"], "traffic": _traffic(self.name),
                "launch_ms": ms, "peak_source": f"hbm_gbs of {source}"}

    def cpu_sample(self, budget_s):
        import oracle

        g = torch.Generator().manual_seed(4)
        levels = [oracle.make_refiner_level_weights(c, 4, g) for _, c in self.levels]
        scale = 4  # the pyramid at 1/4 of the linear size: 1/16 of one direction-image per call
        xs = [torch.randn(1, s // scale, s // scale, c, generator=g).to(torch.bfloat16) for s, c in self.levels]

        def call():
            for x, level in zip(xs, levels):
                oracle.refiner_level_ext(x, level)

        pairs_per_call = 0.5 / (scale * scale)
        return _cpu_loop(call, pairs_per_call, budget_s, "pairs/s",
                         f"1 direction-image at 1/{scale} linear size (1/{2 * scale * scale} pair) per call, scaled by pixels")


WORKLOADS = {"stack": StackWorkload, "conv": ConvWorkload, "int8": Int8Workload, "dw": DepthwiseWorkload}
DEFAULT_WORKLOAD = "stack"


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of each workload's dominant kernel, from the ncu
# captures summarised under profiles/ (file named beside each figure); None where no capture exists.
NCU_TRAFFIC: dict[str, float] = {
    # dw5x5_kernel depthwise + GELU -> MXFP8 on 8 x 400 x 400 x 128 (the launch the stack's roofline times), same shape for
    # every --pairs >= 4: profiles/depthwise_mxfp8_refiner_level_400x400x128.md (418.53 MB read + 154.40 MB written)
    "refiner-stack": 572.93e6,
    # profiles/conv_mxfp8_3x3_100x100x512.md (22.99 MB read; the 20 MB output is still in L2 when the kernel ends)
    "mxfp8-conv-100x100x512-k3": 23.05e6,
    # profiles/conv_int8_3x3_100x100x256.md
    "int8-conv-100x100x256-k3": 5.79e6,
    # profiles/depthwise_gelu_bf16_4x200x200x256.md (88.71 MB read + 36.21 MB written; the rest of the output in L2)
    "depthwise5x5-gelu-4x200x200x256": 124.92e6,
}


def _traffic(name: str):
    if name.startswith("refiner-stack"):
        return NCU_TRAFFIC["refiner-stack"]
    return NCU_TRAFFIC.get(name)


def _cpu_loop(fn, units_per_call: float, budget_s: float, unit: str, sample: str) -> dict:
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    fn()  # warm-up
    calls, start = 0, time.perf_counter()
    while True:
        fn()
        calls += 1
        elapsed = time.perf_counter() - start
        if elapsed >= budget_s or calls >= 1000:
            break
    return {"value": units_per_call * calls / elapsed, "unit": unit, "cores": threads, "kind": "port",
            "sample": f"{sample}; {calls} calls in {elapsed:.1f} s"}


def _cpu_conv_sample(h, c, k, budget_s):
    import oracle

    g = torch.Generator().manual_seed(2)
    x = (torch.randn(1, h, h, c, generator=g)).to(torch.bfloat16)
    ce = oracle.static_block_exponent(x)
    w = torch.empty(c, c, k, k)
    torch.nn.init.kaiming_normal_(w, generator=g)
    wq, we = oracle.pack_mx_conv_weight(w)
    bias = (torch.randn(c, generator=g) * 0.02).to(torch.bfloat16)
    oe = torch.zeros(c // 32, dtype=torch.int8)

    def call():
        q = oracle.quantize_static_mx(x, ce)
        oracle.mxfp8_conv2d_ext(q, ce, wq, we, bias, k, k, 1, 1, k // 2, k // 2, 1, 1, act="gelu", out_exponent=oe)

    return _cpu_loop(call, 2.0 * h * h * c * c * k * k / 1e12, budget_s, "TFLOP/s", "1 of 4 images of the workload per call")


# ---- driver ------------------------------------------------------------------------------------------------------------------


def _timed(fn, steps: int, ranks) -> float:
    """Device time of `steps` calls in ms: CUDA events on the current stream, barrier + synchronise on both sides, max over ranks."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ranks.barrier()
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    ranks.barrier()
    return ranks.max(ms)


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cls = WORKLOADS[args.workload]
    probe = cls.__new__(cls)
    Workload.__init__(probe, None, 0, 1)
    if isinstance(probe, StackWorkload):
        from flashim_b200.refiner import LEVELS

        probe.levels = LEVELS
    budget = 8.0
    for _ in range(args.warmup):
        probe.cpu_sample(0.5)
    samples = [probe.cpu_sample(budget) for _ in range(args.steps)]
    value = statistics.mean(s["value"] for s in samples)
    sample = samples[-1]
    line = {
        "impl": "reference", "metric": cls.metric, "value": value, "unit": cls.unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": cls.scaling, "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": cls.name},
        "cpu_baseline": {**sample, "value": value},
        "e2e": {"value": value, "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU oracle (restatement of FlashIM's torch reference, pinned to the reference's outputs) on all host cores",
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--workload", choices=sorted(WORKLOADS), default=DEFAULT_WORKLOAD)
    parser.add_argument("--impl", choices=["b200", "reference"], default="b200")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--pairs", type=int, default=StackWorkload.PAIRS,
                        help="image pairs of the stack workload (BASELINE config 5 has 64; smaller values are for ncu captures)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    StackWorkload.PAIRS = args.pairs
    StackWorkload.name = f"refiner-stack-{args.pairs}-pairs"

    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sm_100a kernels have no CPU path")

    from flashim_b200.sharding import Ranks

    ranks = Ranks.from_env("nccl")
    rank, world, local = ranks.rank, ranks.world, ranks.local_rank
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    import flashim_b200

    workload = WORKLOADS[args.workload](device, rank, world)
    # clocks are sampled from the warm-up to the end of the end-to-end region (short timed regions fall between samples)
    with ClockSampler(local) as sampler:
        for _ in range(args.warmup):
            workload.step()
        torch.cuda.synchronize()
        flashim_b200.check_status(device)
        ms = _timed(workload.step, args.steps, ranks)
        flashim_b200.check_status(device)
        units = ranks.sum(workload.units_per_step())
        value = units * args.steps / (ms * 1e-3)
        for _ in range(2):
            workload.step_e2e()
        e2e_ms = _timed(workload.step_e2e, args.steps, ranks)
        flashim_b200.check_status(device)
        # keep the device busy long enough for at least a few 200 ms samples
        spin_until = time.perf_counter() + 0.7
        while time.perf_counter() < spin_until:
            workload.step()
        torch.cuda.synchronize()
    h2d, d2h = workload.e2e_bytes()

    roofline = workload.roofline(args.steps) if rank == 0 else None
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = workload.cpu_sample(12.0)
    if rank == 0:
        line = {
            "metric": workload.metric, "value": value, "unit": workload.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": workload.scaling,
            "vs_baseline": None, "dtype": workload.dtype, "data": "synthetic", "config": workload.config(),
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": units * args.steps / (e2e_ms * 1e-3), "unit": workload.unit, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": workload.launches_per_step * args.steps,
            "clocks": sampler.report,
        }
        print(json.dumps(line), flush=True)
    ranks.close()


if __name__ == "__main__":
    main()
