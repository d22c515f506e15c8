#!/usr/bin/env python
"""Benchmark of the sm_100a conv path. One JSON line on stdout (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload stack|conv|dw|int8] [--impl reference]

Workloads (seeded synthetic inputs of the stated shapes and distributions):
  stack  config 5: synthetic refiner stack, 64 image pairs (128 direction-images) over the 3-level bf16 pyramid,
         batch-sharded over the N GPUs with no communication; metric pairs/s ("strong" scaling: 64 pairs in total).
  conv   config 3, H=W=100 C=512->512 3x3, N=4: bf16 -> static MXFP8 quantise -> conv + bias + GELU + MXFP8 requant;
         metric TFLOP/s (algorithmic 2*N*Ho*Wo*Cout*Cin*kh*kw); every GPU runs its own batch ("weak").
  int8   config 2: bf16 [2,100,100,256] -> INT8 quantise -> 256->256 3x3 conv + bias -> bf16; TOP/s.
  dw     config 4: depthwise 5x5 + bias + GELU, bf16 [4,200,200,256]; metric GB/s (algorithmic N*H*W*C*4 bytes).

A step is one pass of the workload over one batch. `value` is measured with inputs resident in HBM, `e2e` through the
public API with pinned host buffers (H2D of the step's inputs and D2H of its result inside the timed region). Inputs
rotate through buffers that together exceed the 126 MB L2, so no step finds its input cached.
`--impl reference` times FlashIM's own CPU implementation of the path on this host's cores: the reference's literal ops
when a FlashIM checkout is importable ($FLASHIM_REFERENCE or a directory `reference` beside this repository), else the
CPU oracle (the restatement of those ops, pinned to the reference's outputs).
The default line also carries `kernels`: the dominant kernels of every workload timed alone (CUDA-graph replay between
CUDA events, rotating inputs larger than L2) with their algorithmic work and roofline fraction, and `shards`: a digest
check that a pair's outputs do not depend on which GPU, or which position of a shard, computed it.
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
    """The conv shape sweep at its largest compute-bound shape: N=4, H=W=100, 512 -> 512, 3x3 pad 1."""

    name, metric, unit, dtype = "mxfp8-conv-100x100x512-k3", "mxfp8_conv_tflops", "TFLOP/s", "fp8_e4m3"
    traffic_key = "conv_mxfp8_3x3_100x100x512"
    launches_per_step = 2
    N, H, C, K = 4, 100, 512, 3
    EPILOGUE = "bias+gelu+mxfp8-requant"

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

    @classmethod
    def describe(cls, world: int) -> dict:
        return {"workload": cls.name, "batch": cls.N, "height": cls.H, "width": cls.H, "cin": cls.C, "cout": cls.C,
                "kernel": cls.K, "epilogue": cls.EPILOGUE, "input": "bf16, quantised in the step",
                "l2": f"{_rotation(cls.N * cls.H * cls.H * cls.C * 2)} rotating input buffers > L2"}

    def config(self):
        return self.describe(self.world)

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
                "frac": achieved / tensor_peak, "traffic": _traffic(self.traffic_key), "launch_ms": ms,
                "peak_source": f"2 x bf16_tflops of {source} (fp8 dense rate is twice bf16)"}

    def cpu_sample(self, budget_s):
        return _cpu_conv_sample(self.H, self.C, self.K, budget_s, getattr(self, "literal", False))


class Int8Workload(ConvWorkload):
    """The INT8 case: INT8 [2,100,100,256] -> 256, 3x3 pad 1, bias, bf16 out."""

    name, metric, unit, dtype = "int8-conv-100x100x256-k3", "int8_conv_tops", "TOP/s", "int8"
    traffic_key = "conv_int8_3x3_100x100x256"
    N, H, C, K = 2, 100, 256, 3
    EPILOGUE = "scales+bias->bf16"

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
        fn, kind = (lambda: oracle.int8_conv2d(*args)), "port"
        if getattr(self, "literal", False):
            from flashim import ops as ref_ops

            fn, kind = (lambda: ref_ops.int8_conv2d.get("reference")(*args)), "reference"
        out = _cpu_loop(fn, ops_per_call, budget_s, "TOP/s", f"1 of {self.N} images of the workload per call")
        out["kind"] = kind
        return out


class DepthwiseWorkload(Workload):
    """The depthwise case: depthwise 5x5 + bias + GELU on bf16 [4,200,200,256] -> bf16."""

    name, metric, unit, dtype = "depthwise5x5-gelu-4x200x200x256", "depthwise_gbs", "GB/s", "f32"
    traffic_key = "depthwise_gelu_bf16_4x200x200x256"
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

    @classmethod
    def describe(cls, world: int) -> dict:
        return {"workload": cls.name, "batch": cls.N, "height": cls.H, "width": cls.H, "channels": cls.C,
                "epilogue": "bias+gelu->bf16", "l2": f"{_rotation(cls.N * cls.H * cls.H * cls.C * 2)} rotating input buffers > L2"}

    def config(self):
        return self.describe(self.world)

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
                "frac": achieved / peak["hbm_gbs"], "traffic": _traffic(self.traffic_key), "launch_ms": ms,
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
    """The refiner stack: 64 pairs (128 direction-images) through the refiner stack, sharded by pairs over the ranks."""

    name, metric, unit, dtype = "refiner-stack-64-pairs", "refiner_stack_pairs_per_s", "pairs/s", "fp8_e4m3"
    traffic_key = "depthwise_mxfp8_refiner_level_400x400x128"
    scaling = "strong"
    PAIRS = 64

    def __init__(self, device, rank, world):
        super().__init__(device, rank, world)
        import flashim_b200
        from flashim_b200.refiner import LEVELS

        # graph replay: the stack is 2304 launches per step, whose host cost would otherwise bound the step
        self.model = flashim_b200.load("refiner-stack", "fp8", device=device, engine="cuda-graph")
        from flashim_b200.sharding import shard_pairs

        first, per_rank = shard_pairs(self.PAIRS, rank, world)
        self.first_pair, self.pairs = first, per_rank
        images = 2 * per_rank
        self.levels = LEVELS
        # The batch is the same 64 pairs whatever the number of GPUs: every pair is drawn from its own seed, and a rank
        # generates exactly the pairs of its shard (on the device; a pinned host mirror feeds the end-to-end path).
        self.inputs = [torch.cat([self.pair_input(level, first + i) for i in range(per_rank)]) for level in range(len(LEVELS))]
        self.host = [x.cpu().pin_memory() for x in self.inputs]
        # the graph's own input buffers hold the resident inputs (`value`) and receive the host copies (`e2e`)
        self.inputs = self.staging = self.model.static_inputs(self.inputs)
        self.result_host = [torch.empty((images, s, s, 32), dtype=torch.bfloat16).pin_memory() for s, _ in LEVELS]
        blocks = len(self.model.levels[0].blocks)
        # per level and chunk: the projection, the kernels of each block (depthwise + the residual MLP as one kernel at 128
        # and 256 channels, else depthwise + up conv + down conv) and the head (the quantisers run inside the convs)
        # (a projection wider than one 256-column tile is fed by the standalone quantiser: one more launch)
        self.launches_per_step = sum(-(-images // self.model.chunk) * (2 + (2 if c in (128, 256) else 3) * blocks
                                                                       + (1 if c > 256 or c % 128 else 0) + (1 if c % 128 else 0))
                                     for _, c in LEVELS)

    def pair_input(self, level: int, pair: int) -> torch.Tensor:
        """The two direction-images of global pair `pair` at pyramid level `level`: bf16 [2, s, s, c] ~ N(0, 1)."""
        size, channels = self.levels[level]
        g = torch.Generator(device=self.device).manual_seed(4_000_000 + 1000 * level + pair)
        return torch.randn(2, size, size, channels, generator=g, device=self.device, dtype=torch.float32).to(torch.bfloat16)

    @staticmethod
    def digest(outputs: list[torch.Tensor]) -> int:
        """Order-sensitive integer checksum of a list of bf16 tensors (exact: int64 arithmetic on the raw bits)."""
        total = 0
        for t in outputs:
            bits = t.contiguous().view(torch.int32).reshape(-1).to(torch.int64)
            weights = torch.arange(bits.numel(), device=bits.device, dtype=torch.int64) % 1021 + 1
            total = (total * 31 + int((bits * weights).sum().item())) % (1 << 61)
        return total

    def shard_check(self, ranks) -> dict:
        """A pair's outputs must not depend on the GPU or the batch position that computed it (no op mixes samples). Every
        rank digests the outputs of each of its pairs from the step just run; rank 0 recomputes the first and last pair of
        every shard on its own GPU as a batch of one pair and compares."""
        outputs = self.model(self.inputs)
        mine = {self.first_pair + i: self.digest([o[2 * i: 2 * i + 2] for o in outputs]) for i in range(self.pairs)}
        gathered = ranks.gather_strings(json.dumps(mine))
        if ranks.rank != 0:
            return {}
        table = {int(k): v for part in gathered for k, v in json.loads(part).items()}
        from flashim_b200.sharding import shard_pairs

        sample = sorted({p for r in range(self.world) for f, n in [shard_pairs(self.PAIRS, r, self.world)] if n
                         for p in (f, f + n - 1)})
        ok = len(table) == self.PAIRS
        for pair in sample:
            alone = self.model([self.pair_input(level, pair) for level in range(len(self.levels))])
            ok = ok and self.digest(list(alone)) == table.get(pair)
        return {"pairs": len(table), "recomputed_on_rank0": sample, "digest_ok": bool(ok),
                "how": "int64 checksum of each pair's head outputs; rank 0 recomputes the first and last pair of every shard as a "
                       "batch of one pair"}

    @classmethod
    def describe(cls, world: int) -> dict:
        from flashim_b200.refiner import LEVELS

        return {"workload": cls.name, "pairs": cls.PAIRS, "images": 2 * cls.PAIRS,
                "pyramid": [[2 * cls.PAIRS, s, s, c] for s, c in LEVELS], "blocks": 4, "preset": "fp8",
                "parallelism": f"batch-sharded x{world}, no collectives",
                "l2": "per-rank pyramid (>= 1.1 GB) exceeds L2"}

    def config(self):
        return self.describe(self.world)

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
                "peak": peak["hbm_gbs"], "unit": "GB/s", "frac": achieved / peak["hbm_gbs"], "traffic": _traffic(self.traffic_key),
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


def kernel_table(device, steps: int) -> list[dict]:
    """The dominant kernel of every workload of the path, each timed alone: a CUDA-graph replay of `steps` launches between
    CUDA events, inputs rotating through buffers larger than L2. Entries carry the algorithmic work of one launch, the
    achieved rate and its fraction of the measured peak (tensor peak for fp8 / int8 = twice the measured bf16 rate)."""
    from flashim_b200 import ops
    from flashim_b200.quant import swizzle_scales

    e4m3, bf16 = torch.float8_e4m3fn, torch.bfloat16
    peak, source = peaks()
    hbm, tensor = peak["hbm_gbs"], 2.0 * peak["bf16_tflops"]
    g = torch.Generator(device=device).manual_seed(7)
    rows: list[dict] = []

    def rotate(make, nbytes):
        buffers = [make() for _ in range(_rotation(nbytes))]
        state = {"i": 0}

        def nxt():
            state["i"] += 1
            return buffers[state["i"] % len(buffers)]
        return nxt

    def randn(*shape, dtype=bf16, scale=1.0):
        return (torch.randn(*shape, generator=g, device=device, dtype=torch.float32) * scale).to(dtype)

    def add(kernel, workload, fn, flops, nbytes, bound, traffic_key=None):
        ms = _time_launches(fn, max(steps, 10))
        tf, gbs = flops / ms / 1e9, nbytes / ms / 1e6
        row = {"kernel": kernel, "workload": workload, "launch_ms": ms, "bound": bound, "tflops": tf, "gbs": gbs,
               "frac_tensor": tf / tensor, "frac_hbm": gbs / hbm, "frac": tf / tensor if bound == "tensor" else gbs / hbm,
               "algorithmic_flop": flops, "algorithmic_bytes": nbytes, "traffic": _traffic(traffic_key) if traffic_key else None}
        rows.append(row)

    fused = ops.mxfp8_conv2d_fused.get("sm100")
    # the conv shape sweep (k = 3): E4M3 in -> conv + bias + GELU + static MXFP8 requantisation, N = 4
    for size, c in ((100, 512), (200, 256), (400, 128), (800, 64)):
        n, k = 4, 3
        nxt = rotate(lambda: randn(n, size, size, c, dtype=e4m3), n * size * size * c)
        ce = torch.zeros(c // 32, dtype=torch.int8, device=device)
        w = randn(c, k * k * c, dtype=e4m3, scale=0.05)
        ws = swizzle_scales(torch.zeros(c, k * k * c // 32, dtype=torch.int8)).to(device)
        bias, oe = randn(c, scale=0.02), torch.zeros(c // 32, dtype=torch.int8, device=device)
        add("conv_kernel<mxfp8> 3x3 + bias + GELU + requant", f"4x{size}x{size}x{c} -> {c}",
            lambda: fused(nxt(), ce, w, ws, bias, k, k, 1, 1, 1, 1, 1, 1, act="gelu", out_exponent=oe),
            2.0 * n * size * size * c * c * k * k, n * size * size * c * 2 + k * k * c * c, "tensor" if c >= 128 else "hbm",
            "conv_mxfp8_3x3_100x100x512" if size == 100 else None)
    # the INT8 case: INT8 3x3, scales + bias -> bf16
    n, size, c, k = 2, 100, 256, 3
    nxt8 = rotate(lambda: torch.randint(-127, 128, (n, size, size, c), generator=g, device=device, dtype=torch.int8), n * size * size * c)
    w8 = torch.randint(-127, 128, (c, k * k * c), generator=g, device=device, dtype=torch.int8)
    a_scale, w_scale = torch.tensor(0.02, device=device), torch.rand(c, generator=g, device=device) * 0.01 + 0.001
    bias8 = randn(c, scale=0.02)
    add("conv_kernel<int8> 3x3 + scales + bias", f"2x{size}x{size}x{c} -> {c}",
        lambda: ops.int8_conv2d.get("sm100")(nxt8(), w8, a_scale, w_scale, bias8, k, k, 1, 1, 1, 1, 1, 1),
        2.0 * n * size * size * c * c * k * k, n * size * size * c * 3 + k * k * c * c, "tensor", "conv_int8_3x3_100x100x256")
    # the depthwise case: depthwise 5x5 + bias + GELU -> bf16
    n, size, c = 4, 200, 256
    nxtd = rotate(lambda: randn(n, size, size, c).permute(0, 3, 1, 2), n * size * size * c * 2)
    dw, db = randn(25, c, scale=0.05), randn(c, dtype=torch.float32)
    add("dw5x5_kernel<bf16, gelu>", f"4x{size}x{size}x{c}", lambda: ops.depthwise5x5_act.get("sm100")(nxtd(), dw, db, "gelu"),
        2.0 * 25 * n * size * size * c, n * size * size * c * 4, "hbm", "depthwise_gelu_bf16_4x200x200x256")
    # the two kernels that dominate a refiner block at the 400 x 400 x 128 level (one 8-image chunk)
    n, size, c = 8, 400, 128
    nxts = rotate(lambda: randn(n, size, size, c).permute(0, 3, 1, 2), n * size * size * c * 2)
    dw, db = randn(25, c, scale=0.05), randn(c, dtype=torch.float32, scale=0.02)
    add("dw5x5_kernel<mxfp8, gelu>", f"8x{size}x{size}x{c}", lambda: ops.depthwise5x5_act_mxfp8.get("sm100")(nxts(), dw, db, "gelu"),
        2.0 * 25 * n * size * size * c, n * size * size * c * (2 + 1 + 1 / 32), "hbm", "depthwise_mxfp8_refiner_level_400x400x128")
    pixels = n * size * size

    def quantised():
        q, sc = ops.quantize_mxfp8_dynamic.get("sm100")(randn(pixels, c))
        return q.view(n, size, size, c), sc
    nxtq = rotate(quantised, pixels * c)
    wu = randn(2 * c, c, dtype=e4m3, scale=0.05)
    su = swizzle_scales(torch.zeros(2 * c, c // 32, dtype=torch.int8)).to(device)
    bu = randn(2 * c, scale=0.02)
    add("conv_kernel<mxfp8> 1x1 up + bias + GELU + dynamic requant", f"8x{size}x{size}x{c} -> {2 * c}",
        lambda: fused(*nxtq(), wu, su, bu, 1, 1, 1, 1, 0, 0, 1, 1, act="gelu", dynamic_out=True),
        2.0 * pixels * c * 2 * c, pixels * (c + 2 * c) * (1 + 1 / 32), "hbm", "conv_mxfp8_1x1_up_400x400x128")
    # the same layer with its down conv in the same kernel (what the stack runs at 128 and 256 channels): the hidden tensor
    # stays on chip, so the launch reads x and the residual and writes the block's output
    wd = randn(c, 2 * c, dtype=e4m3, scale=0.05)
    sd = swizzle_scales(torch.zeros(c, 2 * c // 32, dtype=torch.int8)).to(device)
    bd = randn(c, scale=0.02)
    residual = randn(n, size, size, c)
    add("mlp_kernel<mxfp8> 1x1 up + GELU + requant + 1x1 down + residual", f"8x{size}x{size}x{c}",
        lambda: ops.mxfp8_gelu_mlp_residual.get("sm100")(*nxtq(), wu, su, bu, wd, sd, bd, residual),
        2.0 * pixels * c * 2 * c * 2, pixels * c * (1 + 1 / 32 + 2 + 2), "hbm", "mlp_mxfp8_refiner_level_400x400x128")
    return rows


WORKLOADS = {"stack": StackWorkload, "conv": ConvWorkload, "int8": Int8Workload, "dw": DepthwiseWorkload}
DEFAULT_WORKLOAD = "stack"


def _traffic(name: str):
    """DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the kernel `name`, from the ncu captures
    whose figures are collected in profiles/traffic.json; None where no capture exists."""
    path = ROOT / "profiles" / "traffic.json"
    if not path.is_file():
        return None
    table = json.loads(path.read_text())
    entry = table.get(name)
    return None if entry is None else float(entry["dram_bytes"])


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


def _cpu_conv_sample(h, c, k, budget_s, literal=False):
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

    kind = "port"
    if literal:  # FlashIM's own ops: quantize_mxfp8 -> mxfp8_conv2d -> GELU -> quantize_mxfp8 (the conv op has no GELU of its own)
        import torch.nn.functional as F
        from flashim import ops as ref_ops

        def call():  # noqa: F811
            q = ref_ops.quantize_mxfp8.get("reference")(x, ce)
            y = ref_ops.mxfp8_conv2d.get("reference")(q.values, ce, wq, we, bias, k, k, 1, 1, k // 2, k // 2, 1, 1)
            ref_ops.quantize_mxfp8.get("reference")(F.gelu(y.float()).to(torch.bfloat16), oe)
        kind = "reference"

    out = _cpu_loop(call, 2.0 * h * h * c * c * k * k / 1e12, budget_s, "TFLOP/s", "1 of 4 images of the workload per call")
    out["kind"] = kind
    return out


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


def _reference_checkout() -> bool:
    """Make FlashIM importable from $FLASHIM_REFERENCE or a directory `reference` beside this repository, if there is one."""
    for candidate in (os.environ.get("FLASHIM_REFERENCE"), str(ROOT.parent / "reference")):
        if candidate and (Path(candidate) / "flashim").is_dir():
            if candidate not in sys.path:
                sys.path.append(candidate)
            try:
                import flashim  # noqa: F401
                return True
            except Exception:
                return False
    return False


def run_reference(args) -> None:
    """FlashIM's CPU implementation of the workload on this host's cores, a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cls = WORKLOADS[args.workload]
    probe = cls.__new__(cls)
    Workload.__init__(probe, None, 0, 1)
    if isinstance(probe, StackWorkload):
        from flashim_b200.refiner import LEVELS

        probe.levels = LEVELS
    probe.literal = _reference_checkout() and not isinstance(probe, StackWorkload)
    budget = 8.0
    for _ in range(args.warmup):
        probe.cpu_sample(0.5)
    samples, started = [], time.perf_counter()
    for _ in range(args.steps):
        samples.append(probe.cpu_sample(budget))
    step_ms = (time.perf_counter() - started) * 1e3 / max(args.steps, 1)
    value = statistics.mean(s["value"] for s in samples)
    sample = samples[-1]
    line = {
        "impl": "reference", "metric": cls.metric, "value": value, "unit": cls.unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": cls.scaling, "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": cls.describe(max(args.gpus, 1)),
        "cpu_baseline": {**sample, "value": value},
        "e2e": {"value": value, "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "a step is a bounded sample of the workload (see cpu_baseline.sample): `value` is the rate of that sample, "
                "extrapolated by work units to the whole workload; ms_per_step is the wall time of one sample step",
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
    parser.add_argument("--no-kernel-table", action="store_true", help="skip the per-kernel timings of the `kernels` entry")
    parser.add_argument("--pairs", type=int, default=StackWorkload.PAIRS,
                        help="image pairs of the stack workload (the benchmark has 64; smaller values are for ncu captures)")
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
    launches = workload.launches_per_step

    # after the timed regions: output digests across shards, host-to-device bandwidth, per-kernel table (rank 0)
    shards = workload.shard_check(ranks) if isinstance(workload, StackWorkload) else None
    host_link = _h2d_probe(device, ranks)
    roofline = workload.roofline(args.steps) if rank == 0 else None
    kernels = None
    if rank == 0 and not args.no_kernel_table:
        workload = None  # release the workload's buffers before the table allocates its own
        torch.cuda.empty_cache()
        kernels = kernel_table(device, args.steps)
        workload = WORKLOADS[args.workload].__new__(WORKLOADS[args.workload])
        Workload.__init__(workload, device, rank, world)
        if isinstance(workload, StackWorkload):
            from flashim_b200.refiner import LEVELS

            workload.levels = LEVELS
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = workload.cpu_sample(12.0)
    if rank == 0:
        cls = WORKLOADS[args.workload]
        line = {
            "metric": cls.metric, "value": value, "unit": cls.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": cls.scaling,
            "vs_baseline": None, "dtype": cls.dtype, "data": "synthetic", "config": cls.describe(world),
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": units * args.steps / (e2e_ms * 1e-3), "unit": cls.unit, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps, "host_link": host_link},
            "gpu_launches": launches * args.steps,
            "clocks": sampler.report,
            "kernels": kernels,
            "shards": shards,
        }
        print(json.dumps(line), flush=True)
    ranks.close()


def _h2d_probe(device, ranks) -> dict | None:
    """Pinned-host -> device copy rate of this rank alone and with every rank copying at once (GB/s, 256 MB copies): the
    end-to-end path of N ranks shares the host's memory system and PCIe root, which is what bounds it at N = 8."""
    size = 256 << 20
    host = torch.empty(size, dtype=torch.uint8).pin_memory()
    dev = torch.empty(size, dtype=torch.uint8, device=device)

    def rate() -> float:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dev.copy_(host, non_blocking=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(4):
            dev.copy_(host, non_blocking=True)
        end.record()
        torch.cuda.synchronize()
        return 4 * size / (start.elapsed_time(end) * 1e-3) / 1e9

    alone = None
    for r in range(ranks.world):  # one rank at a time
        ranks.barrier()
        if r == ranks.rank:
            alone = rate()
    ranks.barrier()
    together = rate()  # all ranks at once
    ranks.barrier()
    slowest_alone, slowest_together = -ranks.max(-alone), -ranks.max(-together)
    if ranks.rank != 0:
        return None
    return {"alone_gbs_min": slowest_alone, "all_ranks_gbs_min": slowest_together, "all_ranks_gbs_sum": ranks.world * slowest_together
            if ranks.world > 1 else together}


if __name__ == "__main__":
    main()
