"""Synthetic refiner stack: the benchmark model of the conv path, registered as ``"refiner-stack"``.

Structure per pyramid level (channels C), after RoMaV2's ``ConvRefiner`` (flashim/models/romav2/refiner.py:45-148: a
projection, a run of depthwise-separable blocks, a small head) with the block widened to a residual MLP::

    x bf16 NHWC -> dynamic MXFP8 -> 1x1 conv C->C
      4 x [ depthwise 5x5 + bias + GELU -> dynamic MXFP8 -> 1x1 conv C->2C + bias + GELU -> dynamic MXFP8
            -> 1x1 conv 2C->C + bias + residual ]
    -> dynamic MXFP8 -> 1x1 conv C->4 (warp + confidence; 32 physical output channels)

Every tensor-core product is a block-scaled MXFP8 conv with per-pixel E8M0 activation scales produced by the epilogue
(or the depthwise producer) of the layer before, so no standalone quantisation pass runs between layers. Weights are
random-init (Kaiming normal) from ``arch.seed``; there is no checkpoint. Image pairs are independent: a batch is
processed in chunks, and several GPUs each take a contiguous slice of the pairs with no communication.
"""

from __future__ import annotations

import torch
from torch import Tensor, nn

from flashim_b200 import ops
from flashim_b200.backends.sm100.kernels import check_status
from flashim_b200.build import EAGER, BuildContext, EngineSpec, ModelSpec
from flashim_b200.config import RunConfig
from flashim_b200.quant.tensor import QuantizedWeight, padded_channels, swizzle_scales

LEVELS = ((100, 512), (200, 256), (400, 128))  # (height = width, channels) of the benchmark's feature pyramid


class PointwiseMX(nn.Module):
    """A 1x1 conv with MXFP8 weights: E4M3 ``[Coutp, Cin]`` + swizzled E8M0 scales + bf16 bias ``[Coutp]``."""

    def __init__(self, cin: int, cout: int, generator: torch.Generator) -> None:
        super().__init__()
        weight = torch.empty(cout, cin, 1, 1)
        nn.init.kaiming_normal_(weight, generator=generator)
        packed = QuantizedWeight.from_conv(weight)
        self.cin, self.cout = cin, cout
        self.register_buffer("weight", packed.values.view(torch.uint8))
        self.register_buffer("weight_exponent", packed.scale_exponent)
        self.register_buffer("weight_scales", swizzle_scales(packed.scale_exponent))
        self.register_buffer("bias", (torch.randn(padded_channels(cout), generator=generator) * 0.02).to(torch.bfloat16))

    def forward(self, q: Tensor, scales: Tensor, **epilogue):
        return ops.mxfp8_conv2d_fused(q, scales, self.weight.view(torch.float8_e4m3fn), self.weight_scales, self.bias,
                                      1, 1, 1, 1, 0, 0, 1, 1, **epilogue)


    def forward_bf16(self, x: Tensor, **epilogue):
        """The same layer on bf16 activations: quantised per pixel and 32 channels inside the conv kernel where it takes
        them (Cin a multiple of 128, one tile of output channels), by the standalone quantiser otherwise. Same bits either way."""
        # (a layer wider than one 256-column tile would quantise every activation tile once per column tile: measured
        # slower than the standalone quantiser at 512 -> 512)
        if self.cin % 128 == 0 and self.cout <= 256:
            return ops.mxfp8_conv2d_bf16(x, None, self.weight.view(torch.float8_e4m3fn), self.weight_scales, self.bias, **epilogue)
        q, s = ops.quantize_mxfp8_dynamic(x)
        return self.forward(q, s, **epilogue)


class RefinerBlock(nn.Module):
    def __init__(self, channels: int, generator: torch.Generator) -> None:
        super().__init__()
        self.channels = channels
        self.register_buffer("dw_weight", (torch.randn(25, channels, generator=generator) * 0.05).to(torch.bfloat16))
        self.register_buffer("dw_bias", torch.randn(channels, generator=generator) * 0.02)
        self.up = PointwiseMX(channels, 2 * channels, generator)
        self.down = PointwiseMX(2 * channels, channels, generator)

    def forward(self, x: Tensor) -> Tensor:
        """``x`` bf16 ``[B, H, W, C]`` -> bf16 ``[B, H, W, C]``."""
        b, h, w, c = x.shape
        q, s = ops.depthwise5x5_act_mxfp8(x.permute(0, 3, 1, 2), self.dw_weight, self.dw_bias, "gelu")
        if c in (128, 256) and x.is_contiguous():
            # up conv, GELU, requantisation, down conv and residual add in one launch: the hidden tensor stays on chip
            # (the same bits as the two launches below)
            return ops.mxfp8_gelu_mlp_residual(
                q.view(b, h, w, c), s, self.up.weight.view(torch.float8_e4m3fn), self.up.weight_scales, self.up.bias,
                self.down.weight.view(torch.float8_e4m3fn), self.down.weight_scales, self.down.bias, x)
        hq, hs = self.up(q.view(b, h, w, c), s, act="gelu", dynamic_out=True)
        return self.down(hq, hs, residual=x)


class RefinerLevel(nn.Module):
    def __init__(self, channels: int, blocks: int, generator: torch.Generator) -> None:
        super().__init__()
        self.channels = channels
        # construction order matches oracle.make_refiner_level_weights: proj, head, then the blocks
        self.proj = PointwiseMX(channels, channels, generator)
        self.head = PointwiseMX(channels, 4, generator)
        self.blocks = nn.ModuleList(RefinerBlock(channels, generator) for _ in range(blocks))

    def forward(self, x: Tensor) -> Tensor:
        """bf16 ``[B, H, W, C]`` -> bf16 ``[B, H, W, 32]`` (channels 0-1 warp, 2-3 confidence, the rest padding)."""
        y = self.proj.forward_bf16(x)
        for block in self.blocks:
            y = block(y)
        return self.head.forward_bf16(y)


class RefinerStack(nn.Module):
    """``forward(pyramid)``: a list of bf16 NHWC tensors (one per level, the same batch of direction-images) -> the list of
    head outputs. ``chunk`` images are processed at a time to bound the intermediate tensors."""

    def __init__(self, levels=LEVELS, blocks: int = 4, seed: int = 4, chunk: int = 8, lanes: int = 1) -> None:
        super().__init__()
        generator = torch.Generator().manual_seed(seed)
        self.level_shapes = tuple(levels)
        self.chunk = chunk
        self.lanes = lanes
        self.levels = nn.ModuleList(RefinerLevel(c, blocks, generator) for _, c in levels)
        self._side: dict = {}

    @torch.inference_mode()
    def forward(self, pyramid: list[Tensor]) -> list[Tensor]:
        """Chunks are independent. With ``lanes > 1`` they alternate between that many streams (forked from and joined to
        the current one, also inside a graph capture), so that the prologue of one chunk's kernel overlaps the tail of the
        other's; the results are the same bytes."""
        device = pyramid[0].device
        lanes = self.lanes if device.type == "cuda" else 1
        if lanes > 1:
            main = torch.cuda.current_stream(device)
            if device not in self._side:
                self._side[device] = [torch.cuda.Stream(device) for _ in range(lanes - 1)]
            streams = [main, *self._side[device][: lanes - 1]]
            for stream in streams[1:]:
                stream.wait_stream(main)
        outputs, turn = [], 0
        for level, x in zip(self.levels, pyramid):
            parts = []
            for i in range(0, x.shape[0], self.chunk):
                if lanes > 1:
                    with torch.cuda.stream(streams[turn % lanes]):
                        parts.append(level(x[i: i + self.chunk]))
                    turn += 1
                else:
                    parts.append(level(x[i: i + self.chunk]))
            outputs.append(parts)
        if lanes > 1:
            for stream in streams[1:]:
                main.wait_stream(stream)
        return [parts[0] if len(parts) == 1 else torch.cat(parts) for parts in outputs]

    def flops_per_image(self) -> float:
        """Algorithmic FLOPs of one direction-image through every level (1x1 convs: 2*C_in*C_out per pixel;
        depthwise: 2*25 per element)."""
        total = 0.0
        for (size, c), level in zip(self.level_shapes, self.levels):
            pixels = size * size
            per_pixel = 2 * c * c + len(level.blocks) * (2 * 25 * c + 2 * c * 2 * c + 2 * 2 * c * c) + 2 * c * 4
            total += pixels * per_pixel
        return total


def _load(config: RunConfig) -> nn.Module:
    arch = config.arch
    levels = tuple(tuple(level) for level in arch.get("levels", LEVELS))
    model = RefinerStack(levels, int(arch.get("blocks", 4)), int(arch.get("seed", 4)), int(arch.get("chunk", 8)),
                         int(arch.get("lanes", 2)))
    return model.to(config.device or "cuda").eval()


def _graph_setup(model: nn.Module, ctx: BuildContext) -> None:
    """``cuda-graph`` engine: capture one forward per input-shape signature and replay it (shapes must repeat). The 17
    launches per level and chunk cost more on the host than on the GPU once the kernels are fast; a replay has no host
    cost. ``model.static_inputs(pyramid)`` returns the graph's own input buffers for that signature: a caller that
    writes its inputs there (e.g. the host-to-device copy) and passes them back skips the staging copy.
    After flashim/engines/cuda_graph.py:19-63."""
    eager_forward = model.forward
    graphs: dict = {}

    def signature(pyramid):
        return tuple((tuple(t.shape), t.dtype) for t in pyramid)

    def entry_for(pyramid):
        key = signature(pyramid)
        entry = graphs.get(key)
        if entry is None:
            static_in = [t.clone() for t in pyramid]
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                for _ in range(2):
                    eager_forward(static_in)
            torch.cuda.current_stream().wait_stream(stream)
            check_status(static_in[0].device)  # kernels inside a capture cannot be checked; the warm-up runs of the same shapes can
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_out = eager_forward(static_in)
            entry = graphs[key] = (graph, static_in, static_out)
        return entry

    def forward(pyramid):
        graph, static_in, static_out = entry_for(pyramid)
        for dst, src in zip(static_in, pyramid):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src)
        graph.replay()
        return static_out

    # ---- host-to-host streaming: per-chunk graphs in two slots, copies on their own streams ----
    chunk_graphs: dict = {}
    streams: dict = {}

    def chunk_entry(index: int, level, shape, dtype, device, slot: int):
        key = (index, tuple(shape), dtype, slot)
        entry = chunk_graphs.get(key)
        if entry is None:
            static_in = torch.zeros(shape, dtype=dtype, device=device)
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side), torch.inference_mode():
                for _ in range(2):
                    level(static_in)
            torch.cuda.current_stream(device).wait_stream(side)
            check_status(device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph), torch.inference_mode():
                static_out = level(static_in)
            entry = chunk_graphs[key] = (graph, static_in, static_out)
        return entry

    def forward_host(host_pyramid, host_outputs):
        """Pinned host pyramid -> pinned host head outputs. Chunk ``i + 1`` crosses PCIe while chunk ``i`` computes and
        chunk ``i - 1`` returns: a copy-in stream, the compute stream and a copy-out stream, two buffer slots per level,
        ordered by events only (no host synchronisation until the end)."""
        device = next(model.parameters(), next(model.buffers())).device
        compute = torch.cuda.current_stream(device)
        if device not in streams:
            streams[device] = (torch.cuda.Stream(device), torch.cuda.Stream(device))
        copy_in, copy_out = streams[device]
        copy_in.wait_stream(compute)
        copy_out.wait_stream(compute)
        in_free: dict = {}   # (level, slot) -> event: the graph that read this input buffer has run
        out_free: dict = {}  # (level, slot) -> event: the copy-out of this output buffer has finished
        step = 0
        for index, (level, src, dst) in enumerate(zip(model.levels, host_pyramid, host_outputs)):
            for start in range(0, src.shape[0], model.chunk):
                part = src[start: start + model.chunk]
                slot = step & 1
                step += 1
                graph, static_in, static_out = chunk_entry(index, level, part.shape, part.dtype, device, slot)
                key = (index, tuple(part.shape), slot)
                with torch.cuda.stream(copy_in):
                    if key in in_free:
                        copy_in.wait_event(in_free[key])
                    static_in.copy_(part, non_blocking=True)
                    arrived = torch.cuda.Event()
                    arrived.record(copy_in)
                compute.wait_event(arrived)
                if key in out_free:
                    compute.wait_event(out_free[key])
                graph.replay()
                done = torch.cuda.Event()
                done.record(compute)
                in_free[key] = done
                with torch.cuda.stream(copy_out):
                    copy_out.wait_event(done)
                    dst[start: start + part.shape[0]].copy_(static_out, non_blocking=True)
                    returned = torch.cuda.Event()
                    returned.record(copy_out)
                out_free[key] = returned
        compute.wait_stream(copy_out)
        compute.synchronize()
        return host_outputs

    model.forward = forward
    model.static_inputs = lambda pyramid: entry_for(pyramid)[1]
    model.forward_host = forward_host


def _validate(config: RunConfig) -> None:
    for size, channels in config.arch.get("levels", LEVELS):
        if channels % 64:
            raise ValueError(f"refiner-stack: level channels must be multiples of 64, got {channels}")


SPEC = ModelSpec(
    name="refiner-stack",
    role="dense",
    description="synthetic MXFP8 refiner stack over a 3-level feature pyramid (benchmark model of the conv path)",
    load=_load,
    presets={"fp8": {"precision": {"compute_dtype": "bf16", "quant": "mxfp8-dynamic"}}},
    default_preset="fp8",
    engines={"eager": EAGER, "cuda-graph": EngineSpec(setup=_graph_setup)},
    validate=_validate,
)
