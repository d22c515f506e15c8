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
from flashim_b200.build import EAGER, BuildContext, EngineSpec, ModelSpec
from flashim_b200.config import RunConfig
from flashim_b200.quant.tensor import QuantizedWeight, padded_channels, swizzle_scales

LEVELS = ((100, 512), (200, 256), (400, 128))  # (height = width, channels) of the feature pyramid in BASELINE config 5


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
        q, s = ops.quantize_mxfp8_dynamic(x)
        y = self.proj(q, s)
        for block in self.blocks:
            y = block(y)
        q, s = ops.quantize_mxfp8_dynamic(y)
        return self.head(q, s)


class RefinerStack(nn.Module):
    """``forward(pyramid)``: a list of bf16 NHWC tensors (one per level, the same batch of direction-images) -> the list of
    head outputs. ``chunk`` images are processed at a time to bound the intermediate tensors."""

    def __init__(self, levels=LEVELS, blocks: int = 4, seed: int = 4, chunk: int = 8) -> None:
        super().__init__()
        generator = torch.Generator().manual_seed(seed)
        self.level_shapes = tuple(levels)
        self.chunk = chunk
        self.levels = nn.ModuleList(RefinerLevel(c, blocks, generator) for _, c in levels)

    @torch.inference_mode()
    def forward(self, pyramid: list[Tensor]) -> list[Tensor]:
        outputs = []
        for level, x in zip(self.levels, pyramid):
            parts = [level(x[i: i + self.chunk]) for i in range(0, x.shape[0], self.chunk)]
            outputs.append(parts[0] if len(parts) == 1 else torch.cat(parts))
        return outputs

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
    model = RefinerStack(levels, int(arch.get("blocks", 4)), int(arch.get("seed", 4)), int(arch.get("chunk", 8)))
    return model.to(config.device or "cuda").eval()


def _graph_setup(model: nn.Module, ctx: BuildContext) -> None:
    """``cuda-graph`` engine: capture one forward per input-shape signature and replay it (the launch-bound small
    levels gain; shapes must repeat). After flashim/engines/cuda_graph.py:19-63."""
    eager_forward = model.forward
    graphs: dict = {}

    def forward(pyramid):
        key = tuple((tuple(t.shape), t.dtype) for t in pyramid)
        entry = graphs.get(key)
        if entry is None:
            static_in = [t.clone() for t in pyramid]
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                for _ in range(2):
                    eager_forward(static_in)
            torch.cuda.current_stream().wait_stream(stream)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_out = eager_forward(static_in)
            entry = graphs[key] = (graph, static_in, static_out)
        graph, static_in, static_out = entry
        for dst, src in zip(static_in, pyramid):
            dst.copy_(src)
        graph.replay()
        return static_out

    model.forward = forward


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
