"""Plugging the sm_100a backend into a FlashIM installation.

``register_into_flashim()`` registers the ``"sm100"`` implementations into FlashIM's own op registry
(``flashim.ops.mxfp8_conv2d``, ``int8_conv2d``, ``depthwise5x5_relu_mxfp8``, ``depthwise5x5_relu_int8``,
``quantize_mxfp8``, ``quantize_int8``, ``mxfp8_scaled_mm``, ``int8_linear``) with FlashIM's ``DeviceSpec`` / ``Feature`` types, so ``flashim.load(name,
preset)`` dispatches to them on a compute-capability-10.0 device. It is what an entry point of group
``flashim.backends`` (flashim/backends/_loader.py:63-70) or a ``Backend("sm100", ...)`` row of ``BACKENDS`` would call.

FlashIM keeps its torch references as fallbacks; registering there does not remove them. This package's own registry
(``flashim_b200.ops``) has none.
"""

from __future__ import annotations

_DONE = False


def register_into_flashim() -> list[str]:
    """Register into ``flashim.ops``; returns the names of the ops that gained an ``"sm100"`` implementation."""
    global _DONE
    import flashim.ops as their_ops  # noqa: F401  (raises ImportError when FlashIM is not installed)
    from flashim.ops._registry import DeviceSpec
    from flashim.platforms import Feature

    from flashim_b200.backends.sm100 import kernels

    names = ["mxfp8_conv2d", "int8_conv2d", "depthwise5x5_relu_mxfp8", "depthwise5x5_relu_int8", "quantize_mxfp8",
             "quantize_int8", "mxfp8_scaled_mm", "int8_linear", "int8_conv2d_maxpool", "romav2_refiner_heads", "romav2_refiner_input",
             "mxfp8_linear", "mxfp8_gelu_mlp", "gelu_quantize", "depthwise5x5_relu_pointwise", "depthwise5x5_relu_pointwise_mxfp8",
             "depthwise5x5_relu_pointwise_int8"]
    if not _DONE:
        kernels.register(their_ops, DeviceSpec, Feature)
        _DONE = True
    return [n for n in names if any(i.name == "sm100" for i in getattr(their_ops, n).impls)]


def entry_point() -> None:
    """Target of a ``flashim.backends`` entry point (``flashim_b200.integration:entry_point``)."""
    register_into_flashim()


def enable_sm100_conv_paths(model, capability: tuple[int, int] | None = None) -> list[str]:
    """Point FlashIM's quantised conv modules at the fused conv ops on a B200; returns the names of the modules changed.

    ``StaticMXFP8Conv2d`` decides at construction whether ``forward`` calls ``ops.mxfp8_conv2d`` or gathers an im2col
    matrix for a plain GEMM (``fused_mxfp8_conv2d_worthwhile``, flashim/ops/conv.py:241-306, measured on sm_89 / sm_90 /
    sm_12x), and whether a conv writes the next conv's quantised input from its epilogue (``CHAINED_CAPABILITIES``,
    flashim/quant/methods/conv2d.py:37-40,188-191). Neither table lists compute capability 10.0, so on a B200 a layer with
    more than 36 (tap, 32-channel block) products would never reach the implicit-GEMM kernel registered here. This pass
    sets ``use_fused`` and ``chain_output`` on every such module whose geometry the sm100 kernel takes (strides up to 4,
    zero padding), and ``chain_output`` on ``StaticInt8Conv2d``. It is a post-quantisation pass: run it on the model
    ``flashim.load`` returned, or list :data:`SM100_CONV_PASS` among a ``ModelSpec``'s passes. ``capability`` overrides
    the device query (for tests on a machine without the GPU)."""
    import torch
    from flashim.quant.methods.conv2d import StaticInt8Conv2d, StaticMXFP8Conv2d

    changed = []
    for name, module in model.named_modules():
        if not isinstance(module, (StaticMXFP8Conv2d, StaticInt8Conv2d)):
            continue
        device = next(module.buffers()).device
        have = capability
        if have is None and device.type == "cuda":
            have = torch.cuda.get_device_capability(device)
        stride = module.geometry["stride"]
        stride = (stride, stride) if isinstance(stride, int) else tuple(stride)
        if have != (10, 0) or max(stride) > 4:
            continue
        if isinstance(module, StaticMXFP8Conv2d):
            if module.channel_exponent.shape[0] > 16 * 4:  # static activation scales of at most 2048 channels stay resident
                continue
            module.use_fused = True
        module.chain_output = True
        changed.append(name)
    return changed


def _conv_pass():
    """:func:`enable_sm100_conv_paths` as a FlashIM ``Pass`` (flashim/build.py:48-60), built on first use so that importing
    this module does not import FlashIM."""
    from flashim.build import Pass

    return Pass(apply=lambda model, ctx: enable_sm100_conv_paths(model), stage="post_quant",
                description="route quantised convs through the sm_100a implicit-GEMM kernels")


def __getattr__(name: str):
    if name == "SM100_CONV_PASS":
        return _conv_pass()
    raise AttributeError(name)
