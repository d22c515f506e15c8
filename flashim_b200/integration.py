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
