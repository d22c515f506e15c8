from flashim_b200.quant.tensor import (  # noqa: F401
    BLOCK, Int8Tensor, QuantizedTensor, QuantizedWeight, calibrate_block32_exponent, exponent_to_e8m0, padded_channels, scale_exponent_from_amax,
    swizzle_scales,
)
