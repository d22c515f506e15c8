"""Ops of the quantized conv path. Names and signatures are FlashIM's (flashim/ops/conv.py, flashim/ops/quantize.py)
so a module written against ``flashim.ops`` runs unchanged; ops marked *extension* expose what the sm_100a epilogues add
on top (GELU, per-pixel activation scales, dynamic requantisation, fp32 / int32 outputs).

No op here carries a torch reference: if no registered implementation accepts a call, the call raises
:class:`~flashim_b200.ops._registry.NoImplementation`.
"""

from flashim_b200.ops._registry import (  # noqa: F401
    OPS, DeviceSpec, NoImplementation, Op, call_counts, configure, reset_call_counts, set_strict,
)

# -- FlashIM's ops (same name, same arguments) ---------------------------------------------------------------------
quantize_mxfp8 = Op("quantize_mxfp8", doc="(value [..., C], scale_exponent int8 [Cp/32]) -> QuantizedTensor "
                    "(flashim/ops/quantize.py:80-87)")
quantize_int8 = Op("quantize_int8", doc="(value, scale, *, channel_scale=None) -> Int8Tensor "
                   "(flashim/ops/quantize.py:93-100)")
depthwise5x5_relu_mxfp8 = Op("depthwise5x5_relu_mxfp8", doc="(value [B,C,H,W] channels-last, weight bf16 [25,C], bias fp32 "
                             "[C]) -> (E4M3 [B*H*W, C], swizzled E8M0) (flashim/ops/conv.py:30-44)")
depthwise5x5_relu_int8 = Op("depthwise5x5_relu_int8", doc="(value, weight, bias, scale) -> int8 [B*H*W, C] "
                            "(flashim/ops/conv.py:50-61)")
mxfp8_conv2d = Op("mxfp8_conv2d", doc="(x E4M3 NHWC, channel_exponent, weight E4M3 [Cout, K], weight_exponent int8 "
                  "[Cout, K/32], bias, kh, kw, sh, sw, ph, pw, dh, dw, *, relu, residual, out_exponent) -> bf16 / E4M3 "
                  "NHWC (flashim/ops/conv.py:309-342)")
int8_conv2d = Op("int8_conv2d", doc="(x int8 NHWC, weight int8 [Cout, K], a_scale, w_scale, bias, kh, kw, sh, sw, ph, pw, "
                 "dh, dw, *, relu, residual, out_scale) -> bf16 / int8 NHWC (flashim/ops/conv.py:174-206)")

int8_conv2d_maxpool = Op("int8_conv2d_maxpool", doc="(x, weight, a_scale, w_scale, bias, kh, kw, sh, sw, ph, pw, dh, dw, *, relu, "
                         "out_scale) -> (bf16 [B, Ho, Wo, Cout], int8 [B, Ho/2, Wo/2, Cout]): int8_conv2d and its 2x2 max "
                         "pool quantised with out_scale (flashim/ops/conv.py:209-222)")

romav2_refiner_input = Op("romav2_refiner_input", doc="(f_a, f_b [B, h, w, P] fp32, warp [B, h, w, 2], emb_weight [E, 2(, 1, 1)], "
                          "emb_bias [E], scale_factor [2], radius, pair=0) -> bf16 channels-last [B, 2P + E + K, h, w]: "
                          "[f_a, f_b at the warp, displacement embedding, local correlation] (flashim/ops/romav2.py:36-66)")
romav2_refiner_heads = Op("romav2_refiner_heads", doc="(z [B, C, h, w] channels-last, weight [6, C], bias [6], prev_warp "
                          "[B, h, w, 2], prev_confidence [B, h, w, 1 or 4], refine_init) -> (warp fp32 [B, h, w, 2], confidence "
                          "fp32 [B, h, w, 4]): warp / confidence 1x1 heads, warp update and precision parameters "
                          "(flashim/ops/romav2.py:95-120)")

mxfp8_scaled_mm = Op("mxfp8_scaled_mm", doc="(a E4M3 [M, K], b_t E4M3 [K, N] (the transpose of a row-major [N, K]), a_scale, "
                     "b_scale swizzled E8M0, bias=None) -> bf16 [M, N]: the block-scaled GEMM the pointwise composites end "
                     "in (flashim/ops/gemm.py:40-52)")
int8_linear = Op("int8_linear", doc="(a int8 [M, K], weight int8 [N, K], a_scale, w_scale, bias, *, relu, gelu, residual) -> "
                 "bf16 [M, N] (flashim/ops/gemm.py:82-98)")

mxfp8_linear = Op("mxfp8_linear", doc="(activation QuantizedTensor [rows, K], bias [N] or None, weight QuantizedWeight [N, K]) -> "
                  "bf16 [rows, N]: static MXFP8 linear (flashim/ops/gemm.py:58-72)")
gelu_quantize = Op("gelu_quantize", doc="(value bf16 [..., C], scale_exponent, approximate='none', *, input_bias=None) -> "
                   "QuantizedTensor: quantize_static(GELU(value [+ input_bias])) (flashim/ops/quantize.py:62-74)")
mxfp8_gelu_mlp = Op("mxfp8_gelu_mlp", doc="(x QuantizedTensor, w1 QuantizedWeight, b1, hidden_exponent, w2 QuantizedWeight) -> bf16 "
                    "[rows, N2]: linear, GELU(+ b1), static requantisation, linear (flashim/ops/gemm.py:146-157)")
depthwise5x5_relu_pointwise = Op("depthwise5x5_relu_pointwise", doc="(value [B, C, H, W], dw_weight bf16 [25, C], dw_bias [C], pw_weight "
                                 "bf16 [N, C], pw_bias bf16 [N]) -> bf16 channels-last [B, N, H, W]: the bf16 refiner block "
                                 "(flashim/ops/conv.py:67-87)")
depthwise5x5_relu_pointwise_mxfp8 = Op("depthwise5x5_relu_pointwise_mxfp8", doc="(value, dw_weight, dw_bias, pw_weight E4M3 [N, K], "
                                       "pw_scale_swizzled, pw_scale_u8, pw_bias) -> bf16 [B, N, H, W]: depthwise5x5_relu_mxfp8 then "
                                       "mxfp8_scaled_mm (flashim/ops/conv.py:93-113)")
depthwise5x5_relu_pointwise_int8 = Op("depthwise5x5_relu_pointwise_int8", doc="(value, dw_weight, dw_bias, pw_weight int8 [N, K], "
                                      "pw_wscale, pw_bias, scale) -> bf16 [B, N, H, W]: depthwise5x5_relu_int8 then int8_linear "
                                      "(flashim/ops/conv.py:119-138)")

# -- extensions --------------------------------------------------------------------------------------------------------
quantize_mxfp8_dynamic = Op("quantize_mxfp8_dynamic", doc="(value [..., C]) -> (E4M3 [..., C], swizzled E8M0 bytes): "
                            "per-(row, 32) dynamic MXFP8, the quantiser of flashim/quant/formats/mx.py:50-60 as an op")
depthwise5x5_act = Op("depthwise5x5_act", doc="(value, weight, bias, act='gelu') -> bf16 [B, H, W, C]: depthwise + bias + "
                      "activation with a dense output")
depthwise5x5_act_mxfp8 = Op("depthwise5x5_act_mxfp8", doc="(value, weight, bias, act='gelu') -> (E4M3 [B*H*W, C], swizzled "
                            "E8M0): depthwise5x5_relu_mxfp8 with a selectable activation")
mxfp8_conv2d_fused = Op("mxfp8_conv2d_fused", doc="(x, act_scale, weight, weight_scales, bias, kh, kw, sh, sw, ph, pw, dh, "
                        "dw, *, act, residual, out_exponent, dynamic_out, out_fp32): mxfp8_conv2d with per-pixel activation "
                        "scales (act_scale uint8 swizzled) or static ones (int8 [Cin/32]), pre-swizzled weight scales, and "
                        "the GELU / dynamic-requant / fp32 epilogues")
mxfp8_conv2d_bf16 = Op("mxfp8_conv2d_bf16", doc="(x bf16 [B, H, W, Cin], act_exponent int8 [Cin/32] | None, weight, weight_scales, "
                       "bias, *, act, residual, out_exponent, dynamic_out, out_fp32): a 1x1 mxfp8_conv2d_fused whose "
                       "activation quantiser (static exponents, or per pixel and 32 channels when act_exponent is None) "
                       "runs inside the conv kernel; the same bits as quantising first")
mxfp8_gelu_mlp_residual = Op("mxfp8_gelu_mlp_residual", doc="(x E4M3 [..., C], x_scales uint8 swizzled, w1 E4M3 [2C, C], w1_scales, b1, "
                             "w2 E4M3 [C, 2C], w2_scales, b2, residual bf16 [..., C]) -> bf16 [..., C]: the residual MLP of a refiner "
                             "block (1x1 up conv + GELU + per-pixel requantisation, 1x1 down conv + residual) in one launch, "
                             "the hidden tensor staying on chip; C = 128 or 256; the same bits as the two convs")
int8_conv2d_accumulators = Op("int8_conv2d_accumulators", doc="(x, weight, kh, kw, sh, sw, ph, pw, dh, dw) -> int32 "
                              "[B, Ho, Wo, Cout]: the raw sums of int8_conv2d")

from flashim_b200.backends import load as _load_backends  # noqa: E402

_load_backends()
