/* C ABI of libflashim_sm100.so: hand-written sm_100a (B200) kernels for FlashIM's quantized convolution path.
 *
 * Conventions, the same as FlashIM's own JIT CUDA backend (flashim/backends/cuda/csrc/conv.cu:218-234,
 * flashim/backends/cuda/csrc/depthwise.cu:405-427; Python side flashim/backends/cuda/conv.py:39-47,119-128):
 *   - plain device pointers, ints and `long long` strides only; no framework types;
 *   - the caller allocates every input and output; the library keeps no buffer of its own;
 *   - `stream` is a cudaStream_t passed as void*; every call is asynchronous on it;
 *   - return value: 0 = launched; a positive value is a cudaError_t; FIM_ERR_* (negative) are argument errors
 *     detected before any launch; FIM_ERR_UNSUPPORTED (99) = a geometry this build has no kernel for.
 *   - activations are NHWC (`[B, H, W, C]`, C contiguous), which is the memory of a channels-last `[B, C, H, W]`
 *     tensor; quantized weights are `[Cout, kh*kw*Cin]` in (ky, kx, c) order as FlashIM packs them
 *     (flashim/quant/methods/conv2d.py:91-100,193-205).
 *   - `status` (may be NULL) points to one zero-initialised int32 in device-accessible memory. Kernels that wait on
 *     barriers bound every wait (2 s); a CTA whose wait runs out stores an FIM_STATUS_* code there (first writer wins),
 *     abandons its tile and exits cleanly. A non-zero word after synchronisation means the output is invalid.
 */
#ifndef FLASHIM_SM100_H_
#define FLASHIM_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FIM_ABI_VERSION 1

#define FIM_ERR_LAYOUT (-1)
#define FIM_ERR_ARGUMENT (-2)
#define FIM_ERR_DRIVER (-3)
#define FIM_ERR_UNSUPPORTED 99

#define FIM_DTYPE_F32 0
#define FIM_DTYPE_BF16 1

#define FIM_ACT_NONE 0
#define FIM_ACT_RELU 1
#define FIM_ACT_GELU 2
#define FIM_ACT_RELU_EARLY 3 /* conv epilogues: ReLU before the residual add (the order of flashim/ops/gemm.py:87-98) */

/* What the conv epilogue writes. */
#define FIM_OUT_BF16 0         /* bf16 [B,Ho,Wo,Cout] */
#define FIM_OUT_F32 1          /* fp32, before the bf16 rounding (MXFP8 only) */
#define FIM_OUT_E4M3_STATIC 2  /* E4M3, static exponents `out_exponent[Cout/32]` applied to the bf16 result */
#define FIM_OUT_E4M3_DYNAMIC 3 /* E4M3 + one E8M0 byte per (pixel, 32 channels) of the bf16 result */
#define FIM_OUT_INT8 4         /* int8, static scale `out_scale` applied to the bf16 result (INT8 only) */
#define FIM_OUT_INT32 5        /* raw int32 accumulators (INT8 only) */

#define FIM_STATUS_WAIT_FULL 0x101
#define FIM_STATUS_WAIT_EMPTY 0x102
#define FIM_STATUS_WAIT_TMEM_FULL 0x103
#define FIM_STATUS_WAIT_TMEM_EMPTY 0x104
#define FIM_STATUS_WAIT_ROWS 0x105

/* ABI version of the loaded library (FIM_ABI_VERSION at build time). */
int fim_abi_version(void);

/* ---- standalone quantisers ------------------------------------------------------------------------------------- */

/* Static block-32 MXFP8: out[r, c] = e4m3(sat(value[r, c] / 2**exponent[c / 32])), channels zero-padded to a multiple
 * of 32 in `out` ([rows, ceil32(channels)], 16-byte aligned). `value` is contiguous [rows, channels] of `dtype`.
 * Replaces: ops.quantize_mxfp8 (flashim/ops/quantize.py:80-87; oracle flashim/quant/tensor.py:97-121). */
int fim_quantize_mxfp8_static(const void* value, int dtype, const int8_t* exponent, void* out, long long rows,
                              int channels, void* stream);

/* Dynamic block-32 MXFP8 per (row, 32 channels): e = clamp(ceil(log2(amax / 448))) evaluated in fp32 (-127 for a zero
 * block), out = e4m3(sat(value * 2**-e)); the E8M0 byte e + 127 is stored at [row, group] (`swizzled` == 0) or in the
 * 128-row x 4-group swizzled layout the block-scaled GEMM reads (`swizzled` != 0; the caller zero-fills padding).
 * Replaces: quantize_dynamic_2d + swizzle_scales (flashim/quant/formats/mx.py:50-86). */
int fim_quantize_mxfp8_dynamic(const void* value, int dtype, void* out, void* scales, int swizzled, long long rows,
                               int channels, void* stream);

/* Static per-tensor INT8: out = sat127(round_half_even(value / *scale)), true division.
 * Replaces: ops.quantize_int8 without channel_scale (flashim/ops/quantize.py:93-100; oracle
 * flashim/quant/formats/int8.py:24-26). */
int fim_quantize_int8_static(const void* value, int dtype, const float* scale, void* out, long long count, void* stream);

/* The two static quantisers reading the channels-last view of an NCHW-contiguous tensor: `value` is [batch, channels,
 * pixels] in memory (pixels = H * W), `out` the packed NHWC codes [batch, pixels, ceil32(channels)] (MXFP8, padding
 * channels zero) or [batch, pixels, channels] (INT8, channels % 16 == 0), 16-byte aligned. Bytes equal those of the
 * row-major entry points on `value.permute(0, 2, 1)`.
 * Replaces: the channels-first branch of ops.quantize_mxfp8 / ops.quantize_int8
 * (flashim/backends/triton/quantize.py:217-246, 325-353). */
int fim_quantize_mxfp8_static_nchw(const void* value, int dtype, const int8_t* exponent, void* out, int batch, int channels,
                                   long long pixels, void* stream);
int fim_quantize_int8_static_nchw(const void* value, int dtype, const float* scale, void* out, int batch, int channels,
                                  long long pixels, void* stream);

/* out[b, y, x, c] = int8(max over the 2x2 window of value[b, 2y.., 2x.., c] / *scale): MaxPool2d(2) of a bf16 NHWC tensor
 * (16-byte aligned, channels % 8 == 0) and the static INT8 quantiser in one pass; `out` is int8 [batch, height / 2,
 * width / 2, channels], 8-byte aligned; a trailing odd row / column is dropped.
 * Replaces: the pooled output of ops.int8_conv2d_maxpool (flashim/ops/conv.py:209-222). */
int fim_maxpool2_quantize_int8(const void* value, const float* scale, void* out, int batch, int height, int width, int channels,
                               void* stream);

/* out = e4m3(sat(bf16(GELU(float(value) + input_bias)) / 2**exponent[c / 32])): erf-form GELU of a bf16 matrix
 * `[rows, channels]` (channels % 32 == 0, 16-byte aligned) plus an optional fp32 per-channel bias (NULL: none), rounded
 * to bf16 and quantised with static block-32 exponents.
 * Replaces: ops.gelu_quantize with approximate = "none" (flashim/ops/quantize.py:62-74), the middle step of
 * ops.mxfp8_gelu_mlp (flashim/ops/gemm.py:146-157). */
int fim_gelu_quantize_mxfp8(const void* value, const float* input_bias, const int8_t* exponent, void* out, long long rows,
                            int channels, void* stream);

/* ---- RoMaV2 refiner heads -------------------------------------------------------------------------------------- */

/* The 1x1 convolution of the refiner's last feature map to 2 displacement + 4 precision channels and what follows it:
 *   out[o] = sum_c z[row, c] * weight[o, c] + bias[o]            (fp32, o = 0..5)
 *   warp[row] = prev_warp[row] + (out[0] * inv_norm_x, out[1] * inv_norm_y)
 *   l00 = softplus(out[3]) + 1e-6, l10 = out[4], l11 = softplus(out[5]) + 1e-6
 *   confidence[row] = prev_confidence[row] (zero-padded to 4) + (out[2], l00^2, l00 * l10, l10^2 + l11^2)
 * `z` bf16 [rows, channels] (the NHWC memory of a channels-last tensor, 16-byte aligned, channels % 8 == 0, <= 512),
 * `weight` fp32 [6, channels], `bias` fp32 [6], `prev_warp` / `warp` fp32 [rows, 2], `prev_confidence` fp32
 * [rows, prev_channels] with prev_channels 1 or 4, `confidence` fp32 [rows, 4]; inv_norm = 1 / (refine_init * (w, h)).
 * Replaces: ops.romav2_refiner_heads (flashim/ops/romav2.py:95-120), Triton `_refiner_heads_kernel`
 * (flashim/backends/triton/romav2.py:202-250). */
int fim_romav2_refiner_heads(const void* z, const float* weight, const float* bias, const float* prev_warp,
                             const float* prev_confidence, int prev_channels, float* warp, float* confidence, long long rows,
                             int channels, float inv_norm_x, float inv_norm_y, void* stream);

/* The refiner's input row per pixel of A, bf16 [batch, height, width, 2 * features + embedding + K] (the NHWC memory of a
 * channels-last tensor), K = (2 * radius + 1)^2 or 0 for radius < 0:
 *   [0, P)            f_a
 *   [P, 2P)           f_b sampled bilinearly at warp (x, y in [-1, 1], align_corners = False, zeros outside)
 *   [2P, 2P + E)      emb_weight[e, 0] * scale_x * dx + emb_weight[e, 1] * scale_y * dy + emb_bias[e], (dx, dy) = warp - the
 *                     pixel's own normalised coordinates
 *   [2P + E, .. + K)  sum_c f_a[c] / sqrt(P) * f_b sampled at warp + ((kx - r) * 2 / width, (ky - r) * 2 / height), k = ky * (2r + 1) + kx
 * `f_a`, `f_b` fp32 [batch, height, width, features] (16-byte aligned, features % 4 == 0, <= 256), `warp` fp32 [.., 2],
 * `emb_weight` fp32 [embedding, 2], `emb_bias` fp32 [embedding], radius <= 3. pair > 0: batch == 2 * pair and image i is
 * matched with image (i + pair) % batch of `f_a` (`f_b` is ignored).
 * Replaces: ops.romav2_refiner_input (flashim/ops/romav2.py:36-66), Triton `refiner_input`
 * (flashim/backends/triton/romav2.py). */
int fim_romav2_refiner_input(const float* f_a, const float* f_b, const float* warp, const float* emb_weight, const float* emb_bias,
                             float scale_x, float scale_y, void* out, int batch, int height, int width, int features,
                             int embedding, int radius, int pair, void* stream);

/* ---- depthwise 5x5 (pad 2, stride 1) -------------------------------------------------------------------------- */

/* out[b,y,x,c] = act(sum_{ky,kx} value[b,y+ky-2,x+kx-2,c] * weight[ky*5+kx, c] + bias[c]) with fp32 accumulation
 * over bf16 inputs, written as bf16 NHWC. `value` bf16 NHWC, `weight` bf16 [25, C] (tap-major), `bias` fp32 [C].
 * C must be a multiple of 32. Extension of the reference's depthwise producers (which always end in a quantiser):
 * same operands and arithmetic as flashim/ops/conv.py:30-41. */
int fim_dw5x5_bf16(const void* value, const void* weight, const float* bias, void* out, int batch, int height, int width,
                   int channels, int act, int* status, void* stream);

/* Depthwise + bias + act, the fp32 result quantised per (pixel, 32 channels) to MXFP8 without an intermediate bf16
 * rounding: E4M3 [B*H*W, C] and E8M0 bytes (swizzled != 0: 128x4 swizzled layout; else [B*H*W, C/32]).
 * With act = FIM_ACT_RELU and swizzled = 1 this replaces ops.depthwise5x5_relu_mxfp8 (flashim/ops/conv.py:30-44;
 * kernel flashim/backends/triton/conv.py:47-130). */
int fim_dw5x5_mxfp8(const void* value, const void* weight, const float* bias, void* out, void* scales, int swizzled,
                    int batch, int height, int width, int channels, int act, int* status, void* stream);

/* Depthwise + bias + ReLU rounded to bf16, then static INT8 with *scale (true division): int8 [B*H*W, C].
 * Replaces ops.depthwise5x5_relu_int8 (flashim/ops/conv.py:50-61; C ABI flashim/backends/cuda/csrc/depthwise.cu:407-412). */
int fim_dw5x5_relu_int8(const void* value, const void* weight, const float* bias, const float* scale, void* out, int batch,
                        int height, int width, int channels, int* status, void* stream);

/* ---- implicit-GEMM conv2d on tcgen05 tensor cores ----------------------------------------------------------- */

typedef struct FimConvGeometry {
  int batch, height, width, cin, cout; /* cin, cout: physical (padded) channel counts, multiples of 32 (BF16: cin % 16) */
  int kh, kw, stride_h, stride_w, pad_h, pad_w, dil_h, dil_w;
} FimConvGeometry;

typedef struct FimConvEpilogue {
  const void* bias;          /* bf16 [cout] or NULL */
  const void* residual;      /* bf16, addressed with the four element strides below, or NULL */
  long long res_stride[4];   /* batch, row, column, channel */
  int res_channels;          /* channels present in `residual` (<= cout) */
  int act;                   /* FIM_ACT_*: GELU is applied before the residual add, ReLU after it */
  int out_mode;              /* FIM_OUT_* */
  const int8_t* out_exponent;/* FIM_OUT_E4M3_STATIC: int8 [cout/32] */
  void* out_scales;          /* FIM_OUT_E4M3_DYNAMIC: E8M0 bytes, swizzled 128x4 layout over rows = B*Ho*Wo */
  const float* out_scale;    /* FIM_OUT_INT8: one fp32 */
} FimConvEpilogue;

/* Block-scaled MXFP8 conv: x E4M3 NHWC; activation scales either static (`act_exponent` int8 [cin/32], shared by every
 * pixel and tap) or per pixel (`act_scales_swizzled`: E8M0 bytes in the 128x4 swizzled layout over rows = B*H*W; 1x1
 * stride-1 unpadded convs only). Strides 1 to 4 are supported (a strided conv reads every stride-th pixel through the
 * tensor map's element strides); weight E4M3 [cout, kh*kw*cin]; `weight_scales_swizzled`: E8M0 bytes of the
 * [cout, kh*kw*cin/32] exponents in the 128x4 swizzled layout. fp32 accumulation in tensor memory, epilogue
 * bias -> bf16 rounding -> GELU -> residual add (one more bf16 rounding) -> ReLU -> requantisation, as `epilogue` selects:
 * GELU acts before the residual is added, ReLU after it (relu(out + residual), flashim/ops/conv.py:198-203).
 * Replaces ops.mxfp8_conv2d (flashim/ops/conv.py:309-342; kernel flashim/backends/triton/conv.py:1122-1192) and, with
 * per-pixel scales, ops.mxfp8_scaled_mm (flashim/ops/gemm.py:40-52). */
int fim_mxfp8_conv2d(const void* x, const int8_t* act_exponent, const void* act_scales_swizzled, const void* weight,
                     const void* weight_scales_swizzled, const FimConvGeometry* geometry, const FimConvEpilogue* epilogue,
                     void* out, int* status, void* stream);

/* The same conv on bf16 activations, with the activation quantiser inside the kernel (1x1, stride 1, unpadded,
 * cin % 128 == 0 only; anything else returns FIM_ERR_UNSUPPORTED and the caller quantises first): converter warps turn
 * each bf16 tile into E4M3 on its way to the MMAs, with the static exponents `act_exponent` (int8 [cin/32]) or, when that
 * is NULL, with one exponent per pixel and 32 channels formed on the fly. The result equals fim_quantize_mxfp8_static /
 * fim_quantize_mxfp8_dynamic followed by fim_mxfp8_conv2d bit for bit. Replaces the quantize_mxfp8 + mxfp8_conv2d pair of
 * StaticMXFP8Conv2d.forward (flashim/quant/methods/conv2d.py:217-251) for such layers. */
int fim_mxfp8_conv2d_bf16(const void* x_bf16, const int8_t* act_exponent, const void* weight, const void* weight_scales_swizzled,
                          const FimConvGeometry* geometry, const FimConvEpilogue* epilogue, void* out, int* status, void* stream);

/* INT8 conv: x int8 NHWC, weight int8 [cout, kh*kw*cin]; exact int32 accumulation in tensor memory; epilogue
 * float(acc) * (*a_scale * w_scale[n]) + bias (separately rounded), ReLU, bf16, residual, optional INT8 requantisation.
 * Replaces ops.int8_conv2d (flashim/ops/conv.py:174-206; kernel flashim/backends/triton/conv.py:702-805). */
int fim_int8_conv2d(const void* x, const void* weight, const float* a_scale, const float* w_scale,
                    const FimConvGeometry* geometry, const FimConvEpilogue* epilogue, void* out, int* status, void* stream);

/* fim_int8_conv2d (FIM_OUT_BF16 only) whose epilogue also writes the second output of ops.int8_conv2d_maxpool: `pooled`,
 * int8 [B, Ho / 2, Wo / 2, cout], the 2x2 / stride-2 max pool of the bf16 output quantised with `epilogue->out_scale`
 * (a trailing odd row or column is dropped, as F.max_pool2d does). The pool is taken from the bf16 tile while it lies in
 * shared memory for its own store: the output is not read back. Ho, Wo >= 2 and cin % 64 == 0, else
 * FIM_ERR_UNSUPPORTED (the caller then runs fim_int8_conv2d and fim_maxpool2_quantize_int8). Replaces
 * ops.int8_conv2d_maxpool (flashim/ops/conv.py:209-222; the POOL epilogue of flashim/backends/triton/conv.py:798-805). */
int fim_int8_conv2d_maxpool(const void* x, const void* weight, const float* a_scale, const float* w_scale,
                            const FimConvGeometry* geometry, const FimConvEpilogue* epilogue, void* out, void* pooled, int* status,
                            void* stream);

/* BF16 conv: x bf16 NHWC, weight bf16 [cout, kh*kw*cin] in (ky, kx, c) order, fp32 accumulation on the tensor cores
 * (kind::f16), epilogue bias -> bf16 (FIM_OUT_BF16) or fp32 (FIM_OUT_F32), activation and residual as above. The
 * pointwise product of ops.depthwise5x5_relu_pointwise (flashim/ops/conv.py:67-87; kernel
 * flashim/backends/cuda/csrc/depthwise.cu:165-401) runs through this entry point as a 1x1 conv. */
int fim_bf16_conv2d(const void* x, const void* weight, const FimConvGeometry* geometry, const FimConvEpilogue* epilogue, void* out,
                    int* status, void* stream);

/* The residual MLP of a refiner block in one launch: out = (quantise(GELU(x W1^T + b1)) W2^T + b2) + residual over `rows`
 * pixels of `channels` (128 or 256, else FIM_ERR_UNSUPPORTED) channels. x: E4M3 [rows, C] with per-pixel scales
 * (`x_scales_swizzled`, E8M0 bytes in the 128x4 swizzled layout over rows, as the depthwise producer writes them); w1 E4M3
 * [2C, C], w2 E4M3 [C, 2C], their scales swizzled; b1 bf16 [2C], b2 bf16 [C]; residual and out bf16 [rows, C], dense. The
 * hidden activations (bias -> bf16 -> GELU -> one E8M0 exponent per pixel and 32 channels -> E4M3) stay in shared memory
 * as the operand of the second product. Bit-identical to fim_mxfp8_conv2d with FIM_ACT_GELU + FIM_OUT_E4M3_DYNAMIC
 * followed by fim_mxfp8_conv2d with a residual. The counterpart in the reference keeps the hidden tile on chip the same
 * way: _mxfp8_gelu_mlp_kernel (flashim/backends/triton/gemm.py:558-613, op flashim/ops/gemm.py:146-157), there with
 * static scales and without the residual. */
int fim_mxfp8_gelu_mlp_residual(const void* x, const void* x_scales_swizzled, const void* w1, const void* w1_scales_swizzled,
                                const void* bias1, const void* w2, const void* w2_scales_swizzled, const void* bias2,
                                const void* residual, void* out, long long rows, int channels, int* status, void* stream);

/* Tile configuration the conv entry points would use for a geometry (for reports and tests): writes
 * {tile_rows, tile_cols, block_n, block_k, stages, ctas}. Returns 0 or FIM_ERR_UNSUPPORTED. */
int fim_conv_plan(const FimConvGeometry* geometry, int int8, int per_pixel_scales, int plan[6]);

/* The work list of the persistent CTAs for a geometry (for reports and tests): writes {tiles, full_width_tiles,
 * tiles_after_the_tail_split, ctas, cta_pairs (0 / 1), resident_k_iterations, channel_tile_major_order (0 / 1),
 * accumulator_buffers}. The last partial round of tiles runs as half-width tiles when at most half of the CTAs would
 * otherwise have work in it: then tiles_after_the_tail_split > tiles. Returns 0 or FIM_ERR_UNSUPPORTED. */
int fim_conv_schedule(const FimConvGeometry* geometry, int int8, int per_pixel_scales, int schedule[8]);

#ifdef __cplusplus
}
#endif
#endif /* FLASHIM_SM100_H_ */
