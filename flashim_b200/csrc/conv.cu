// Implicit-GEMM conv2d (NHWC, stride 1) on the tcgen05 tensor cores of sm_100a: block-scaled MXFP8
// (kind::mxf8f6f4, E8M0 scale per 32 along K) and INT8 (kind::i8, int32 accumulation).
//
// One persistent CTA per SM walks output tiles of 128 pixels (a tile_h x tile_w patch of one image) x BN output
// channels. Warp 0 is the TMA producer: per (tap, channel chunk) it loads the shifted activation patch (a 4-D box whose
// out-of-image part TMA fills with zeros: the conv padding, no im2col buffer) and the weight tile into a ring of
// swizzled K-major stages, plus the 512-byte scale tiles. Warp 1 issues tcgen05.mma from one lane, accumulating in
// tensor memory; scale tiles go shared memory -> tensor memory with tcgen05.cp in front of the MMAs that use them, into
// the stage's own column set, so a copy never waits for the MMAs of another stage. Warps 2-17 are the epilogue: four
// column groups of four warps, one per 32-lane quarter of tensor memory. They tcgen05.ld 32 columns at a time, add the
// bias, round to bf16x2 words and hand the accumulator back at once; activation / residual / requantisation then run on
// packed pairs in registers, the 32-column panel of the tile goes to swizzled shared memory and on to a TMA store,
// which clips the ragged image edge. Accumulators are double-buffered in tensor memory when two of them fit, so the
// epilogue of tile i overlaps the main loop of tile i + 1. The producer and MMA loops keep stage addresses, descriptors
// and phase bits in registers: a single lane issues them and every instruction there is on the critical path of the
// tensor pipe.
//
// Rounding points follow FlashIM's torch reference: flashim/ops/conv.py:174-206,309-342 and flashim/ops/gemm.py:58-98.
#include <cstdio>

#include "common.cuh"
#include "flashim_sm100.h"
#include "flashim_sm100_tune.h"

namespace fim {
namespace {

constexpr int kThreads = 576;  // producer warp, MMA warp, 16 epilogue warps
// A layer that takes bf16 activations adds eight converter warps, which quantise each 128 x 128 tile on its way from the
// TMA landing ring into the K-major stage the MMAs read (four warps measured 10 to 18 % slower: the quantiser arithmetic
// of a tile, not its bytes, is what such a layer waits for).
constexpr int kConverterWarps = 8, kConvertThreads = kThreads + 32 * kConverterWarps;
constexpr int kRawStages = 2;                       // landing ring of bf16 tiles
constexpr uint32_t kRawBytes = 128u * 128u * 2u;    // 128 pixels x 128 channels of bf16
constexpr int kTileM = 128;
constexpr uint32_t kTmemColumns = 512;
constexpr int kMaxStages = 12;  // a short K loop is bound by the latency of a stage's round trip: more stages in flight
constexpr int kSmemLimit = 226 * 1024;

// Division of a tile index by a run-time constant without the integer-division sequence (some forty instructions, which a
// warp that owns 32 columns of a tile would pay several times per tile): q = floor(x * floor(2**32 / d) / 2**32) is the
// quotient or one below it for every x < 2**32, so one compare-and-step finishes it. `magic` = floor(2**32 / d), or
// 2**32 - 1 for d = 1 (which the same two steps turn into x).
struct FastDiv {
  uint32_t divisor, magic;
};
__host__ inline FastDiv make_fastdiv(int divisor) {
  FastDiv f;
  f.divisor = static_cast<uint32_t>(divisor < 1 ? 1 : divisor);
  f.magic = f.divisor == 1 ? 0xFFFFFFFFu : static_cast<uint32_t>((1ull << 32) / f.divisor);
  return f;
}
__device__ __forceinline__ void divmod(int x, const FastDiv& f, int& quotient, int& remainder) {
  uint32_t q = __umulhi(static_cast<uint32_t>(x), f.magic);
  uint32_t r = static_cast<uint32_t>(x) - q * f.divisor;
  if (r >= f.divisor) ++q, r -= f.divisor;
  quotient = static_cast<int>(q), remainder = static_cast<int>(r);
}

struct ConvParams {
  int cin, cout, out_h, out_w;
  int kh, kw, pad_h, pad_w, dil_h, dil_w, stride_h, stride_w;
  int tile_h, tile_w, tiles_x, tiles_y, tiles_n, total_tiles;
  int row_tiles;   // row tiles (of a CTA pair: pairs of them) per output-channel tile
  FastDiv div_row_tiles, div_tiles_n, div_tiles_x, div_tiles_y;  // the same counts prepared for divmod()
  int n_major;     // tile order: 1 = all row tiles of an output-channel tile before the next (keeps weight scales resident)
  int batch;       // images (rows of a flattened 1x1 conv count as one)
  int full_tiles;  // tiles [0, full_tiles) are BN wide; the rest are the halves (BN / 2 columns) of the last few tiles
  int k_chunks, stages;
  int resident_k;  // weight-scale tiles of the first resident_k K iterations stay in tensor memory from tile to tile
  int panels_per_half;  // output panels each column group of the epilogue rotates through (1 or 2)
  // scales (MXFP8)
  const int8_t* act_exponent;     // static: [cin / 32]
  const uint8_t* act_scales;      // per pixel: swizzled tiles over rows = pixels
  int act_scale_tiles;            // 4-group tiles per row tile in act_scales
  const uint8_t* weight_scales;   // swizzled tiles over rows = cout
  int weight_scale_tiles, weight_row_tiles;
  // INT8
  const float* a_scale;
  const float* w_scale;
  // epilogue
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long res_stride[4];
  int res_channels, act, out_mode, out_elem;  // out_elem: bytes per output element
  const int8_t* out_exponent;
  uint8_t* out_scales;
  const float* out_scale;
  int* status;
  uint32_t poll_backoff_ns;  // sleep between polls of the epilogue's wait for an accumulator
  int b_slots;               // weight (and weight-scale) tiles held in shared memory: `stages`, or every K step of a tile (resident)
  int weights_resident;      // 1: the layer's whole weight matrix is loaded once per CTA and stays in shared memory
  int convert_static;        // bf16 activations: 1 = quantise with act_exponent, 0 = per pixel and 32 channels on the fly
  int warp_panels;           // flat 1x1 convs: every epilogue warp stages and stores its own 32 rows (no barrier between warps)
  int pool;                  // INT8, bf16 output: the 2x2 max pool of the output also leaves the epilogue, as INT8 codes (out_scale)
  int debug;  // probe builds only (FIM_PROBE_BUILD): 1 = no activation loads, 2 = no weight loads, 4 = no output stores, 8 = no scale copies
};

// Measurement switches that make results invalid exist only in a build with -DFIM_PROBE_BUILD=1; the shipped kernels carry
// no test of them.
#ifndef FIM_PROBE_BUILD
#define FIM_PROBE_BUILD 0
#endif
__device__ __forceinline__ int probe_flags(const ConvParams& p) { return FIM_PROBE_BUILD ? p.debug : 0; }

struct SharedControl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t weights_ready;          // resident weights: their one-time copies have landed
  uint64_t raw_full[kRawStages];   // bf16 landing ring of a converting layer
  uint64_t raw_empty[kRawStages];
  uint32_t tmem_base;
  int abort_flag;
  int group_go[4][2];  // epilogue: did the accumulator of tile (parity) arrive? One decision per column group
};

constexpr int kMaxStaticScaleTiles = 16;  // input channels / 128 whose activation scales stay resident in tensor memory
__host__ __device__ constexpr int acc_stages(int bn) {
  return 2 * bn + 4 * kMaxStaticScaleTiles + kMaxStages * (bn < 128 ? 4 : bn / 32) <= 512 ? 2 : 1;
}
__host__ __device__ constexpr int scale_tiles_b(int bn) { return bn <= 128 ? 1 : bn / 128; }

__device__ __forceinline__ uint32_t idesc_mxf8(int block_n, int block_m = kTileM) {
  // E4M3 x E4M3 (format 0), both K-major, UE8M0 scales, M = block_m (256 for a CTA pair), N = block_n; scale ids are
  // OR-ed in per MMA
  return (static_cast<uint32_t>(block_n >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(block_m >> 4) << 24);
}
__device__ __forceinline__ uint32_t idesc_i8(int block_n, int block_m = kTileM) {
  // S32 accumulator (2), signed 8-bit A and B (1), both K-major, M = block_m, N = block_n
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(block_n >> 3) << 17) |
         (static_cast<uint32_t>(block_m >> 4) << 24);
}

#include "gelu_table.inc"
constexpr uint32_t kGeluSmemBytes = (kGeluEntries * 4u + 1023u) / 1024u * 1024u;  // keeps the tiles behind it 1024-byte aligned

// GELU of two bf16 values in one word, as bf16: the erf form torch evaluates (x * 0.5 * (1 + erf(x / sqrt 2)) in fp32,
// rounded to bf16), looked up instead of computed. `table` locates the shared-memory copy of kGeluTable: per magnitude a
// 16-bit delta for either sign; result magnitude = max(a + delta, 0), result sign = input sign. Magnitudes below
// kGeluBase share entry 0 (half the value: the exponent drops by one; zero stays zero), those above the table share the
// last entry (x itself for positive values, -0 for negative ones). Exact for every bf16 input except subnormals, which
// become zero. Eleven instructions per pair and no MUFU; the arithmetic form costs about forty.
struct GeluTable {
  uint32_t low2;    // the low 16 bits of the table's shared-memory address, in both halves of the word
  uint32_t window;  // its upper 16 bits: zero for a single CTA; in a cluster the CTA's rank sits up there
};
__device__ __forceinline__ GeluTable gelu_table_at(uint32_t smem_address) {
  GeluTable t;
  t.low2 = (smem_address & 0xFFFFu) * 0x00010001u;
  t.window = smem_address & 0xFFFF0000u;
  return t;
}
__device__ __forceinline__ uint32_t gelu_bf16x2(uint32_t r, const GeluTable& table) {
  constexpr uint32_t kNegBase = ((0x10000u - static_cast<uint32_t>(kGeluBase - 1)) & 0xFFFFu) * 0x00010001u;
  constexpr uint32_t kLast = static_cast<uint32_t>(kGeluEntries - 1) * 0x00010001u;
  const uint32_t a = r & 0x7FFF7FFFu;
  const uint32_t t = __viaddmin_s16x2_relu(a, kNegBase, kLast);  // clamp(a - (base - 1), 0, entries - 1) in each half
  // both entry addresses with one multiply-add: the table sits in the first 64 KB of the CTA's shared window, so the low
  // 16 bits of an address fit a half and neither half carries into the other; a byte permute then puts each half under
  // the window's upper bits
  const uint32_t at = t * 4u + table.low2;
  uint32_t w0, w1, negative;
  asm("ld.shared.b32 %0, [%1];" : "=r"(w0) : "r"(__byte_perm(at, table.window, 0x7610)));
  asm("ld.shared.b32 %0, [%1];" : "=r"(w1) : "r"(__byte_perm(at, table.window, 0x7632)));
  // byte 0 of `negative` = 0xFF when the low value is negative, byte 1 the same for the high value (sign replication of
  // bytes 1 and 3); each byte steers two selector nibbles: bytes 2-3 of w0 / w1 (the delta for negative values) or 0-1
  asm("prmt.b32 %0, %1, %2, 0x00B9;" : "=r"(negative) : "r"(r), "r"(0u));
  const uint32_t delta = __byte_perm(w0, w1, (negative & 0x2222u) | 0x5410u);
  return __viaddmax_s16x2(a, delta, 0u) | (r & 0x80008000u);
}

__device__ __forceinline__ uint32_t idesc_bf16(int block_n, int block_m = kTileM) {
  // F32 accumulator (1), BF16 A and B (1), both K-major, M = block_m, N = block_n (kind::f16)
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(block_n >> 3) << 17) |
         (static_cast<uint32_t>(block_m >> 4) << 24);
}

// What the epilogue does, as template argument EPI of the kernel. 0 = the general epilogue with every switch read from
// ConvParams at run time. kEpiFixed = the same code with the switches below as compile-time constants (bias present, two
// panels per group), which removes the tests, the parameter loads and the register moves at their joins: about a third
// of the epilogue's instructions. kEpiLean = the shorter epilogue of a flat block-scaled 1x1 layer (bias present; bf16
// output, or E4M3 with per-pixel scales when kEpiDynamic; GELU when kEpiGelu; a dense bf16 residual over every output
// channel when kEpiResidual): the layers a refiner block is made of. kEpiPool = the general epilogue of an INT8 conv with
// bf16 output that also writes the 2x2 max pool of its tiles as INT8 codes.
constexpr uint32_t kPoolPanelBytes = 1024;  // 32 pooled pixels x 32 INT8 channels
constexpr int kEpiGelu = 1, kEpiDynamic = 2, kEpiResidual = 4, kEpiLean = 8, kEpiFixed = 16, kEpiStatic = 32, kEpiPool = 64;

struct EpilogueSwitches {
  int act, out_mode;
  uint32_t out_elem, panels;  // bytes per output element; output panels per group
  bool has_bias, has_residual;
};
template <int EPI>
__device__ __forceinline__ EpilogueSwitches epilogue_switches(const ConvParams& p) {
  EpilogueSwitches sw;
  if constexpr ((EPI & kEpiFixed) != 0) {
    sw.act = (EPI & kEpiGelu) ? kActGelu : kActNone;
    sw.out_mode = (EPI & kEpiStatic) ? FIM_OUT_E4M3_STATIC : ((EPI & kEpiDynamic) ? FIM_OUT_E4M3_DYNAMIC : FIM_OUT_BF16);
    sw.out_elem = sw.out_mode == FIM_OUT_BF16 ? 2u : 1u;
    sw.panels = 2u;
    sw.has_bias = true;
    sw.has_residual = (EPI & kEpiResidual) != 0;
  } else {
    sw.act = p.act, sw.out_mode = p.out_mode;
    sw.out_elem = static_cast<uint32_t>(p.out_elem), sw.panels = static_cast<uint32_t>(p.panels_per_half);
    sw.has_bias = p.bias != nullptr, sw.has_residual = p.residual != nullptr;
  }
  return sw;
}

// ---- epilogue arithmetic on 32 consecutive output channels of one pixel ----------------------------------------------
// Fills `w` with the output bytes of the chunk (32 * out_elem bytes, little end first). The block-scaled path works on
// packed pairs throughout: fp32 pairs (one issue slot for two channels) up to the bf16 rounding, bf16x2 words after it
// (residual add, ReLU and the block maximum are single bf16x2 instructions; a bf16 add of two bf16 values rounds once,
// like the reference's fp32 add followed by a bf16 rounding, because the fp32 sum of two 8-bit significands is exact
// whenever it can matter). `bias_at` is the shared-memory address of this chunk's 32 fp32 bias values.
__device__ __forceinline__ void load_bias_pairs(uint32_t bias_at, int i, uint64_t& b0, uint64_t& b1) {
  asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(b0), "=l"(b1) : "r"(bias_at + i * 16));
}

// bf16x2 words r[IN] -> E4M3 codes of value * 2**-e (e in [-127, 127]), four per output word. The scaling is one
// mixed-precision FMA per value (fp32 = bf16 * bf16 + -0, exact: a bf16 times a power of two; the addend -0 keeps the
// sign of a zero product), which reads the halves of the packed word directly and runs at the full fp32 rate; unpacking
// with shifts and masks first costs two half-rate integer instructions per pair.
template <int IN, int WORDS>  // IN bf16x2 words in, IN / 2 words of `w` written
__device__ __forceinline__ void scale_to_e4m3(const uint32_t (&r)[IN], int e, uint32_t (&w)[WORDS]) {
  static_assert(IN % 2 == 0 && WORDS >= IN / 2, "four codes per output word");
  // 2**-e as bf16 bits in both halves; 2**-127 (e = 127) is a bf16 subnormal, which the instruction takes as it is
  const uint32_t inv16 = e == 127 ? 0x0040u : static_cast<uint32_t>(127 - e) << 7;
  const uint32_t inv = inv16 * 0x00010001u;
#pragma unroll
  for (int i = 0; i < IN / 2; ++i) {
    float a, b, c, d;
    asm("{\n\t.reg .b16 xl, xh, yl, yh, s, t;\n\t"
        "mov.b32 {xl, xh}, %4;\n\tmov.b32 {yl, yh}, %5;\n\tmov.b32 {s, t}, %6;\n\t"
        "fma.rn.f32.bf16 %0, xl, s, 0f80000000;\n\tfma.rn.f32.bf16 %1, xh, s, 0f80000000;\n\t"
        "fma.rn.f32.bf16 %2, yl, s, 0f80000000;\n\tfma.rn.f32.bf16 %3, yh, s, 0f80000000;\n\t}"
        : "=f"(a), "=f"(b), "=f"(c), "=f"(d)
        : "r"(r[2 * i]), "r"(r[2 * i + 1]), "r"(inv));
    w[i] = e4m3x4(a, b, c, d);
  }
}

// fp32 value (+ INT8 dequantisation) + bias of one chunk, as 16 packed pairs
template <bool INT8>
__device__ __forceinline__ void biased_chunk(const ConvParams& p, const EpilogueSwitches& sw, const uint32_t (&raw)[32], int n,
                                             uint32_t bias_at, float a_scale, uint64_t (&v2)[16]) {
  if (INT8) {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float4 s = __ldg(reinterpret_cast<const float4*>(p.w_scale + n + i));
      v2[i / 2] = pack2(__fmul_rn(__int2float_rn(static_cast<int>(raw[i])), __fmul_rn(a_scale, s.x)),
                        __fmul_rn(__int2float_rn(static_cast<int>(raw[i + 1])), __fmul_rn(a_scale, s.y)));
      v2[i / 2 + 1] = pack2(__fmul_rn(__int2float_rn(static_cast<int>(raw[i + 2])), __fmul_rn(a_scale, s.z)),
                            __fmul_rn(__int2float_rn(static_cast<int>(raw[i + 3])), __fmul_rn(a_scale, s.w)));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v2[i] = pack2(__uint_as_float(raw[2 * i]), __uint_as_float(raw[2 * i + 1]));
  }
  if (sw.has_bias) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint64_t b0, b1;
      load_bias_pairs(bias_at, i, b0, b1);
      v2[2 * i] = add2(v2[2 * i], b0);
      v2[2 * i + 1] = add2(v2[2 * i + 1], b1);
    }
  }
}

// Four-byte outputs: the int32 accumulators as they are, or the biased fp32 values
template <bool INT8>
__device__ __forceinline__ void wide_chunk(const ConvParams& p, const EpilogueSwitches& sw, const uint32_t (&raw)[32], int n,
                                           uint32_t bias_at, float a_scale, uint32_t (&w)[32]) {
  if (INT8 && sw.out_mode == FIM_OUT_INT32) {
#pragma unroll
    for (int i = 0; i < 32; ++i) w[i] = raw[i];
    return;
  }
  uint64_t v2[16];
  biased_chunk<INT8>(p, sw, raw, n, bias_at, a_scale, v2);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float lo, hi;
    unpack2(v2[i], lo, hi);
    w[2 * i] = __float_as_uint(lo), w[2 * i + 1] = __float_as_uint(hi);
  }
}

// First step of the other outputs: one bf16 rounding of the biased values, 16 bf16x2 words. This step is short, so the
// accumulator can go back to the MMA warp before the long arithmetic starts.
template <bool INT8>
__device__ __forceinline__ void round_chunk(const ConvParams& p, const EpilogueSwitches& sw, const uint32_t (&raw)[32], int n,
                                            uint32_t bias_at, float a_scale, uint32_t (&r)[16]) {
  uint64_t v2[16];
  biased_chunk<INT8>(p, sw, raw, n, bias_at, a_scale, v2);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    float lo, hi;
    unpack2(v2[i], lo, hi);
    r[i] = pack_bf16(lo, hi);
  }
}

// Second step, on the rounded values: activation (ReLU waits for the residual when there is one), residual, and the
// output format.
template <bool INT8>
__device__ __forceinline__ void finish_chunk(const ConvParams& p, const EpilogueSwitches& sw, uint32_t (&r)[16], int n, size_t pixel,
                                             int b, int y, int x, bool valid, const GeluTable& gelu_table, uint32_t (&w)[16]) {
  const bool has_res = sw.has_residual;
  if (sw.act == kActGelu) {
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = gelu_bf16x2(r[i], gelu_table);
  } else if (sw.act == kActReluEarly || (sw.act == kActRelu && !has_res)) {
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = bf16x2_max(r[i], 0u);
  }
  if (has_res) {
    const int limit = p.res_channels - n;  // channels of this chunk present in the residual
    if (valid && limit > 0) {
      const __nv_bfloat16* rp = p.residual + b * p.res_stride[0] + y * p.res_stride[1] + x * p.res_stride[2];
      const bool vec = p.res_stride[3] == 1 && limit >= 32 && ((reinterpret_cast<uintptr_t>(rp + n) & 15u) == 0);
      if (vec) {
        const uint4* r4 = reinterpret_cast<const uint4*>(rp + n);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 q = __ldg(r4 + i);
          r[4 * i] = bf16x2_add(r[4 * i], q.x);
          r[4 * i + 1] = bf16x2_add(r[4 * i + 1], q.y);
          r[4 * i + 2] = bf16x2_add(r[4 * i + 2], q.z);
          r[4 * i + 3] = bf16x2_add(r[4 * i + 3], q.w);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint32_t lo = 2 * i < limit ? __bfloat16_as_ushort(rp[(n + 2 * i) * p.res_stride[3]]) : 0u;
          const uint32_t hi = 2 * i + 1 < limit ? __bfloat16_as_ushort(rp[(n + 2 * i + 1) * p.res_stride[3]]) : 0u;
          r[i] = bf16x2_add(r[i], lo | (hi << 16));
        }
      }
    }
    if (sw.act == kActRelu) {
#pragma unroll
      for (int i = 0; i < 16; ++i) r[i] = bf16x2_max(r[i], 0u);
    }
  }
  if (sw.out_mode == FIM_OUT_BF16) {
#pragma unroll
    for (int i = 0; i < 16; ++i) w[i] = r[i];
    return;
  }
  if (INT8) {  // FIM_OUT_INT8
    const Int8Quantizer quantizer = make_int8_quantizer(__ldg(p.out_scale));
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      w[i] = int8_pack4(quantizer, bf16_lo(r[2 * i]), bf16_hi(r[2 * i]), bf16_lo(r[2 * i + 1]), bf16_hi(r[2 * i + 1]));
    }
    return;
  }
  int e;
  if (sw.out_mode == FIM_OUT_E4M3_STATIC) {
    e = static_cast<int>(__ldg(p.out_exponent + (n >> 5)));
  } else {
    // block maximum of |value| on bf16x2 words: max.xorsign.abs keeps the larger magnitude in both halves (signs are
    // masked off at the end); a bf16 magnitude shifted left by 16 is the same number in fp32
    uint32_t m[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = bf16x2_absmax(r[2 * i], r[2 * i + 1]);
#pragma unroll
    for (int i = 0; i < 4; ++i) m[i] = bf16x2_absmax(m[2 * i], m[2 * i + 1]);
    m[0] = bf16x2_absmax(bf16x2_absmax(m[0], m[1]), bf16x2_absmax(m[2], m[3]));
    const uint32_t top = max(m[0] & 0x7FFFu, (m[0] >> 16) & 0x7FFFu);
    e = e8m0_exponent_bits(top << 16);
    if (valid) {
      const int groups = p.cout >> 5;
      p.out_scales[swizzled_scale_offset(pixel, n >> 5, (groups + 3) >> 2)] = static_cast<uint8_t>(e + 127);
    }
  }
  scale_to_e4m3(r, e, w);
}

// Write this row's 32 * elem bytes of a panel into swizzled shared memory (the layout a TMA store with swizzle mode
// 32 * elem bytes reads): 16-byte slot i of row r lands in slot i ^ ((r * pitch / 128) mod slots).
template <int WORDS>
__device__ __forceinline__ void stage_row(uint32_t panel, int row, int elem, const uint32_t (&w)[WORDS]) {
  const uint32_t pitch = 32u * elem;           // 32, 64 or 128 bytes
  const uint32_t slots = pitch >> 4;           // 2, 4 or 8
  const uint32_t phase = ((static_cast<uint32_t>(row) * pitch) >> 7) & (slots - 1);
  const uint32_t base = panel + row * pitch;
#pragma unroll
  for (uint32_t i = 0; i < WORDS / 4; ++i) {
    if (i < slots) {
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(base + ((i ^ phase) << 4)), "r"(w[4 * i]), "r"(w[4 * i + 1]),
                   "r"(w[4 * i + 2]), "r"(w[4 * i + 3])
                   : "memory");
    }
  }
}

// Tile index -> row tile, first output channel and width. The tiles of the last, partial round of the persistent CTAs are
// split into two half-width tiles each when that lets the round finish in half the time (the host decides: full_tiles).
template <int BN>
__device__ __forceinline__ void decode_tile(const ConvParams& p, int tile, int& m_tile, int& n0, int& width) {
  int whole = tile, half = 0;
  width = BN;
  if (tile >= p.full_tiles) {
    const int h = tile - p.full_tiles;
    whole = p.full_tiles + (h >> 1);
    half = h & 1;
    width = BN / 2;
  }
  int nt;
  if (p.n_major) {
    divmod(whole, p.div_row_tiles, nt, m_tile);
  } else {
    divmod(whole, p.div_tiles_n, m_tile, nt);
  }
  n0 = nt * BN + half * (BN / 2);
}

// PAIR: the kernel runs as clusters of two CTAs that share one tcgen05 instruction stream (cta_group::2): a pair owns
// 256 pixels (128 per CTA) x BN channels, each CTA loads its own pixels and half of the weight rows, the even CTA (the
// leader) issues M = 256 MMAs that read both halves, and each CTA drains its own 128 accumulator rows. A CTA then moves
// 2/3 of the operand bytes per MMA through its shared memory, which is what bounds the single-CTA form. Barriers: the
// stage's "full" barrier lives in the leader and counts both CTAs' bytes; "empty" and "accumulator full" exist in both
// CTAs and the leader's commits arrive on both; "accumulator empty" lives in the leader and collects both epilogues.
// FMT: 0 = block-scaled MXFP8, 1 = INT8, 2 = BF16 (plain kind::f16 MMAs on 2-byte elements; every size below is in bytes
// of K, so a BF16 layer is a conv over 2 * Cin "channels" of one byte without scales).
constexpr int kFmtMx = 0, kFmtI8 = 1, kFmtBf16 = 2;

// CONVERT: the activations arrive as bf16 rows of a flat 1x1 layer (through `act_map`, 128 x 128 boxes without swizzle) and
// are quantised to E4M3 on chip — with the static exponents of `act_exponent`, or per pixel and 32 channels, in which case
// the converter warps also write the stage's activation-scale tile — by exactly the arithmetic of the standalone
// quantisers, so the result equals quantising first and convolving then, bit for bit.
template <int FMT, int BN, int BK, bool PAIR, int EPI, bool CONVERT>
__global__ void __launch_bounds__(CONVERT ? kConvertThreads : kThreads, 1)
conv_kernel(const __grid_constant__ CUtensorMap act_map, const __grid_constant__ CUtensorMap weight_map,
            const __grid_constant__ CUtensorMap out_map, const __grid_constant__ CUtensorMap sfb_map,
            const __grid_constant__ CUtensorMap sfa_map, const __grid_constant__ CUtensorMap out_warp_map, const ConvParams p) {
  static_assert(!PAIR || BN == 256 || (BN == 128 && FMT == kFmtMx), "CTA pairs are built for 256-wide tiles (and 128-wide block-scaled ones)");
  static_assert(!CONVERT || (FMT == kFmtMx && !PAIR && BK == 128), "the converter feeds flat block-scaled layers");
  constexpr int kBlockThreads = CONVERT ? kConvertThreads : kThreads;
  static_assert((EPI & kEpiPool) == 0 || (FMT == kFmtI8 && EPI == kEpiPool), "the pooled output belongs to the INT8 conv's general epilogue");
  static_assert((EPI & kEpiLean) == 0 || (FMT == kFmtMx && !PAIR && BN >= 128), "the short epilogues serve flat block-scaled layers");
  constexpr bool INT8 = FMT == kFmtI8;
  constexpr bool SCALED = FMT == kFmtMx;  // operands carry E8M0 block scales
  constexpr int kAccStages = acc_stages(BN);
  constexpr int kScaleTilesB = scale_tiles_b(BN);
  constexpr int kKSteps = BK / 32;
  constexpr uint32_t kABytes = kTileM * BK, kBBytes = (PAIR ? BN / 2 : BN) * BK;  // per CTA
  constexpr int kWeightBoxRows = BN < 128 ? BN : 128;  // rows of one weight TMA box
  constexpr uint32_t kSfbColumns = BN < 128 ? 4 : BN / 32;
  constexpr uint32_t kSfbColumn = kAccStages * BN;                        // one set of kSfbColumns per stage
  // then the activation scales (static: 4 columns per 128 input channels, copied once; per-pixel: 4 columns per stage),
  // then the resident weight scales (kSfbColumns per K iteration, kept while consecutive tiles share their channels)
  const uint32_t sfa_column = kSfbColumn + static_cast<uint32_t>(p.stages) * kSfbColumns;
  const uint32_t resident_column =
      sfa_column + 4u * static_cast<uint32_t>(SCALED && (CONVERT ? p.convert_static == 0 : p.act_scales != nullptr) ? p.stages : (p.cin + 127) / 128);
  constexpr int kEpiGroups = BN >= 128 ? 4 : 2;          // column groups of the epilogue, four warps (one per lane quarter) each
  constexpr int kChunksPerWarp = BN / (32 * kEpiGroups); // 32-column chunks each epilogue warp owns
  // A 64-wide tile has two column groups; the other eight epilogue warps form a second set, and the sets drain alternate
  // tiles (set s always meets accumulator stage s), so a narrow layer has all sixteen warps at work too.
  constexpr int kTileSets = BN >= 128 ? 1 : 2;
  static_assert(kTileSets == 1 || kAccStages == 2, "each set of epilogue warps needs an accumulator stage of its own");
  constexpr int kPanelGroups = 4;                        // four-warp groups that own output panels

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) SharedControl ctl;

  // dynamic shared memory, 1024-byte aligned:
  // [GELU table][stages x A][stages x B][output panels][stages x scale tiles B][stages x scale tile A][static A scale tiles][bias]
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t panel_bytes = 4096u * p.out_elem;
  const uint32_t smem_gelu = base;  // kGeluTable first, when the epilogue applies GELU: within 64 KB of the window's start
  const uint32_t smem_a = base + (p.act == kActGelu ? kGeluSmemBytes : 0u);
  const uint32_t smem_b = smem_a + p.stages * kABytes;
  const uint32_t smem_out = smem_b + static_cast<uint32_t>(p.b_slots) * kBBytes;
  const uint32_t smem_pool = smem_out + kPanelGroups * p.panels_per_half * panel_bytes;  // pooled panels: two of 1 KB per group
  const uint32_t smem_sfb = smem_pool + (p.pool ? kPanelGroups * 2u * kPoolPanelBytes : 0u);
  const uint32_t smem_sfa = smem_sfb + static_cast<uint32_t>(p.b_slots) * kScaleTilesB * 512;
  const uint32_t smem_sfa_static = smem_sfa + p.stages * 512;
  const uint32_t smem_bias = smem_sfa_static + ((p.cin + 127) / 128) * 512;  // fp32, tiles_n * BN entries
  const uint32_t smem_raw = (smem_bias + static_cast<uint32_t>(p.tiles_n * BN) * 4u + 1023u) & ~1023u;  // CONVERT: bf16 landing ring

  // (the warp index through a shuffle: the compiler then treats it, and every address or coordinate derived from it, as
  // uniform over the warp)
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  // per-pixel activation scales: read from HBM tiles, or written into the stage by the converter warps
  const bool dynamic_a = SCALED && (CONVERT ? p.convert_static == 0 : p.act_scales != nullptr);
  const int taps = p.kh * p.kw;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;                   // 0: the CTA that issues the MMAs
  const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);  // tile walker index
  const int workers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&ctl.full[s], CONVERT ? 1 + kConverterWarps : 1);  // the producer's bytes (+ the converter warps' tile)
      mbar_init(&ctl.empty[s], 1);
    }
    mbar_init(&ctl.weights_ready, 1);
    if (CONVERT) {
      for (int s = 0; s < kRawStages; ++s) {
        mbar_init(&ctl.raw_full[s], 1);
        mbar_init(&ctl.raw_empty[s], kConverterWarps);
      }
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl.tmem_full[s], 1);
      mbar_init(&ctl.tmem_empty[s], (PAIR ? 2 : 1) * 4 * kEpiGroups);
    }
    mbar_fence_init();
    tma_prefetch_desc(&act_map);
    tma_prefetch_desc(&weight_map);
    tma_prefetch_desc(&out_map);
    if (p.warp_panels || p.pool) tma_prefetch_desc(&out_warp_map);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(&ctl.tmem_base, kTmemColumns);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&ctl.tmem_base, kTmemColumns);
      tmem_relinquish();
    }
  }
  if (warp == 2 && SCALED && !dynamic_a) {
    // static activation scales: one 512-byte tile per 128 input channels, the same 4 bytes in all 128 rows
    const int tiles = (p.cin + 127) / 128;
    const int groups = p.cin / 32;
    for (int t = 0; t < tiles; ++t) {
      uint32_t word = 0;
      for (int g = 0; g < 4; ++g) {
        const int idx = t * 4 + g;
        const uint32_t byte = idx < groups ? static_cast<uint32_t>(static_cast<int>(p.act_exponent[idx]) + 127) : 127u;
        word |= (byte & 0xFFu) << (8 * g);
      }
      asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(smem_sfa_static + t * 512 + lane * 16), "r"(word) : "memory");
    }
    fence_async_proxy();
  }
  if (p.bias != nullptr) {
    // the bias widened to fp32 once per CTA (zero for the columns a ragged last tile pads)
    for (int i = threadIdx.x; i < p.tiles_n * BN; i += kBlockThreads) {
      const float value = i < p.cout ? __bfloat162float(p.bias[i]) : 0.0f;
      asm volatile("st.shared.f32 [%0], %1;" ::"r"(smem_bias + i * 4), "f"(value) : "memory");
    }
  }
  if (p.act == kActGelu) {
    for (int i = threadIdx.x; i < kGeluEntries; i += kBlockThreads) {
      asm volatile("st.shared.b32 [%0], %1;" ::"r"(smem_gelu + i * 4), "r"(kGeluTable[i]) : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync();  // the other CTA's barriers and static scale tiles exist before anything refers to them
  tc_fence_after();
  const uint32_t tmem = ctl.tmem_base;
  const uint32_t full0 = smem_u32(&ctl.full[0]), empty0 = smem_u32(&ctl.empty[0]);
  const uint32_t tfull0 = smem_u32(&ctl.tmem_full[0]), tempty0 = smem_u32(&ctl.tmem_empty[0]);
  const uint32_t raw_full0 = smem_u32(&ctl.raw_full[0]), raw_empty0 = smem_u32(&ctl.raw_empty[0]);
  volatile int* abort_flag = &ctl.abort_flag;

  // how the producer and MMA warps walk their loops (see the producer): one elected lane alone, or the whole warp
  constexpr bool kLaneLoop = BN <= 128;
  auto loop_wait = [&](uint32_t bar, uint32_t parity, int code) -> bool {
    return kLaneLoop ? mbar_wait_addr(bar, parity, abort_flag, p.status, code) : mbar_wait_warp(bar, parity, abort_flag, p.status, code);
  };
  if (warp == 0) {
    // ===== TMA producer =====
    // The issuing lane is picked by elect.sync rather than by its lane number: the compiler then knows that a single lane
    // runs the code and keeps coordinates, addresses and byte counts in uniform registers, which is where the copy
    // instructions take them from (behind `lane == 0` every operand of every copy went through a vector-to-uniform move,
    // several hundred cycles per K step in a chain this lane walks alone). Narrow tiles, whose K steps are short, let that
    // one lane walk the whole loop (kLaneLoop); for 256-wide tiles the whole warp walks it, polls the barriers together
    // and elects the issuer per K step, which measured 3 % faster there and 10 % slower on the narrow ones.
    if (kLaneLoop ? elect_one() : true) {
      const uint32_t a_box_bytes = in_register(static_cast<uint32_t>(p.tile_h * p.tile_w) * BK);
      // loop parameters, once into registers (a kernel parameter read in the loop is a constant-bank load per iteration)
      const uint32_t stages = in_register(static_cast<uint32_t>(p.stages));
      const int k_chunks = static_cast<int>(in_register(static_cast<uint32_t>(p.k_chunks)));
      const int kh = static_cast<int>(in_register(static_cast<uint32_t>(p.kh))), kw = static_cast<int>(in_register(static_cast<uint32_t>(p.kw)));
      const int dil_h = static_cast<int>(in_register(static_cast<uint32_t>(p.dil_h))), dil_w = static_cast<int>(in_register(static_cast<uint32_t>(p.dil_w)));
      const int resident_bytes = static_cast<int>(in_register(static_cast<uint32_t>(p.resident_k * BK)));
      const bool load_a = !(probe_flags(p) & 1), load_b = !(probe_flags(p) & 2);
      uint32_t s = 0, phase = 0, raw_s = 0, raw_phase = 0;
      bool alive = true;
      int last_n0 = -1;
      const bool resident_b = in_register(static_cast<uint32_t>(p.weights_resident)) != 0;
      if (resident_b && worker < p.total_tiles && (kLaneLoop || elect_one())) {
        // A layer with one output-channel tile whose weights fit beside the activation ring: every K step's weight tile
        // and scale tiles are copied once and stay; the loop below then moves activations only.
        const int k_total = kh * kw * k_chunks;
        mbar_expect_tx_addr(smem_u32(&ctl.weights_ready), static_cast<uint32_t>(k_total) * (kBBytes + (SCALED ? kScaleTilesB * 512u : 0u)));
        for (int ki = 0; ki < k_total; ++ki) {
#pragma unroll
          for (int part = 0; part < BN / kWeightBoxRows; ++part) {
            tma_load_2d_addr(smem_b + ki * kBBytes + part * kWeightBoxRows * BK, &weight_map, smem_u32(&ctl.weights_ready), ki * BK,
                             part * kWeightBoxRows);
          }
          if (SCALED) {
#pragma unroll
            for (int i = 0; i < kScaleTilesB; ++i) {
              const int row_tile = min(i, p.weight_row_tiles - 1);
              bulk_load_addr(smem_sfb + (ki * kScaleTilesB + i) * 512,
                             p.weight_scales + (static_cast<size_t>(row_tile) * p.weight_scale_tiles + ((ki * BK) >> 7)) * 512, 512,
                             smem_u32(&ctl.weights_ready));
            }
          }
        }
      }
      for (int tile = worker; tile < p.total_tiles && alive; tile += workers) {
        int m_tile, n0, width;
        decode_tile<BN>(p, tile, m_tile, n0, width);
        if (PAIR) m_tile = 2 * m_tile + static_cast<int>(rank);  // a pair owns two consecutive row tiles
        int m = m_tile;
        int tx, ty, b;
        divmod(m, p.div_tiles_x, m, tx);
        divmod(m, p.div_tiles_y, b, ty);
        const int x0 = tx * p.tile_w * p.stride_w - p.pad_w, y0 = ty * p.tile_h * p.stride_h - p.pad_h;
        // the weight tile arrives in boxes of kWeightBoxRows rows (a 256-wide tile is two boxes, its half one)
        const int b_parts = PAIR ? 1 : width / kWeightBoxRows;
        const int scale_tiles = BN <= 128 ? 1 : width / 128;
        // a pair's barrier (in the leader) counts the bytes of both CTAs, which load the same amounts
        // (a pair's weight box always has BN / 2 rows: for a half-width tile only the first width / 2 of them are used)
        // (a converting layer's activation tile and scale tile are written by the converter warps, not counted here)
        const uint32_t operand_bytes = (load_a && !CONVERT ? a_box_bytes : 0u) +
                                       (load_b && !resident_b ? (PAIR ? kBBytes : static_cast<uint32_t>(width) * BK) : 0u) +
                                       (dynamic_a && !CONVERT ? 512u : 0u);
        const uint32_t sfb_bytes = SCALED ? scale_tiles * 512u : 0u;
        // weight scales of the first resident_k iterations are already in tensor memory when the tile before this one
        // had the same output channels
        const bool fresh = n0 != last_n0;
        last_n0 = n0;
        const uint8_t* sfb_src[kScaleTilesB];
#pragma unroll
        for (int i = 0; i < kScaleTilesB; ++i) {
          const int row_tile = min(n0 / 128 + i, p.weight_row_tiles - 1);
          sfb_src[i] = p.weight_scales + static_cast<size_t>(row_tile) * p.weight_scale_tiles * 512;
        }
        const uint8_t* sfa_src = dynamic_a && !CONVERT ? p.act_scales + static_cast<size_t>(m_tile) * p.act_scale_tiles * 512 : nullptr;
        int k0 = 0;  // offset along the weight's K axis
        for (int ky = 0; ky < kh && alive; ++ky) {
          for (int kx = 0; kx < kw && alive; ++kx) {
            const int cx = x0 + kx * dil_w, cy = y0 + ky * dil_h;
            for (int j = 0; j < k_chunks; ++j, k0 += BK) {
              if (CONVERT) {
                // the bf16 tile of this K step into the landing ring: 128 rows of the pixel matrix x 128 channels
                if (!loop_wait(raw_empty0 + 8 * raw_s, raw_phase ^ 1, kStatusWaitEmpty)) {
                  alive = false;
                  break;
                }
                if (kLaneLoop || elect_one()) {
                  mbar_expect_tx_addr(raw_full0 + 8 * raw_s, kRawBytes);
                  tma_load_4d_addr(smem_raw + raw_s * kRawBytes, &act_map, raw_full0 + 8 * raw_s, j * 128, m_tile * kTileM, 0, 0);
                }
                if (++raw_s == kRawStages) raw_s = 0, raw_phase ^= 1;
              }
              if (!loop_wait(empty0 + 8 * s, phase ^ 1, kStatusWaitEmpty)) {
                alive = false;
                break;
              }
              const uint32_t bar = PAIR ? ((full0 + 8 * s) & ~kPeerBit) : full0 + 8 * s;
              const bool load_sfb = SCALED && !resident_b && (fresh || k0 >= resident_bytes);
              const uint32_t tx_bytes = (PAIR ? 2u : 1u) * (operand_bytes + (load_sfb ? sfb_bytes : 0u));
              const bool issuer = kLaneLoop || elect_one();
              if (issuer && (!PAIR || rank == 0)) {
                if (tx_bytes != 0) {
                  mbar_expect_tx_addr(full0 + 8 * s, tx_bytes);
                } else {
                  mbar_arrive_addr(full0 + 8 * s);
                }
              }
              if (PAIR) {
                if (issuer) {
                if (load_a) tma_load_4d_pair(smem_a + s * kABytes, &act_map, bar, j * BK, cx, cy, b);
                if (load_b) tma_load_2d_pair(smem_b + s * kBBytes, &weight_map, bar, k0, n0 + static_cast<int>(rank) * (width / 2));
                if (SCALED) {
                  // scale tiles through their tensor maps (128 words of 4 bytes per tile): only a tiled load can count
                  // on a barrier in the other CTA
                  const int w_tile = k0 >> 7;
                  if (load_sfb) {
#pragma unroll
                    for (int i = 0; i < kScaleTilesB; ++i) {
                      const int row_tile = min(n0 / 128 + i, p.weight_row_tiles - 1);
                      tma_load_2d_pair(smem_sfb + (s * kScaleTilesB + i) * 512, &sfb_map, bar, 0, row_tile * p.weight_scale_tiles + w_tile);
                    }
                  }
                  if (dynamic_a) {
                    tma_load_2d_pair(smem_sfa + s * 512, &sfa_map, bar, 0, m_tile * p.act_scale_tiles + ((j * BK) >> 7));
                  }
                }
                }
                if (++s == stages) s = 0, phase ^= 1;
                continue;
              }
              if (issuer) {
              if (load_a && !CONVERT) tma_load_4d_addr(smem_a + s * kABytes, &act_map, bar, j * BK, cx, cy, b);
              if (load_b && !resident_b) {
#pragma unroll
                for (int part = 0; part < BN / kWeightBoxRows; ++part) {
                  if (part < b_parts) {
                    tma_load_2d_addr(smem_b + s * kBBytes + part * kWeightBoxRows * BK, &weight_map, bar, k0, n0 + part * kWeightBoxRows);
                  }
                }
              }
              if (SCALED) {
                const int w_tile = k0 >> 7;
#pragma unroll
                for (int i = 0; i < kScaleTilesB; ++i) {
                  if (i < scale_tiles && load_sfb) {
                    bulk_load_addr(smem_sfb + (s * kScaleTilesB + i) * 512, sfb_src[i] + static_cast<size_t>(w_tile) * 512, 512, bar);
                  }
                }
                if (dynamic_a && !CONVERT) bulk_load_addr(smem_sfa + s * 512, sfa_src + static_cast<size_t>((j * BK) >> 7) * 512, 512, bar);
              }
              }
              if (++s == stages) s = 0, phase ^= 1;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer (of a pair: the leader CTA's) =====
    // (one lane picked by elect.sync, as in the producer: it issues the tcgen05 instructions and their commits)
    if (rank == 0 && (kLaneLoop ? elect_one() : true)) {
      const uint64_t a_desc0 = kmajor_desc(smem_a, BK), b_desc0 = kmajor_desc(smem_b, BK);
      const uint64_t sfb_desc0 = scale_desc(smem_sfb), sfa_desc0 = scale_desc(dynamic_a ? smem_sfa : smem_sfa_static);
      const int k_iters = static_cast<int>(in_register(static_cast<uint32_t>(taps * p.k_chunks)));
      const bool copy_scales = SCALED && !(probe_flags(p) & 8);
      // loop parameters, once into registers
      const uint32_t stages = in_register(static_cast<uint32_t>(p.stages));
      const int k_chunks = static_cast<int>(in_register(static_cast<uint32_t>(p.k_chunks)));
      const int resident_k = static_cast<int>(in_register(static_cast<uint32_t>(p.resident_k)));
      const uint32_t sfa_base = in_register(tmem + sfa_column), sfb_stage_base = in_register(tmem + kSfbColumn);
      const uint32_t sfb_resident_base = in_register(tmem + resident_column);
      const bool per_stage_a = in_register(dynamic_a ? 1u : 0u) != 0;
      if (SCALED && !dynamic_a && (kLaneLoop || elect_one())) {
        // static activation scales never change: all tiles go to tensor memory once, ahead of the first MMA
        const int tiles = (p.cin + 127) / 128;
        for (int t = 0; t < tiles; ++t) {
          if (PAIR) {
            tc_copy_scales_pair(tmem + sfa_column + 4 * t, sfa_desc0 + static_cast<uint64_t>((t * 512) >> 4));
          } else {
            tc_copy_scales(tmem + sfa_column + 4 * t, sfa_desc0 + static_cast<uint64_t>((t * 512) >> 4));
          }
        }
      }
      uint32_t s = 0, phase = 0, tile_it = 0;
      bool alive = true;
      int last_n0 = -1;
      const bool resident_b = in_register(static_cast<uint32_t>(p.weights_resident)) != 0;
      if (resident_b && worker < p.total_tiles) alive = loop_wait(smem_u32(&ctl.weights_ready), 0, kStatusWaitFull);
#if FIM_PROBE_BUILD
      long long c_wait = 0, c_issue = 0, c_tile = 0, c_rounds = 0;
      const long long c_start = clock64();
#endif
      for (int tile = worker; tile < p.total_tiles && alive; tile += workers, ++tile_it) {
#if FIM_PROBE_BUILD
        const long long c_t0 = clock64();
#endif
        const uint32_t acc = kAccStages == 2 ? (tile_it & 1u) : 0u;
        const uint32_t acc_phase = kAccStages == 2 ? ((tile_it >> 1) & 1u) : (tile_it & 1u);
        if (!loop_wait(tempty0 + 8 * acc, acc_phase ^ 1, kStatusWaitTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem + acc * BN;
        int m_tile, n0, width;
        decode_tile<BN>(p, tile, m_tile, n0, width);
        const uint32_t idesc = INT8 ? idesc_i8(width, PAIR ? 256 : kTileM)
                                    : (SCALED ? idesc_mxf8(width, PAIR ? 256 : kTileM) : idesc_bf16(width, PAIR ? 256 : kTileM));
        const int scale_tiles = BN <= 128 ? 1 : width / 128;
        const bool fresh = n0 != last_n0;  // the resident weight scales belong to other output channels
        last_n0 = n0;
        int j = 0;            // channel chunk within the tap
        uint32_t b_id = 0;    // (32-channel block index along the weight's K) mod 4 at the start of the stage
#if FIM_PROBE_BUILD
        c_tile += clock64() - c_t0;
#endif
        for (int ki = 0; ki < k_iters; ++ki) {
#if FIM_PROBE_BUILD
          const long long c_a = clock64();
#endif
          if (!loop_wait(full0 + 8 * s, phase, kStatusWaitFull)) {
            alive = false;
            break;
          }
          tc_fence_after();
#if FIM_PROBE_BUILD
          const long long c_b = clock64();
          c_wait += c_b - c_a;
#endif
          uint32_t a_id = 0;
          const uint32_t kb_a = j * kKSteps;  // 32-channel block index of the activation chunk
          if (BK != 128) a_id = kb_a & 3;
          // scale tiles of this stage: shared memory -> the stage's own tensor-memory columns, in front of its MMAs (the
          // tensor pipe runs both in issue order; a column set is rewritten only after the MMAs that read it, a whole
          // ring of stages earlier). Issuing a stage's copies one stage early was measured: no gain, the pipe serialises
          // copies and MMAs either way.
          // the first resident_k iterations keep their weight scales in columns of their own from tile to tile
          const bool resident = ki < resident_k;
          const uint32_t sfb_tmem = resident ? sfb_resident_base + kSfbColumns * ki : sfb_stage_base + kSfbColumns * s;
          const uint32_t sfa_tmem = sfa_base + 4 * (per_stage_a ? s : (kb_a >> 2));
          const uint64_t a_desc = a_desc0 + static_cast<uint64_t>((s * kABytes) >> 4);
          // weights: the stage's tile, or K step ki of the resident matrix (a half-width tile starts n0 rows into it)
          const uint32_t b_slot = resident_b ? static_cast<uint32_t>(ki) : s;
          const uint32_t b_row0 = resident_b ? static_cast<uint32_t>(n0) : 0u;
          const uint64_t b_desc = b_desc0 + static_cast<uint64_t>((b_slot * kBBytes + b_row0 * BK) >> 4);
          const uint64_t sfb_from = sfb_desc0 + static_cast<uint64_t>(((b_slot * kScaleTilesB + (b_row0 >> 7)) * 512) >> 4);
          const uint64_t sfa_from = sfa_desc0 + static_cast<uint64_t>((s * 512) >> 4);
          const bool copy_b = copy_scales && (fresh || !resident), copy_a = copy_scales && per_stage_a;
          const uint32_t scaled0 = idesc | (a_id << 29) | (b_id << 4);  // the scale ids advance by one per K step
          const uint32_t first = ki > 0 ? 1u : 0u;
          if (kLaneLoop || elect_one()) {
#pragma unroll
            for (int i = 0; i < kScaleTilesB; ++i) {
              if (i < scale_tiles && copy_b) {
                if (PAIR) {
                  tc_copy_scales_pair(sfb_tmem + 4 * i, sfb_from + 32 * i);
                } else {
                  tc_copy_scales(sfb_tmem + 4 * i, sfb_from + 32 * i);
                }
              }
            }
            if (copy_a) {
              if (PAIR) {
                tc_copy_scales_pair(sfa_tmem, sfa_from);
              } else {
                tc_copy_scales(sfa_tmem, sfa_from);
              }
            }
#pragma unroll
            for (int k = 0; k < kKSteps; ++k) {
              const uint32_t accumulate = k > 0 ? 1u : first;
              if (INT8) {
                if (PAIR) {
                  tc_mma_i8_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, accumulate);
                } else {
                  tc_mma_i8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, accumulate);
                }
              } else if (!SCALED) {
                tc_mma_bf16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, accumulate);
              } else {
                const uint32_t scaled = scaled0 + static_cast<uint32_t>(k) * ((1u << 29) | (1u << 4));
                if (PAIR) {
                  tc_mma_mxf8_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, scaled, sfa_tmem, sfb_tmem, accumulate);
                } else {
                  tc_mma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, scaled, sfa_tmem, sfb_tmem, accumulate);
                }
              }
            }
            // the stage is free once these MMAs have read it (of a pair: in both CTAs)
            if (PAIR) {
              tc_commit_pair(empty0 + 8 * s);
              tc_commit_pair((empty0 + 8 * s) | kPeerBit);
            } else {
              tc_commit(&ctl.empty[s]);
            }
          }
#if FIM_PROBE_BUILD
          c_issue += clock64() - c_b;
          ++c_rounds;
#endif
          if (++s == stages) s = 0, phase ^= 1;
          if (++j == k_chunks) j = 0;
          if (BK != 128) b_id = (b_id + kKSteps) & 3;
        }
        if (alive && (kLaneLoop || elect_one())) {
          if (PAIR) {
            tc_commit_pair(tfull0 + 8 * acc);
            tc_commit_pair((tfull0 + 8 * acc) | kPeerBit);
          } else {
            tc_commit(&ctl.tmem_full[acc]);
          }
        }
      }
#if FIM_PROBE_BUILD
      if ((p.debug & 8192) && blockIdx.x == 0 && (kLaneLoop || lane == 0)) {
        printf("mma warp: %lld K rounds, per round wait %.1f issue %.1f clk; per tile head %.1f clk over %u tiles; total %lld clk\n", c_rounds,
               double(c_wait) / double(c_rounds), double(c_issue) / double(c_rounds), double(c_tile) / double(tile_it), tile_it, clock64() - c_start);
      }
#endif
    }
  } else if (CONVERT && warp >= 2 + 16) {
    // ===== converter: bf16 landing tile -> E4M3 K-major stage (+ the stage's activation-scale tile) =====
    // 1024 pieces of 16 channels per tile, four per thread: piece t = (row t / 8, channels 16 * (t % 8) ...); the two
    // lanes of a 32-channel block are neighbours. A warp reads 1 KB of consecutive shared memory per step and writes four
    // rows of the 128-byte-swizzled stage, both without bank conflicts.
    const int ctid = static_cast<int>(threadIdx.x) - 32 * (2 + 16);
    const int piece = ctid & 7, group = piece >> 1;
    uint32_t s = 0, phase = 0, raw_s = 0, raw_phase = 0;
    bool alive = true;
    for (int tile = worker; tile < p.total_tiles && alive; tile += workers) {
      for (int j = 0; j < p.k_chunks; ++j) {
        if (!mbar_wait_addr(raw_full0 + 8 * raw_s, raw_phase, abort_flag, p.status, kStatusWaitFull) ||
            !mbar_wait_addr(empty0 + 8 * s, phase ^ 1, abort_flag, p.status, kStatusWaitEmpty)) {
          alive = false;
          break;
        }
        const uint32_t from = smem_raw + raw_s * kRawBytes, to = smem_a + s * kABytes, scale_tile = smem_sfa + s * 512;
        const int static_e = p.convert_static ? static_cast<int>(__ldg(p.act_exponent + j * 4 + group)) : 0;
        constexpr int kRowsPerPass = 4 * kConverterWarps;  // eight threads per row
#pragma unroll 2
        for (int i = 0; i < kTileM / kRowsPerPass; ++i) {
          const int row = i * kRowsPerPass + (ctid >> 3);
          uint32_t w[8];
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]) : "r"(from + row * 256 + piece * 32));
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7]) : "r"(from + row * 256 + piece * 32 + 16));
          // the arithmetic of the conv epilogue's requantiser, on the packed words (the same bits as the standalone
          // quantisers, which work in fp32: a bf16 maximum, an exact power-of-two scaling)
          int e = static_e;
          if (!p.convert_static) {
            uint32_t m = bf16x2_absmax(bf16x2_absmax(bf16x2_absmax(w[0], w[1]), bf16x2_absmax(w[2], w[3])),
                                       bf16x2_absmax(bf16x2_absmax(w[4], w[5]), bf16x2_absmax(w[6], w[7])));
            uint32_t top = max(m & 0x7FFFu, (m >> 16) & 0x7FFFu);
            top = max(top, __shfl_xor_sync(0xffffffffu, top, 1));
            e = e8m0_exponent_bits(top << 16);
            if ((piece & 1) == 0) {
              asm volatile("st.shared.u8 [%0], %1;" ::"r"(scale_tile + (row & 31) * 16 + (row >> 5) * 4 + group), "r"(e + 127) : "memory");
            }
          }
          uint32_t q[4];
          scale_to_e4m3(w, e, q);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(to + row * 128 + ((piece ^ (row & 7)) << 4)), "r"(q[0]), "r"(q[1]),
                       "r"(q[2]), "r"(q[3])
                       : "memory");
        }
        fence_async_proxy();  // the MMAs (and the scale copy) read these bytes through the async proxy
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_addr(full0 + 8 * s);
          mbar_arrive_addr(raw_empty0 + 8 * raw_s);
        }
        if (++s == static_cast<uint32_t>(p.stages)) s = 0, phase ^= 1;
        if (++raw_s == kRawStages) raw_s = 0, raw_phase ^= 1;
      }
    }
  } else {
    // ===== epilogue: warp w owns tensor-memory lanes 32 * (w % 4) ... + 31 and one column group of the tile =====
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    if constexpr ((EPI & kEpiLean) != 0) {
      // ----- short epilogue of a flat 1x1 layer: a tile is 128 consecutive rows of the pixel matrix, this warp owns 32 of
      // them and kChunksPerWarp chunks of 32 channels, stages each chunk in two panels of its own and stores it itself
      constexpr bool kGelu = (EPI & kEpiGelu) != 0, kDynamic = (EPI & kEpiDynamic) != 0, kResidual = (EPI & kEpiResidual) != 0;
      constexpr uint32_t kElem = kDynamic ? 1u : 2u;            // bytes per output element
      constexpr uint32_t kPitch = 32u * kElem, kSlots = kPitch >> 4;
      constexpr uint32_t kPanelBytes = 32u * kPitch;
      constexpr int kGroupColumns = BN / kEpiGroups;
      constexpr uint32_t kPanels = CONVERT ? 1u : 2u;  // a converting layer gives the second panel's room to its landing ring
      const uint32_t my_panels = smem_out + static_cast<uint32_t>(warp - 2) * kPanels * kPanelBytes;
      // 16-byte slot i of this lane's row sits at row_at ^ (i << 4) (the swizzle a TMA store of kPitch-byte rows reads)
      const uint32_t row_at = static_cast<uint32_t>(lane) * kPitch + ((((static_cast<uint32_t>(lane) * kPitch) >> 7) & (kSlots - 1)) << 4);
      const uint32_t bias_at = smem_bias + static_cast<uint32_t>(group * kGroupColumns) * 4u;
      const uint32_t lane_tmem = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + group * kGroupColumns;
      const GeluTable gelu2 = gelu_table_at(smem_gelu);
      const int row = quarter * 32 + lane;
      const int scale_tiles = ((p.cout >> 5) + 3) >> 2;         // 4-group tiles per row tile of the output scales
      const uint32_t scale_at = static_cast<uint32_t>(lane * 16 + quarter * 4);
      const long long res_pitch = p.res_stride[2];
      uint32_t tile_it = 0, chunk_it = 0;
      for (int tile = worker; tile < p.total_tiles; tile += workers, ++tile_it) {
        int m, n0, width;
        decode_tile<BN>(p, tile, m, n0, width);
        const int pixel = m * kTileM + row;  // the host keeps rows below 2**31
        const bool valid = pixel < p.out_w;
        const uint32_t acc = kAccStages == 2 ? (tile_it & 1u) : 0u;
        const uint32_t acc_phase = kAccStages == 2 ? ((tile_it >> 1) & 1u) : (tile_it & 1u);
        const int column0 = group * kGroupColumns;  // first column of this warp inside the tile
        const __nv_bfloat16* res_row = nullptr;
        if (kResidual) {
          res_row = p.residual + static_cast<long long>(pixel) * res_pitch + n0 + column0;
          // ask for the line in L2 before the wait for the accumulator (a prefetch holds no registers)
          if (valid && column0 < width) asm volatile("prefetch.global.L2 [%0];" ::"l"(res_row));
        }
        // (the warp leaves together: its stores are issued through elect.sync, which every lane must reach)
        if (!mbar_wait_warp(tfull0 + 8 * acc, acc_phase, abort_flag, p.status, kStatusWaitTmemFull, true, p.poll_backoff_ns)) break;
        tc_fence_after();
        uint32_t q[kChunksPerWarp][16];
#pragma unroll
        for (int g = 0; g < kChunksPerWarp; ++g) {
          uint32_t raw[32];
          tmem_load_32(lane_tmem + acc * BN + g * 32, raw);
          tmem_load_wait();
          if (g + 1 == kChunksPerWarp) {  // the accumulator goes back to the MMA warp before the long arithmetic
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_addr(tempty0 + 8 * acc);
          }
          if (column0 + g * 32 >= width) continue;  // a half-width tile of a split last round: nothing behind this chunk
          const uint32_t bias_chunk = bias_at + static_cast<uint32_t>(n0 + g * 32) * 4u;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint64_t b0, b1;
            load_bias_pairs(bias_chunk, i, b0, b1);
            float v0, v1, v2, v3;
            unpack2(add2(pack2(__uint_as_float(raw[4 * i]), __uint_as_float(raw[4 * i + 1])), b0), v0, v1);
            unpack2(add2(pack2(__uint_as_float(raw[4 * i + 2]), __uint_as_float(raw[4 * i + 3])), b1), v2, v3);
            q[g][2 * i] = pack_bf16(v0, v1);
            q[g][2 * i + 1] = pack_bf16(v2, v3);
          }
        }
#pragma unroll
        for (int g = 0; g < kChunksPerWarp; ++g) {
          if (column0 + g * 32 >= width) continue;
          uint32_t(&r)[16] = q[g];
          if (kGelu) {
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = gelu_bf16x2(r[i], gelu2);
          }
          if (kResidual) {
            if (valid) {
              const uint4* r4 = reinterpret_cast<const uint4*>(res_row + g * 32);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint4 v = __ldg(r4 + i);
                r[4 * i] = bf16x2_add(r[4 * i], v.x);
                r[4 * i + 1] = bf16x2_add(r[4 * i + 1], v.y);
                r[4 * i + 2] = bf16x2_add(r[4 * i + 2], v.z);
                r[4 * i + 3] = bf16x2_add(r[4 * i + 3], v.w);
              }
            }
          }
          const uint32_t panel = my_panels + (chunk_it & (kPanels - 1u)) * kPanelBytes;
          ++chunk_it;
          const uint32_t at = panel + row_at;
          if (kDynamic) {
            uint32_t mx[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) mx[i] = bf16x2_absmax(r[2 * i], r[2 * i + 1]);
#pragma unroll
            for (int i = 0; i < 4; ++i) mx[i] = bf16x2_absmax(mx[2 * i], mx[2 * i + 1]);
            mx[0] = bf16x2_absmax(bf16x2_absmax(mx[0], mx[1]), bf16x2_absmax(mx[2], mx[3]));
            const uint32_t top = max(mx[0] & 0x7FFFu, (mx[0] >> 16) & 0x7FFFu);
            const int e = e8m0_exponent_bits(top << 16);
            if (valid) {
              const int kg = (n0 + column0 + g * 32) >> 5;
              p.out_scales[(static_cast<size_t>(m) * scale_tiles + (kg >> 2)) * 512 + scale_at + (kg & 3)] = static_cast<uint8_t>(e + 127);
            }
            uint32_t w[8];
            scale_to_e4m3(r, e, w);
            if (elect_one()) bulk_wait_read<kPanels - 1>();  // the store that last read this panel has finished with it
            __syncwarp();
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(at), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(at ^ 16u), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
          } else {
            if (elect_one()) bulk_wait_read<kPanels - 1>();
            __syncwarp();
#pragma unroll
            for (uint32_t i = 0; i < 4; ++i) {
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(at ^ (i << 4)), "r"(r[4 * i]), "r"(r[4 * i + 1]),
                           "r"(r[4 * i + 2]), "r"(r[4 * i + 3])
                           : "memory");
            }
          }
          fence_async_proxy();
          __syncwarp();
          if (elect_one()) {  // always the same lane (the lowest): the bulk groups it commits are the ones it waits for
            tma_store_4d(&out_warp_map, panel, (n0 + column0 + g * 32) * static_cast<int>(kElem), m * kTileM + quarter * 32, 0, 0);
            bulk_commit();
          }
        }
      }
      if (elect_one()) bulk_wait_read<0>();
    } else
    if (group < kEpiGroups * kTileSets) {
    const int cgroup = group & (kEpiGroups - 1);  // column group inside the tile
    const uint32_t tile_set = static_cast<uint32_t>(group / kEpiGroups);
    const EpilogueSwitches sw = epilogue_switches<EPI>(p);
    const uint32_t panel_bytes_ = 4096u * sw.out_elem;
    // the warp whose elected lane issues the TMA stores of its group (always the same lane: it waits for the groups it commits)
    const bool leader_warp = ((warp - 2) & 3) == 0;
    const uint32_t bar_id = 1 + group;
    const int row = quarter * 32 + lane;
    const int ry = row / p.tile_w, rx = row - ry * p.tile_w;
    const bool row_in_tile = row < p.tile_h * p.tile_w;
    const float a_scale = INT8 && p.a_scale != nullptr ? __ldg(p.a_scale) : 1.0f;
    const uint32_t panels = smem_out + group * sw.panels * panel_bytes_;
    // A flat 1x1 conv (a tile = 128 consecutive rows of the pixel matrix) lets every warp stage and store its own 32 rows:
    // the four warps of a group then never wait for each other. The panels take the same shared memory either way.
    const bool own = p.warp_panels != 0;
    const uint32_t own_bytes = 1024u * sw.out_elem;
    const uint32_t own_panels = smem_out + static_cast<uint32_t>(warp - 2) * sw.panels * own_bytes;
    const bool store = !(probe_flags(p) & 4);
    constexpr int kGroupColumns = BN / kEpiGroups;
    // The pooled second output (int8_conv2d_maxpool): once a chunk's 128 rows x 32 channels lie staged as bf16 for their
    // own store, thread t takes eight channels (one 16-byte slot) of pooled pixel t / 4: the maximum over the four rows of
    // its 2x2 window, quantised to INT8, into a panel of 32 pooled pixels x 32 bytes that a second TMA store writes through
    // `out_warp_map` (here: the tensor map of the pooled output, boxes of tile_w / 2 x tile_h / 2 pixels). The tile's
    // origin and sides are even (the host's choice), so every window lies inside one tile.
    constexpr bool pool = (EPI & kEpiPool) != 0;  // a kernel of its own: the general epilogue pays nothing for it
    uint32_t pool_from[4] = {0u, 0u, 0u, 0u}, pool_to = 0u;  // byte offsets into a staged panel / a pooled panel
    const uint32_t pool_panels = smem_pool + group * 2u * kPoolPanelBytes;
    bool pool_active = false;
    Int8Quantizer pool_quantizer = {};
    if (pool) {
      const int half_w = p.tile_w >> 1, pp = row >> 2, slot = row & 3;
      const int py = pp / half_w, px = pp - py * half_w;
      pool_active = pp < half_w * (p.tile_h >> 1);
      const int r00 = 2 * py * p.tile_w + 2 * px;
      const int rows4[4] = {r00, r00 + 1, r00 + p.tile_w, r00 + p.tile_w + 1};
#pragma unroll
      for (int i = 0; i < 4; ++i) {  // where stage_row<16> put that slot of a 64-byte row
        pool_from[i] = static_cast<uint32_t>(rows4[i]) * 64u + ((static_cast<uint32_t>(slot) ^ ((static_cast<uint32_t>(rows4[i]) >> 1) & 3u)) << 4);
      }
      pool_to = static_cast<uint32_t>(pp) * 32u + static_cast<uint32_t>(slot) * 8u;
      pool_quantizer = make_int8_quantizer(__ldg(p.out_scale));
    }
    uint32_t tile_it = 0, chunk_it = 0;
    for (int tile = worker; tile < p.total_tiles; tile += workers, ++tile_it) {
      if (kTileSets == 2 && (tile_it & 1u) != tile_set) continue;  // the other set's tile
      int m, n0, width;
      decode_tile<BN>(p, tile, m, n0, width);
      if (PAIR) m = 2 * m + static_cast<int>(rank);
      const int n_end = min(p.cout, n0 + width);  // columns of this tile that exist
      int tx, ty, b;
      divmod(m, p.div_tiles_x, m, tx);
      divmod(m, p.div_tiles_y, b, ty);
      const int x0 = tx * p.tile_w, y0 = ty * p.tile_h;
      const int x = x0 + rx, y = y0 + ry;
      const bool valid = row_in_tile && x < p.out_w && y < p.out_h && b < p.batch;
      const size_t pixel = (static_cast<size_t>(b) * p.out_h + y) * p.out_w + x;
      const uint32_t acc = kAccStages == 2 ? (tile_it & 1u) : 0u;
      const uint32_t acc_phase = kAccStages == 2 ? ((tile_it >> 1) & 1u) : (tile_it & 1u);
      if (sw.has_residual && valid && p.res_stride[3] == 1) {
        // ask for this row's residual line in L2 before the wait for the accumulator, so that the loads in the epilogue
        // do not pay the DRAM latency (a prefetch holds no registers)
        const int n_first = n0 + cgroup * kGroupColumns;
        if (n_first < p.res_channels) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(p.residual + b * p.res_stride[0] + y * p.res_stride[1] + x * p.res_stride[2] +
                                                          n_first));
        }
      }
      // One warp of the group waits for the accumulator (sleeping between polls: the main loop of a tile takes
      // microseconds) and publishes whether it arrived; the four warps then take the same decision, so none of them can
      // be left alone at a named barrier below when a wait runs out. The word alternates from one tile of the group to its next: the
      // deciding warp cannot be two tiles ahead of a sibling, which it meets at this barrier every tile.
      if (own) {
        // no barrier joins the warps below, so each waits for itself
        if (!mbar_wait_warp(tfull0 + 8 * acc, acc_phase, abort_flag, p.status, kStatusWaitTmemFull, true, p.poll_backoff_ns)) break;
      } else {
        volatile int* go = &ctl.group_go[group][(tile_it >> (kTileSets - 1)) & 1u];
        if (quarter == 0) {
          const bool arrived = mbar_wait_addr(tfull0 + 8 * acc, acc_phase, abort_flag, p.status, kStatusWaitTmemFull, false, p.poll_backoff_ns);
          if (lane == 0) *go = arrived ? 1 : 0;
          __syncwarp();
        }
        named_barrier(bar_id, 128);
        if (*go == 0) break;
        mbar_try_addr(tfull0 + 8 * acc, acc_phase);  // the phase is complete: this observes it for this warp too
      }
      tc_fence_after();
      const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN + cgroup * kGroupColumns;
      // Drain: every chunk of this warp is read, biased and rounded to bf16x2 words first (16 registers per chunk), and
      // the accumulator goes back to the MMA warp right after the last read; the long arithmetic follows. Four-byte
      // outputs cannot be held that compactly: their chunks are finished one by one.
      const bool wide = sw.out_elem == 4;
      auto take_panel = [&]() -> uint32_t {  // a free output panel of this group (of this warp: `own`)
        const uint32_t slot = chunk_it & (sw.panels - 1);
        const uint32_t panel = own ? own_panels + slot * own_bytes : panels + slot * panel_bytes_;
        ++chunk_it;
        if ((own || leader_warp) && elect_one()) {  // the store that last read this panel has finished with it
          if (sw.panels == 2) {
            bulk_wait_read<1>();
          } else {
            bulk_wait_read<0>();
          }
        }
        if (own) {
          __syncwarp();
        } else {
          named_barrier(bar_id, 128);
        }
        return panel;
      };
      auto send_panel = [&](uint32_t panel, int n, bool commit = true) {
        fence_async_proxy();
        if (own) {
          __syncwarp();
          if (store && elect_one()) {
            tma_store_4d(&out_warp_map, panel, n * static_cast<int>(sw.out_elem), x0 + quarter * 32, y0, b);
            bulk_commit();
          }
          return;
        }
        named_barrier(bar_id, 128);
        if (leader_warp && store && elect_one()) {
          tma_store_4d(&out_map, panel, n * static_cast<int>(sw.out_elem), x0, y0, b);
          if (commit) bulk_commit();
        }
      };
      // the pooled panel of the chunk staged in `panel` (every row of it: send_panel's barrier has passed); its store joins
      // the bulk group of the chunk's own store, so the wait that frees an output panel frees the pooled panel of the
      // same parity with it
      auto send_pooled = [&](uint32_t panel, uint32_t parity, int n) {
        const uint32_t pooled = pool_panels + parity * kPoolPanelBytes;
        if (pool_active) {
          uint32_t v[4][4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[i][0]), "=r"(v[i][1]), "=r"(v[i][2]), "=r"(v[i][3]) : "r"(panel + pool_from[i]));
          }
          uint32_t m[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) m[j] = bf16x2_max(bf16x2_max(v[0][j], v[1][j]), bf16x2_max(v[2][j], v[3][j]));
          const uint32_t q0 = int8_pack4(pool_quantizer, bf16_lo(m[0]), bf16_hi(m[0]), bf16_lo(m[1]), bf16_hi(m[1]));
          const uint32_t q1 = int8_pack4(pool_quantizer, bf16_lo(m[2]), bf16_hi(m[2]), bf16_lo(m[3]), bf16_hi(m[3]));
          asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(pooled + pool_to), "r"(q0), "r"(q1) : "memory");
        }
        fence_async_proxy();
        named_barrier(bar_id, 128);
        if (leader_warp && elect_one()) {
          // (a tile past the last whole window, next to an odd edge, has no pooled pixel)
          if (store && (x0 >> 1) < (p.out_w >> 1) && (y0 >> 1) < (p.out_h >> 1)) {
            tma_store_4d(&out_warp_map, pooled, n, x0 >> 1, y0 >> 1, b);
          }
          bulk_commit();
        }
      };
      const int panel_row = own ? lane : row;
      auto release_accumulator = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) {
            mbar_arrive_cluster((tempty0 + 8 * acc) & ~kPeerBit);  // the barrier the leader's MMA thread waits on
          } else {
            mbar_arrive_addr(tempty0 + 8 * acc);
          }
        }
      };
      if (wide) {
#pragma unroll
        for (int g = 0; g < kChunksPerWarp; ++g) {
          const int n = n0 + cgroup * kGroupColumns + g * 32;
          uint32_t raw[32], w[32];
          tmem_load_32(lane_addr + g * 32, raw);
          tmem_load_wait();
          if (g + 1 == kChunksPerWarp) release_accumulator();
          if (n >= n_end) continue;  // uniform over the four warps of this group
          wide_chunk<INT8>(p, sw, raw, n, smem_bias + static_cast<uint32_t>(n) * 4u, a_scale, w);
          const uint32_t panel = take_panel();
          stage_row<32>(panel, panel_row, sw.out_elem, w);
          send_panel(panel, n);
        }
      } else {
        uint32_t q[kChunksPerWarp][16];
#pragma unroll
        for (int g = 0; g < kChunksPerWarp; ++g) {
          const int n = n0 + cgroup * kGroupColumns + g * 32;
          uint32_t raw[32];
          tmem_load_32(lane_addr + g * 32, raw);
          tmem_load_wait();
          if (g + 1 == kChunksPerWarp) release_accumulator();
          if (n < n_end) round_chunk<INT8>(p, sw, raw, n, smem_bias + static_cast<uint32_t>(n) * 4u, a_scale, q[g]);
        }
#pragma unroll
        for (int g = 0; g < kChunksPerWarp; ++g) {
          const int n = n0 + cgroup * kGroupColumns + g * 32;
          if (n >= n_end) continue;  // uniform over the four warps of this group
          uint32_t w[16];
          finish_chunk<INT8>(p, sw, q[g], n, pixel, b, y, x, valid, gelu_table_at(smem_gelu), w);
          const uint32_t parity = chunk_it & 1u;
          const uint32_t panel = take_panel();
          stage_row<16>(panel, panel_row, sw.out_elem, w);
          send_panel(panel, n, !pool);
          if (pool) send_pooled(panel, parity, n);
        }
      }
    }
    if ((own || leader_warp) && elect_one()) bulk_wait_read<0>();
    }
  }

  if (ctl.abort_flag) {
    // a wait ran out somewhere in this CTA: let copies in flight land before shared memory goes away
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync();  // neither CTA leaves while the other may still touch its barriers or tensor memory
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) {
      tmem_dealloc_pair(tmem, kTmemColumns);
    } else {
      tmem_dealloc(tmem, kTmemColumns);
    }
  }
}

// ---- residual MLP of a refiner block: x W1^T + b1 -> GELU -> per-pixel MXFP8 -> W2^T + b2 + residual, one kernel ----------
//
// The 1x1 up conv (C -> 2C, GELU, dynamic requantisation) and the 1x1 down conv (2C -> C, residual) of a block as one
// persistent kernel: the hidden tensor never leaves the SM. Per tile of 128 pixels the MMA warp forms the hidden
// activations 128 channels at a time in one tensor-memory accumulator; sixteen hidden-block warps (32 pixels x 32 hidden
// channels each: exactly one scale block per lane) add the bias, round to bf16, apply the table GELU, form the block's
// E8M0 exponent and write the E4M3 bytes straight into a K-major swizzled operand tile in shared memory, with the scale
// bytes in a 512-byte scale tile beside it; the MMA warp then multiplies that tile into the second accumulator (all C
// output channels) while the next 128 hidden channels are being formed (the first product of block g + 1 is issued
// ahead of the second product of block g, across tile boundaries too). Eight output warps, two per lane quarter of
// tensor memory (they take alternate 32-channel chunks), add bias and residual to the finished second accumulator and
// store bf16 rows; the residual reaches them by TMA, in panels of the output panels' shape, two chunks ahead. The same
// MMAs in the same order as the two separate launches, the same epilogue arithmetic: the same bits. KC = C / 128 (1 or
// 2). 26 warps: TMA producer, MMA issuer, 16 hidden-block warps, 8 output warps. (Four interleaved copies of the GELU
// table, so that lanes of different copies never share a bank, measured no faster: 267 against 263 us.)
constexpr uint32_t kMlpTile = 128u * 128u;  // bytes of one operand tile: 128 rows x 128 bytes of K
constexpr int kMlpOutWarps = 8;  // output warps: two per lane quarter of tensor memory, which take alternate 32-channel chunks
constexpr int kMlpThreads = kThreads + 32 * kMlpOutWarps;
constexpr uint32_t kMlpPanels = 2, kMlpPanelBytes = 32u * 64u;  // output panels per output warp: 32 rows x 32 bf16 channels
constexpr uint32_t kMlpResidualSlots = 2;  // residual panels (same shape) each output warp keeps in flight
struct MlpParams {
  int rows, row_tiles, stages;
  const uint8_t* x_scales;   // per-pixel scales of x: swizzled tiles, KC per row tile
  const uint8_t* w1_scales;  // [2C / 128 row tiles][KC] tiles
  const uint8_t* w2_scales;  // [KC row tiles][2C / 128] tiles
  const __nv_bfloat16* bias1;  // [2C]
  const __nv_bfloat16* bias2;  // [C]
  const __nv_bfloat16* residual;  // [rows, C], dense
  int* status;
  uint32_t poll_backoff_ns;
  int debug;  // probe builds only (FIM_PROBE_BUILD): 1 = no residual loads, 2 = the output warps only drain, 4 = no GELU / requantisation arithmetic
};
__device__ __forceinline__ int probe_flags(const MlpParams& p) { return FIM_PROBE_BUILD ? p.debug : 0; }

struct MlpControl {
  uint64_t w_full[kMaxStages], w_empty[kMaxStages];
  uint64_t x_full, x_empty, acc1_full, acc1_empty, acc2_full, acc2_empty;
  uint64_t h_full[2], h_empty[2];
  uint64_t res_full[kMlpOutWarps][kMlpResidualSlots];  // per output warp: its residual panels have landed
  uint32_t tmem_base;
  int abort_flag;
};


template <int KC>
__global__ void __launch_bounds__(kMlpThreads, 1)
mlp_kernel(const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w1_map, const __grid_constant__ CUtensorMap w2_map,
           const __grid_constant__ CUtensorMap out_map, const __grid_constant__ CUtensorMap res_map, const MlpParams p) {
  constexpr int C = 128 * KC, HB = 2 * KC;            // channels; hidden blocks of 128 channels
  constexpr uint32_t kUnitBytes = KC * kMlpTile;      // a weight unit: W1 rows of one hidden block, or W2 columns of one
  constexpr uint32_t kPanels = kMlpPanels, kPanelBytes = kMlpPanelBytes;
  constexpr uint32_t kAcc1 = 0, kAcc2 = 128, kSfa1 = 128 + C, kSfa2 = kSfa1 + 4 * KC, kSfbRing = kSfa2 + 8;

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) MlpControl ctl;

  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  const uint32_t smem_gelu = base;
  const uint32_t smem_x = base + kGeluSmemBytes;
  const uint32_t smem_w = smem_x + kUnitBytes;
  const uint32_t smem_h = smem_w + static_cast<uint32_t>(p.stages) * kUnitBytes;
  const uint32_t smem_out = smem_h + 2u * kMlpTile;
  const uint32_t smem_res = smem_out + kMlpOutWarps * kPanels * kPanelBytes;  // residual panels: kMlpResidualSlots per output warp
  const uint32_t smem_xsf = smem_res + kMlpOutWarps * kMlpResidualSlots * kPanelBytes;
  const uint32_t smem_wsf = smem_xsf + KC * 512u;
  const uint32_t smem_hsf = smem_wsf + static_cast<uint32_t>(p.stages) * KC * 512u;
  const uint32_t smem_bias1 = smem_hsf + 2u * 512u;  // fp32 [2C]
  const uint32_t smem_bias2 = smem_bias1 + 2u * C * 4u;  // fp32 [C]

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  const int worker = static_cast<int>(blockIdx.x), workers = static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&ctl.w_full[s], 1);
      mbar_init(&ctl.w_empty[s], 1);
    }
    mbar_init(&ctl.x_full, 1);
    mbar_init(&ctl.x_empty, 1);
    mbar_init(&ctl.acc1_full, 1);
    mbar_init(&ctl.acc1_empty, 16);
    mbar_init(&ctl.acc2_full, 1);
    mbar_init(&ctl.acc2_empty, kMlpOutWarps);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ctl.h_full[b], 16);
      mbar_init(&ctl.h_empty[b], 1);
    }
    for (int w = 0; w < kMlpOutWarps; ++w) {
      for (uint32_t i = 0; i < kMlpResidualSlots; ++i) mbar_init(&ctl.res_full[w][i], 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&x_map);
    tma_prefetch_desc(&w1_map);
    tma_prefetch_desc(&w2_map);
    tma_prefetch_desc(&out_map);
    tma_prefetch_desc(&res_map);
  }
  if (warp == 1) {
    tmem_alloc(&ctl.tmem_base, kTmemColumns);
    tmem_relinquish();
  }
  for (int i = threadIdx.x; i < 3 * C; i += kMlpThreads) {  // both biases widened to fp32 once per CTA
    const float value = __bfloat162float(i < 2 * C ? p.bias1[i] : p.bias2[i - 2 * C]);
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(smem_bias1 + i * 4), "f"(value) : "memory");
  }
  for (int i = threadIdx.x; i < kGeluEntries; i += kMlpThreads) {
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(smem_gelu + i * 4), "r"(kGeluTable[i]) : "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl.tmem_base;
  volatile int* abort_flag = &ctl.abort_flag;
  const uint32_t w_full0 = smem_u32(&ctl.w_full[0]), w_empty0 = smem_u32(&ctl.w_empty[0]);
  const uint32_t x_full = smem_u32(&ctl.x_full), x_empty = smem_u32(&ctl.x_empty);
  const uint32_t acc1_full = smem_u32(&ctl.acc1_full), acc1_empty = smem_u32(&ctl.acc1_empty);
  const uint32_t acc2_full = smem_u32(&ctl.acc2_full), acc2_empty = smem_u32(&ctl.acc2_empty);
  const uint32_t h_full0 = smem_u32(&ctl.h_full[0]), h_empty0 = smem_u32(&ctl.h_empty[0]);

  if (warp == 0) {
    // ===== TMA producer: the tile's activations, then its weight units in the order the MMA warp takes them =====
    if (elect_one()) {
      const uint32_t stages = in_register(static_cast<uint32_t>(p.stages));
      uint32_t s = 0, phase = 0;
      bool alive = true;
      // one weight unit into the ring: KC tiles of 128 rows x 128 bytes and their KC scale tiles
      auto unit = [&](const CUtensorMap* map, int k0, int k_step, int row0, int row_step, const uint8_t* scales, int scale_step) {
        if (!mbar_wait_addr(w_empty0 + 8 * s, phase ^ 1, abort_flag, p.status, kStatusWaitEmpty)) {
          alive = false;
          return;
        }
        const uint32_t bar = w_full0 + 8 * s;
        mbar_expect_tx_addr(bar, KC * (kMlpTile + 512u));
#pragma unroll
        for (int i = 0; i < KC; ++i) {
          tma_load_2d_addr(smem_w + s * kUnitBytes + i * kMlpTile, map, bar, k0 + i * k_step, row0 + i * row_step);
          bulk_load_addr(smem_wsf + (s * KC + i) * 512u, scales + static_cast<size_t>(i) * scale_step * 512, 512, bar);
        }
        if (++s == stages) s = 0, phase ^= 1;
      };
      // The units follow the MMA warp's order over the CTA's hidden blocks g = 0, 1, ... (HB per tile, across tiles): the
      // first product of block g + 1 is issued before the second product of block g, so that a block's accumulator is
      // ready when the epilogue warps finish the block before it, also across a tile boundary.
      const int my_tiles = worker < p.row_tiles ? (p.row_tiles - worker + workers - 1) / workers : 0;
      const uint32_t blocks = static_cast<uint32_t>(my_tiles) * HB;
      auto activations = [&](uint32_t t) {  // the t-th tile of this CTA: its pixels and their scale tiles
        if (!mbar_wait_addr(x_empty, (t & 1u) ^ 1u, abort_flag, p.status, kStatusWaitEmpty)) {
          alive = false;
          return;
        }
        const int m = worker + static_cast<int>(t) * workers;
        mbar_expect_tx_addr(x_full, KC * (kMlpTile + 512u));
#pragma unroll
        for (int j = 0; j < KC; ++j) {
          tma_load_4d_addr(smem_x + j * kMlpTile, &x_map, x_full, j * 128, m * kTileM, 0, 0);
          bulk_load_addr(smem_xsf + j * 512u, p.x_scales + (static_cast<size_t>(m) * KC + j) * 512, 512, x_full);
        }
      };
      // W1 rows of hidden block h: K chunks j at columns 128 j; scale tiles (row tile h, K tile j)
      auto first_unit = [&](uint32_t g) {
        const int h = static_cast<int>(g & (HB - 1));
        if (h == 0) activations(g / HB);
        if (alive) unit(&w1_map, 0, 128, h * 128, 0, p.w1_scales + static_cast<size_t>(h) * KC * 512, 1);
      };
      if (blocks != 0) first_unit(0);
      for (uint32_t g = 0; g < blocks && alive; ++g) {
        if (g + 1 < blocks) first_unit(g + 1);
        // W2 columns of hidden block h: row tiles i at rows 128 i; scale tiles (row tile i, K tile h)
        const int h = static_cast<int>(g & (HB - 1));
        if (alive) unit(&w2_map, h * 128, 0, 0, 128, p.w2_scales + static_cast<size_t>(h) * 512, HB);
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer =====
    if (elect_one()) {
      const uint32_t stages = in_register(static_cast<uint32_t>(p.stages));
      const uint64_t x_desc = kmajor_desc(smem_x, 128), w_desc0 = kmajor_desc(smem_w, 128), h_desc0 = kmajor_desc(smem_h, 128);
      const uint64_t xsf_desc = scale_desc(smem_xsf), wsf_desc0 = scale_desc(smem_wsf), hsf_desc0 = scale_desc(smem_hsf);
      const uint32_t idesc1 = idesc_mxf8(128), idesc2 = idesc_mxf8(C);
      uint32_t s = 0, phase = 0;
      bool alive = true;
      const int my_tiles = worker < p.row_tiles ? (p.row_tiles - worker + workers - 1) / workers : 0;
      const uint32_t blocks = static_cast<uint32_t>(my_tiles) * HB;  // hidden blocks of this CTA, across its tiles
      // the first product of hidden block g: acc1 = x W1[block]^T
      auto first = [&](uint32_t g) {
        const uint32_t h = g & (HB - 1), t = g / HB;
        if (h == 0) {
          if (!mbar_wait_addr(x_full, t & 1u, abort_flag, p.status, kStatusWaitFull)) {
            alive = false;
            return;
          }
          tc_fence_after();
#pragma unroll
          for (int j = 0; j < KC; ++j) tc_copy_scales(tmem + kSfa1 + 4 * j, xsf_desc + static_cast<uint64_t>((j * 512u) >> 4));
        }
        if (!mbar_wait_addr(acc1_empty, (g & 1u) ^ 1u, abort_flag, p.status, kStatusWaitTmemEmpty) ||
            !mbar_wait_addr(w_full0 + 8 * s, phase, abort_flag, p.status, kStatusWaitFull)) {
          alive = false;
          return;
        }
        tc_fence_after();
        const uint32_t sfb = tmem + kSfbRing + s * 4 * KC;
#pragma unroll
        for (int j = 0; j < KC; ++j) tc_copy_scales(sfb + 4 * j, wsf_desc0 + static_cast<uint64_t>(((s * KC + j) * 512u) >> 4));
#pragma unroll
        for (int j = 0; j < KC; ++j) {
          const uint64_t a_desc = x_desc + static_cast<uint64_t>((j * kMlpTile) >> 4);
          const uint64_t b_desc = w_desc0 + static_cast<uint64_t>((s * kUnitBytes + j * kMlpTile) >> 4);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t scaled = idesc1 + static_cast<uint32_t>(k) * ((1u << 29) | (1u << 4));
            tc_mma_mxf8(tmem + kAcc1, a_desc + 2 * k, b_desc + 2 * k, scaled, tmem + kSfa1 + 4 * j, sfb + 4 * j, (j > 0 || k > 0) ? 1u : 0u);
          }
        }
        tc_commit(&ctl.w_empty[s]);
        tc_commit(&ctl.acc1_full);
        if (h == HB - 1) tc_commit(&ctl.x_empty);  // the tile's activations have been read for the last time
        if (++s == stages) s = 0, phase ^= 1;
      };
      // the second product of hidden block g: acc2 (+)= H[buffer] x W2 unit
      auto second = [&](uint32_t g) {
        const uint32_t b = g & 1u, h = g & (HB - 1), t = g / HB;
        if (h == 0 && !mbar_wait_addr(acc2_empty, (t & 1u) ^ 1u, abort_flag, p.status, kStatusWaitTmemEmpty)) {
          alive = false;
          return;
        }
        if (!mbar_wait_addr(h_full0 + 8 * b, (g >> 1) & 1u, abort_flag, p.status, kStatusWaitFull) ||
            !mbar_wait_addr(w_full0 + 8 * s, phase, abort_flag, p.status, kStatusWaitFull)) {
          alive = false;
          return;
        }
        tc_fence_after();
        const uint32_t sfa = tmem + kSfa2 + 4 * b, sfb = tmem + kSfbRing + s * 4 * KC;
        tc_copy_scales(sfa, hsf_desc0 + static_cast<uint64_t>((b * 512u) >> 4));
#pragma unroll
        for (int i = 0; i < KC; ++i) tc_copy_scales(sfb + 4 * i, wsf_desc0 + static_cast<uint64_t>(((s * KC + i) * 512u) >> 4));
        const uint64_t a_desc = h_desc0 + static_cast<uint64_t>((b * kMlpTile) >> 4);
        const uint64_t b_desc = w_desc0 + static_cast<uint64_t>((s * kUnitBytes) >> 4);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t scaled = idesc2 + static_cast<uint32_t>(k) * ((1u << 29) | (1u << 4));
          tc_mma_mxf8(tmem + kAcc2, a_desc + 2 * k, b_desc + 2 * k, scaled, sfa, sfb, (k > 0 || h != 0) ? 1u : 0u);
        }
        tc_commit(&ctl.w_empty[s]);
        tc_commit(&ctl.h_empty[b]);
        if (h == HB - 1) tc_commit(&ctl.acc2_full);
        if (++s == stages) s = 0, phase ^= 1;
      };
      // block g + 1's first product goes ahead of block g's second one: its accumulator is then ready when the epilogue
      // warps finish block g, also where block g + 1 opens the next tile
      if (blocks != 0) first(0);
      for (uint32_t g = 0; g < blocks && alive; ++g) {
        if (g + 1 < blocks) first(g + 1);
        if (alive) second(g);
      }
    }
  } else if (warp < 2 + 16) {
    // ===== hidden-block warps: lanes 32 * (w % 4) ... of tensor memory, 32 hidden channels (w - 2) / 4 of every block =====
    const int quarter = warp & 3, group = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const GeluTable gelu2 = gelu_table_at(smem_gelu);
    const uint32_t lane_tmem = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + kAcc1 + group * 32;
    // where this lane's 32 hidden bytes go in a K-major 128-byte-swizzled tile, and its scale byte in the scale tile
    const uint32_t h_row = static_cast<uint32_t>(row) * 128u;
    const uint32_t h_at0 = h_row + (((2u * group) ^ (static_cast<uint32_t>(row) & 7u)) << 4);
    const uint32_t h_at1 = h_row + (((2u * group + 1u) ^ (static_cast<uint32_t>(row) & 7u)) << 4);
    const uint32_t hsf_at = static_cast<uint32_t>(lane * 16 + quarter * 4 + group);
    const int my_tiles = worker < p.row_tiles ? (p.row_tiles - worker + workers - 1) / workers : 0;
    const uint32_t blocks = static_cast<uint32_t>(my_tiles) * HB;
#if FIM_PROBE_BUILD
    long long c_wait = 0, c_load = 0, c_math = 0, c_hwait = 0, c_write = 0;
    const long long c_start = clock64();
#endif
    for (uint32_t g = 0; g < blocks; ++g) {
#if FIM_PROBE_BUILD
      const long long c0 = clock64();
#endif
      if (!mbar_wait_warp(acc1_full, g & 1u, abort_flag, p.status, kStatusWaitTmemFull, true, p.poll_backoff_ns)) break;
      tc_fence_after();
#if FIM_PROBE_BUILD
      const long long c1 = clock64();
#endif
      uint32_t raw[32], r[16];
      tmem_load_32(lane_tmem, raw);
      tmem_load_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_addr(acc1_empty);  // the accumulator goes back before the long arithmetic
#if FIM_PROBE_BUILD
      const long long c2 = clock64();
#endif
      const uint32_t bias_chunk = smem_bias1 + ((g & (HB - 1)) * 128u + static_cast<uint32_t>(group) * 32u) * 4u;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint64_t b0, b1;
        load_bias_pairs(bias_chunk, i, b0, b1);
        float v0, v1, v2, v3;
        unpack2(add2(pack2(__uint_as_float(raw[4 * i]), __uint_as_float(raw[4 * i + 1])), b0), v0, v1);
        unpack2(add2(pack2(__uint_as_float(raw[4 * i + 2]), __uint_as_float(raw[4 * i + 3])), b1), v2, v3);
        r[2 * i] = pack_bf16(v0, v1);
        r[2 * i + 1] = pack_bf16(v2, v3);
      }
      int e = 0;
      uint32_t w[8];
      if (!(probe_flags(p) & 4)) {
#pragma unroll
      for (int i = 0; i < 16; ++i) r[i] = gelu_bf16x2(r[i], gelu2);
      uint32_t mx[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) mx[i] = bf16x2_absmax(r[2 * i], r[2 * i + 1]);
#pragma unroll
      for (int i = 0; i < 4; ++i) mx[i] = bf16x2_absmax(mx[2 * i], mx[2 * i + 1]);
      mx[0] = bf16x2_absmax(bf16x2_absmax(mx[0], mx[1]), bf16x2_absmax(mx[2], mx[3]));
      const uint32_t top = max(mx[0] & 0x7FFFu, (mx[0] >> 16) & 0x7FFFu);
      e = e8m0_exponent_bits(top << 16);
      scale_to_e4m3(r, e, w);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = r[i];
      }
      // the operand buffer of this hidden block: free once the second product that last read it has completed
      const uint32_t b = g & 1u;
#if FIM_PROBE_BUILD
      const long long c3 = clock64();
#endif
      if (!mbar_wait_warp(h_empty0 + 8 * b, ((g >> 1) & 1u) ^ 1u, abort_flag, p.status, kStatusWaitEmpty)) break;
#if FIM_PROBE_BUILD
      const long long c4 = clock64();
#endif
      const uint32_t tile_at = smem_h + b * kMlpTile;
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile_at + h_at0), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(tile_at + h_at1), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
      asm volatile("st.shared.u8 [%0], %1;" ::"r"(smem_hsf + b * 512u + hsf_at), "r"(e + 127) : "memory");
      fence_async_proxy();  // the second product reads these bytes through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive_addr(h_full0 + 8 * b);
#if FIM_PROBE_BUILD
      const long long c5 = clock64();
      c_wait += c1 - c0, c_load += c2 - c1, c_math += c3 - c2, c_hwait += c4 - c3, c_write += c5 - c4;
#endif
    }
#if FIM_PROBE_BUILD
    if ((p.debug & 8192) && blockIdx.x == 0 && lane == 0 && (warp == 2 || warp == 17)) {
      printf("hidden warp %d: %u blocks; per block wait %.0f load %.0f math %.0f buffer wait %.0f write %.0f clk; total %lld clk\n", warp, blocks,
             double(c_wait) / blocks, double(c_load) / blocks, double(c_math) / blocks, double(c_hwait) / blocks, double(c_write) / blocks,
             clock64() - c_start);
    }
#endif
  } else {
    // ===== output warps: two per lane quarter; bias, residual and bf16 rows of every other 32-channel chunk of its 32 pixels.
    // Few instructions but a long chain per chunk (tensor-memory load, residual panel, store): warps of their own keep
    // that latency off the hidden-block warps, whose arithmetic is what a tile takes. =====
    const int quarter = warp & 3;
    const uint32_t lane_tmem = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + kAcc2;
    const uint32_t my_panels = smem_out + static_cast<uint32_t>(warp - 18) * kPanels * kPanelBytes;
    // 16-byte slot i of this lane's 64-byte panel row sits at row_at ^ (i << 4) (the swizzle a TMA store of such rows reads)
    const uint32_t row_at = static_cast<uint32_t>(lane) * 64u + ((((static_cast<uint32_t>(lane) * 64u) >> 7) & 3u) << 4);
    constexpr int kShare = kMlpOutWarps / 4;  // warps per lane quarter: warp `turn` of them takes chunks turn, turn + kShare, ...
    constexpr int kChunks = 4 * KC / kShare;   // chunks of a tile this warp handles
    const int turn = (warp - 18) >> 2;
    // The residual of this warp's 32 pixels arrives by TMA, one panel of 32 channels per copy (the shape and swizzle of an
    // output panel), kMlpResidualSlots chunks ahead of its use; rows past the end of the tensor arrive as zeros. The
    // lane that issued a copy is the one that re-issues into the slot after the warp has read it.
    const uint32_t my_res = smem_res + static_cast<uint32_t>(warp - 18) * kMlpResidualSlots * kPanelBytes;
    const uint32_t res_full0 = smem_u32(&ctl.res_full[warp - 18][0]);
    const int my_tiles = worker < p.row_tiles ? (p.row_tiles - worker + workers - 1) / workers : 0;
    const uint32_t chunks = static_cast<uint32_t>(my_tiles) * kChunks;
    const bool load_residual = !(probe_flags(p) & 1);
    auto ask = [&](uint32_t n) {  // chunk n of this CTA's sequence into slot n % slots
      if (n < chunks && elect_one()) {
        const uint32_t slot = n & (kMlpResidualSlots - 1u);
        const int m = worker + static_cast<int>(n / kChunks) * workers, c = static_cast<int>(n % kChunks) * kShare + turn;
        if (load_residual) {
          mbar_expect_tx_addr(res_full0 + 8 * slot, kPanelBytes);
          tma_load_4d_addr(my_res + slot * kPanelBytes, &res_map, res_full0 + 8 * slot, c * 64, m * kTileM + quarter * 32, 0, 0);
        } else {
          mbar_arrive_addr(res_full0 + 8 * slot);
        }
      }
    };
    for (uint32_t n = 0; n < kMlpResidualSlots; ++n) ask(n);
    uint32_t tile_it = 0, chunk_it = 0;
    bool alive = true;
    for (int m = worker; m < p.row_tiles && alive; m += workers, ++tile_it) {
      if (!mbar_wait_warp(acc2_full, tile_it & 1u, abort_flag, p.status, kStatusWaitTmemFull, true, p.poll_backoff_ns)) break;
      tc_fence_after();
#pragma unroll
      for (int mine = 0; mine < kChunks; ++mine) {
        const int c = mine * kShare + turn;
        uint32_t raw[32], r[16];
        tmem_load_32(lane_tmem + c * 32, raw);
        tmem_load_wait();
        if (mine + 1 == kChunks) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_addr(acc2_empty);
        }
        if (probe_flags(p) & 2) continue;
        const uint32_t bias_chunk = smem_bias2 + static_cast<uint32_t>(c * 32) * 4u;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint64_t b0, b1;
          load_bias_pairs(bias_chunk, i, b0, b1);
          float v0, v1, v2, v3;
          unpack2(add2(pack2(__uint_as_float(raw[4 * i]), __uint_as_float(raw[4 * i + 1])), b0), v0, v1);
          unpack2(add2(pack2(__uint_as_float(raw[4 * i + 2]), __uint_as_float(raw[4 * i + 3])), b1), v2, v3);
          r[2 * i] = pack_bf16(v0, v1);
          r[2 * i + 1] = pack_bf16(v2, v3);
        }
        {
          const uint32_t slot = chunk_it & (kMlpResidualSlots - 1u);
          if (!mbar_wait_warp(res_full0 + 8 * slot, (chunk_it / kMlpResidualSlots) & 1u, abort_flag, p.status, kStatusWaitFull)) {
            alive = false;
            break;
          }
          const uint32_t from = my_res + slot * kPanelBytes + row_at;
#pragma unroll
          for (uint32_t i = 0; i < 4; ++i) {
            uint4 v;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(from ^ (i << 4)));
            r[4 * i] = bf16x2_add(r[4 * i], v.x);
            r[4 * i + 1] = bf16x2_add(r[4 * i + 1], v.y);
            r[4 * i + 2] = bf16x2_add(r[4 * i + 2], v.z);
            r[4 * i + 3] = bf16x2_add(r[4 * i + 3], v.w);
          }
          __syncwarp();  // every lane has read the slot
          ask(chunk_it + kMlpResidualSlots);
        }
        const uint32_t panel = my_panels + (chunk_it & (kPanels - 1u)) * kPanelBytes;
        ++chunk_it;
        const uint32_t at = panel + row_at;
        if (elect_one()) bulk_wait_read<kPanels - 1>();  // the store that last read this panel has finished with it
        __syncwarp();
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(at ^ (i << 4)), "r"(r[4 * i]), "r"(r[4 * i + 1]), "r"(r[4 * i + 2]),
                       "r"(r[4 * i + 3])
                       : "memory");
        }
        fence_async_proxy();
        __syncwarp();
        if (elect_one()) {
          tma_store_4d(&out_map, panel, c * 64, m * kTileM + quarter * 32, 0, 0);
          bulk_commit();
        }
      }
    }
    if (elect_one()) bulk_wait_read<0>();
  }

  if (ctl.abort_flag) {
    // a wait ran out somewhere in this CTA: let copies in flight land before shared memory goes away
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemColumns);
  }
}

// ---- host ------------------------------------------------------------------------------------------------------------

int g_forced_block_n = 0;
int g_max_ctas = 0;
int g_debug_flags = 0;

struct Plan {
  int tile_h, tile_w, block_n, block_k, stages, ctas, panels_per_half;
  int tiles_x, tiles_y, tiles_n, total_tiles;
  bool flat;
  bool pair;  // clusters of two CTAs driving one cta_group::2 instruction stream
  bool convert = false;    // bf16 activations, quantised on chip
  bool resident_b = false; // the whole weight matrix stays in shared memory (one output-channel tile, small K)
  int fixed_epilogue = 0;  // kEpiLean | switches when one of the compile-time epilogues serves this call, else 0
  int out_h, out_w;
  size_t smem;
};

int out_elem_bytes(int out_mode) {
  switch (out_mode) {
    case FIM_OUT_BF16: return 2;
    case FIM_OUT_F32:
    case FIM_OUT_INT32: return 4;
    default: return 1;
  }
}

int make_plan(const FimConvGeometry& g, int fmt, bool per_pixel, bool allow_flat, int out_elem, bool gelu, Plan* plan,
              bool convert = false, bool pool = false) {
  // `g.cin` counts bytes of K per tap here (a BF16 layer arrives with its channel count doubled)
  const bool int8 = fmt == kFmtI8, scaled = fmt == kFmtMx;
  if (g.batch <= 0 || g.height <= 0 || g.width <= 0 || g.cin <= 0 || g.cout <= 0) return kBadArgument;
  if (g.cin % 32 || g.cout % 32) return kUnsupported;
  if (g.stride_h < 1 || g.stride_w < 1) return kBadArgument;
  if (g.stride_h > 4 || g.stride_w > 4) return kUnsupported;
  if (g.kh < 1 || g.kw < 1 || g.dil_h < 1 || g.dil_w < 1 || g.pad_h < 0 || g.pad_w < 0) return kBadArgument;
  const int span_h = g.height + 2 * g.pad_h - g.dil_h * (g.kh - 1), span_w = g.width + 2 * g.pad_w - g.dil_w * (g.kw - 1);
  if (span_h <= 0 || span_w <= 0) return kBadArgument;
  const int out_h = (span_h - 1) / g.stride_h + 1, out_w = (span_w - 1) / g.stride_w + 1;
  const bool pointwise = g.kh == 1 && g.kw == 1 && g.pad_h == 0 && g.pad_w == 0 && g.stride_h == 1 && g.stride_w == 1;
  if (per_pixel && !(pointwise && allow_flat)) return kUnsupported;
  if (scaled && !per_pixel && (g.cin + 127) / 128 > kMaxStaticScaleTiles) return kUnsupported;
  Plan pl;
  pl.out_h = out_h, pl.out_w = out_w;
  pl.block_k = g.cin % 128 == 0 ? 128 : (g.cin % 64 == 0 ? 64 : 32);
  // Output-channel tile: 256 halves the activation re-reads of a wide layer; narrower layers keep two accumulators in
  // tensor memory so the epilogue overlaps the next tile.
  // A block-scaled 1x1 layer that writes at least as much as it reads is bound by its epilogue: the wide tile halves the
  // per-tile work of the epilogue warps (measured 5 to 16 % faster at 256 and 512 input channels); one that reads more
  // than it writes keeps the narrow tile, whose smaller stages hold more activation bytes in flight.
  const bool wide_pointwise = fmt == kFmtMx && pointwise && allow_flat && g.cout >= g.cin;
  int bn = g.cout <= 64 ? 64 : (g.cout % 256 == 0 && (g.kh * g.kw * g.cin >= 1024 || wide_pointwise) ? 256 : 128);
  if (g_forced_block_n == 256 && g.cout > 128) bn = 256;
  if (g_forced_block_n == 128 && g.cout > 64) bn = 128;
  if (g_forced_block_n == 64) bn = 64;
  if (fmt == kFmtBf16 && bn == 256) bn = 128;  // BF16 layers on this path are narrow pointwise products
  if (bn == 64 && g.cout > 64 && scaled) bn = 128;  // a 64-wide tile may only start at column 0 of its scale tile
  pl.block_n = bn;
  pl.flat = pointwise && allow_flat;
  pl.convert = convert;
  if (convert && !(fmt == kFmtMx && pl.flat && pl.block_k == 128)) return kUnsupported;
  if (pl.flat) {
    pl.tile_h = 1, pl.tile_w = kTileM;
    const long long rows = static_cast<long long>(g.batch) * out_h * out_w;
    const long long tiles = (rows + kTileM - 1) / kTileM;
    if (tiles > 0x3fffffffLL) return kUnsupported;
    pl.tiles_x = static_cast<int>(tiles), pl.tiles_y = 1;
  } else {
    double best = -1.0;
    pl.tile_h = 1, pl.tile_w = kTileM;
    for (int tw = 4; tw <= kTileM; ++tw) {
      const int th = kTileM / tw;
      if (pool && ((tw | th) & 1)) continue;  // every 2x2 pooling window inside one tile
      if (tw * g.stride_w > 256 || th * g.stride_h > 256) continue;  // a TMA box spans at most 256 positions per dimension
      const double covered = static_cast<double>(ceil_div(out_w, tw)) * ceil_div(out_h, th) * kTileM;
      const double eff = static_cast<double>(out_w) * out_h / covered;
      if (eff > best + 1e-9 || (eff > best - 1e-9 && tw > pl.tile_w)) {
        best = eff;
        pl.tile_h = th, pl.tile_w = tw;
      }
    }
    pl.tiles_x = ceil_div(out_w, pl.tile_w), pl.tiles_y = ceil_div(out_h, pl.tile_h);
  }
  pl.tiles_n = ceil_div(g.cout, bn);
  const long long row_tiles = static_cast<long long>(pl.tiles_x) * pl.tiles_y * (pl.flat ? 1 : g.batch);
  // CTA pairs for the wide, compute-bound INT8 tiles: a pair owns two consecutive row tiles (the last one may not exist:
  // its loads are zero-filled and its stores clipped). The block-scaled form is correct too but measured slower than
  // single CTAs (its scale copies serialise the pair's tensor pipes): it only runs when asked for (tuning flag 128).
  pl.pair = bn == 256 && row_tiles >= 2 && !(g_debug_flags & 64) && (int8 || (g_debug_flags & 128)) && !convert;
  // A 128-wide block-scaled tile moves as many operand bytes through shared memory per MMA as the tensor pipe takes
  // twice as fast; a pair halves the weight bytes per CTA (64 rows each). Worth it for a spatial conv with many tiles
  // (3x3 128 -> 128 at 400 x 400: 118 -> 107 us), not for a small one, not for a flat 1x1 layer, whose short epilogue
  // serves single CTAs only, and not with a GELU epilogue (117 -> 123 us: the two epilogues of a pair release one shared
  // accumulator barrier, and the heavier they are the longer the MMAs wait for the slower one); flag 16384 forces it.
  if (bn == 128 && scaled && pl.block_k == 128 && row_tiles >= 2 && !convert && !(g_debug_flags & 64) &&
      ((g_debug_flags & 16384) || (!pl.flat && !gelu && row_tiles >= 8LL * sm_count()))) {
    pl.pair = true;
  }
  const long long total = (pl.pair ? (row_tiles + 1) / 2 : row_tiles) * pl.tiles_n;
  if (total > 0x3fffffffLL) return kUnsupported;
  pl.total_tiles = static_cast<int>(total);
  // shared memory: alignment slack + output panels + static activation-scale tiles + the stage ring. A layer with few
  // K iterations per tile is bound by its stores: it gets more panels in flight; a long main loop gets the stages.
  const int k_iters = g.kh * g.kw * (g.cin / pl.block_k);
  pl.panels_per_half = out_elem == 4 || convert ? 1 : 2;  // 16 KB panels of a 4-byte output: one per column group
  (void)k_iters;
  const int stage_bytes = kTileM * pl.block_k + (pl.pair ? bn / 2 : bn) * pl.block_k + scale_tiles_b(bn) * 512 + 512;
  const int bias_bytes = pl.tiles_n * bn * 4;
  if (bias_bytes > 32 * 1024) return kUnsupported;
  const int epilogue_groups = 4;  // four-warp groups with output panels of their own
  const int gelu_bytes = gelu ? static_cast<int>(kGeluSmemBytes) : 0;
  const int raw_bytes = convert ? 1024 + kRawStages * static_cast<int>(kRawBytes) : 0;  // landing ring (+ its alignment)
  const int pool_bytes = pool ? epilogue_groups * 2 * static_cast<int>(kPoolPanelBytes) : 0;
  const int fixed = 1024 + epilogue_groups * pl.panels_per_half * 4096 * out_elem + ((g.cin + 127) / 128) * 512 + bias_bytes + gelu_bytes +
                    raw_bytes + pool_bytes;
  pl.stages = (kSmemLimit - fixed) / stage_bytes;
  if (pl.stages > kMaxStages) pl.stages = kMaxStages;
  if (pl.stages < 2) return kUnsupported;
  pl.smem = static_cast<size_t>(fixed) + static_cast<size_t>(pl.stages) * stage_bytes;
  // One output-channel tile and a weight matrix that fits beside at least three activation stages: the weights (and their
  // scale tiles) are copied once per CTA instead of once per tile and K step, which leaves the producer one copy per K
  // step. Used for 64-wide tiles, where the producer's copies are what a K step waits for (3x3 64 -> 64: 377 -> 345 us);
  // measured without gain at 128 and slower at 256 columns (1x1 128 -> 256: 163 -> 175 us), flag 4096 asks for it there.
  if (pl.tiles_n == 1 && !pl.pair && !convert && g.cout <= bn && !(g_debug_flags & 2048) && (bn == 64 || (g_debug_flags & 4096))) {
    const int all_b = k_iters * (bn * pl.block_k + scale_tiles_b(bn) * 512);
    const int a_stage = kTileM * pl.block_k + 512;
    if (fixed + all_b + 3 * a_stage <= kSmemLimit) {
      pl.resident_b = true;
      pl.stages = (kSmemLimit - fixed - all_b) / a_stage;
      if (pl.stages > kMaxStages) pl.stages = kMaxStages;
      pl.smem = static_cast<size_t>(fixed) + all_b + static_cast<size_t>(pl.stages) * a_stage;
    }
  }
  const int device_sms = sm_count();
  const int sms = g_max_ctas > 0 && g_max_ctas < device_sms ? g_max_ctas : device_sms;
  pl.ctas = pl.total_tiles < sms ? pl.total_tiles : sms;
  if (pl.pair) pl.ctas = 2 * (pl.total_tiles < sms / 2 ? pl.total_tiles : sms / 2);
  *plan = pl;
  return kOk;
}

// What the persistent CTAs walk: the tile list (with the last partial round cut into half-width tiles when that halves
// its duration), the tile order and how many K iterations keep their weight scales resident in tensor memory.
struct Schedule {
  int total_tiles, full_tiles, resident_k, n_major;
};

Schedule make_schedule(const FimConvGeometry& g, const Plan& pl, bool int8, bool per_pixel) {
  Schedule sc;
  sc.total_tiles = pl.total_tiles, sc.full_tiles = pl.total_tiles, sc.resident_k = 0, sc.n_major = 0;
  const int walkers = pl.pair ? pl.ctas / 2 : pl.ctas;  // a CTA pair walks the tile list as one
  if (pl.block_n == 256 && (!pl.pair || int8) && pl.total_tiles > walkers) {
    // the last round of the persistent CTAs: when at most half of them would have a tile, two half-width tiles each
    // finish it in half the time (block-scaled CTA pairs keep whole tiles: their scale tiles are laid out for 256 columns)
    const int rest = pl.total_tiles % walkers;
    if (rest > 0 && 2 * rest <= walkers && !(g_debug_flags & 16)) {
      sc.full_tiles = pl.total_tiles - rest;
      sc.total_tiles = sc.full_tiles + 2 * rest;
    }
  }
  if (!int8 && pl.block_k == 128 && !(g_debug_flags & 256)) {
    // Tensor-memory columns left after the accumulators, the per-stage scale sets and the activation scales hold the
    // weight scales of the first K iterations for as long as consecutive tiles of a CTA share their output channels.
    // That needs the row tiles of one channel tile to follow each other, which re-reads the activations once per channel
    // tile: fine when they stay in L2 or the layer is compute-bound, not for a wide memory-bound layer.
    const int sfb_columns = pl.block_n < 128 ? 4 : pl.block_n / 32;
    const int sfa_columns = 4 * (per_pixel ? pl.stages : (g.cin + 127) / 128);
    const int room = 512 - acc_stages(pl.block_n) * pl.block_n - pl.stages * sfb_columns - sfa_columns;
    const int k_iters = g.kh * g.kw * (g.cin / pl.block_k);
    const long long activation_bytes = static_cast<long long>(g.batch) * g.height * g.width * g.cin;
    const bool cheap_reread = pl.tiles_n == 1 || k_iters >= 8 || activation_bytes <= (48LL << 20);
    if (room >= sfb_columns && cheap_reread) {
      sc.resident_k = room / sfb_columns < k_iters ? room / sfb_columns : k_iters;
      sc.n_major = 1;
    }
  }
  return sc;
}

struct ConvMaps {
  CUtensorMap act, weight, out, sfb, sfa, out_warp;
};

template <int FMT, int BN, int BK, bool PAIR, int EPI = 0, bool CONVERT = false>
int launch_conv(const ConvMaps& maps, const ConvParams& p, const Plan& pl, cudaStream_t stream) {
  // the shared-memory opt-in is a per-device attribute of the function: set once per device and instantiation
  static bool configured[kMaxDevices] = {};
  const int device = current_device();
  if (device < 0 || device >= kMaxDevices || !configured[device]) {
    const cudaError_t e =
        cudaFuncSetAttribute(conv_kernel<FMT, BN, BK, PAIR, EPI, CONVERT>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (device >= 0 && device < kMaxDevices) configured[device] = true;
  }
  if (PAIR) {
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(pl.ctas), 1, 1);
    config.blockDim = dim3(kThreads, 1, 1);
    config.dynamicSmemBytes = pl.smem;
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2, attribute.val.clusterDim.y = 1, attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&config, conv_kernel<FMT, BN, BK, PAIR, EPI, CONVERT>, maps.act, maps.weight, maps.out, maps.sfb,
                                               maps.sfa, maps.out_warp, p));
  }
  conv_kernel<FMT, BN, BK, PAIR, EPI, CONVERT><<<pl.ctas, CONVERT ? kConvertThreads : kThreads, pl.smem, stream>>>(maps.act, maps.weight, maps.out, maps.sfb, maps.sfa, maps.out_warp, p);
  return static_cast<int>(cudaGetLastError());
}

template <int FMT, int BN>
int launch_conv_k(const ConvMaps& maps, const ConvParams& p, const Plan& pl, cudaStream_t stream) {
  // the general epilogue with its switches fixed at compile time, for the layers measured most: a block-scaled conv with
  // bias, GELU and static requantisation at each tile width's usual K step, and the INT8 conv with bias and bf16 output
  constexpr int kGeluStatic = kEpiFixed | kEpiGelu | kEpiStatic;
  if constexpr (FMT == kFmtMx) {
    if (pl.convert) {  // bf16 activations quantised on chip (flat layers, 128 channels per K step)
      if constexpr (BN >= 128) {
        if (pl.fixed_epilogue == kEpiLean) return launch_conv<FMT, BN, 128, false, kEpiLean, true>(maps, p, pl, stream);
      }
      return launch_conv<FMT, BN, 128, false, 0, true>(maps, p, pl, stream);
    }
  }
  if constexpr (FMT == kFmtMx) {
    if (pl.fixed_epilogue == kGeluStatic && !pl.pair) {
      if constexpr (BN == 64) {
        if (pl.block_k == 64) return launch_conv<FMT, BN, 64, false, kGeluStatic>(maps, p, pl, stream);
      } else {
        if (pl.block_k == 128) return launch_conv<FMT, BN, 128, false, kGeluStatic>(maps, p, pl, stream);
      }
    }
  }
  if constexpr (FMT == kFmtI8) {
    if (pl.fixed_epilogue == kEpiPool) {  // the general epilogue + the pooled second output
      if (pl.block_k != 128 && pl.block_k != 64) return kUnsupported;
      if constexpr (BN == 256) {
        if (pl.pair) {
          return pl.block_k == 128 ? launch_conv<FMT, BN, 128, true, kEpiPool>(maps, p, pl, stream)
                                   : launch_conv<FMT, BN, 64, true, kEpiPool>(maps, p, pl, stream);
        }
      }
      return pl.block_k == 128 ? launch_conv<FMT, BN, 128, false, kEpiPool>(maps, p, pl, stream)
                               : launch_conv<FMT, BN, 64, false, kEpiPool>(maps, p, pl, stream);
    }
  }
  if constexpr (FMT == kFmtI8 && BN == 256) {
    if (pl.fixed_epilogue == kEpiFixed && pl.pair && pl.block_k == 128) {
      return launch_conv<FMT, BN, 128, true, kEpiFixed>(maps, p, pl, stream);
    }
  }
  if constexpr (BN == 128 && FMT == kFmtMx) {
    if (pl.pair) {
      if (pl.fixed_epilogue == kGeluStatic) return launch_conv<FMT, BN, 128, true, kGeluStatic>(maps, p, pl, stream);
      return launch_conv<FMT, BN, 128, true>(maps, p, pl, stream);
    }
  }
  if constexpr (BN == 256 && FMT != kFmtBf16) {
    if (pl.pair) {
      if (pl.block_k == 128) return launch_conv<FMT, BN, 128, true>(maps, p, pl, stream);
      if (pl.block_k == 64) return launch_conv<FMT, BN, 64, true>(maps, p, pl, stream);
      return launch_conv<FMT, BN, 32, true>(maps, p, pl, stream);
    }
  }
  if constexpr (FMT == kFmtMx && BN >= 128) {
    if (pl.block_k == 128) {  // the epilogues fixed at compile time: the three 1x1 layers of a refiner block
      switch (pl.fixed_epilogue) {
        case kEpiLean: return launch_conv<FMT, BN, 128, false, kEpiLean>(maps, p, pl, stream);
        case kEpiLean | kEpiResidual: return launch_conv<FMT, BN, 128, false, kEpiLean | kEpiResidual>(maps, p, pl, stream);
        case kEpiLean | kEpiGelu | kEpiDynamic:
          return launch_conv<FMT, BN, 128, false, kEpiLean | kEpiGelu | kEpiDynamic>(maps, p, pl, stream);
        default: break;
      }
    }
  }
  if (pl.block_k == 128) return launch_conv<FMT, BN, 128, false>(maps, p, pl, stream);
  if (pl.block_k == 64) return launch_conv<FMT, BN, 64, false>(maps, p, pl, stream);
  return launch_conv<FMT, BN, 32, false>(maps, p, pl, stream);
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

int run_conv(int fmt, const void* x, const int8_t* act_exponent, const void* act_scales, const void* weight,
             const void* weight_scales, const float* a_scale, const float* w_scale, const FimConvGeometry* geometry,
             const FimConvEpilogue* ep, void* out, int* status, void* stream, bool convert = false, void* pooled = nullptr) {
  const bool int8 = fmt == kFmtI8;
  if (geometry == nullptr || ep == nullptr) return kBadArgument;
  if (geometry->batch == 0 || geometry->height == 0 || geometry->width == 0) return kOk;
  if (x == nullptr || weight == nullptr || out == nullptr) return kBadArgument;
  if (ep->act < 0 || ep->act > 3 || ep->out_mode < 0 || ep->out_mode > 5) return kBadArgument;
  // the kernel counts K in bytes: a BF16 layer is a layer of 2 * Cin one-byte channels
  FimConvGeometry bytes = *geometry;
  if (fmt == kFmtBf16) {
    if (geometry->cin % 16) return kUnsupported;
    bytes.cin = 2 * geometry->cin;
  }
  const FimConvGeometry* g = &bytes;
  if (int8) {
    if (ep->out_mode != FIM_OUT_INT32 && (a_scale == nullptr || w_scale == nullptr)) return kBadArgument;
    if (ep->out_mode != FIM_OUT_BF16 && ep->out_mode != FIM_OUT_INT8 && ep->out_mode != FIM_OUT_INT32) return kBadArgument;
    if (ep->out_mode == FIM_OUT_INT8 && ep->out_scale == nullptr) return kBadArgument;
  } else if (fmt == kFmtBf16) {
    if (ep->out_mode != FIM_OUT_BF16 && ep->out_mode != FIM_OUT_F32) return kBadArgument;
  } else {
    if (weight_scales == nullptr) return kBadArgument;
    if (convert ? act_scales != nullptr : (act_exponent == nullptr) == (act_scales == nullptr)) return kBadArgument;
    if (ep->out_mode == FIM_OUT_INT8 || ep->out_mode == FIM_OUT_INT32) return kBadArgument;
    if (ep->out_mode == FIM_OUT_E4M3_STATIC && ep->out_exponent == nullptr) return kBadArgument;
    if (ep->out_mode == FIM_OUT_E4M3_DYNAMIC && ep->out_scales == nullptr) return kBadArgument;
  }
  if (!aligned16(x) || !aligned16(weight) || !aligned16(out) || (ep->bias && !aligned16(ep->bias)) ||
      (weight_scales && !aligned16(weight_scales)) || (act_scales && !aligned16(act_scales)) || (w_scale && !aligned16(w_scale))) {
    return kBadLayout;
  }
  const bool pool = pooled != nullptr;
  if (pool && !(int8 && ep->out_mode == FIM_OUT_BF16 && ep->out_scale != nullptr && aligned16(pooled))) return kBadArgument;
  if (pool && geometry->cin % 64) return kUnsupported;
  const int out_elem = out_elem_bytes(ep->out_mode);
  // one activation scale per pixel and 32 channels: given by the caller, or formed on chip from bf16 activations
  const bool per_pixel = act_scales != nullptr || (convert && act_exponent == nullptr);

  // a 1x1 conv is a plain GEMM over flattened pixels when the residual (if any) is dense NHWC
  bool allow_flat = !pool;  // pooling windows need the tile to be a patch of the image
  Plan pl;
  if (allow_flat) {
    Plan probe;
    const int rc0 = make_plan(*g, fmt, per_pixel, true, out_elem, ep->act == FIM_ACT_GELU, &probe, convert);
    if (rc0 != kOk) return rc0;
    if (probe.flat && ep->residual != nullptr) {
      const long long c = ep->res_stride[3], xs = ep->res_stride[2], ys = ep->res_stride[1], bs = ep->res_stride[0];
      const bool dense = c == 1 && ys == xs * probe.out_w && bs == ys * probe.out_h;
      if (!dense) allow_flat = false;
    }
  }
  const int rc = make_plan(*g, fmt, per_pixel, allow_flat, out_elem, ep->act == FIM_ACT_GELU, &pl, convert, pool);
  if (rc != kOk) return rc;
  if (pool && (pl.out_h < 2 || pl.out_w < 2 || pl.panels_per_half != 2)) return kUnsupported;  // no whole window: nothing to pool

  const Schedule sc = make_schedule(*g, pl, fmt != kFmtMx, per_pixel);
  ConvParams p;
  p.cin = g->cin, p.cout = g->cout;
  p.out_h = pl.out_h, p.out_w = pl.out_w;
  p.kh = g->kh, p.kw = g->kw, p.pad_h = g->pad_h, p.pad_w = g->pad_w, p.dil_h = g->dil_h, p.dil_w = g->dil_w;
  p.stride_h = g->stride_h, p.stride_w = g->stride_w;
  p.tile_h = pl.tile_h, p.tile_w = pl.tile_w, p.tiles_x = pl.tiles_x, p.tiles_y = pl.tiles_y, p.tiles_n = pl.tiles_n;
  p.total_tiles = sc.total_tiles;
  p.full_tiles = sc.full_tiles;
  p.batch = pl.flat ? 1 : g->batch;
  p.k_chunks = g->cin / pl.block_k, p.stages = pl.stages, p.panels_per_half = pl.panels_per_half;
  p.row_tiles = pl.total_tiles / pl.tiles_n;
  p.div_row_tiles = make_fastdiv(p.row_tiles), p.div_tiles_n = make_fastdiv(pl.tiles_n);
  p.div_tiles_x = make_fastdiv(pl.tiles_x), p.div_tiles_y = make_fastdiv(pl.tiles_y);
  p.resident_k = sc.resident_k, p.n_major = sc.n_major;
  p.act_exponent = act_exponent;
  p.convert_static = convert && act_exponent != nullptr ? 1 : 0;
  p.weights_resident = pl.resident_b ? 1 : 0;
  p.b_slots = pl.resident_b ? g->kh * g->kw * (g->cin / pl.block_k) : pl.stages;
  p.act_scales = static_cast<const uint8_t*>(act_scales);
  p.act_scale_tiles = (g->cin / 32 + 3) / 4;
  p.weight_scales = static_cast<const uint8_t*>(weight_scales);
  p.weight_scale_tiles = (g->kh * g->kw * g->cin / 32 + 3) / 4;
  p.weight_row_tiles = (g->cout + 127) / 128;
  p.a_scale = a_scale, p.w_scale = w_scale;
  p.bias = static_cast<const __nv_bfloat16*>(ep->bias);
  p.residual = static_cast<const __nv_bfloat16*>(ep->residual);
  for (int i = 0; i < 4; ++i) p.res_stride[i] = ep->res_stride[i];
  p.res_channels = ep->res_channels > 0 ? ep->res_channels : g->cout;
  p.act = ep->act, p.out_mode = ep->out_mode, p.out_elem = out_elem;
  p.out_exponent = ep->out_exponent;
  p.out_scales = static_cast<uint8_t*>(ep->out_scales);
  p.out_scale = ep->out_scale;
  p.pool = pool ? 1 : 0;
  p.status = status;
  p.debug = g_debug_flags;
  p.poll_backoff_ns = (g_debug_flags & 32) ? 0u : 200u;

  // tensor maps: activations [B, H, W, Cin] and outputs [B, Ho, Wo, Cout * elem bytes] (a flat 1x1 conv sees one row of
  // B*H*W pixels), weights [Cout, K]
  long long in_b = g->batch, in_h = g->height, in_w = g->width, o_b = g->batch, o_h = pl.out_h, o_w = pl.out_w;
  if (pl.flat) {
    in_w = o_w = static_cast<long long>(g->batch) * g->height * g->width;
    in_h = o_h = 1, in_b = o_b = 1;
    p.out_h = 1, p.out_w = static_cast<int>(o_w);
    if (p.residual != nullptr) p.res_stride[0] = 0, p.res_stride[1] = 0;  // dense: the flat column index addresses it
  }
  ConvMaps maps;
  CUtensorMap& act_map = maps.act;
  CUtensorMap& weight_map = maps.weight;
  CUtensorMap& out_map = maps.out;
  if (convert) {
    // bf16 rows of the pixel matrix, landing as they lie in memory (256 bytes per row of a 128-channel box)
    const uint64_t dims[4] = {static_cast<uint64_t>(g->cin), static_cast<uint64_t>(in_w), 1, 1};
    const uint64_t strides[3] = {static_cast<uint64_t>(g->cin) * 2, static_cast<uint64_t>(in_w) * g->cin * 2,
                                 static_cast<uint64_t>(in_w) * g->cin * 2};
    const uint32_t box[4] = {128, static_cast<uint32_t>(kTileM), 1, 1};
    const int rcm = make_tensor_map(&act_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rcm != kOk) return rcm;
  } else {
    const uint64_t dims[4] = {static_cast<uint64_t>(g->cin), static_cast<uint64_t>(in_w), static_cast<uint64_t>(in_h),
                              static_cast<uint64_t>(in_b)};
    const uint64_t strides[3] = {static_cast<uint64_t>(g->cin), static_cast<uint64_t>(in_w) * g->cin,
                                 static_cast<uint64_t>(in_h) * in_w * g->cin};
    // a strided conv reads every stride-th pixel of a box stride times as wide: the copy lands densely in shared memory
    const uint32_t box[4] = {static_cast<uint32_t>(pl.block_k), static_cast<uint32_t>(pl.tile_w * g->stride_w),
                             static_cast<uint32_t>(pl.tile_h * g->stride_h), 1};
    const uint32_t steps[4] = {1, static_cast<uint32_t>(g->stride_w), static_cast<uint32_t>(g->stride_h), 1};
    const int rcm = make_tensor_map(&act_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, x, dims, strides, box, swizzle_for_bytes(pl.block_k),
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, steps);
    if (rcm != kOk) return rcm;
  }
  {
    const uint64_t k_total = static_cast<uint64_t>(g->kh) * g->kw * g->cin;
    const uint64_t dims[2] = {k_total, static_cast<uint64_t>(g->cout)};
    const uint64_t strides[1] = {k_total};
    // rows per copy: a whole narrow tile, 128 rows of a wide one, or the half of the tile a CTA of a pair holds
    const uint32_t box[2] = {static_cast<uint32_t>(pl.block_k), static_cast<uint32_t>(pl.pair ? pl.block_n / 2 : (pl.block_n < 128 ? pl.block_n : 128))};
    const int rcm = make_tensor_map(&weight_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, weight, dims, strides, box, swizzle_for_bytes(pl.block_k));
    if (rcm != kOk) return rcm;
  }
  {
    const uint64_t row = static_cast<uint64_t>(g->cout) * out_elem;
    const uint64_t dims[4] = {row, static_cast<uint64_t>(o_w), static_cast<uint64_t>(o_h), static_cast<uint64_t>(o_b)};
    const uint64_t strides[3] = {row, static_cast<uint64_t>(o_w) * row, static_cast<uint64_t>(o_h) * o_w * row};
    const uint32_t box[4] = {static_cast<uint32_t>(32 * out_elem), static_cast<uint32_t>(pl.tile_w), static_cast<uint32_t>(pl.tile_h), 1};
    const int rcm = make_tensor_map(&out_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, out, dims, strides, box, swizzle_for_bytes(32 * out_elem));
    if (rcm != kOk) return rcm;
    maps.out_warp = out_map;
    p.warp_panels = 0;
    if (pl.flat && !(g_debug_flags & 512)) {  // one store per warp: 32 rows of the pixel matrix x 32 channels
      const uint32_t warp_box[4] = {static_cast<uint32_t>(32 * out_elem), 32, 1, 1};
      const int rcw = make_tensor_map(&maps.out_warp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, out, dims, strides, warp_box,
                                      swizzle_for_bytes(32 * out_elem));
      if (rcw != kOk) return rcw;
      p.warp_panels = 1;
    }
    if (pool) {  // the pooled output [B, Ho / 2, Wo / 2, Cout] INT8, stored in boxes of a quarter tile x 32 channels
      const uint64_t prow = static_cast<uint64_t>(g->cout), ph = static_cast<uint64_t>(pl.out_h / 2), pw = static_cast<uint64_t>(pl.out_w / 2);
      const uint64_t pdims[4] = {prow, pw, ph, static_cast<uint64_t>(o_b)};
      const uint64_t pstrides[3] = {prow, pw * prow, ph * pw * prow};
      const uint32_t pbox[4] = {32, static_cast<uint32_t>(pl.tile_w / 2), static_cast<uint32_t>(pl.tile_h / 2), 1};
      const int rcp = make_tensor_map(&maps.out_warp, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, pooled, pdims, pstrides, pbox, CU_TENSOR_MAP_SWIZZLE_NONE);
      if (rcp != kOk) return rcp;
    }
  }
  if (fmt == kFmtMx && p.warp_panels && !pl.pair && pl.block_n >= 128 && pl.block_k == 128 && p.bias != nullptr &&
      !(g_debug_flags & 1024)) {
    const bool plain = p.act == kActNone && p.out_mode == FIM_OUT_BF16;
    const bool res_ok = p.residual != nullptr && p.res_stride[3] == 1 && p.res_channels >= p.cout && p.res_stride[2] % 8 == 0 &&
                        reinterpret_cast<uintptr_t>(p.residual) % 16 == 0;
    if (plain && p.residual == nullptr) pl.fixed_epilogue = kEpiLean;
    if (plain && res_ok) pl.fixed_epilogue = kEpiLean | kEpiResidual;
    if (p.act == kActGelu && p.out_mode == FIM_OUT_E4M3_DYNAMIC && p.residual == nullptr) {
      pl.fixed_epilogue = kEpiLean | kEpiGelu | kEpiDynamic;
    }
  }
  if (pl.fixed_epilogue == 0 && p.bias != nullptr && p.residual == nullptr && pl.panels_per_half == 2 && !(g_debug_flags & 1024)) {
    if (fmt == kFmtMx && p.act == kActGelu && p.out_mode == FIM_OUT_E4M3_STATIC) pl.fixed_epilogue = kEpiFixed | kEpiGelu | kEpiStatic;
    if (fmt == kFmtI8 && p.act == kActNone && p.out_mode == FIM_OUT_BF16 && !pool) pl.fixed_epilogue = kEpiFixed;
  }

  if (pool) pl.fixed_epilogue = kEpiPool;

  // scale tiles as tensors of 128 four-byte words per 512-byte tile: the loads of a CTA pair go through these
  maps.sfb = act_map, maps.sfa = act_map;
  if (pl.pair && !int8) {
    const uint64_t dims[2] = {128, static_cast<uint64_t>(p.weight_row_tiles) * p.weight_scale_tiles};
    const uint64_t strides[1] = {512};
    const uint32_t box[2] = {128, 1};
    const int rcm = make_tensor_map(&maps.sfb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, weight_scales, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rcm != kOk) return rcm;
    if (act_scales != nullptr) {
      const long long pixel_rows = static_cast<long long>(g->batch) * g->height * g->width;
      const uint64_t adims[2] = {128, static_cast<uint64_t>((pixel_rows + 127) / 128) * p.act_scale_tiles};
      const int rca = make_tensor_map(&maps.sfa, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, act_scales, adims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
      if (rca != kOk) return rca;
    }
  }

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int8) {
    if (pl.block_n == 64) return launch_conv_k<kFmtI8, 64>(maps, p, pl, s);
    if (pl.block_n == 128) return launch_conv_k<kFmtI8, 128>(maps, p, pl, s);
    return launch_conv_k<kFmtI8, 256>(maps, p, pl, s);
  }
  if (fmt == kFmtBf16) {
    if (pl.block_n == 64) return launch_conv_k<kFmtBf16, 64>(maps, p, pl, s);
    if (pl.block_n == 128) return launch_conv_k<kFmtBf16, 128>(maps, p, pl, s);
    return kUnsupported;
  }
  if (pl.block_n == 64) return launch_conv_k<kFmtMx, 64>(maps, p, pl, s);
  if (pl.block_n == 128) return launch_conv_k<kFmtMx, 128>(maps, p, pl, s);
  return launch_conv_k<kFmtMx, 256>(maps, p, pl, s);
}

template <int KC>
int launch_mlp(const CUtensorMap& x_map, const CUtensorMap& w1_map, const CUtensorMap& w2_map, const CUtensorMap& out_map,
               const CUtensorMap& res_map, const MlpParams& p, int ctas, size_t smem, cudaStream_t stream) {
  static bool configured[kMaxDevices] = {};
  const int device = current_device();
  if (device < 0 || device >= kMaxDevices || !configured[device]) {
    const cudaError_t e = cudaFuncSetAttribute(mlp_kernel<KC>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (device >= 0 && device < kMaxDevices) configured[device] = true;
  }
  mlp_kernel<KC><<<ctas, kMlpThreads, smem, stream>>>(x_map, w1_map, w2_map, out_map, res_map, p);
  return static_cast<int>(cudaGetLastError());
}

int run_mlp(const void* x, const void* x_scales, const void* w1, const void* w1_scales, const void* bias1, const void* w2,
            const void* w2_scales, const void* bias2, const void* residual, void* out, long long rows, int channels, int* status,
            void* stream) {
  if (rows < 0 || channels <= 0) return kBadArgument;
  if (rows == 0) return kOk;
  if (x == nullptr || x_scales == nullptr || w1 == nullptr || w1_scales == nullptr || bias1 == nullptr || w2 == nullptr ||
      w2_scales == nullptr || bias2 == nullptr || residual == nullptr || out == nullptr) {
    return kBadArgument;
  }
  if (channels != 128 && channels != 256) return kUnsupported;  // the second accumulator holds every output channel
  if (rows > 0x7fffffffLL - kTileM) return kUnsupported;
  for (const void* ptr : {x, x_scales, w1, w1_scales, bias1, w2, w2_scales, bias2, residual, static_cast<const void*>(out)}) {
    if (!aligned16(ptr)) return kBadLayout;
  }
  const int kc = channels / 128, c = channels;
  const uint32_t unit = static_cast<uint32_t>(kc) * (kMlpTile + 512u);
  const uint32_t fixed = 1024u + kGeluSmemBytes + unit + 2u * (kMlpTile + 512u) + kMlpOutWarps * (kMlpPanels + kMlpResidualSlots) * kMlpPanelBytes + 3u * c * 4u;
  int stages = static_cast<int>((kSmemLimit - fixed) / unit);
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) return kUnsupported;
  const size_t smem = fixed + static_cast<size_t>(stages) * unit;

  MlpParams p;
  p.rows = static_cast<int>(rows);
  p.row_tiles = static_cast<int>((rows + kTileM - 1) / kTileM);
  p.stages = stages;
  p.x_scales = static_cast<const uint8_t*>(x_scales);
  p.w1_scales = static_cast<const uint8_t*>(w1_scales);
  p.w2_scales = static_cast<const uint8_t*>(w2_scales);
  p.bias1 = static_cast<const __nv_bfloat16*>(bias1);
  p.bias2 = static_cast<const __nv_bfloat16*>(bias2);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.status = status;
  p.poll_backoff_ns = (g_debug_flags & 32) ? 0u : 200u;
  p.debug = g_debug_flags;

  CUtensorMap x_map, w1_map, w2_map, out_map, res_map;
  {
    const uint64_t dims[4] = {static_cast<uint64_t>(c), static_cast<uint64_t>(rows), 1, 1};
    const uint64_t strides[3] = {static_cast<uint64_t>(c), static_cast<uint64_t>(rows) * c, static_cast<uint64_t>(rows) * c};
    const uint32_t box[4] = {128, static_cast<uint32_t>(kTileM), 1, 1};
    const int rc = make_tensor_map(&x_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, x, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != kOk) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(c), static_cast<uint64_t>(2 * c)};
    const uint64_t strides[1] = {static_cast<uint64_t>(c)};
    const uint32_t box[2] = {128, 128};
    const int rc = make_tensor_map(&w1_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w1, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != kOk) return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(2 * c), static_cast<uint64_t>(c)};
    const uint64_t strides[1] = {static_cast<uint64_t>(2 * c)};
    const uint32_t box[2] = {128, 128};
    const int rc = make_tensor_map(&w2_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != kOk) return rc;
  }
  {
    const uint64_t row = static_cast<uint64_t>(c) * 2;
    const uint64_t dims[4] = {row, static_cast<uint64_t>(rows), 1, 1};
    const uint64_t strides[3] = {row, static_cast<uint64_t>(rows) * row, static_cast<uint64_t>(rows) * row};
    const uint32_t box[4] = {64, 32, 1, 1};
    const int rc = make_tensor_map(&out_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, out, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc != kOk) return rc;
    const int rcr = make_tensor_map(&res_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, residual, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B);
    if (rcr != kOk) return rcr;
  }
  const int device_sms = sm_count();
  const int sms = g_max_ctas > 0 && g_max_ctas < device_sms ? g_max_ctas : device_sms;
  const int ctas = p.row_tiles < sms ? p.row_tiles : sms;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return kc == 1 ? launch_mlp<1>(x_map, w1_map, w2_map, out_map, res_map, p, ctas, smem, s)
                 : launch_mlp<2>(x_map, w1_map, w2_map, out_map, res_map, p, ctas, smem, s);
}

}  // namespace
}  // namespace fim

using namespace fim;

extern "C" int fim_mxfp8_conv2d(const void* x, const int8_t* act_exponent, const void* act_scales_swizzled, const void* weight,
                                const void* weight_scales_swizzled, const FimConvGeometry* geometry,
                                const FimConvEpilogue* epilogue, void* out, int* status, void* stream) {
  return run_conv(kFmtMx, x, act_exponent, act_scales_swizzled, weight, weight_scales_swizzled, nullptr, nullptr, geometry, epilogue,
                  out, status, stream);
}

extern "C" int fim_mxfp8_conv2d_bf16(const void* x_bf16, const int8_t* act_exponent, const void* weight,
                                     const void* weight_scales_swizzled, const FimConvGeometry* geometry,
                                     const FimConvEpilogue* epilogue, void* out, int* status, void* stream) {
  if (geometry != nullptr && geometry->cin % 128) return kUnsupported;
  return run_conv(kFmtMx, x_bf16, act_exponent, nullptr, weight, weight_scales_swizzled, nullptr, nullptr, geometry, epilogue, out,
                  status, stream, true);
}

extern "C" int fim_int8_conv2d(const void* x, const void* weight, const float* a_scale, const float* w_scale,
                               const FimConvGeometry* geometry, const FimConvEpilogue* epilogue, void* out, int* status,
                               void* stream) {
  return run_conv(kFmtI8, x, nullptr, nullptr, weight, nullptr, a_scale, w_scale, geometry, epilogue, out, status, stream);
}

extern "C" int fim_int8_conv2d_maxpool(const void* x, const void* weight, const float* a_scale, const float* w_scale,
                                       const FimConvGeometry* geometry, const FimConvEpilogue* epilogue, void* out, void* pooled,
                                       int* status, void* stream) {
  if (pooled == nullptr) return kBadArgument;
  return run_conv(kFmtI8, x, nullptr, nullptr, weight, nullptr, a_scale, w_scale, geometry, epilogue, out, status, stream, false, pooled);
}

extern "C" int fim_bf16_conv2d(const void* x, const void* weight, const FimConvGeometry* geometry, const FimConvEpilogue* epilogue,
                               void* out, int* status, void* stream) {
  return run_conv(kFmtBf16, x, nullptr, nullptr, weight, nullptr, nullptr, nullptr, geometry, epilogue, out, status, stream);
}

extern "C" int fim_mxfp8_gelu_mlp_residual(const void* x, const void* x_scales_swizzled, const void* w1, const void* w1_scales_swizzled,
                                           const void* bias1, const void* w2, const void* w2_scales_swizzled, const void* bias2,
                                           const void* residual, void* out, long long rows, int channels, int* status, void* stream) {
  return run_mlp(x, x_scales_swizzled, w1, w1_scales_swizzled, bias1, w2, w2_scales_swizzled, bias2, residual, out, rows, channels, status,
                 stream);
}

extern "C" int fim_conv_plan(const FimConvGeometry* geometry, int int8, int per_pixel_scales, int plan[6]) {
  if (geometry == nullptr || plan == nullptr) return kBadArgument;
  Plan pl;
  const int rc = make_plan(*geometry, int8 != 0 ? kFmtI8 : kFmtMx, per_pixel_scales != 0, true, 2, false, &pl);
  if (rc != kOk) return rc;
  plan[0] = pl.tile_h, plan[1] = pl.tile_w, plan[2] = pl.block_n, plan[3] = pl.block_k, plan[4] = pl.stages, plan[5] = pl.ctas;
  return kOk;
}

extern "C" int fim_conv_schedule(const FimConvGeometry* geometry, int int8, int per_pixel_scales, int schedule[8]) {
  if (geometry == nullptr || schedule == nullptr) return kBadArgument;
  Plan pl;
  const int rc = make_plan(*geometry, int8 != 0 ? kFmtI8 : kFmtMx, per_pixel_scales != 0, true, 2, false, &pl);
  if (rc != kOk) return rc;
  const Schedule sc = make_schedule(*geometry, pl, int8 != 0, per_pixel_scales != 0);
  schedule[0] = pl.total_tiles, schedule[1] = sc.full_tiles, schedule[2] = sc.total_tiles, schedule[3] = pl.ctas;
  schedule[4] = pl.pair ? 1 : 0, schedule[5] = sc.resident_k, schedule[6] = sc.n_major, schedule[7] = acc_stages(pl.block_n);
  return kOk;
}

extern "C" void fim_conv_tune(int block_n, int max_ctas, int flags) {
  g_forced_block_n = block_n;
  g_max_ctas = max_ctas;
  g_debug_flags = flags;
}
