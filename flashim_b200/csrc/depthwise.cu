// Depthwise 5x5 (pad 2, stride 1) + bias + activation on bf16 NHWC, with three epilogues: bf16, dynamic MXFP8,
// static INT8. Arithmetic follows FlashIM's torch reference (flashim/ops/conv.py:30-61): bf16 inputs and weights,
// fp32 FMA chain ordered (ky, kx) from zero, bias added last.
//
// Layout of the work. A CTA works on strips of 64 channels x (COLS * WARPS) columns of one image, five output rows (a
// unit) at a time; the persistent CTAs split the sequence of all units evenly. Input rows (with their 2-pixel halo,
// zero-filled outside the image by TMA) arrive five at a time in a ring of shared-memory chunks. A lane owns one bf16x2
// channel pair and COLS adjacent columns, keeps the 25 weight pairs and five rows of partial sums in registers as packed
// fp32 pairs (fma.rn.f32x2: both channels in one issue slot), and finishes one output row per input row.
//
// What bounds it is the fp32 pipe (25 FMAs per element, plus the polynomial of the GELU) and, next to it, the issue slots
// of everything else. Two things keep the pipe fed: (1) every warp computes - there is no producer warp holding
// registers; lane 0 of warp 0 issues the TMA copy four chunks ahead whenever it hands a chunk back - so that three CTAs
// of four warps fit on an SM at 168 registers and the latency of one warp's shared-memory reads and shuffles hides
// behind the FMAs of the others; (2) the epilogue is written for issue
// slots: the five rows of a chunk are one straight-line block (accumulator slots, shared-memory offsets and weights are
// all compile-time), barriers are touched once per chunk, a fresh accumulator starts with a multiply instead of being
// zeroed, GELU is one MUFU and a Horner polynomial with immediate operands per value, and the MX block maximum over 16
// lanes is a transposing butterfly.
#include "common.cuh"
#include "flashim_sm100.h"
#include "flashim_sm100_tune.h"

namespace fim {
namespace {

#ifndef FIM_PROBE_BUILD
#define FIM_PROBE_BUILD 0
#endif

// store only where `on` is non-zero, as a predicated instruction (no branch, the warp stays converged)
__device__ __forceinline__ void store_if(uint32_t* at, uint32_t v, uint32_t on) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %2, 0;\n\t@q st.global.b32 [%0], %1;\n\t}" ::"l"(at), "r"(v), "r"(on) : "memory");
}
__device__ __forceinline__ void store_if(uint16_t* at, uint16_t v, uint32_t on) {
  asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %2, 0;\n\t@q st.global.b16 [%0], %1;\n\t}" ::"l"(at), "h"(v), "r"(on) : "memory");
}

// The 25 * COLS multiply-adds per output row and channel pair as mixed-precision FMAs (fp32 += bf16 * bf16, one per
// channel, operands read from the halves of the packed words as they arrive from shared memory) instead of packed fp32
// FMAs on unpacked values: the same bits (a bf16 product is exact in fp32), no unpacking, and the weights stay packed
// (25 registers instead of 50). Measured per epilogue at 8x400x400x128: bf16 outputs 7-10 % faster (GELU 255 -> 238 us,
// ReLU 205 -> 185), ReLU -> MXFP8 7 % faster, GELU -> MXFP8 unchanged at first (its long epilogue is short of issue slots,
// and this form issues two instructions where the packed one issues one) and 8 % faster (329 -> 304 us) once the
// registers the packed weights free hold the coefficient pairs of a packed GELU polynomial; ReLU -> INT8 4 % slower: it
// keeps the packed fp32 form.
#ifndef FIM_DW_MIXED_FMA
#define FIM_DW_MIXED_FMA 1
#endif
__host__ __device__ constexpr bool mixed_fma_for(int mode, int min_ctas) {
  // (four CTAs per SM leave 128 registers per thread: only the packed weights fit)
  return FIM_DW_MIXED_FMA != 0 && (min_ctas >= 4 || mode != 2 /* every output but INT8 */);
}

// d = a * w + c per half of the packed bf16x2 words a and w, in fp32 (one rounding each)
__device__ __forceinline__ void fma_bf16x2(uint32_t a, uint32_t w, float c0, float c1, float& d0, float& d1) {
  asm("{\n\t.reg .b16 al, ah, wl, wh;\n\tmov.b32 {al, ah}, %2;\n\tmov.b32 {wl, wh}, %3;\n\t"
      "fma.rn.f32.bf16 %0, al, wl, %4;\n\tfma.rn.f32.bf16 %1, ah, wh, %5;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "r"(a), "r"(w), "f"(c0), "f"(c1));
}

constexpr int kChannels = 64;    // per CTA: one 128-byte line per pixel
constexpr int kChunkRows = 5;    // input rows per ring chunk = accumulator slots
// chunks in the ring: copies run up to 20 rows ahead (a chunk takes ~2 us to arrive); four CTAs per SM have room for four
__host__ __device__ constexpr int ring_stages(int min_ctas) { return min_ctas >= 4 ? 4 : 5; }

enum { kOutBf16 = 0, kOutMx = 1, kOutInt8 = 2 };

struct DwParams {
  const uint32_t* weight;  // bf16x2 words, [25][C/2]
  const float* bias;
  void* out;
  uint8_t* scales;
  const float* scale;  // INT8
  int batch, height, width, channels;
  int tiles_x, channel_tiles;  // a strip = (image, 64-channel tile, column tile), all rows of the image
  int strip_chunks, total_units;  // 5-row output chunks per strip; work units = strips * strip_chunks
  int act, swizzled;
  int* status;
  int debug;  // probe builds only: 1 = no FMAs, 2 = no epilogue, 4 = no loads and no waits for them
};

// GELU(x) = x * Phi(x) on an fp32 value. With p = Phi(-|x|) = 2**q(-|x|), q the degree-7 minimax polynomial of
// log2 Phi on [-5.5, 0] (relative error of p below 4e-6; q keeps falling beyond -5.5, so p underflows to 0 for large |x|),
// the value is max(x, 0) - |x| p for either sign. One MUFU; the Horner steps take their coefficients as immediates, so the
// constants occupy no registers beside the 25 weight pairs. For x < -4.4 torch's own fp32 expression
// x * 0.5 * (1 + erf(x / sqrt 2)) is dominated by the rounding of 1 + erf; this form stays accurate there.
__device__ __forceinline__ float gelu_phi(float x) {
  const float u = -fabsf(x);
  float q = 1.793454771359393e-06f;
  q = fmaf(q, u, 6.090417082305066e-05f);
  q = fmaf(q, u, 0.000926029053516686f);
  q = fmaf(q, u, 0.00849375780671835f);
  q = fmaf(q, u, 0.053937844932079315f);
  q = fmaf(q, u, -0.45848050713539124f);
  q = fmaf(q, u, 1.1512467861175537f);
  q = fmaf(q, u, -0.9999954700469971f);
  float p;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(q));
  return fmaf(u, p, fmaxf(x, 0.0f));
}

// The same on a pair of values with packed FMAs (one issue slot per Horner step of both); the coefficient pairs then live
// in registers, which only the kernels with packed weights have to spare.
__device__ __forceinline__ uint64_t gelu_phi2(uint64_t x2) {
  float x0, x1;
  unpack2(x2, x0, x1);
  const uint64_t u = pack2(-fabsf(x0), -fabsf(x1));
  uint64_t q = pack2(1.793454771359393e-06f, 1.793454771359393e-06f);
  q = fma2(q, u, pack2(6.090417082305066e-05f, 6.090417082305066e-05f));
  q = fma2(q, u, pack2(0.000926029053516686f, 0.000926029053516686f));
  q = fma2(q, u, pack2(0.00849375780671835f, 0.00849375780671835f));
  q = fma2(q, u, pack2(0.053937844932079315f, 0.053937844932079315f));
  q = fma2(q, u, pack2(-0.45848050713539124f, -0.45848050713539124f));
  q = fma2(q, u, pack2(1.1512467861175537f, 1.1512467861175537f));
  q = fma2(q, u, pack2(-0.9999954700469971f, -0.9999954700469971f));
  float q0, q1, p0, p1;
  unpack2(q, q0, q1);
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p0) : "f"(q0));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p1) : "f"(q1));
  return fma2(u, pack2(p0, p1), pack2(fmaxf(x0, 0.0f), fmaxf(x1, 0.0f)));
}

template <int ACT, bool PACKED_GELU = false>
__device__ __forceinline__ uint64_t activate2(uint64_t v) {
  if (ACT == kActNone) return v;
  if (ACT == kActGelu && PACKED_GELU) return gelu_phi2(v);
  float lo, hi;
  unpack2(v, lo, hi);
  if (ACT == kActGelu) return pack2(gelu_phi(lo), gelu_phi(hi));
  return pack2(fmaxf(lo, 0.0f), fmaxf(hi, 0.0f));
}

// Finish one output row of this lane: bias, activation and the epilogue of MODE for the lane's COLS pixels.
// `out_row` points at this lane's channel pair of pixel (row, x0) in units of output pairs; `pixel0` is that pixel's
// index in the batch; `cols_ok` has bit j set when column x0 + j exists (0 for a lane without channels).
template <int MODE, int ACT, int COLS, bool PACKED_GELU = false>
__device__ __forceinline__ void emit_row(const DwParams& p, const uint64_t (&acc)[COLS], uint64_t bias2, void* out_row,
                                         size_t pixel0, int c, uint32_t cols_ok, const Int8Quantizer& int8, int lane) {
  const size_t pair_stride = static_cast<size_t>(p.channels >> 1);
  uint64_t v[COLS];
#pragma unroll
  for (int j = 0; j < COLS; ++j) v[j] = activate2<ACT, PACKED_GELU>(add2(acc[j], bias2));
  if (MODE == kOutBf16) {
    uint32_t* out = static_cast<uint32_t*>(out_row);
#pragma unroll
    for (int j = 0; j < COLS; ++j) {
      float lo, hi;
      unpack2(v[j], lo, hi);
      store_if(out + j * pair_stride, pack_bf16(lo, hi), cols_ok & (1u << j));
    }
  } else if (MODE == kOutMx) {
    // amax of each pixel over the 16 lanes of its 32-channel block by a transposing butterfly: every exchange halves the
    // pixels a lane keeps until it holds one, whose maximum the remaining exchanges complete. With four pixels lane l
    // ends up with pixel ((l & 1) << 1) | ((l >> 1) & 1), with two pixels with pixel l & 1. The lane computes that
    // pixel's exponent; the first lanes of each half-warp store the scale bytes; 2**-e goes back with one shuffle per pixel.
    float m[COLS];
#pragma unroll
    for (int j = 0; j < COLS; ++j) {
      float lo, hi;
      unpack2(v[j], lo, hi);
      m[j] = fmaxf(fabsf(lo), fabsf(hi));
    }
    int mine;  // the pixel this lane holds after the butterfly
    if (COLS == 4) {
      const bool odd = lane & 1;  // even lanes keep pixels 0, 1 and odd lanes pixels 2, 3
      const float s0 = __shfl_xor_sync(0xffffffffu, odd ? m[0] : m[2], 1);
      const float s1 = __shfl_xor_sync(0xffffffffu, odd ? m[1] : m[3], 1);
      m[0] = fmaxf(odd ? m[2] : m[0], s0);
      m[1] = fmaxf(odd ? m[3] : m[1], s1);
      const bool up = lane & 2;  // then bit 1 of the lane picks the second of the pair
      const float s2 = __shfl_xor_sync(0xffffffffu, up ? m[0] : m[1], 2);
      m[0] = fmaxf(up ? m[1] : m[0], s2);
      mine = ((lane & 1) << 1) | ((lane >> 1) & 1);
    } else {
      const bool odd = lane & 1;  // even lanes keep pixel 0, odd lanes pixel 1
      const float s0 = __shfl_xor_sync(0xffffffffu, odd ? m[0] : m[1], 1);
      m[0] = fmaxf(odd ? m[1] : m[0], s0);
      m[0] = fmaxf(m[0], __shfl_xor_sync(0xffffffffu, m[0], 2));
      mine = lane & 1;
    }
    m[0] = fmaxf(m[0], __shfl_xor_sync(0xffffffffu, m[0], 4));
    m[0] = fmaxf(m[0], __shfl_xor_sync(0xffffffffu, m[0], 8));
    const int e = e8m0_exponent_bits(__float_as_uint(m[0]));
    const float inv_mine = exp2_int(-e);
    {
      // the owner lanes (the first COLS of each half-warp) store their pixel's scale byte; the address is computed by all
      // lanes and only the store is predicated, which keeps the warp converged
      const size_t pixel = pixel0 + mine;
      const int groups = p.channels >> 5;
      const int g = c >> 5;
      const size_t at = p.swizzled ? swizzled_scale_offset(pixel, g, (groups + 3) >> 2) : pixel * groups + g;
      const uint32_t owner = ((lane & 15) < COLS && ((cols_ok >> mine) & 1u)) ? 1u : 0u;
      asm volatile("{\n\t.reg .pred q;\n\tsetp.ne.u32 q, %2, 0;\n\t@q st.global.u8 [%0], %1;\n\t}" ::"l"(p.scales + at),
                   "r"(static_cast<uint32_t>(e + 127)), "r"(owner)
                   : "memory");
    }
    const int half = lane & 16;
    uint16_t* out = static_cast<uint16_t*>(out_row);
#pragma unroll
    for (int j = 0; j < COLS; ++j) {
      const int holder = COLS == 4 ? (((j >> 1) & 1) | ((j & 1) << 1)) : j;  // a lane of this half-warp that holds pixel j
      const float inv = __shfl_sync(0xffffffffu, inv_mine, half | holder);
      float lo, hi;
      unpack2(mul2(v[j], pack2(inv, inv)), lo, hi);
      store_if(out + j * pair_stride, e4m3x2(lo, hi), cols_ok & (1u << j));
    }
  } else {
    uint16_t* out = static_cast<uint16_t*>(out_row);
#pragma unroll
    for (int j = 0; j < COLS; ++j) {
      float lo, hi;
      unpack2(v[j], lo, hi);
      const uint32_t rounded = pack_bf16(lo, hi);  // one packed conversion instead of two scalar ones
      const uint16_t codes = static_cast<uint16_t>(int8_pack2(int8, bf16_lo(rounded), bf16_hi(rounded)));
      store_if(out + j * pair_stride, codes, cols_ok & (1u << j));
    }
  }
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// Where the copies of a CTA stand: the chunk sequence of its unit range [u, u_end), span by span.
struct CopyCursor {
  int u, u_end;       // next unit that starts a span
  int g, len;         // next chunk of the current span (0 .. len) and the span's length in units
  int k0, tx, ct, b;  // the span's first unit within its strip and the strip's coordinates
};

// Thread layout: WARPS compute warps; warp w owns columns COLS * w .. COLS * w + COLS - 1 of the tile. Lane 0 of warp 0
// also issues the copies.
template <int MODE, int ACT, int COLS, int WARPS, int MIN_CTAS, bool PROBE>
__global__ void __launch_bounds__(32 * WARPS, MIN_CTAS) dw5x5_kernel(const __grid_constant__ CUtensorMap in_map, const DwParams p) {
  constexpr bool kMixedFma = mixed_fma_for(MODE, MIN_CTAS);
  constexpr int kStages = ring_stages(MIN_CTAS);
  constexpr int kTileCols = WARPS * COLS;
  constexpr uint32_t kRowBytes = (kTileCols + 4) * kChannels * 2;
  constexpr uint32_t kChunkBytes = kChunkRows * kRowBytes;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ int abort_flag;

  // (the warp index through a shuffle: uniform to the compiler, and so is everything derived from it)
  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;

  // Persistent CTAs over work units of five output rows. A strip is one (image, channel tile, column tile) over all rows;
  // the units of all strips form one sequence, of which this CTA owns the contiguous range [u_begin, u_end): an equal
  // share to within one unit, cut into spans where it crosses a strip. A span of `len` units reads len + 1 input chunks
  // (its rows plus the halo above and below), so the chunk ring flows on from span to span without draining.
  const int u_begin = static_cast<int>(static_cast<long long>(blockIdx.x) * p.total_units / gridDim.x);
  const int u_end = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * p.total_units / gridDim.x);
  const bool loads = !(PROBE && (p.debug & 4));

  const uint32_t smem0 = smem_u32(smem_raw), full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], WARPS);
    }
    mbar_fence_init();
    fence_async_proxy();
    tma_prefetch_desc(&in_map);
  }
  __syncthreads();
  if (u_end <= u_begin) return;

  // ---- copies: issued by one lane of warp 0 (the cursor lives in every lane of that warp, uniformly) ----
  CopyCursor cur;
  cur.u = u_begin, cur.u_end = u_end, cur.g = 1, cur.len = 0, cur.k0 = 0, cur.tx = 0, cur.ct = 0, cur.b = 0;
  uint32_t copy_stage = 0;
  // Issue the next chunk of the sequence into ring stage `copy_stage`; false when the sequence has ended.
  auto issue_copy = [&]() -> bool {
    if (cur.g > cur.len) {  // the span is complete: open the next one
      if (cur.u >= cur.u_end) return false;
      const int strip = cur.u / p.strip_chunks;
      cur.k0 = cur.u - strip * p.strip_chunks;
      cur.len = min(p.strip_chunks - cur.k0, cur.u_end - cur.u);
      cur.u += cur.len;
      int t = strip;
      cur.tx = t % p.tiles_x; t /= p.tiles_x;
      cur.ct = t % p.channel_tiles;
      cur.b = t / p.channel_tiles;
      cur.g = 0;
    }
    if (elect_one()) {  // one lane, known to the compiler as one: the copy's operands stay in uniform registers
      mbar_expect_tx_addr(full0 + 8 * copy_stage, kChunkBytes);
      tma_load_4d_addr(smem0 + copy_stage * kChunkBytes, &in_map, full0 + 8 * copy_stage, cur.ct * kChannels,
                       cur.tx * kTileCols - 2, (cur.k0 + cur.g) * kChunkRows - 2, cur.b);
    }
    ++cur.g;
    if (++copy_stage == kStages) copy_stage = 0;
    return true;
  };
  bool copies_left = loads;
  if (warp == 0) {
    // the ring starts with all stages but one in flight; from then on every chunk handed back is answered by one copy
    for (int i = 0; i < kStages - 1 && copies_left; ++i) copies_left = issue_copy();
  }

  // ---- compute ----
  const Int8Quantizer int8_scale = make_int8_quantizer(MODE == kOutInt8 ? __ldg(p.scale) : 1.0f);
  const uint32_t lane_smem = smem0 + (warp * COLS * (kChannels / 2) + lane) * 4;
  constexpr int kOutBytes = MODE == kOutBf16 ? 4 : 2;  // per channel pair
  const size_t pair_stride = static_cast<size_t>(p.channels >> 1);
  const size_t row_pairs = static_cast<size_t>(p.width) * pair_stride;

  // per-span state
  uint64_t wreg[kMixedFma ? 1 : 25];   // unpacked weight pairs (packed-fp32 form)
  uint32_t wpack[kMixedFma ? 25 : 1];  // bf16x2 weight words (mixed-precision form)
  uint64_t bias2 = 0ull;
  int c = 0, last_ct = -1, y_base = 0, y_end = 0, y_out = 0;
  uint32_t cols_ok = 0;
  size_t pixel0 = 0;
  uint8_t* out_row = nullptr;
#pragma unroll
  for (int k = 0; k < (kMixedFma ? 1 : 25); ++k) wreg[k] = 0ull;
#pragma unroll
  for (int k = 0; k < (kMixedFma ? 25 : 1); ++k) wpack[k] = 0u;
  uint64_t acc[kMixedFma ? 1 : kChunkRows][COLS];
  float facc[kMixedFma ? kChunkRows : 1][COLS][2];
#pragma unroll
  for (int s = 0; s < (kMixedFma ? 1 : kChunkRows); ++s)
#pragma unroll
    for (int j = 0; j < COLS; ++j) acc[s][j] = 0ull;  // a slot is read for real only after its first multiply
#pragma unroll
  for (int s = 0; s < (kMixedFma ? kChunkRows : 1); ++s)
#pragma unroll
    for (int j = 0; j < COLS; ++j) facc[s][j][0] = facc[s][j][1] = 0.0f;

  uint32_t s = 0, phase = 0, taken = 0;  // ring position of the chunk in use; chunks handed back so far
  uint32_t raw[COLS + 4];  // bf16x2 words of the input row about to be used
  bool ok = !loads || mbar_wait_addr(full0, 0, &abort_flag, p.status, kStatusWaitRows);
  bool alive = __all_sync(0xffffffffu, ok);
  if (alive) {
#pragma unroll
    for (int j = 0; j < COLS + 4; ++j) raw[j] = lds32(lane_smem + j * (kChannels * 2));
  }
  for (int u = u_begin; u < u_end && alive;) {
    const int strip = u / p.strip_chunks, k0 = u - strip * p.strip_chunks;
    const int len = min(p.strip_chunks - k0, u_end - u);
    u += len;
    {
      int t = strip;
      const int tx = t % p.tiles_x; t /= p.tiles_x;
      const int ct = t % p.channel_tiles;
      const int b = t / p.channel_tiles;
      c = ct * kChannels + 2 * lane;
      const bool lane_active = c < p.channels;
      if (ct != last_ct) {  // uniform: a new channel tile brings new weights and bias
        last_ct = ct;
#pragma unroll
        for (int k = 0; k < 25; ++k) {
          const uint32_t word = lane_active ? __ldg(p.weight + ((static_cast<size_t>(k) * p.channels + c) >> 1)) : 0u;
          if (kMixedFma) {
            wpack[k] = word;
          } else {
            wreg[k] = bf16x2_to_f32x2(word);
          }
        }
        bias2 = lane_active ? pack2(__ldg(p.bias + c), __ldg(p.bias + c + 1)) : pack2(0.f, 0.f);
      }
      const int x0 = tx * kTileCols + warp * COLS;
      cols_ok = 0;
#pragma unroll
      for (int j = 0; j < COLS; ++j) cols_ok |= (lane_active && x0 + j < p.width) ? (1u << j) : 0u;
      y_base = k0 * kChunkRows;
      y_end = min(y_base + len * kChunkRows, p.height);
      y_out = y_base - 4;  // where the span's first input row would "finish": four rows above the span
      pixel0 = (static_cast<size_t>(b) * p.height + y_base) * p.width + x0;  // of output row y_base, advanced per emitted row
      out_row = static_cast<uint8_t*>(p.out) + (pixel0 * pair_stride + (c >> 1)) * kOutBytes;
    }
    for (int g = 0; g <= len && alive; ++g) {
      const bool more = g < len || u < u_end;  // another chunk follows, in this span or the next
      const uint32_t chunk = lane_smem + s * kChunkBytes;
      const uint32_t s_next = s + 1 == kStages ? 0u : s + 1;
      const uint32_t phase_next = s + 1 == kStages ? phase ^ 1u : phase;
#pragma unroll
      for (int ph = 0; ph < kChunkRows; ++ph) {
        uint64_t in[kMixedFma ? 1 : COLS + 4];
        uint32_t row[kMixedFma ? COLS + 4 : 1];  // this row's packed words, while `raw` takes the next row
#pragma unroll
        for (int j = 0; j < COLS + 4; ++j) {
          if (kMixedFma) {
            row[j] = raw[j];
          } else {
            in[j] = bf16x2_to_f32x2(raw[j]);
          }
        }
        // fetch the next input row while this one is in the FMAs
        if (ph + 1 < kChunkRows) {
#pragma unroll
          for (int j = 0; j < COLS + 4; ++j) raw[j] = lds32(chunk + (ph + 1) * kRowBytes + j * (kChannels * 2));
        } else {
          // every word of this chunk is in registers: hand it back, then take the first row of the next chunk (which
          // may already belong to the next tile)
          __syncwarp();
          if (lane == 0 && loads) mbar_arrive_addr(empty0 + 8 * s);
          if (warp == 0 && copies_left) {
            // One copy per chunk handed back, into the stage handed back one chunk ago: the other warps have had a whole
            // chunk's time to release it, so this wait rarely spins. Stage (taken - 1) mod kStages has then been released
            // (taken - 1) / kStages + 1 times; the first kStages - 1 copies went out before the loop.
            bool free_stage = true;
            if (taken >= 1) {
              const uint32_t round = (taken - 1) / kStages;
              // (the warp agrees on the outcome: the copy below is issued through elect.sync, which every lane must reach)
              free_stage = __all_sync(0xffffffffu, mbar_wait_addr(empty0 + 8 * copy_stage, round & 1u, &abort_flag, p.status, kStatusWaitRows));
            }
            copies_left = free_stage && issue_copy();
          }
          ++taken;
          if (more) {
            ok = !loads || mbar_wait_addr(full0 + 8 * s_next, phase_next, &abort_flag, p.status, kStatusWaitRows);
            alive = __all_sync(0xffffffffu, ok);
#pragma unroll
            for (int j = 0; j < COLS + 4; ++j) raw[j] = lds32(lane_smem + s_next * kChunkBytes + j * (kChannels * 2));
          }
        }
        if (!(PROBE && (p.debug & 1))) {
          // 25 * COLS packed FMAs: input row r = 5 g + ph feeds tap row ky of the output row in slot (ph - ky) mod 5. Tap
          // column outermost, so neighbouring instructions belong to 5 * COLS different accumulators and nothing waits on
          // the FMA latency. Tap row 0 opens a new output row: its first term is a plain product (0 + a*b == a*b).
#pragma unroll
          for (int kx = 0; kx < 5; ++kx) {
#pragma unroll
            for (int ky = 0; ky < 5; ++ky) {
              const int slot = (ph - ky + 5) % 5;
#pragma unroll
              for (int j = 0; j < COLS; ++j) {
                if (kMixedFma) {
                  // (a new output row starts from -0: the sum then keeps the sign of a zero first product, like a plain multiply)
                  const bool first = ky == 0 && kx == 0;
                  fma_bf16x2(row[j + kx], wpack[ky * 5 + kx], first ? -0.0f : facc[slot][j][0], first ? -0.0f : facc[slot][j][1],
                             facc[slot][j][0], facc[slot][j][1]);
                } else {
                  acc[slot][j] = (ky == 0 && kx == 0) ? mul2(in[j], wreg[0]) : fma2(in[j + kx], wreg[ky * 5 + kx], acc[slot][j]);
                }
              }
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < COLS; ++j) {  // keep the loads alive
            if (kMixedFma) {
              facc[(ph + 1) % 5][j][0] = __uint_as_float(row[j]), facc[(ph + 1) % 5][j][1] = __uint_as_float(row[j + 4]);
            } else {
              acc[(ph + 1) % 5][j] = in[j] ^ in[j + 4];
            }
          }
        }
        // The output row in slot (ph + 1) mod 5 has now received all five input rows: finish it (bias, activation, stores)
        // straight from its accumulators. Nothing branches here: a row outside the span has an empty store mask, so the
        // compiler is free to overlap this epilogue with the FMAs of the next input row.
        {
          const bool valid = y_out >= y_base && y_out < y_end;
          if (!(PROBE && (p.debug & 2))) {
            if (kMixedFma) {
              uint64_t done[COLS];
#pragma unroll
              for (int j = 0; j < COLS; ++j) done[j] = pack2(facc[(ph + 1) % 5][j][0], facc[(ph + 1) % 5][j][1]);
              emit_row<MODE, ACT, COLS, true>(p, done, bias2, out_row, pixel0, c, valid ? cols_ok : 0u, int8_scale, lane);
            } else {
              emit_row<MODE, ACT, COLS>(p, acc[(ph + 1) % 5], bias2, out_row, pixel0, c, valid ? cols_ok : 0u, int8_scale, lane);
            }
          }
          pixel0 += valid ? static_cast<size_t>(p.width) : 0;
          out_row += valid ? row_pairs * kOutBytes : 0;
        }
        ++y_out;
      }
      s = s_next, phase = phase_next;
    }
  }
  if (abort_flag) {
    // a wait ran out: give copies that are still in flight time to land before the shared memory is released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

int g_dw_variant = 0;
int g_dw_probe = 0;

// Thread layouts that are compiled in: columns per lane, warps per CTA and the CTAs an SM is meant to hold (which caps
// the registers). Tiles are COLS * WARPS columns wide.
struct Variant {
  int cols, warps, ctas_per_sm;
};
constexpr Variant kVariants[] = {
    {4, 4, 3},  // 1: 16 columns, 12 warps per SM at 168 registers
    {4, 5, 2},  // 2: 20 columns, 10 warps per SM
    {2, 8, 2},  // 3: 16 columns, 16 warps per SM at 128 registers (two columns per lane)
    {4, 4, 4},  // 4: 16 columns, 16 warps per SM at 128 registers (mixed-precision FMAs, packed weights, four-chunk ring)
};
constexpr int kVariantCount = sizeof(kVariants) / sizeof(kVariants[0]);

int pick_variant(int width) {
  if (g_dw_variant >= 1 && g_dw_variant <= kVariantCount) return g_dw_variant - 1;
  // Measured on 100- to 400-pixel-wide images with every epilogue: four columns per lane on three CTAs of four warps is the
  // fastest layout throughout. Two columns per lane hold sixteen warps on an SM but spend more instructions per element
  // (dw -> MXFP8 on 8 x 400 x 400 x 128: 463 us against 369 us); 20-column tiles fit 100 and 200 columns exactly yet lose
  // more to the fifth warp doubling up on one scheduler. Four CTAs per SM (128 registers with the packed weights of the
  // mixed-precision form) measured 2-8 % slower than three: more warps do not buy the FMA pipe any time.
  (void)width;
  return 0;
}

template <int MODE, int COLS, int WARPS, int MIN_CTAS>
cudaError_t launch_kernel(const CUtensorMap& map, const DwParams& p, int act, unsigned grid, cudaStream_t s) {
  constexpr unsigned kBlock = WARPS * 32;
  constexpr size_t kSmem = static_cast<size_t>(ring_stages(MIN_CTAS)) * kChunkRows * (WARPS * COLS + 4) * kChannels * 2;
  // every instantiation gets the opt-in limit once per device (some chunk rings exceed the 48 KB default)
  static bool configured[kMaxDevices] = {};
  const int device = current_device();
  if (device < 0 || device >= kMaxDevices || !configured[device]) {
    cudaError_t e = cudaSuccess;
    auto set = [&](auto kernel) {
      if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmem));
    };
    set(dw5x5_kernel<MODE, kActNone, COLS, WARPS, MIN_CTAS, false>);
    set(dw5x5_kernel<MODE, kActRelu, COLS, WARPS, MIN_CTAS, false>);
    set(dw5x5_kernel<MODE, kActGelu, COLS, WARPS, MIN_CTAS, false>);
#if FIM_PROBE_BUILD
    set(dw5x5_kernel<MODE, kActRelu, COLS, WARPS, MIN_CTAS, true>);
    set(dw5x5_kernel<MODE, kActGelu, COLS, WARPS, MIN_CTAS, true>);
#endif
    if (e != cudaSuccess) return e;
    if (device >= 0 && device < kMaxDevices) configured[device] = true;
  }
#if FIM_PROBE_BUILD
  if (g_dw_probe != 0) {  // measurement hooks: a separate instantiation, so the production kernel carries no flag tests
    if (act == kActGelu) dw5x5_kernel<MODE, kActGelu, COLS, WARPS, MIN_CTAS, true><<<grid, kBlock, kSmem, s>>>(map, p);
    else dw5x5_kernel<MODE, kActRelu, COLS, WARPS, MIN_CTAS, true><<<grid, kBlock, kSmem, s>>>(map, p);
    return cudaGetLastError();
  }
#endif
  if (act == kActGelu) {
    dw5x5_kernel<MODE, kActGelu, COLS, WARPS, MIN_CTAS, false><<<grid, kBlock, kSmem, s>>>(map, p);
  } else if (act == kActRelu) {
    dw5x5_kernel<MODE, kActRelu, COLS, WARPS, MIN_CTAS, false><<<grid, kBlock, kSmem, s>>>(map, p);
  } else {
    dw5x5_kernel<MODE, kActNone, COLS, WARPS, MIN_CTAS, false><<<grid, kBlock, kSmem, s>>>(map, p);
  }
  return cudaGetLastError();
}

template <int MODE>
int launch(const void* value, const void* weight, const float* bias, void* out, void* scales, const float* scale, int swizzled,
           int batch, int height, int width, int channels, int act, int* status, void* stream) {
  if (batch < 0 || height < 0 || width < 0 || channels <= 0 || act < 0 || act > 2) return kBadArgument;
  if (channels % 32) return kUnsupported;
  if (batch == 0 || height == 0 || width == 0) return kOk;
  if (value == nullptr || weight == nullptr || bias == nullptr || out == nullptr) return kBadArgument;
  if ((reinterpret_cast<uintptr_t>(value) & 15u) || (reinterpret_cast<uintptr_t>(weight) & 3u) ||
      (reinterpret_cast<uintptr_t>(out) & 3u)) {
    return kBadLayout;
  }
  const Variant variant = kVariants[pick_variant(width)];
  const int tile_cols = variant.cols * variant.warps;
  DwParams p;
  p.weight = static_cast<const uint32_t*>(weight);
  p.bias = bias;
  p.out = out;
  p.scales = static_cast<uint8_t*>(scales);
  p.scale = scale;
  p.batch = batch, p.height = height, p.width = width, p.channels = channels;
  p.tiles_x = ceil_div(width, tile_cols);
  p.channel_tiles = ceil_div(channels, kChannels);
  p.strip_chunks = ceil_div(height, kChunkRows);
  p.act = act, p.swizzled = swizzled, p.status = status, p.debug = g_dw_probe;
  const long long units = static_cast<long long>(p.tiles_x) * p.channel_tiles * batch * p.strip_chunks;
  if (units > 0x7fffffffLL) return kUnsupported;
  p.total_units = static_cast<int>(units);

  CUtensorMap map;
  const uint64_t dims[4] = {static_cast<uint64_t>(channels), static_cast<uint64_t>(width), static_cast<uint64_t>(height),
                            static_cast<uint64_t>(batch)};
  const uint64_t strides[3] = {static_cast<uint64_t>(channels) * 2, static_cast<uint64_t>(width) * channels * 2,
                               static_cast<uint64_t>(height) * width * channels * 2};
  const uint32_t box[4] = {kChannels, static_cast<uint32_t>(tile_cols + 4), kChunkRows, 1};
  // a CTA reads 128 bytes (64 channels) of every pixel: with more channels than that, fetching 256-byte granules into L2
  // would drag in the neighbouring channel tile, which another CTA reads much later
  const int rc = make_tensor_map(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, value, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE,
                                 channels > kChannels ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
  if (rc != kOk) return rc;

  // persistent CTAs, as many as the SMs hold; a small problem gets fewer, each with at least four units so the halo chunk
  // stays cheap
  const long long resident = static_cast<long long>(sm_count()) * variant.ctas_per_sm;
  const long long want = (units + 3) / 4;
  const unsigned grid = static_cast<unsigned>(want < resident ? want : resident);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (variant.cols == 2) e = launch_kernel<MODE, 2, 8, 2>(map, p, act, grid, s);
  else if (variant.warps == 4 && variant.ctas_per_sm == 4) e = launch_kernel<MODE, 4, 4, 4>(map, p, act, grid, s);
  else if (variant.warps == 4) e = launch_kernel<MODE, 4, 4, 3>(map, p, act, grid, s);
  else e = launch_kernel<MODE, 4, 5, 2>(map, p, act, grid, s);
  return static_cast<int>(e);
}

}  // namespace
}  // namespace fim

using namespace fim;

extern "C" int fim_dw5x5_bf16(const void* value, const void* weight, const float* bias, void* out, int batch, int height,
                              int width, int channels, int act, int* status, void* stream) {
  return launch<kOutBf16>(value, weight, bias, out, nullptr, nullptr, 0, batch, height, width, channels, act, status, stream);
}

extern "C" int fim_dw5x5_mxfp8(const void* value, const void* weight, const float* bias, void* out, void* scales, int swizzled,
                               int batch, int height, int width, int channels, int act, int* status, void* stream) {
  if (scales == nullptr && batch > 0 && height > 0 && width > 0) return kBadArgument;
  return launch<kOutMx>(value, weight, bias, out, scales, nullptr, swizzled, batch, height, width, channels, act, status, stream);
}

extern "C" int fim_dw5x5_relu_int8(const void* value, const void* weight, const float* bias, const float* scale, void* out,
                                   int batch, int height, int width, int channels, int* status, void* stream) {
  if (scale == nullptr && batch > 0 && height > 0 && width > 0) return kBadArgument;
  return launch<kOutInt8>(value, weight, bias, out, nullptr, scale, 0, batch, height, width, channels, kActRelu, status, stream);
}

extern "C" void fim_dw_tune(int variant, int probe_flags) {
  g_dw_variant = variant;
  g_dw_probe = probe_flags;
}

extern "C" int fim_abi_version(void) { return FIM_ABI_VERSION; }
