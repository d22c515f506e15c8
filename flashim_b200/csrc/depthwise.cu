// Depthwise 5x5 (pad 2, stride 1) + bias + activation on bf16 NHWC, with three epilogues: bf16, dynamic MXFP8,
// static INT8. Arithmetic follows FlashIM's torch reference (flashim/ops/conv.py:30-61): bf16 inputs and weights,
// fp32 FMA chain ordered (ky, kx) from zero, bias added last.
//
// Layout of the work. A CTA owns 64 channels x (4 * warps) columns x `tile_rows` rows of one image. Input rows
// (with their 2-pixel halo, zero-filled outside the image by TMA) stream through a ring of single-row stages in
// shared memory; a lane owns one bf16x2 channel pair and four adjacent columns, keeps the 25 weight pairs and five rows
// of partial sums in registers as packed fp32 pairs (fma.rn.f32x2: both channels in one issue slot), and finishes one
// output row per input row. The kernel is bound by the fp32 pipe (25 FMAs per element), not by HBM alone, so the issue
// slots beside the FMAs are what is budgeted: one 32-bit shared-memory load per input word, packed bias / GELU math, one
// redux per 32-channel MX block (16 adjacent lanes).
#include "common.cuh"
#include "flashim_sm100.h"

namespace fim {
namespace {

constexpr int kChannels = 64;  // per CTA: one 128-byte line per pixel
constexpr int kCols = 4;       // output columns per lane
constexpr int kStages = 8;     // single-row stages in the ring
constexpr int kMinWarps = 4, kMaxWarps = 5;  // compute warps per CTA (plus one producer warp)

enum { kOutBf16 = 0, kOutMx = 1, kOutInt8 = 2 };

struct DwParams {
  const uint32_t* weight;  // bf16x2 words, [25][C/2]
  const float* bias;
  void* out;
  uint8_t* scales;
  const float* scale;  // INT8
  int batch, height, width, channels;
  int tile_rows, tiles_x, tiles_y, channel_tiles;
  int act, swizzled;
  int* status;
  int debug;  // timing experiments only: 1 = no FMAs, 2 = no epilogue, 4 = no loads and no waits for them
};

template <int ACT>
__device__ __forceinline__ uint64_t activate2(uint64_t v) {
  if (ACT == kActGelu) return gelu_fast2(v);
  if (ACT == kActRelu) {
    float lo, hi;
    unpack2(v, lo, hi);
    return pack2(fmaxf(lo, 0.0f), fmaxf(hi, 0.0f));
  }
  return v;
}

// Finish one output row of this lane: bias, activation and the epilogue of MODE for the lane's four pixels. It is
// inlined next to the FMA block of the following input row, with which it shares no data, so the two interleave.
template <int MODE, int ACT>
__device__ __forceinline__ void emit_row(const DwParams& p, const uint64_t (&acc)[kCols], uint64_t bias2, size_t row_pixel,
                                         int x0, int c, bool lane_active, float int8_scale) {
  float lo[kCols], hi[kCols];
#pragma unroll
  for (int j = 0; j < kCols; ++j) unpack2(activate2<ACT>(add2(acc[j], bias2)), lo[j], hi[j]);
  if (MODE == kOutBf16) {
    uint32_t* out = reinterpret_cast<uint32_t*>(p.out) + (((row_pixel + x0) * p.channels + c) >> 1);
#pragma unroll
    for (int j = 0; j < kCols; ++j) {
      if (lane_active && x0 + j < p.width) out[static_cast<size_t>(j) * (p.channels >> 1)] = pack_bf16(lo[j], hi[j]);
    }
  } else if (MODE == kOutMx) {
    // amax of each pixel over the 16 lanes of its 32-channel block by a transposing butterfly: after the exchanges lane
    // l holds the block maximum of one pixel (5 shuffles instead of 16), computes that pixel's exponent once, and the
    // four exponents are read back with one shuffle each.
    float m[kCols];
#pragma unroll
    for (int j = 0; j < kCols; ++j) m[j] = lane_active ? fmaxf(fabsf(lo[j]), fabsf(hi[j])) : 0.0f;
    const int lane = threadIdx.x & 31;
    {
      const bool odd = lane & 1;  // even lanes keep pixels 0, 1 and odd lanes pixels 2, 3
      const float s0 = __shfl_xor_sync(0xffffffffu, odd ? m[0] : m[2], 1);
      const float s1 = __shfl_xor_sync(0xffffffffu, odd ? m[1] : m[3], 1);
      m[0] = fmaxf(odd ? m[2] : m[0], s0);
      m[1] = fmaxf(odd ? m[3] : m[1], s1);
    }
    {
      const bool up = lane & 2;  // then bit 1 of the lane picks the second of the pair
      const float s0 = __shfl_xor_sync(0xffffffffu, up ? m[0] : m[1], 2);
      m[0] = fmaxf(up ? m[1] : m[0], s0);
    }
    m[0] = fmaxf(m[0], __shfl_xor_sync(0xffffffffu, m[0], 4));
    m[0] = fmaxf(m[0], __shfl_xor_sync(0xffffffffu, m[0], 8));
    // this lane now holds pixel ((lane & 1) << 1) | ((lane >> 1) & 1) of its half-warp
    const int mine = e8m0_exponent(m[0]);
    const int half = lane & 16;
    const int groups = p.channels >> 5;
    uint16_t* out = reinterpret_cast<uint16_t*>(p.out) + (((row_pixel + x0) * p.channels + c) >> 1);
#pragma unroll
    for (int j = 0; j < kCols; ++j) {
      const int e = __shfl_sync(0xffffffffu, mine, half | ((j >> 1) & 1) | ((j & 1) << 1));
      const float inv = exp2_int(-e);
      if (lane_active && x0 + j < p.width) {
        out[static_cast<size_t>(j) * (p.channels >> 1)] = e4m3x2(lo[j] * inv, hi[j] * inv);
        if ((lane & 15) == 0) {
          const size_t pixel = row_pixel + x0 + j;
          const int g = c >> 5;
          const size_t at = p.swizzled ? swizzled_scale_offset(pixel, g, (groups + 3) >> 2) : pixel * groups + g;
          p.scales[at] = static_cast<uint8_t>(e + 127);
        }
      }
    }
  } else {
    uint16_t* out = reinterpret_cast<uint16_t*>(p.out) + (((row_pixel + x0) * p.channels + c) >> 1);
#pragma unroll
    for (int j = 0; j < kCols; ++j) {
      const int qlo = int8_code(bf16_round(lo[j]), int8_scale), qhi = int8_code(bf16_round(hi[j]), int8_scale);
      if (lane_active && x0 + j < p.width) {
        out[static_cast<size_t>(j) * (p.channels >> 1)] = static_cast<uint16_t>((qlo & 0xFF) | ((qhi & 0xFF) << 8));
      }
    }
  }
}

__device__ __forceinline__ uint64_t lds64(uint32_t addr) {
  uint64_t v;
  asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(addr));
  return v;
}

// Thread layout: `warps` compute warps (warp w owns columns 4w .. 4w+3 of the tile) and one producer warp whose lane 0
// streams input rows into the ring. Shared memory: [kStages rows][25 x 32 weight pairs as packed fp32].
template <int MODE, int ACT, bool WREG, bool PROBE>
__global__ void __launch_bounds__(32 * (kMaxWarps + 1), 2) dw5x5_kernel(const __grid_constant__ CUtensorMap in_map, const DwParams p) {
  extern __shared__ __align__(128) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ int abort_flag;

  const int warps = (blockDim.x >> 5) - 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_cols = warps * kCols;
  const uint32_t row_bytes = (tile_cols + 4) * kChannels * 2;

  // tile decode: x fastest, then y, channel tile, batch
  int t = blockIdx.x;
  const int tx = t % p.tiles_x; t /= p.tiles_x;
  const int ty = t % p.tiles_y; t /= p.tiles_y;
  const int ct = t % p.channel_tiles;
  const int b = t / p.channel_tiles;
  const int x_base = tx * tile_cols, y_base = ty * p.tile_rows, c_base = ct * kChannels;
  const int rows_out = min(p.tile_rows, p.height - y_base);
  const int rows_in = rows_out + 4;
  const bool loads = !(PROBE && (p.debug & 4));

  const uint32_t smem0 = smem_u32(smem_raw), full0 = smem_u32(&full_bar[0]), empty0 = smem_u32(&empty_bar[0]);
  const uint32_t wsm = smem0 + kStages * row_bytes;
  const int c = c_base + 2 * lane;
  const bool lane_active = c < p.channels;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], warps);
    }
    mbar_fence_init();
    fence_async_proxy();
    tma_prefetch_desc(&in_map);
  }
  if (warp == 0 && !WREG) {
    // the 25 weight pairs of this lane's channels, widened to fp32 once per CTA
    for (int k = 0; k < 25; ++k) {
      const uint64_t w2 = bf16x2_to_f32x2(lane_active ? __ldg(p.weight + ((static_cast<size_t>(k) * p.channels + c) >> 1)) : 0u);
      asm volatile("st.shared.b64 [%0], %1;" ::"r"(wsm + (k * 32 + lane) * 8), "l"(w2) : "memory");
    }
  }
  __syncthreads();

  if (warp == warps) {
    // ===== producer: one input row per stage, kStages rows ahead of the consumers =====
    if (lane == 0 && loads) {
      for (int r = 0; r < rows_in; ++r) {
        const int s = r % kStages;
        if (r >= kStages && !mbar_wait_addr(empty0 + 8 * s, ((r / kStages) - 1) & 1, &abort_flag, p.status, kStatusWaitRows)) break;
        mbar_expect_tx_addr(full0 + 8 * s, row_bytes);
        tma_load_4d_addr(smem0 + s * row_bytes, &in_map, full0 + 8 * s, c_base, x_base - 2, y_base - 2 + r, b);
      }
    }
  } else {
    // ===== consumers =====
    const uint64_t bias2 = lane_active ? pack2(__ldg(p.bias + c), __ldg(p.bias + c + 1)) : pack2(0.f, 0.f);
    const float int8_scale = MODE == kOutInt8 ? __ldg(p.scale) : 1.0f;
    const uint32_t lane_smem = smem0 + (warp * kCols * (kChannels / 2) + lane) * 4;
    const uint32_t lane_w = wsm + lane * 8;
    const int x0 = x_base + warp * kCols;
    const size_t image_pixel = static_cast<size_t>(b) * p.height * p.width;

    uint64_t wreg[WREG ? 25 : 1];
    if (WREG) {
#pragma unroll
      for (int k = 0; k < 25; ++k) {
        wreg[k] = bf16x2_to_f32x2(lane_active ? __ldg(p.weight + ((static_cast<size_t>(k) * p.channels + c) >> 1)) : 0u);
      }
    }
    uint64_t acc[5][kCols];
#pragma unroll
    for (int s = 0; s < 5; ++s)
#pragma unroll
      for (int j = 0; j < kCols; ++j) acc[s][j] = 0ull;  // two +0.0f
    uint64_t fin[kCols];   // the row completed by the previous input row, emitted beside this row's FMAs
    int fin_y = -1;
    uint32_t raw[kCols + 4];  // bf16x2 words of the next input row

    auto fetch = [&](int r) -> bool {  // wait for input row r and read this lane's words of it
      const int s = r % kStages;
      if (loads && !mbar_wait_addr(full0 + 8 * s, (r / kStages) & 1, &abort_flag, p.status, kStatusWaitRows)) return false;
#pragma unroll
      for (int j = 0; j < kCols + 4; ++j) {
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(raw[j]) : "r"(lane_smem + s * row_bytes + j * (kChannels * 2)));
      }
      return true;
    };

    bool alive = fetch(0);
    for (int r0 = 0; r0 < rows_in && alive; r0 += 5) {
#pragma unroll
      for (int ph = 0; ph < 5; ++ph) {
        const int r = r0 + ph;
        if (r >= rows_in) break;
        uint64_t in[kCols + 4];
#pragma unroll
        for (int j = 0; j < kCols + 4; ++j) in[j] = bf16x2_to_f32x2(raw[j]);
        // the words of row r are in registers: release its stage, then start on row r + 1
        __syncwarp();
        if (lane == 0 && loads) mbar_arrive_addr(empty0 + 8 * (r % kStages));
        if (r + 1 < rows_in && !fetch(r + 1)) {
          alive = false;
          break;
        }
        if (fin_y >= 0 && !(PROBE && (p.debug & 2))) {
          emit_row<MODE, ACT>(p, fin, bias2, image_pixel + static_cast<size_t>(fin_y) * p.width, x0, c, lane_active, int8_scale);
        }
        if (!(PROBE && (p.debug & 1))) {
          // 100 packed FMAs in one basic block: tap column outermost, so consecutive instructions belong to 20 different
          // accumulators and nothing waits on the FMA latency. Rows above / below the tile accumulate too (into sums that
          // are dropped): a branch per tap row would split the block. Weights come from shared memory per use.
#pragma unroll
          for (int kx = 0; kx < 5; ++kx) {
#pragma unroll
            for (int ky = 0; ky < 5; ++ky) {
              const int slot = (ph - ky + 5) % 5;  // output row r - ky of this tile
              const uint64_t w2 = WREG ? wreg[ky * 5 + kx] : lds64(lane_w + (ky * 5 + kx) * 256);
#pragma unroll
              for (int j = 0; j < kCols; ++j) acc[slot][j] = fma2(in[j + kx], w2, acc[slot][j]);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < kCols; ++j) acc[ph][j] = in[j] ^ in[j + 4];  // keep the loads alive
        }
        // output row r - 4 has now received all five input rows
        const int done = (ph + 1) % 5;
        fin_y = r - 4 >= 0 ? y_base + r - 4 : -1;
#pragma unroll
        for (int j = 0; j < kCols; ++j) {
          fin[j] = acc[done][j];
          acc[done][j] = 0ull;
        }
      }
    }
    if (alive && fin_y >= 0 && !(PROBE && (p.debug & 2))) {
      emit_row<MODE, ACT>(p, fin, bias2, image_pixel + static_cast<size_t>(fin_y) * p.width, x0, c, lane_active, int8_scale);
    }
  }
  if (abort_flag) {
    // a wait ran out: give copies that are still in flight time to land before the shared memory is released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
}

int g_dw_debug = 0;

int pick_warps(int width) {
  // fewest idle columns in the last tile of a row; on ties the narrower CTA (more CTAs per SM, better latency hiding)
  int best = kMinWarps;
  double best_eff = 0.0;
  for (int w = kMinWarps; w <= kMaxWarps; ++w) {
    const int cols = w * kCols;
    const double eff = static_cast<double>(width) / (static_cast<double>(ceil_div(width, cols)) * cols);
    if (eff > best_eff + 1e-9) {
      best_eff = eff;
      best = w;
    }
  }
  return best;
}

int pick_tile_rows(int height, long long tiles_per_row_band) {
  // Rows per CTA: tall enough that the 4 halo rows (loaded, not computed on) cost little, short enough that the grid
  // fills the 148 SMs several times over at 3-4 resident CTAs each.
  const int candidates[] = {64, 50, 40, 32, 25, 20, 16, 10, 8};
  for (int rows : candidates) {
    if (rows > height && rows != 8) continue;
    const long long ctas = tiles_per_row_band * ceil_div(height, rows);
    if (ctas >= 148LL * 3 * 3) return rows;  // three waves of three resident CTAs per SM
  }
  return height < 8 ? height : 8;
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
  const int warps = pick_warps(width);
  const int tile_cols = warps * kCols;
  DwParams p;
  p.weight = static_cast<const uint32_t*>(weight);
  p.bias = bias;
  p.out = out;
  p.scales = static_cast<uint8_t*>(scales);
  p.scale = scale;
  p.batch = batch, p.height = height, p.width = width, p.channels = channels;
  p.tiles_x = ceil_div(width, tile_cols);
  p.channel_tiles = ceil_div(channels, kChannels);
  p.tile_rows = pick_tile_rows(height, static_cast<long long>(p.tiles_x) * p.channel_tiles * batch);
  p.tiles_y = ceil_div(height, p.tile_rows);
  p.act = act, p.swizzled = swizzled, p.status = status, p.debug = g_dw_debug;
  const long long ctas = static_cast<long long>(p.tiles_x) * p.tiles_y * p.channel_tiles * batch;
  if (ctas > 0x7fffffffLL) return kUnsupported;

  CUtensorMap map;
  const uint64_t dims[4] = {static_cast<uint64_t>(channels), static_cast<uint64_t>(width), static_cast<uint64_t>(height),
                            static_cast<uint64_t>(batch)};
  const uint64_t strides[3] = {static_cast<uint64_t>(channels) * 2, static_cast<uint64_t>(width) * channels * 2,
                               static_cast<uint64_t>(height) * width * channels * 2};
  const uint32_t box[4] = {kChannels, static_cast<uint32_t>(tile_cols + 4), 1, 1};
  const int rc = make_tensor_map(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, value, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != kOk) return rc;

  const size_t smem = static_cast<size_t>(kStages) * (tile_cols + 4) * kChannels * 2 + 25 * 32 * 8;
  const unsigned grid = static_cast<unsigned>(ctas), block = (warps + 1) * 32;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (g_dw_debug != 0) {  // measurement hooks: a separate instantiation, so the production kernel carries no flag tests
    if (act == kActGelu) dw5x5_kernel<MODE, kActGelu, true, true><<<grid, block, smem, s>>>(map, p);
    else dw5x5_kernel<MODE, kActRelu, true, true><<<grid, block, smem, s>>>(map, p);
  } else if (act == kActGelu) {
    dw5x5_kernel<MODE, kActGelu, true, false><<<grid, block, smem, s>>>(map, p);
  } else if (act == kActRelu) {
    dw5x5_kernel<MODE, kActRelu, true, false><<<grid, block, smem, s>>>(map, p);
  } else {
    dw5x5_kernel<MODE, kActNone, true, false><<<grid, block, smem, s>>>(map, p);
  }
  return static_cast<int>(cudaGetLastError());
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

extern "C" void fim_dw_tune(int debug_flags) { g_dw_debug = debug_flags; }

extern "C" int fim_abi_version(void) { return FIM_ABI_VERSION; }
