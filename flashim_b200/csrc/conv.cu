// Implicit-GEMM conv2d (NHWC, stride 1) on the tcgen05 tensor cores of sm_100a: block-scaled MXFP8
// (kind::mxf8f6f4, E8M0 scale per 32 along K) and INT8 (kind::i8, int32 accumulation).
//
// One persistent CTA per SM walks output tiles of 128 pixels (a tile_h x tile_w patch of one image) x BN output
// channels. Warp 0 is the TMA producer: per (tap, channel chunk) it loads the shifted activation patch (a 4-D box whose
// out-of-image part TMA fills with zeros: the conv padding, no im2col buffer) and the weight tile into a ring of
// swizzled K-major stages, plus the 512-byte scale tiles. Warp 1 issues tcgen05.mma from one lane, accumulating in
// tensor memory; scale tiles go shared memory -> tensor memory with tcgen05.cp in front of the MMAs that use them.
// Warps 2-5 are the epilogue: tcgen05.ld their 32 accumulator rows, apply bias / bf16 rounding / activation / residual
// / requantisation in registers and store. Accumulators are double-buffered in tensor memory when 2 * BN columns fit,
// so the epilogue of tile i overlaps the main loop of tile i + 1.
//
// Rounding points follow FlashIM's torch reference: flashim/ops/conv.py:174-206,309-342 and flashim/ops/gemm.py:58-98.
#include "common.cuh"
#include "flashim_sm100.h"

namespace fim {
namespace {

constexpr int kThreads = 192;
constexpr int kTileM = 128;
constexpr uint32_t kTmemColumns = 512;
constexpr int kMaxStages = 8;
constexpr int kSmemBudget = 200 * 1024;

struct ConvParams {
  int batch, height, width, cin, cout, out_h, out_w;
  int kh, kw, pad_h, pad_w, dil_h, dil_w;
  int tile_h, tile_w, tiles_x, tiles_y, tiles_n, total_tiles;
  int block_k, k_chunks, stages;
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
  int res_channels, act, out_mode;
  const int8_t* out_exponent;
  uint8_t* out_scales;
  const float* out_scale;
  void* out;
  int* status;
  int debug;  // timing experiments only: 1 = no activation loads, 2 = no weight loads, 4 = no output stores
};

struct SharedControl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ uint32_t idesc_mxf8(int block_n, uint32_t a_id, uint32_t b_id) {
  // E4M3 x E4M3 (format 0), both K-major, UE8M0 scales, M = 128, N = block_n
  return (b_id << 4) | (static_cast<uint32_t>(block_n >> 3) << 17) | (1u << 23) | (static_cast<uint32_t>(kTileM >> 4) << 24) |
         (a_id << 29);
}
__device__ __forceinline__ uint32_t idesc_i8(int block_n) {
  // S32 accumulator (2), signed 8-bit A and B (1), both K-major, M = 128, N = block_n
  return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(block_n >> 3) << 17) |
         (static_cast<uint32_t>(kTileM >> 4) << 24);
}

// ---- epilogue on 32 consecutive output channels of one pixel -------------------------------------------------------
template <bool INT8>
__device__ __forceinline__ void finish_chunk(const ConvParams& p, const uint32_t (&raw)[32], int n, size_t pixel, int b, int y,
                                             int x, float a_scale) {
  float v[32];
  if (INT8) {
    if (p.out_mode == FIM_OUT_INT32) {
      uint4* dst = reinterpret_cast<uint4*>(static_cast<int32_t*>(p.out) + pixel * p.cout + n);
#pragma unroll
      for (int i = 0; i < 8; ++i) dst[i] = make_uint4(raw[4 * i], raw[4 * i + 1], raw[4 * i + 2], raw[4 * i + 3]);
      return;
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float scale = __fmul_rn(a_scale, __ldg(p.w_scale + n + i));
      v[i] = __fmul_rn(__int2float_rn(static_cast<int>(raw[i])), scale);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
  }
  if (p.bias != nullptr) {
    const uint4* bp = reinterpret_cast<const uint4*>(p.bias + n);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 w = __ldg(bp + i);
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[8 * i + 2 * j] = __fadd_rn(v[8 * i + 2 * j], bf16_lo(ws[j]));
        v[8 * i + 2 * j + 1] = __fadd_rn(v[8 * i + 2 * j + 1], bf16_hi(ws[j]));
      }
    }
  }
  if (!INT8 && p.out_mode == FIM_OUT_F32) {
    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.out) + pixel * p.cout + n);
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    return;
  }
  const bool has_res = p.residual != nullptr;
  // one bf16 rounding, activation on the rounded value (ReLU waits for the residual when there is one)
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    float h = bf16_round(v[i]);
    if (p.act == kActGelu) h = bf16_round(gelu_erf(h));
    if (p.act == kActRelu && !has_res) h = fmaxf(h, 0.0f);
    v[i] = h;
  }
  if (has_res) {
    const __nv_bfloat16* rp = p.residual + b * p.res_stride[0] + y * p.res_stride[1] + x * p.res_stride[2];
    const int limit = p.res_channels - n;  // channels of this chunk present in the residual
    const bool vec = p.res_stride[3] == 1 && limit >= 32 && ((reinterpret_cast<uintptr_t>(rp + n) & 15u) == 0);
    if (vec) {
      const uint4* r4 = reinterpret_cast<const uint4*>(rp + n);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 w = __ldg(r4 + i);
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          v[8 * i + 2 * j] += bf16_lo(ws[j]);
          v[8 * i + 2 * j + 1] += bf16_hi(ws[j]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (i < limit) v[i] += __bfloat162float(rp[(n + i) * p.res_stride[3]]);
      }
    }
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = bf16_round(p.act == kActRelu ? fmaxf(v[i], 0.0f) : v[i]);
  }
  if (p.out_mode == FIM_OUT_BF16) {
    uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + pixel * p.cout + n);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      dst[i] = make_uint4(pack_bf16(v[8 * i], v[8 * i + 1]), pack_bf16(v[8 * i + 2], v[8 * i + 3]),
                          pack_bf16(v[8 * i + 4], v[8 * i + 5]), pack_bf16(v[8 * i + 6], v[8 * i + 7]));
    }
    return;
  }
  if (INT8) {  // FIM_OUT_INT8
    const float scale = __ldg(p.out_scale);
    uint32_t q[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t w = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) w |= (static_cast<uint32_t>(int8_code(v[4 * i + k], scale)) & 0xFFu) << (8 * k);
      q[i] = w;
    }
    uint4* dst = reinterpret_cast<uint4*>(static_cast<int8_t*>(p.out) + pixel * p.cout + n);
    dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
    dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
    return;
  }
  int e;
  if (p.out_mode == FIM_OUT_E4M3_STATIC) {
    e = static_cast<int>(__ldg(p.out_exponent + (n >> 5)));
  } else {
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    e = e8m0_exponent(amax);
    const int groups = p.cout >> 5;
    p.out_scales[swizzled_scale_offset(pixel, n >> 5, (groups + 3) >> 2)] = static_cast<uint8_t>(e + 127);
  }
  const float inv = exp2_int(-e);
  uint32_t q[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] = e4m3x4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
  uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.out) + pixel * p.cout + n);
  dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
  dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
}

template <bool INT8, int BN>
__global__ void __launch_bounds__(kThreads, 1)
conv_kernel(const __grid_constant__ CUtensorMap act_map, const __grid_constant__ CUtensorMap weight_map, const ConvParams p) {
  constexpr int kAccStages = (2 * BN + 4 + (BN < 128 ? 4 : BN / 32)) <= static_cast<int>(kTmemColumns) ? 2 : 1;
  constexpr int kScaleTilesB = BN <= 128 ? 1 : BN / 128;
  constexpr uint32_t kSfaColumn = kAccStages * BN;
  constexpr uint32_t kSfbColumn = kSfaColumn + 4;

  extern __shared__ uint8_t smem_dyn[];
  __shared__ __align__(8) SharedControl ctl;

  // dynamic shared memory, 1024-byte aligned: [stages x A][stages x B][stages x scale tiles B][stages x scale tile A][static A tiles]
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023u) & ~static_cast<uintptr_t>(1023u));
  const uint32_t a_bytes = kTileM * p.block_k;
  const uint32_t b_bytes = BN * p.block_k;
  uint8_t* smem_a = base;
  uint8_t* smem_b = smem_a + static_cast<size_t>(p.stages) * a_bytes;
  uint8_t* smem_sfb = smem_b + static_cast<size_t>(p.stages) * b_bytes;
  uint8_t* smem_sfa = smem_sfb + static_cast<size_t>(p.stages) * kScaleTilesB * 512;
  uint8_t* smem_sfa_static = smem_sfa + static_cast<size_t>(p.stages) * 512;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool dynamic_a = !INT8 && p.act_scales != nullptr;
  const int taps = p.kh * p.kw;
  const int k_iters = taps * p.k_chunks;

  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&ctl.full[s], 1);
      mbar_init(&ctl.empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl.tmem_full[s], 1);
      mbar_init(&ctl.tmem_empty[s], 4);
    }
    mbar_fence_init();
    tma_prefetch_desc(&act_map);
    tma_prefetch_desc(&weight_map);
  }
  if (warp == 1) {
    tmem_alloc(&ctl.tmem_base, kTmemColumns);
    tmem_relinquish();
  }
  if (warp == 2 && !INT8 && !dynamic_a) {
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
      *reinterpret_cast<uint4*>(smem_sfa_static + t * 512 + lane * 16) = make_uint4(word, word, word, word);
    }
    fence_async_proxy();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl.tmem_base;

  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      const uint32_t a_box_bytes = static_cast<uint32_t>(p.tile_h * p.tile_w) * p.block_k;
      const bool load_a = !(p.debug & 1), load_b = !(p.debug & 2);
      const uint32_t tx_bytes = (load_a ? a_box_bytes : 0u) + (load_b ? b_bytes : 0u) +
                                (INT8 ? 0u : kScaleTilesB * 512u + (dynamic_a ? 512u : 0u));
      uint32_t it = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < p.total_tiles && alive; tile += gridDim.x) {
        const int nt = tile % p.tiles_n;
        int m = tile / p.tiles_n;
        const int tx = m % p.tiles_x; m /= p.tiles_x;
        const int ty = m % p.tiles_y;
        const int b = m / p.tiles_y;
        const int x0 = tx * p.tile_w, y0 = ty * p.tile_h, n0 = nt * BN;
        const int m_tile = tile / p.tiles_n;  // row tile of the per-pixel scale layout (flat 1x1 convs)
        for (int tap = 0; tap < taps && alive; ++tap) {
          const int ky = tap / p.kw, kx = tap - ky * p.kw;
          for (int j = 0; j < p.k_chunks; ++j, ++it) {
            const int s = it % p.stages;
            if (!mbar_wait(&ctl.empty[s], ((it / p.stages) & 1) ^ 1, &ctl.abort_flag, p.status, kStatusWaitEmpty)) {
              alive = false;
              break;
            }
            if (tx_bytes != 0) {
              mbar_expect_tx(&ctl.full[s], tx_bytes);
            } else {
              mbar_arrive(&ctl.full[s]);
            }
            if (load_a) {
              tma_load_4d(smem_a + static_cast<size_t>(s) * a_bytes, &act_map, &ctl.full[s], j * p.block_k,
                          x0 + kx * p.dil_w - p.pad_w, y0 + ky * p.dil_h - p.pad_h, b);
            }
            const int k0 = tap * p.cin + j * p.block_k;
            if (load_b) tma_load_2d(smem_b + static_cast<size_t>(s) * b_bytes, &weight_map, &ctl.full[s], k0, n0);
            if (!INT8) {
              const int w_tile = (k0 >> 5) >> 2;
#pragma unroll
              for (int i = 0; i < kScaleTilesB; ++i) {
                const int row_tile = min(n0 / 128 + i, p.weight_row_tiles - 1);
                bulk_load(smem_sfb + (static_cast<size_t>(s) * kScaleTilesB + i) * 512,
                          p.weight_scales + (static_cast<size_t>(row_tile) * p.weight_scale_tiles + w_tile) * 512, 512,
                          &ctl.full[s]);
              }
              if (dynamic_a) {
                const int a_tile = ((j * p.block_k) >> 5) >> 2;
                bulk_load(smem_sfa + static_cast<size_t>(s) * 512,
                          p.act_scales + (static_cast<size_t>(m_tile) * p.act_scale_tiles + a_tile) * 512, 512, &ctl.full[s]);
              }
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer =====
    if (lane == 0) {
      uint32_t it = 0, tile_it = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < p.total_tiles && alive; tile += gridDim.x, ++tile_it) {
        const uint32_t acc = tile_it % kAccStages;
        if (!mbar_wait(&ctl.tmem_empty[acc], ((tile_it / kAccStages) & 1) ^ 1, &ctl.abort_flag, p.status, kStatusWaitTmemEmpty)) {
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem + acc * BN;
        for (int ki = 0; ki < k_iters; ++ki, ++it) {
          const int s = it % p.stages;
          if (!mbar_wait(&ctl.full[s], (it / p.stages) & 1, &ctl.abort_flag, p.status, kStatusWaitFull)) {
            alive = false;
            break;
          }
          tc_fence_after();
          const int tap = ki / p.k_chunks, j = ki - tap * p.k_chunks;
          uint32_t a_id0 = 0, b_id0 = 0;
          if (!INT8) {
            const int kb_w = (tap * p.cin + j * p.block_k) >> 5;
            const int kb_a = (j * p.block_k) >> 5;
            a_id0 = kb_a & 3, b_id0 = kb_w & 3;
#pragma unroll
            for (int i = 0; i < kScaleTilesB; ++i) {
              tc_copy_scales(tmem + kSfbColumn + 4 * i, scale_desc(smem_u32(smem_sfb + (static_cast<size_t>(s) * kScaleTilesB + i) * 512)));
            }
            const uint8_t* sfa = dynamic_a ? smem_sfa + static_cast<size_t>(s) * 512 : smem_sfa_static + (kb_a >> 2) * 512;
            tc_copy_scales(tmem + kSfaColumn, scale_desc(smem_u32(sfa)));
          }
          const uint64_t a_desc = kmajor_desc(smem_u32(smem_a + static_cast<size_t>(s) * a_bytes), p.block_k);
          const uint64_t b_desc = kmajor_desc(smem_u32(smem_b + static_cast<size_t>(s) * b_bytes), p.block_k);
          const int k_steps = p.block_k >> 5;
          for (int k = 0; k < k_steps; ++k) {
            const uint32_t accumulate = (ki > 0 || k > 0) ? 1u : 0u;
            if (INT8) {
              tc_mma_i8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc_i8(BN), accumulate);
            } else {
              tc_mma_mxf8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc_mxf8(BN, a_id0 + k, b_id0 + k), tmem + kSfaColumn,
                          tmem + kSfbColumn, accumulate);
            }
          }
          tc_commit(&ctl.empty[s]);  // the stage is free once these MMAs have read it
        }
        if (alive) tc_commit(&ctl.tmem_full[acc]);
      }
    }
  } else {
    // ===== epilogue: warp w owns tensor-memory lanes 32 * (w % 4) ... + 31 =====
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int ry = row / p.tile_w, rx = row - ry * p.tile_w;
    const bool row_in_tile = row < p.tile_h * p.tile_w;
    const float a_scale = INT8 && p.a_scale != nullptr ? __ldg(p.a_scale) : 1.0f;
    uint32_t tile_it = 0;
    for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++tile_it) {
      const int nt = tile % p.tiles_n;
      int m = tile / p.tiles_n;
      const int tx = m % p.tiles_x; m /= p.tiles_x;
      const int ty = m % p.tiles_y;
      const int b = m / p.tiles_y;
      const int x = tx * p.tile_w + rx, y = ty * p.tile_h + ry, n0 = nt * BN;
      const bool valid = row_in_tile && x < p.out_w && y < p.out_h;
      const size_t pixel = (static_cast<size_t>(b) * p.out_h + y) * p.out_w + x;
      const uint32_t acc = tile_it % kAccStages;
      if (!mbar_wait(&ctl.tmem_full[acc], (tile_it / kAccStages) & 1, &ctl.abort_flag, p.status, kStatusWaitTmemFull)) break;
      tc_fence_after();
      const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (n0 + c0 >= p.cout) break;  // warp-uniform
        uint32_t raw[32];
        tmem_load_32(lane_addr + c0, raw);
        tmem_load_wait();
        if (valid && !(p.debug & 4)) finish_chunk<INT8>(p, raw, n0 + c0, pixel, b, y, x, a_scale);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.tmem_empty[acc]);
    }
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
  int tile_h, tile_w, block_n, block_k, stages, ctas;
  int tiles_x, tiles_y, tiles_n, total_tiles;
  bool flat;
  int out_h, out_w;
};

int make_plan(const FimConvGeometry& g, bool int8, bool per_pixel, bool allow_flat, Plan* plan) {
  if (g.batch <= 0 || g.height <= 0 || g.width <= 0 || g.cin <= 0 || g.cout <= 0) return kBadArgument;
  if (g.cin % 32 || g.cout % 32) return kUnsupported;
  if (g.stride_h != 1 || g.stride_w != 1) return kUnsupported;
  if (g.kh < 1 || g.kw < 1 || g.dil_h < 1 || g.dil_w < 1 || g.pad_h < 0 || g.pad_w < 0) return kBadArgument;
  const int out_h = g.height + 2 * g.pad_h - g.dil_h * (g.kh - 1);
  const int out_w = g.width + 2 * g.pad_w - g.dil_w * (g.kw - 1);
  if (out_h <= 0 || out_w <= 0) return kBadArgument;
  const bool pointwise = g.kh == 1 && g.kw == 1 && g.pad_h == 0 && g.pad_w == 0;
  if (per_pixel && !(pointwise && allow_flat)) return kUnsupported;
  Plan pl;
  pl.out_h = out_h, pl.out_w = out_w;
  pl.block_k = g.cin % 128 == 0 ? 128 : (g.cin % 64 == 0 ? 64 : 32);
  int bn = g.cout <= 64 ? 64 : 128;
  if (g_forced_block_n == 256 && g.cout > 128) bn = 256;
  if (g_forced_block_n == 128 && g.cout > 64) bn = 128;
  pl.block_n = bn;
  pl.flat = pointwise && allow_flat;
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
  const long long total = static_cast<long long>(pl.tiles_x) * pl.tiles_y * (pl.flat ? 1 : g.batch) * pl.tiles_n;
  if (total > 0x7fffffffLL) return kUnsupported;
  pl.total_tiles = static_cast<int>(total);
  const int scale_bytes = int8 ? 0 : ((bn <= 128 ? 1 : bn / 128) * 512 + 512);
  const int stage_bytes = kTileM * pl.block_k + bn * pl.block_k + scale_bytes;
  pl.stages = kSmemBudget / stage_bytes;
  if (pl.stages > kMaxStages) pl.stages = kMaxStages;
  if (pl.stages < 2) return kUnsupported;
  const int sms = g_max_ctas > 0 && g_max_ctas < 148 ? g_max_ctas : 148;
  pl.ctas = pl.total_tiles < sms ? pl.total_tiles : sms;
  *plan = pl;
  return kOk;
}

template <bool INT8, int BN>
int launch_conv(const CUtensorMap& act_map, const CUtensorMap& weight_map, const ConvParams& p, int ctas, cudaStream_t stream) {
  const int scale_tiles_b = BN <= 128 ? 1 : BN / 128;
  const size_t smem = 1024 + static_cast<size_t>(p.stages) * (kTileM * p.block_k + BN * p.block_k + scale_tiles_b * 512 + 512) +
                      static_cast<size_t>((p.cin + 127) / 128) * 512;
  static bool configured = false;
  if (!configured) {
    const cudaError_t e = cudaFuncSetAttribute(conv_kernel<INT8, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  if (smem > 226 * 1024) return kUnsupported;
  conv_kernel<INT8, BN><<<ctas, kThreads, smem, stream>>>(act_map, weight_map, p);
  return static_cast<int>(cudaGetLastError());
}

bool aligned16(const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

int run_conv(bool int8, const void* x, const int8_t* act_exponent, const void* act_scales, const void* weight,
             const void* weight_scales, const float* a_scale, const float* w_scale, const FimConvGeometry* g,
             const FimConvEpilogue* ep, void* out, int* status, void* stream) {
  if (x == nullptr || weight == nullptr || g == nullptr || ep == nullptr || out == nullptr) return kBadArgument;
  if (int8) {
    if (ep->out_mode != FIM_OUT_INT32 && (a_scale == nullptr || w_scale == nullptr)) return kBadArgument;
    if (ep->out_mode != FIM_OUT_BF16 && ep->out_mode != FIM_OUT_INT8 && ep->out_mode != FIM_OUT_INT32) return kBadArgument;
    if (ep->out_mode == FIM_OUT_INT8 && ep->out_scale == nullptr) return kBadArgument;
    if (ep->act == FIM_ACT_GELU) return kUnsupported;
  } else {
    if (weight_scales == nullptr || (act_exponent == nullptr) == (act_scales == nullptr)) return kBadArgument;
    if (ep->out_mode == FIM_OUT_INT8 || ep->out_mode == FIM_OUT_INT32) return kBadArgument;
    if (ep->out_mode == FIM_OUT_E4M3_STATIC && ep->out_exponent == nullptr) return kBadArgument;
    if (ep->out_mode == FIM_OUT_E4M3_DYNAMIC && ep->out_scales == nullptr) return kBadArgument;
  }
  if (ep->act < 0 || ep->act > 2 || ep->out_mode < 0 || ep->out_mode > 5) return kBadArgument;
  if (!aligned16(x) || !aligned16(weight) || !aligned16(out) || (ep->bias && !aligned16(ep->bias)) ||
      (weight_scales && !aligned16(weight_scales)) || (act_scales && !aligned16(act_scales))) {
    return kBadLayout;
  }
  if (g->batch == 0 || g->height == 0 || g->width == 0) return kOk;

  // a 1x1 conv is a plain GEMM over flattened pixels when the residual (if any) is dense NHWC
  bool allow_flat = true;
  Plan pl;
  {
    Plan probe;
    const int rc0 = make_plan(*g, int8, act_scales != nullptr, true, &probe);
    if (rc0 != kOk) return rc0;
    if (probe.flat && ep->residual != nullptr) {
      const long long c = ep->res_stride[3], xs = ep->res_stride[2], ys = ep->res_stride[1], bs = ep->res_stride[0];
      const bool dense = c == 1 && ys == xs * probe.out_w && bs == ys * probe.out_h;
      if (!dense) allow_flat = false;
    }
  }
  const int rc = make_plan(*g, int8, act_scales != nullptr, allow_flat, &pl);
  if (rc != kOk) return rc;

  ConvParams p;
  p.batch = g->batch, p.height = g->height, p.width = g->width, p.cin = g->cin, p.cout = g->cout;
  p.out_h = pl.out_h, p.out_w = pl.out_w;
  p.kh = g->kh, p.kw = g->kw, p.pad_h = g->pad_h, p.pad_w = g->pad_w, p.dil_h = g->dil_h, p.dil_w = g->dil_w;
  p.tile_h = pl.tile_h, p.tile_w = pl.tile_w, p.tiles_x = pl.tiles_x, p.tiles_y = pl.tiles_y, p.tiles_n = pl.tiles_n;
  p.total_tiles = pl.total_tiles;
  p.block_k = pl.block_k, p.k_chunks = g->cin / pl.block_k, p.stages = pl.stages;
  p.act_exponent = act_exponent;
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
  p.act = ep->act, p.out_mode = ep->out_mode;
  p.out_exponent = ep->out_exponent;
  p.out_scales = static_cast<uint8_t*>(ep->out_scales);
  p.out_scale = ep->out_scale;
  p.out = out;
  p.status = status;
  p.debug = g_debug_flags;

  // tensor maps: activations [B, H, W, Cin] (flat: [1, 1, B*H*W, Cin]) and weights [Cout, K]
  long long eff_b = g->batch, eff_h = g->height, eff_w = g->width;
  if (pl.flat) {
    eff_w = static_cast<long long>(g->batch) * g->height * g->width;
    eff_h = 1, eff_b = 1;
    p.batch = 1, p.height = 1, p.out_h = 1;
    p.width = p.out_w = static_cast<int>(eff_w);
    if (p.residual != nullptr) p.res_stride[0] = 0, p.res_stride[1] = 0;  // dense: the flat column index addresses it
  }
  CUtensorMap act_map, weight_map;
  const uint64_t adims[4] = {static_cast<uint64_t>(g->cin), static_cast<uint64_t>(eff_w), static_cast<uint64_t>(eff_h),
                             static_cast<uint64_t>(eff_b)};
  const uint64_t astrides[3] = {static_cast<uint64_t>(g->cin), static_cast<uint64_t>(eff_w) * g->cin,
                                static_cast<uint64_t>(eff_h) * eff_w * g->cin};
  const uint32_t abox[4] = {static_cast<uint32_t>(pl.block_k), static_cast<uint32_t>(pl.tile_w), static_cast<uint32_t>(pl.tile_h), 1};
  int rcm = make_tensor_map(&act_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, x, adims, astrides, abox, swizzle_for_bytes(pl.block_k));
  if (rcm != kOk) return rcm;
  const uint64_t k_total = static_cast<uint64_t>(g->kh) * g->kw * g->cin;
  const uint64_t wdims[2] = {k_total, static_cast<uint64_t>(g->cout)};
  const uint64_t wstrides[1] = {k_total};
  const uint32_t wbox[2] = {static_cast<uint32_t>(pl.block_k), static_cast<uint32_t>(pl.block_n)};
  rcm = make_tensor_map(&weight_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, weight, wdims, wstrides, wbox, swizzle_for_bytes(pl.block_k));
  if (rcm != kOk) return rcm;

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int8) {
    if (pl.block_n == 64) return launch_conv<true, 64>(act_map, weight_map, p, pl.ctas, s);
    if (pl.block_n == 128) return launch_conv<true, 128>(act_map, weight_map, p, pl.ctas, s);
    return launch_conv<true, 256>(act_map, weight_map, p, pl.ctas, s);
  }
  if (pl.block_n == 64) return launch_conv<false, 64>(act_map, weight_map, p, pl.ctas, s);
  if (pl.block_n == 128) return launch_conv<false, 128>(act_map, weight_map, p, pl.ctas, s);
  return launch_conv<false, 256>(act_map, weight_map, p, pl.ctas, s);
}

}  // namespace
}  // namespace fim

using namespace fim;

extern "C" int fim_mxfp8_conv2d(const void* x, const int8_t* act_exponent, const void* act_scales_swizzled, const void* weight,
                                const void* weight_scales_swizzled, const FimConvGeometry* geometry,
                                const FimConvEpilogue* epilogue, void* out, int* status, void* stream) {
  return run_conv(false, x, act_exponent, act_scales_swizzled, weight, weight_scales_swizzled, nullptr, nullptr, geometry, epilogue,
                  out, status, stream);
}

extern "C" int fim_int8_conv2d(const void* x, const void* weight, const float* a_scale, const float* w_scale,
                               const FimConvGeometry* geometry, const FimConvEpilogue* epilogue, void* out, int* status,
                               void* stream) {
  return run_conv(true, x, nullptr, nullptr, weight, nullptr, a_scale, w_scale, geometry, epilogue, out, status, stream);
}

extern "C" int fim_conv_plan(const FimConvGeometry* geometry, int int8, int per_pixel_scales, int plan[6]) {
  if (geometry == nullptr || plan == nullptr) return kBadArgument;
  Plan pl;
  const int rc = make_plan(*geometry, int8 != 0, per_pixel_scales != 0, true, &pl);
  if (rc != kOk) return rc;
  plan[0] = pl.tile_h, plan[1] = pl.tile_w, plan[2] = pl.block_n, plan[3] = pl.block_k, plan[4] = pl.stages, plan[5] = pl.ctas;
  return kOk;
}

extern "C" void fim_conv_tune(int block_n, int max_ctas, int debug_flags) {
  g_forced_block_n = block_n;
  g_max_ctas = max_ctas;
  g_debug_flags = debug_flags;
}
