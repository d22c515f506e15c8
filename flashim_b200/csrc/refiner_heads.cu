// RoMaV2 refiner heads: the 1x1 convolution to 2 warp + 4 confidence channels with the warp update and the precision
// parametrisation behind it, one pass over the last block's output (flashim/ops/romav2.py:95-120; Triton kernel
// flashim/backends/triton/romav2.py:202-250). Six fp32 dot products per pixel on the CUDA cores, exact fp32 like the
// reference's (a 6-column GEMM would waste the tensor cores); HBM-bound: 2 * C bytes read and 24 bytes written per pixel.
#include "common.cuh"
#include "flashim_sm100.h"

namespace fim {
namespace {

constexpr int kHeadThreads = 256;
constexpr int kHeadOutputs = 6;
constexpr int kHeadMaxChannels = 512;

__device__ __forceinline__ float softplus(float x) { return x > 20.0f ? x : log1pf(expf(x)); }  // torch's threshold

// Eight lanes share four consecutive pixels: each reads 16 bytes (8 channels) of every pixel per 64-channel step and
// reuses the six weight vectors it fetched from shared memory for all four, keeping 24 partial sums. The sums are added
// across the eight lanes by a transposing butterfly (12 + 6 + 3 exchanges instead of 24 x 3): afterwards lane l of the
// group holds sums 3l .. 3l+2 of the 24, i.e. lanes 2p and 2p+1 hold outputs 0-2 and 3-5 of pixel p, which is how the
// epilogue splits: the even lane finishes the warp and the first confidence channel, the odd lane the precision terms.
constexpr int kHeadPixels = 4;

__global__ void __launch_bounds__(kHeadThreads) refiner_heads_kernel(const uint4* __restrict__ z, const float* __restrict__ weight,
                                                                     const float* __restrict__ bias, const float* __restrict__ prev_warp,
                                                                     const float* __restrict__ prev_conf, int prev_channels,
                                                                     float* __restrict__ warp_out, float* __restrict__ conf_out,
                                                                     long long rows, int channels, float inv_norm_x, float inv_norm_y) {
  __shared__ __align__(16) float w[kHeadOutputs * kHeadMaxChannels];
  for (int i = threadIdx.x; i < kHeadOutputs * channels; i += kHeadThreads) w[i] = __ldg(weight + i);
  __syncthreads();
  const int part = threadIdx.x & 7;
  const uint32_t group = 0xFFu << ((threadIdx.x & 31) & ~7);
  const long long stride = static_cast<long long>(gridDim.x) * (kHeadThreads / 8) * kHeadPixels;
  const int row_words = channels / 8;  // 16-byte words per pixel
  // the loop bound is the same for the eight lanes of a group and the shuffles stay inside the group
  for (long long base = (blockIdx.x * static_cast<long long>(kHeadThreads / 8) + (threadIdx.x >> 3)) * kHeadPixels; base < rows;
       base += stride) {
    float sum[kHeadPixels * kHeadOutputs];
#pragma unroll
    for (int k = 0; k < kHeadPixels * kHeadOutputs; ++k) sum[k] = 0.0f;
    // the loads of the next 64-channel step are issued before the arithmetic of this one
    uint4 next[kHeadPixels];
#pragma unroll
    for (int p = 0; p < kHeadPixels; ++p) {
      next[p] = (base + p < rows && part < row_words) ? __ldg(z + (base + p) * row_words + part) : make_uint4(0u, 0u, 0u, 0u);
    }
    for (int word = part; word < row_words; word += 8) {
      float v[kHeadPixels][8];
      uint4 now[kHeadPixels];
#pragma unroll
      for (int p = 0; p < kHeadPixels; ++p) {
        now[p] = next[p];
        if (word + 8 < row_words) next[p] = base + p < rows ? __ldg(z + (base + p) * row_words + word + 8) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int p = 0; p < kHeadPixels; ++p) {
        const uint4 q = now[p];
        v[p][0] = bf16_lo(q.x), v[p][1] = bf16_hi(q.x), v[p][2] = bf16_lo(q.y), v[p][3] = bf16_hi(q.y);
        v[p][4] = bf16_lo(q.z), v[p][5] = bf16_hi(q.z), v[p][6] = bf16_lo(q.w), v[p][7] = bf16_hi(q.w);
      }
#pragma unroll
      for (int o = 0; o < kHeadOutputs; ++o) {
        const float4 a = *reinterpret_cast<const float4*>(w + o * channels + word * 8);
        const float4 b = *reinterpret_cast<const float4*>(w + o * channels + word * 8 + 4);
        const float c[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int p = 0; p < kHeadPixels; ++p) {
#pragma unroll
          for (int j = 0; j < 8; ++j) sum[p * kHeadOutputs + o] = fmaf(v[p][j], c[j], sum[p * kHeadOutputs + o]);
        }
      }
    }
    float r12[12], r6[6], r3[3];
    {
      const bool upper = part & 4;
#pragma unroll
      for (int i = 0; i < 12; ++i) r12[i] = (upper ? sum[12 + i] : sum[i]) + __shfl_xor_sync(group, upper ? sum[i] : sum[12 + i], 4);
    }
    {
      const bool upper = part & 2;
#pragma unroll
      for (int i = 0; i < 6; ++i) r6[i] = (upper ? r12[6 + i] : r12[i]) + __shfl_xor_sync(group, upper ? r12[i] : r12[6 + i], 2);
    }
    {
      const bool upper = part & 1;
#pragma unroll
      for (int i = 0; i < 3; ++i) r3[i] = (upper ? r6[3 + i] : r6[i]) + __shfl_xor_sync(group, upper ? r6[i] : r6[3 + i], 1);
    }
    const long long row = base + (part >> 1);
    if (row >= rows) continue;
    if ((part & 1) == 0) {
      const float d0 = r3[0] + __ldg(bias + 0), d1 = r3[1] + __ldg(bias + 1), c0 = r3[2] + __ldg(bias + 2);
      const float2 pw = __ldg(reinterpret_cast<const float2*>(prev_warp) + row);
      reinterpret_cast<float2*>(warp_out)[row] = make_float2(pw.x + d0 * inv_norm_x, pw.y + d1 * inv_norm_y);
      conf_out[row * 4] = __ldg(prev_conf + row * prev_channels) + c0;
    } else {
      const float x1 = r3[0] + __ldg(bias + 3), l10 = r3[1] + __ldg(bias + 4), x3 = r3[2] + __ldg(bias + 5);
      const float l00 = softplus(x1) + 1e-6f, l11 = softplus(x3) + 1e-6f;
      float c1 = l00 * l00, c2 = l00 * l10, c3 = l10 * l10 + l11 * l11;
      if (prev_channels == 4) {
        c1 += __ldg(prev_conf + row * 4 + 1), c2 += __ldg(prev_conf + row * 4 + 2), c3 += __ldg(prev_conf + row * 4 + 3);
      }
      conf_out[row * 4 + 1] = c1, conf_out[row * 4 + 2] = c2, conf_out[row * 4 + 3] = c3;
    }
  }
}

}  // namespace
}  // namespace fim

using namespace fim;

extern "C" int fim_romav2_refiner_heads(const void* z, const float* weight, const float* bias, const float* prev_warp,
                                        const float* prev_confidence, int prev_channels, float* warp, float* confidence,
                                        long long rows, int channels, float inv_norm_x, float inv_norm_y, void* stream) {
  if (rows < 0 || channels <= 0 || (prev_channels != 1 && prev_channels != 4)) return kBadArgument;
  if (channels % 8 || channels > kHeadMaxChannels) return kUnsupported;
  if (rows == 0) return kOk;
  if (z == nullptr || weight == nullptr || bias == nullptr || prev_warp == nullptr || prev_confidence == nullptr ||
      warp == nullptr || confidence == nullptr) {
    return kBadArgument;
  }
  const auto misaligned = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) != 0; };
  if (misaligned(z, 16) || misaligned(prev_warp, 8) || misaligned(warp, 8) || misaligned(confidence, 16) ||
      misaligned(prev_confidence, prev_channels == 4 ? 16 : 4)) {
    return kBadLayout;
  }
  const long long per_block = (kHeadThreads / 8) * kHeadPixels;
  const long long blocks = (rows + per_block - 1) / per_block;
  const unsigned grid = static_cast<unsigned>(blocks < 148LL * 8 ? blocks : 148LL * 8);
  refiner_heads_kernel<<<grid, kHeadThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(z), weight, bias, prev_warp, prev_confidence, prev_channels, warp, confidence, rows, channels,
      inv_norm_x, inv_norm_y);
  return static_cast<int>(cudaGetLastError());
}
