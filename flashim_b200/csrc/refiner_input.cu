// RoMaV2 refiner input: for every pixel of A the channels-last bf16 row [f_a, f_b sampled at the warp, embedding of the
// scaled displacement, local correlation of f_a / sqrt(P) with f_b over a (2r+1)^2 window around the warp]
// (flashim/ops/romav2.py:36-66; local correlation flashim/ops/correlation.py:13-39; bilinear sampling with zeros padding
// and align_corners = False as F.grid_sample).
//
// The window positions are one feature pixel apart, so all (2r+1)^2 bilinear samples share one fractional offset and
// their corners form a (2r+2)^2 patch of f_b around the warped position. A warp owns a pixel: its lanes first form the
// dot products of f_a / sqrt(P) with each pixel of the patch (eight lanes per patch pixel, f_a from shared memory),
// then every correlation value is the bilinear blend of four neighbouring dot products: (2r+2)^2 reads of P channels
// instead of 4 (2r+1)^2. The four centre pixels of the patch are also the corners of the f_b sample.
#include "common.cuh"
#include "flashim_sm100.h"

namespace fim {
namespace {

constexpr int kInputWarps = 8;
constexpr int kInputMaxFeatures = 256;  // P
constexpr int kInputMaxRadius = 3;
constexpr int kInputMaxPatch = (2 * kInputMaxRadius + 2) * (2 * kInputMaxRadius + 2);

struct InputParams {
  const float* f_a;
  const float* f_b;
  const float* warp;
  const float* emb_weight;  // [E, 2]
  const float* emb_bias;    // [E]
  __nv_bfloat16* out;       // [B, h, w, 2P + E + K]
  int batch, height, width, features, embedding, radius, pair;
  float scale_x, scale_y, root_features;
};

__device__ __forceinline__ void store_bf16(__nv_bfloat16* at, float v) { *at = __float2bfloat16_rn(v); }

__global__ void __launch_bounds__(32 * kInputWarps) refiner_input_kernel(const InputParams p) {
  __shared__ __align__(16) float scaled_a[kInputWarps][kInputMaxFeatures];
  __shared__ float dots[kInputWarps][kInputMaxPatch];
  const int warp_id = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int P = p.features, E = p.embedding;
  const int r = p.radius < 0 ? 0 : p.radius;
  const int side = 2 * r + 2, window = 2 * r + 1;
  const int K = p.radius < 0 ? 0 : window * window;
  const int C = 2 * P + E + K;
  const long long pixels = static_cast<long long>(p.batch) * p.height * p.width;
  float* a_row = scaled_a[warp_id];
  float* dot = dots[warp_id];

  for (long long pixel = blockIdx.x * static_cast<long long>(kInputWarps) + warp_id; pixel < pixels;
       pixel += static_cast<long long>(gridDim.x) * kInputWarps) {
    const unsigned flat = static_cast<unsigned>(pixel);  // the host refuses more than 2**31 pixels
    const int x = static_cast<int>(flat % static_cast<unsigned>(p.width));
    const int y = static_cast<int>((flat / static_cast<unsigned>(p.width)) % static_cast<unsigned>(p.height));
    const int b = static_cast<int>(flat / (static_cast<unsigned>(p.width) * static_cast<unsigned>(p.height)));
    const int b_other = p.pair > 0 ? (b + p.batch - p.pair) % p.batch : b;  // f_b = roll(f_a, pair) along the batch
    const float* other = p.f_b + static_cast<long long>(b_other) * p.height * p.width * P;
    __nv_bfloat16* out = p.out + pixel * C;

    // f_a: copied to the output, and divided by sqrt(P) into shared memory for the dot products
    for (int c = 4 * lane; c < P; c += 128) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(p.f_a + pixel * P + c));
      store_bf16(out + c, a.x), store_bf16(out + c + 1, a.y), store_bf16(out + c + 2, a.z), store_bf16(out + c + 3, a.w);
      *reinterpret_cast<float4*>(a_row + c) = make_float4(a.x / p.root_features, a.y / p.root_features, a.z / p.root_features,
                                                          a.w / p.root_features);
    }
    const float2 at = __ldg(reinterpret_cast<const float2*>(p.warp) + pixel);
    // pixel coordinates of the warped position (align_corners = False) and its bilinear weights
    const float ix = ((at.x + 1.0f) * p.width - 1.0f) * 0.5f, iy = ((at.y + 1.0f) * p.height - 1.0f) * 0.5f;
    const float fx0 = floorf(ix), fy0 = floorf(iy);
    const float tx = ix - fx0, ty = iy - fy0;
    const float w_nw = (1.0f - tx) * (1.0f - ty), w_ne = tx * (1.0f - ty), w_sw = (1.0f - tx) * ty, w_se = tx * ty;
    // far outside the image (or not finite) every sample is zero; clamping keeps the integer arithmetic in range
    const int x0 = static_cast<int>(fminf(fmaxf(fx0, -16.0f), static_cast<float>(p.width) + 16.0f));
    const int y0 = static_cast<int>(fminf(fmaxf(fy0, -16.0f), static_cast<float>(p.height) + 16.0f));
    const bool finite = fabsf(ix) < 1e9f && fabsf(iy) < 1e9f;
    __syncwarp();

    // dot products with the patch pixels (y0 - r + j, x0 - r + i): eight lanes per patch pixel read its channels in
    // 16-byte pieces (a warp-wide load touches four pixels' contiguous rows, not 32 scattered lines) and add up by shuffles
    {
      const int group = lane >> 3, sub = lane & 7;
      for (int first = 0; first < side * side; first += 4) {
        const int pos = first + group;
        const int yy = y0 - r + pos / side, xx = x0 - r + pos % side;
        float sum = 0.0f;
        if (K > 0 && finite && pos < side * side && yy >= 0 && yy < p.height && xx >= 0 && xx < p.width) {
          const float* src = other + (static_cast<long long>(yy) * p.width + xx) * P;
          for (int c = 4 * sub; c < P; c += 32) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(src + c));
            const float4 a = *reinterpret_cast<const float4*>(a_row + c);
            sum = fmaf(a.x, v.x, sum), sum = fmaf(a.y, v.y, sum), sum = fmaf(a.z, v.z, sum), sum = fmaf(a.w, v.w, sum);
          }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if (sub == 0 && pos < side * side) dot[pos] = sum;
      }
    }
    // f_b sampled at the warp: the four centre pixels of the patch, a lane per four channels
    {
      const bool north = finite && y0 >= 0 && y0 < p.height, south = finite && y0 + 1 >= 0 && y0 + 1 < p.height;
      const bool west = x0 >= 0 && x0 < p.width, east = x0 + 1 >= 0 && x0 + 1 < p.width;
      const float* base = other + (static_cast<long long>(y0) * p.width + x0) * P;
      const long long down = static_cast<long long>(p.width) * P;
      const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int c = 4 * lane; c < P; c += 128) {
        const float4 nw = north && west ? __ldg(reinterpret_cast<const float4*>(base + c)) : zero;
        const float4 ne = north && east ? __ldg(reinterpret_cast<const float4*>(base + P + c)) : zero;
        const float4 sw = south && west ? __ldg(reinterpret_cast<const float4*>(base + down + c)) : zero;
        const float4 se = south && east ? __ldg(reinterpret_cast<const float4*>(base + down + P + c)) : zero;
        store_bf16(out + P + c, nw.x * w_nw + ne.x * w_ne + sw.x * w_sw + se.x * w_se);
        store_bf16(out + P + c + 1, nw.y * w_nw + ne.y * w_ne + sw.y * w_sw + se.y * w_se);
        store_bf16(out + P + c + 2, nw.z * w_nw + ne.z * w_ne + sw.z * w_sw + se.z * w_se);
        store_bf16(out + P + c + 3, nw.w * w_nw + ne.w * w_ne + sw.w * w_sw + se.w * w_se);
      }
    }
    // embedding of the scaled displacement from the identity grid (pixel centres: -1 + (2x + 1) / w)
    {
      const float dx = p.scale_x * (at.x - (-1.0f + (2.0f * x + 1.0f) / p.width));
      const float dy = p.scale_y * (at.y - (-1.0f + (2.0f * y + 1.0f) / p.height));
      for (int e = lane; e < E; e += 32) {
        const float2 weight = __ldg(reinterpret_cast<const float2*>(p.emb_weight) + e);
        store_bf16(out + 2 * P + e, fmaf(weight.y, dy, weight.x * dx) + __ldg(p.emb_bias + e));
      }
    }
    __syncwarp();
    // correlation values: the bilinear blend of four neighbouring dot products
    for (int k = lane; k < K; k += 32) {
      const int at_patch = (k / window) * side + k % window;
      const float v = dot[at_patch] * w_nw + dot[at_patch + 1] * w_ne + dot[at_patch + side] * w_sw + dot[at_patch + side + 1] * w_se;
      store_bf16(out + 2 * P + E + k, v);
    }
    __syncwarp();  // the next pixel overwrites this warp's shared rows
  }
}

// Without a correlation window (radius < 0, RoMaV2's full-resolution refiner with 12 features) a pixel is little work:
// eight lanes share one, so a warp handles four pixels at a time.
__global__ void __launch_bounds__(256) refiner_input_plain_kernel(const InputParams p) {
  const int P = p.features, E = p.embedding, C = 2 * P + E;
  const unsigned pixels = static_cast<unsigned>(p.batch) * p.height * p.width;
  const int sub = threadIdx.x & 7;
  for (unsigned pixel = blockIdx.x * 32u + (threadIdx.x >> 3); pixel < pixels; pixel += gridDim.x * 32u) {
    const int x = static_cast<int>(pixel % static_cast<unsigned>(p.width));
    const int y = static_cast<int>((pixel / static_cast<unsigned>(p.width)) % static_cast<unsigned>(p.height));
    const int b = static_cast<int>(pixel / (static_cast<unsigned>(p.width) * static_cast<unsigned>(p.height)));
    const int b_other = p.pair > 0 ? (b + p.batch - p.pair) % p.batch : b;
    const float* other = p.f_b + static_cast<long long>(b_other) * p.height * p.width * P;
    __nv_bfloat16* out = p.out + static_cast<long long>(pixel) * C;
    const float2 at = __ldg(reinterpret_cast<const float2*>(p.warp) + pixel);
    const float ix = ((at.x + 1.0f) * p.width - 1.0f) * 0.5f, iy = ((at.y + 1.0f) * p.height - 1.0f) * 0.5f;
    const float fx0 = floorf(ix), fy0 = floorf(iy);
    const float tx = ix - fx0, ty = iy - fy0;
    const float w_nw = (1.0f - tx) * (1.0f - ty), w_ne = tx * (1.0f - ty), w_sw = (1.0f - tx) * ty, w_se = tx * ty;
    const int x0 = static_cast<int>(fminf(fmaxf(fx0, -16.0f), static_cast<float>(p.width) + 16.0f));
    const int y0 = static_cast<int>(fminf(fmaxf(fy0, -16.0f), static_cast<float>(p.height) + 16.0f));
    const bool finite = fabsf(ix) < 1e9f && fabsf(iy) < 1e9f;
    const bool north = finite && y0 >= 0 && y0 < p.height, south = finite && y0 + 1 >= 0 && y0 + 1 < p.height;
    const bool west = x0 >= 0 && x0 < p.width, east = x0 + 1 >= 0 && x0 + 1 < p.width;
    const float* base = other + (static_cast<long long>(y0) * p.width + x0) * P;
    const long long down = static_cast<long long>(p.width) * P;
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c = 4 * sub; c < P; c += 32) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(p.f_a + static_cast<long long>(pixel) * P + c));
      const float4 nw = north && west ? __ldg(reinterpret_cast<const float4*>(base + c)) : zero;
      const float4 ne = north && east ? __ldg(reinterpret_cast<const float4*>(base + P + c)) : zero;
      const float4 sw = south && west ? __ldg(reinterpret_cast<const float4*>(base + down + c)) : zero;
      const float4 se = south && east ? __ldg(reinterpret_cast<const float4*>(base + down + P + c)) : zero;
      store_bf16(out + c, a.x), store_bf16(out + c + 1, a.y), store_bf16(out + c + 2, a.z), store_bf16(out + c + 3, a.w);
      store_bf16(out + P + c, nw.x * w_nw + ne.x * w_ne + sw.x * w_sw + se.x * w_se);
      store_bf16(out + P + c + 1, nw.y * w_nw + ne.y * w_ne + sw.y * w_sw + se.y * w_se);
      store_bf16(out + P + c + 2, nw.z * w_nw + ne.z * w_ne + sw.z * w_sw + se.z * w_se);
      store_bf16(out + P + c + 3, nw.w * w_nw + ne.w * w_ne + sw.w * w_sw + se.w * w_se);
    }
    const float dx = p.scale_x * (at.x - (-1.0f + (2.0f * x + 1.0f) / p.width));
    const float dy = p.scale_y * (at.y - (-1.0f + (2.0f * y + 1.0f) / p.height));
    for (int e = sub; e < E; e += 8) {
      const float2 weight = __ldg(reinterpret_cast<const float2*>(p.emb_weight) + e);
      store_bf16(out + 2 * P + e, fmaf(weight.y, dy, weight.x * dx) + __ldg(p.emb_bias + e));
    }
  }
}

}  // namespace
}  // namespace fim

using namespace fim;

extern "C" int fim_romav2_refiner_input(const float* f_a, const float* f_b, const float* warp, const float* emb_weight,
                                        const float* emb_bias, float scale_x, float scale_y, void* out, int batch, int height,
                                        int width, int features, int embedding, int radius, int pair, void* stream) {
  if (batch < 0 || height < 0 || width < 0 || features <= 0 || embedding < 0 || pair < 0) return kBadArgument;
  if (features % 4 || features > kInputMaxFeatures || radius > kInputMaxRadius) return kUnsupported;
  if (pair > 0 && batch != 2 * pair) return kBadArgument;
  if (batch == 0 || height == 0 || width == 0) return kOk;
  if (f_a == nullptr || f_b == nullptr || warp == nullptr || out == nullptr || (embedding > 0 && (emb_weight == nullptr || emb_bias == nullptr))) {
    return kBadArgument;
  }
  const auto misaligned = [](const void* q, uintptr_t a) { return (reinterpret_cast<uintptr_t>(q) & (a - 1)) != 0; };
  if (misaligned(f_a, 16) || misaligned(f_b, 16) || misaligned(warp, 8) || misaligned(emb_weight, 8) || misaligned(out, 2)) return kBadLayout;
  InputParams p;
  p.f_a = f_a, p.f_b = pair > 0 ? f_a : f_b, p.warp = warp, p.emb_weight = emb_weight, p.emb_bias = emb_bias;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.batch = batch, p.height = height, p.width = width, p.features = features, p.embedding = embedding, p.radius = radius, p.pair = pair;
  p.scale_x = scale_x, p.scale_y = scale_y;
  p.root_features = static_cast<float>(sqrt(static_cast<double>(features)));
  const long long pixels = static_cast<long long>(batch) * height * width;
  if (pixels >= 0x7fffffffLL) return kUnsupported;
  if (radius < 0) {
    const long long plain_blocks = (pixels + 31) / 32;
    refiner_input_plain_kernel<<<static_cast<unsigned>(plain_blocks < 148LL * 32 ? plain_blocks : 148LL * 32), 256, 0,
                                 static_cast<cudaStream_t>(stream)>>>(p);
    return static_cast<int>(cudaGetLastError());
  }
  const long long blocks = (pixels + kInputWarps - 1) / kInputWarps;
  const unsigned grid = static_cast<unsigned>(blocks < 148LL * 16 ? blocks : 148LL * 16);
  refiner_input_kernel<<<grid, 32 * kInputWarps, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}
