// Standalone activation quantisers (memory-bound, one pass): static and dynamic block-32 MXFP8, static INT8.
// Byte-exact with the FlashIM torch reference (flashim/quant/tensor.py:97-121,148-151; flashim/quant/formats/mx.py:50-60).
#include <type_traits>

#include "common.cuh"
#include "flashim_sm100.h"

namespace fim {
namespace {

constexpr int kThreads = 256;

template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&v)[16]);

template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[16]) {
  const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  const uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = bf16_lo(w[i]);
    v[2 * i + 1] = bf16_hi(w[i]);
  }
}
template <>
__device__ __forceinline__ void load16<float>(const float* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 f = __ldg(reinterpret_cast<const float4*>(p) + i);
    v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
  }
}
// Ragged tail of a row whose channel count is not a multiple of 16: element loads, zero padding.
template <typename T>
__device__ __forceinline__ void load_tail(const T* p, int valid, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = i < valid ? static_cast<float>(p[i]) : 0.0f;
}

// x / 2**e (exact power-of-two scaling), saturate, E4M3; 16 codes per thread.
template <typename T>
__global__ void __launch_bounds__(kThreads) quantize_mx_static_kernel(const T* __restrict__ in, const int8_t* __restrict__ exps,
                                                                      uint8_t* __restrict__ out, long long rows, int channels,
                                                                      int padded, bool aligned) {
  const int chunks = padded / 16;
  const long long total = rows * chunks;
  for (long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kThreads) {
    const long long row = i / chunks;
    const int c0 = static_cast<int>(i - row * chunks) * 16;
    float v[16];
    const T* src = in + row * channels + c0;
    if (c0 + 16 <= channels && aligned) {
      load16<T>(src, v);
    } else {
      load_tail<T>(src, max(0, min(16, channels - c0)), v);
    }
    const float inv = exp2_int(-static_cast<int>(exps[c0 >> 5]));
    uint32_t q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = e4m3x4(v[4 * j] * inv, v[4 * j + 1] * inv, v[4 * j + 2] * inv, v[4 * j + 3] * inv);
    *reinterpret_cast<uint4*>(out + row * padded + c0) = make_uint4(q[0], q[1], q[2], q[3]);
  }
}

// One 32-channel block per pair of lanes: amax -> exponent -> x * 2**-e -> E4M3; E8M0 byte stored swizzled or plain.
template <typename T>
__global__ void __launch_bounds__(kThreads) quantize_mx_dynamic_kernel(const T* __restrict__ in, uint8_t* __restrict__ out,
                                                                       uint8_t* __restrict__ scales, long long rows, int channels,
                                                                       int swizzled) {
  const int chunks = channels / 16;
  const int groups = channels / 32;
  const int group_tiles = (groups + 3) / 4;
  const long long total = rows * chunks;  // even: channels % 32 == 0, so a lane pair never splits across the bound
  const int lane = threadIdx.x & 31;
  // The loop condition is warp-uniform so that every lane reaches the shuffle; lanes past the end carry zeros.
  for (long long i0 = blockIdx.x * static_cast<long long>(kThreads) + (threadIdx.x - lane); i0 < total;
       i0 += static_cast<long long>(gridDim.x) * kThreads) {
    const long long i = i0 + lane;
    const bool valid = i < total;
    const long long row = valid ? i / chunks : 0;
    const int chunk = valid ? static_cast<int>(i - row * chunks) : 0;
    float v[16];
    if (valid) {
      load16<T>(in + row * channels + chunk * 16, v);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = 0.0f;
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const int e = e8m0_exponent(amax);
    const float inv = exp2_int(-e);
    uint32_t q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) q[j] = e4m3x4(v[4 * j] * inv, v[4 * j + 1] * inv, v[4 * j + 2] * inv, v[4 * j + 3] * inv);
    if (!valid) continue;
    *reinterpret_cast<uint4*>(out + row * channels + chunk * 16) = make_uint4(q[0], q[1], q[2], q[3]);
    if ((chunk & 1) == 0) {
      const int g = chunk >> 1;
      const size_t at = swizzled ? swizzled_scale_offset(static_cast<size_t>(row), g, group_tiles)
                                 : static_cast<size_t>(row) * groups + g;
      scales[at] = static_cast<uint8_t>(e + 127);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) quantize_int8_kernel(const T* __restrict__ in, const float* __restrict__ scale_ptr,
                                                                 int8_t* __restrict__ out, long long count) {
  const Int8Quantizer quantizer = make_int8_quantizer(__ldg(scale_ptr));
  const long long chunks = count / 16;
  for (long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x; i < chunks;
       i += static_cast<long long>(gridDim.x) * kThreads) {
    float v[16];
    load16<T>(in + i * 16, v);
    uint32_t q[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      q[j] = int8_pack4(quantizer, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
    *reinterpret_cast<uint4*>(out + i * 16) = make_uint4(q[0], q[1], q[2], q[3]);
  }
  // tail shorter than one chunk
  const long long done = chunks * 16;
  if (blockIdx.x == 0 && threadIdx.x < count - done) {
    out[done + threadIdx.x] = static_cast<int8_t>(int8_code(quantizer, static_cast<float>(in[done + threadIdx.x])));
  }
}

int grid_for(long long work_items, int multiple) {
  const long long blocks = (work_items + kThreads - 1) / kThreads;
  const long long cap = 148LL * multiple;
  return static_cast<int>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Static quantisers that read the channels-last *view* of an NCHW-contiguous tensor ([B, C, P] in memory, P = H * W) and
// write packed NHWC codes ([B, P, Cp]): the layout change rides on the quantiser instead of costing a copy pass
// (flashim/backends/triton/quantize.py:217-234 does the same with a two-dimensional tile). A block owns 128 pixels x 64
// channels: warps read along pixels (contiguous in the source), the code bytes cross through shared memory, and the tile
// leaves as 16-byte pieces along channels (contiguous in the output). Per-element arithmetic is that of the row-major
// kernels above, so the bytes are identical.
constexpr int kTilePixels = 128, kTileChannels = 64, kTilePitch = kTileChannels + 4;

// four consecutive pixels of one channel row (`valid` of them exist); VEC: one aligned 8- or 16-byte load
template <typename T, bool VEC>
__device__ __forceinline__ void load_pixels4(const T* p, int valid, float (&v)[4]);
template <>
__device__ __forceinline__ void load_pixels4<__nv_bfloat16, true>(const __nv_bfloat16* p, int valid, float (&v)[4]) {
  const uint2 w = valid > 0 ? __ldg(reinterpret_cast<const uint2*>(p)) : make_uint2(0u, 0u);
  v[0] = bf16_lo(w.x), v[1] = bf16_hi(w.x), v[2] = bf16_lo(w.y), v[3] = bf16_hi(w.y);
}
template <>
__device__ __forceinline__ void load_pixels4<float, true>(const float* p, int valid, float (&v)[4]) {
  const float4 w = valid > 0 ? __ldg(reinterpret_cast<const float4*>(p)) : make_float4(0.f, 0.f, 0.f, 0.f);
  v[0] = w.x, v[1] = w.y, v[2] = w.z, v[3] = w.w;
}
template <>
__device__ __forceinline__ void load_pixels4<__nv_bfloat16, false>(const __nv_bfloat16* p, int valid, float (&v)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = j < valid ? __bfloat162float(p[j]) : 0.0f;
}
template <>
__device__ __forceinline__ void load_pixels4<float, false>(const float* p, int valid, float (&v)[4]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = j < valid ? p[j] : 0.0f;
}

// A thread quantises 4 channels x 4 pixels per step (lane = pixel quad, so a warp reads 128 consecutive pixels of a
// channel row), turns the four code words (one per channel, a byte per pixel) into four words of 4 channels per pixel
// with byte permutes, and stores those to the shared tile.
template <typename T, bool INT8, bool VEC>
__global__ void __launch_bounds__(kThreads) quantize_nchw_kernel(const T* __restrict__ in, const int8_t* __restrict__ exps,
                                                                 const float* __restrict__ scale_ptr, uint8_t* __restrict__ out,
                                                                 int channels, int padded, long long pixels, int pixel_tiles,
                                                                 int channel_tiles) {
  __shared__ __align__(16) uint8_t tile[kTilePixels * kTilePitch];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long t = blockIdx.x;
  const int ct = static_cast<int>(t % channel_tiles);
  t /= channel_tiles;
  const long long pt = t % pixel_tiles;
  const long long b = t / pixel_tiles;
  const int c0 = ct * kTileChannels;
  const long long p0 = pt * kTilePixels + 4 * lane;
  const int valid = static_cast<int>(pixels - p0 < 4 ? (pixels - p0 < 0 ? 0 : pixels - p0) : 4);
  const Int8Quantizer quantizer = make_int8_quantizer(INT8 ? __ldg(scale_ptr) : 1.0f);

  float v[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int c = c0 + 4 * (warp + 8 * i) + k;
      load_pixels4<T, VEC>(in + (b * channels + (c < channels ? c : 0)) * pixels + p0, c < channels ? valid : 0, v[i][k]);
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int cq = warp + 8 * i;
    if (c0 + 4 * cq >= padded) break;  // warp-uniform; channels in [channels, padded) were loaded as zeros
    uint32_t r[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (INT8) {
        r[k] = int8_pack4(quantizer, v[i][k][0], v[i][k][1], v[i][k][2], v[i][k][3]);
      } else {
        const int c = min(c0 + 4 * cq + k, padded - 1);
        const float inv = exp2_int(-static_cast<int>(exps[c >> 5]));
        r[k] = e4m3x4(v[i][k][0] * inv, v[i][k][1] * inv, v[i][k][2] * inv, v[i][k][3] * inv);
      }
    }
    const uint32_t t0 = __byte_perm(r[0], r[1], 0x5140), t1 = __byte_perm(r[2], r[3], 0x5140);
    const uint32_t t2 = __byte_perm(r[0], r[1], 0x7362), t3 = __byte_perm(r[2], r[3], 0x7362);
    uint32_t* dst = reinterpret_cast<uint32_t*>(tile + (4 * lane) * kTilePitch + 4 * cq);
    dst[0] = __byte_perm(t0, t1, 0x5410);
    dst[kTilePitch / 4] = __byte_perm(t0, t1, 0x7632);
    dst[2 * (kTilePitch / 4)] = __byte_perm(t2, t3, 0x5410);
    dst[3 * (kTilePitch / 4)] = __byte_perm(t2, t3, 0x7632);
  }
  __syncthreads();
  const int part = threadIdx.x & 3;  // 16 channels
  if (c0 + part * 16 >= padded) return;
  const long long tile_p0 = pt * kTilePixels;
#pragma unroll
  for (int j = 0; j < kTilePixels / (kThreads / 4); ++j) {
    const int p = (threadIdx.x >> 2) + j * (kThreads / 4);
    if (tile_p0 + p >= pixels) break;
    const uint32_t* row = reinterpret_cast<const uint32_t*>(tile + p * kTilePitch + part * 16);
    *reinterpret_cast<uint4*>(out + (b * pixels + tile_p0 + p) * padded + c0 + part * 16) = make_uint4(row[0], row[1], row[2], row[3]);
  }
}

// 2x2 / stride-2 max pool of a bf16 NHWC tensor followed by the static INT8 quantiser: the second output of
// int8_conv2d_maxpool (flashim/ops/conv.py:209-222). A thread owns eight channels of one pooled pixel: four 16-byte loads,
// three packed bf16 maxima per word, eight codes, one 8-byte store. A trailing odd row or column is dropped, as
// F.max_pool2d does.
__global__ void __launch_bounds__(kThreads) maxpool2_int8_kernel(const uint4* __restrict__ in, const float* __restrict__ scale_ptr,
                                                                 uint2* __restrict__ out, int batch, int height, int width,
                                                                 int channels) {
  const Int8Quantizer quantizer = make_int8_quantizer(__ldg(scale_ptr));
  const int ho = height / 2, wo = width / 2, groups = channels / 8;
  const long long total = static_cast<long long>(batch) * ho * wo * groups;
  const long long row = static_cast<long long>(width) * groups;  // in 16-byte units
  for (long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kThreads) {
    long long t = i;
    const int g = static_cast<int>(t % groups); t /= groups;
    const int x = static_cast<int>(t % wo); t /= wo;
    const int y = static_cast<int>(t % ho);
    const long long b = t / ho;
    const uint4* src = in + ((b * height + 2 * y) * width + 2 * x) * groups + g;
    const uint4 a = __ldg(src), c = __ldg(src + groups), d = __ldg(src + row), e = __ldg(src + row + groups);
    const uint32_t m[4] = {bf16x2_max(bf16x2_max(a.x, c.x), bf16x2_max(d.x, e.x)), bf16x2_max(bf16x2_max(a.y, c.y), bf16x2_max(d.y, e.y)),
                           bf16x2_max(bf16x2_max(a.z, c.z), bf16x2_max(d.z, e.z)), bf16x2_max(bf16x2_max(a.w, c.w), bf16x2_max(d.w, e.w))};
    const uint32_t q[2] = {int8_pack4(quantizer, bf16_lo(m[0]), bf16_hi(m[0]), bf16_lo(m[1]), bf16_hi(m[1])),
                           int8_pack4(quantizer, bf16_lo(m[2]), bf16_hi(m[2]), bf16_lo(m[3]), bf16_hi(m[3]))};
    out[i] = make_uint2(q[0], q[1]);
  }
}

template <bool INT8>
int launch_nchw(const void* value, int dtype, const int8_t* exponent, const float* scale, void* out, int batch, int channels,
                long long pixels, int padded, void* stream) {
  if (batch < 0 || channels <= 0 || pixels < 0) return kBadArgument;
  if (batch == 0 || pixels == 0) return kOk;
  if (value == nullptr || out == nullptr || (INT8 ? scale == nullptr : exponent == nullptr)) return kBadArgument;
  if (!aligned16(out) || padded % 16) return kBadLayout;
  const long long pixel_tiles = (pixels + kTilePixels - 1) / kTilePixels;
  const int channel_tiles = (padded + kTileChannels - 1) / kTileChannels;
  const long long blocks = pixel_tiles * channel_tiles * batch;
  if (blocks > 0x7fffffffLL) return kUnsupported;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(blocks);
  auto launch = [&](auto zero, auto vec) {
    using T = decltype(zero);
    // one aligned load per four pixels needs every channel row to start on such a boundary
    quantize_nchw_kernel<T, INT8, decltype(vec)::value><<<grid, kThreads, 0, s>>>(
        static_cast<const T*>(value), exponent, scale, static_cast<uint8_t*>(out), channels, padded, pixels,
        static_cast<int>(pixel_tiles), channel_tiles);
  };
  const size_t elem = dtype == FIM_DTYPE_BF16 ? 2 : 4;
  const bool vec = pixels % 4 == 0 && (reinterpret_cast<uintptr_t>(value) % (4 * elem)) == 0;
  if (dtype == FIM_DTYPE_BF16) {
    if (vec) launch(__nv_bfloat16{}, std::true_type{});
    else launch(__nv_bfloat16{}, std::false_type{});
  } else if (dtype == FIM_DTYPE_F32) {
    if (vec) launch(0.0f, std::true_type{});
    else launch(0.0f, std::false_type{});
  } else {
    return kBadArgument;
  }
  return static_cast<int>(cudaGetLastError());
}


// GELU (erf form, evaluated in fp32) of a bf16 matrix plus an optional per-column bias, rounded to bf16, then the static
// block-32 quantiser: out = e4m3(sat(bf16(gelu(float(v) + bias)) / 2**e)). 16 elements per thread; channels % 32 == 0.
__global__ void __launch_bounds__(kThreads) gelu_quantize_mx_kernel(const __nv_bfloat16* __restrict__ in, const float* __restrict__ bias,
                                                                    const int8_t* __restrict__ exps, uint8_t* __restrict__ out,
                                                                    long long rows, int channels) {
  const int chunks = channels / 16;
  const long long total = rows * chunks;
  for (long long i = blockIdx.x * static_cast<long long>(kThreads) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kThreads) {
    const long long row = i / chunks;
    const int c0 = static_cast<int>(i - row * chunks) * 16;
    float v[16];
    load16<__nv_bfloat16>(in + row * channels + c0, v);
    const float inv = exp2_int(-static_cast<int>(exps[c0 >> 5]));
    float q[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float x = bias != nullptr ? v[j] + __ldg(bias + c0 + j) : v[j];
      q[j] = bf16_round(gelu_erf(x)) * inv;
    }
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) w[j] = e4m3x4(q[4 * j], q[4 * j + 1], q[4 * j + 2], q[4 * j + 3]);
    *reinterpret_cast<uint4*>(out + row * channels + c0) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

}  // namespace
}  // namespace fim

using namespace fim;

extern "C" int fim_quantize_mxfp8_static(const void* value, int dtype, const int8_t* exponent, void* out, long long rows,
                                         int channels, void* stream) {
  if (rows == 0 && channels > 0) return kOk;
  if (value == nullptr || exponent == nullptr || out == nullptr || rows < 0 || channels <= 0) return kBadArgument;
  const int padded = (channels + 31) / 32 * 32;
  if (!aligned16(out)) return kBadLayout;
  const int elem = dtype == FIM_DTYPE_BF16 ? 2 : 4;
  const bool vec = aligned16(value) && (static_cast<long long>(channels) * elem) % 16 == 0;
  const int grid = grid_for(rows * (padded / 16), 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == FIM_DTYPE_BF16) {
    quantize_mx_static_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(value), exponent,
                                                                      static_cast<uint8_t*>(out), rows, channels, padded, vec);
  } else if (dtype == FIM_DTYPE_F32) {
    quantize_mx_static_kernel<float><<<grid, kThreads, 0, s>>>(static_cast<const float*>(value), exponent,
                                                              static_cast<uint8_t*>(out), rows, channels, padded, vec);
  } else {
    return kBadArgument;
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fim_quantize_mxfp8_dynamic(const void* value, int dtype, void* out, void* scales, int swizzled, long long rows,
                                          int channels, void* stream) {
  if (rows == 0 && channels > 0) return kOk;
  if (value == nullptr || out == nullptr || scales == nullptr || rows < 0 || channels <= 0) return kBadArgument;
  if (channels % 32) return kBadLayout;
  if (!aligned16(value) || !aligned16(out)) return kBadLayout;
  const int grid = grid_for(rows * (channels / 16), 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == FIM_DTYPE_BF16) {
    quantize_mx_dynamic_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(value),
                                                                       static_cast<uint8_t*>(out), static_cast<uint8_t*>(scales),
                                                                       rows, channels, swizzled);
  } else if (dtype == FIM_DTYPE_F32) {
    quantize_mx_dynamic_kernel<float><<<grid, kThreads, 0, s>>>(static_cast<const float*>(value), static_cast<uint8_t*>(out),
                                                               static_cast<uint8_t*>(scales), rows, channels, swizzled);
  } else {
    return kBadArgument;
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fim_quantize_int8_static(const void* value, int dtype, const float* scale, void* out, long long count,
                                        void* stream) {
  if (count == 0) return kOk;
  if (value == nullptr || scale == nullptr || out == nullptr || count < 0) return kBadArgument;
  if (!aligned16(value) || !aligned16(out)) return kBadLayout;
  const int grid = grid_for(count / 16 + 1, 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == FIM_DTYPE_BF16) {
    quantize_int8_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(value), scale,
                                                                 static_cast<int8_t*>(out), count);
  } else if (dtype == FIM_DTYPE_F32) {
    quantize_int8_kernel<float><<<grid, kThreads, 0, s>>>(static_cast<const float*>(value), scale, static_cast<int8_t*>(out),
                                                         count);
  } else {
    return kBadArgument;
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fim_quantize_mxfp8_static_nchw(const void* value, int dtype, const int8_t* exponent, void* out, int batch,
                                              int channels, long long pixels, void* stream) {
  return launch_nchw<false>(value, dtype, exponent, nullptr, out, batch, channels, pixels, (channels + 31) / 32 * 32, stream);
}

extern "C" int fim_quantize_int8_static_nchw(const void* value, int dtype, const float* scale, void* out, int batch, int channels,
                                             long long pixels, void* stream) {
  if (channels % 16) return kBadLayout;  // INT8 activations are not padded: the packed rows must stay 16-byte pieces
  return launch_nchw<true>(value, dtype, nullptr, scale, out, batch, channels, pixels, channels, stream);
}

extern "C" int fim_maxpool2_quantize_int8(const void* value, const float* scale, void* out, int batch, int height, int width,
                                          int channels, void* stream) {
  if (batch < 0 || height < 0 || width < 0 || channels <= 0) return kBadArgument;
  if (channels % 8) return kBadLayout;
  if (batch == 0 || height < 2 || width < 2) return kOk;
  if (value == nullptr || scale == nullptr || out == nullptr) return kBadArgument;
  if (!aligned16(value) || (reinterpret_cast<uintptr_t>(out) & 7u)) return kBadLayout;
  const long long work = static_cast<long long>(batch) * (height / 2) * (width / 2) * (channels / 8);
  maxpool2_int8_kernel<<<grid_for(work, 16), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(value), scale, static_cast<uint2*>(out), batch, height, width, channels);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int fim_gelu_quantize_mxfp8(const void* value, const float* input_bias, const int8_t* exponent, void* out, long long rows,
                                       int channels, void* stream) {
  if (rows == 0 && channels > 0) return kOk;
  if (value == nullptr || exponent == nullptr || out == nullptr || rows < 0 || channels <= 0) return kBadArgument;
  if (channels % 32) return kBadLayout;
  if (!aligned16(value) || !aligned16(out)) return kBadLayout;
  gelu_quantize_mx_kernel<<<grid_for(rows * (channels / 16), 16), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(value), input_bias, exponent, static_cast<uint8_t*>(out), rows, channels);
  return static_cast<int>(cudaGetLastError());
}
