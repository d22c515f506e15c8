// Standalone activation quantisers (memory-bound, one pass): static and dynamic block-32 MXFP8, static INT8.
// Byte-exact with the FlashIM torch reference (flashim/quant/tensor.py:97-121,148-151; flashim/quant/formats/mx.py:50-60).
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
      uint32_t w = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) w |= (static_cast<uint32_t>(int8_code(quantizer, v[4 * j + k])) & 0xFFu) << (8 * k);
      q[j] = w;
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
