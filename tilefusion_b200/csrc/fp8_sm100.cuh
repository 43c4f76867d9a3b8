// 8-bit floating-point storage: conversion kernels between fp16/bf16 and the
// OCP e4m3 / e5m2 formats.  TileFusion declares the two types and converts
// single values through the CUDA constructors (include/types/base.hpp:13-39,
// from_float / to_float at :70-107; checked by tests/cpp/types/test_fp8.cu);
// these kernels are the bulk form a K/V cache writer needs: round to nearest
// even, saturating to the largest finite value, an optional per-tensor factor
// applied in fp32 before the rounding.
//
// Both kernels are bound by HBM bandwidth (3 bytes per element): 16 elements
// per thread and step, 16-byte vector accesses on the 8-bit side and 2 x 16 on
// the 16-bit side, a grid-stride loop over a grid sized to the SM count.
#pragma once

#include <cuda_fp8.h>

#include <type_traits>

#include "sm100_ptx.cuh"

namespace tfb {

constexpr int kFp8ConvertThreads = 256;
constexpr int kFp8ElemsPerThread = 16;

template <bool kE4M3>
__device__ __forceinline__ uint32_t fp8x2_from(float a, float b) {
  return (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, kE4M3 ? __NV_E4M3 : __NV_E5M2);
}

template <bool kE4M3>
__device__ __forceinline__ float2 fp8x2_to(uint32_t two) {
  const __half2 h(__nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)two, kE4M3 ? __NV_E4M3 : __NV_E5M2));
  return __half22float2(h);
}

// dst[i] = fp8(src[i] * factor); src is T (fp16 / bf16), n elements.
template <typename T, bool kE4M3>
__global__ void __launch_bounds__(kFp8ConvertThreads) fp8_quantize_kernel(const T* __restrict__ src,
                                                                          uint8_t* __restrict__ dst, long long n,
                                                                          float factor) {
  const long long n_vec = n / kFp8ElemsPerThread;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    const uint4 a = __ldcs(reinterpret_cast<const uint4*>(src) + 2 * i);
    const uint4 b = __ldcs(reinterpret_cast<const uint4*>(src) + 2 * i + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t out[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 lo = unpack2<T>(w[2 * e]), hi = unpack2<T>(w[2 * e + 1]);
      out[e] = fp8x2_from<kE4M3>(lo.x * factor, lo.y * factor) |
               (fp8x2_from<kE4M3>(hi.x * factor, hi.y * factor) << 16);
    }
    __stcs(reinterpret_cast<uint4*>(dst) + i, make_uint4(out[0], out[1], out[2], out[3]));
  }
  // ragged tail: fewer than 16 elements, one thread each
  const long long tail = n_vec * kFp8ElemsPerThread + (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (tail < n) {
    const uint16_t raw = reinterpret_cast<const uint16_t*>(src)[tail];
    const float x = unpack2<T>((uint32_t)raw).x * factor;
    dst[tail] = (uint8_t)(fp8x2_from<kE4M3>(x, 0.f) & 0xffu);
  }
}

// dst[i] = T(float(src[i]) * factor); dst is fp16 / bf16.
template <typename T, bool kE4M3>
__global__ void __launch_bounds__(kFp8ConvertThreads) fp8_dequantize_kernel(const uint8_t* __restrict__ src,
                                                                            T* __restrict__ dst, long long n,
                                                                            float factor) {
  const long long n_vec = n / kFp8ElemsPerThread;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
    const uint4 a = __ldcs(reinterpret_cast<const uint4*>(src) + i);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
    uint32_t out[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 lo = fp8x2_to<kE4M3>(w[e] & 0xffffu), hi = fp8x2_to<kE4M3>(w[e] >> 16);
      out[2 * e] = pack2<T>(lo.x * factor, lo.y * factor);
      out[2 * e + 1] = pack2<T>(hi.x * factor, hi.y * factor);
    }
    __stcs(reinterpret_cast<uint4*>(dst) + 2 * i, make_uint4(out[0], out[1], out[2], out[3]));
    __stcs(reinterpret_cast<uint4*>(dst) + 2 * i + 1, make_uint4(out[4], out[5], out[6], out[7]));
  }
  const long long tail = n_vec * kFp8ElemsPerThread + (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (tail < n) {
    const float x = fp8x2_to<kE4M3>((uint32_t)src[tail]).x * factor;
    reinterpret_cast<uint16_t*>(dst)[tail] = (uint16_t)(pack2<T>(x, 0.f) & 0xffffu);
  }
}

}  // namespace tfb
