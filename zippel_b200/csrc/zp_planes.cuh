// 16-bit "plane" storage of fp32 values for the tensor-core contraction.
//
//   bf16 planes   x = x0 + x1 + x2, xi bf16 (x0 = rn(x), x1 = rn(x - x0), ...).  One plane keeps
//                 bf16 precision, three keep ~24 bits; bf16 has fp32's exponent range, so no scale.
//   fp16 planes   x = s * (h0 + h1), hi fp16, s a power of two shared by the whole tensor.  Two
//                 planes keep 22 bits for every element within 2^19 of the tensor's largest
//                 magnitude (smaller ones keep an absolute error below 2^-25 s, invisible in any
//                 norm).  s is chosen from an upper bound on the tensor's magnitude so that the
//                 bound maps to 2^15 (fp16 overflows at 65504); it lives in device memory because
//                 it is computed on the device, between kernels, without a host round trip.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

struct ZpPlanes {
  void *base;              // plane 0 (16-bit elements)
  int64_t plane_stride;    // elements between planes
  int64_t ld;              // row stride in elements (multiple of 8)
  int planes;              // 1..3
  int fp16;                // 0: bf16 planes, 1: fp16 planes with a scale
  const float *scale;      // device pointer to s (fp16 planes only; null means 1)
};

__device__ __forceinline__ float zp_inv_scale(const ZpPlanes &p) {
  return (p.fp16 && p.scale) ? 1.f / *p.scale : 1.f;        // s is a power of two: exact
}
__device__ __forceinline__ float zp_scale(const ZpPlanes &p) {
  return (p.fp16 && p.scale) ? *p.scale : 1.f;
}

// s such that `bound` maps to 2^15; 1 for a zero / non-finite bound
__device__ __forceinline__ float zp_scale_for_bound(float bound) {
  if (!(bound > 0.f) || !(bound < 3.0e38f)) return 1.f;
  int e;
  frexpf(bound, &e);                 // bound = f * 2^e, f in [0.5, 1)  ->  bound <= 2^e
  return ldexpf(1.f, e - 15);
}

// writes VEC (2 or 4) consecutive values at element offset `idx` of every plane;
// `inv` = zp_inv_scale(p), read once per thread.  The format is chosen by ONE warp-uniform branch
// around the whole conversion (a per-element choice makes the compiler issue both conversions).
template <int VEC, bool FP16>
__device__ __forceinline__ void zp_store_planes_fmt(const ZpPlanes &p, int64_t idx, float (&x)[VEC]) {
  static_assert(VEC == 2 || VEC == 4, "pairs of values");
#pragma unroll
  for (int pl = 0; pl < 3; ++pl) {
    if (pl >= p.planes) break;
    // two values per conversion instruction (the one-value conversions run on the quarter-rate
    // special-function pipe and were a large share of the producer kernels' time there)
    uint32_t w[VEC / 2];
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) {
      if (FP16) {
        const __half2 q = __floats2half2_rn(x[2 * i], x[2 * i + 1]);       // low half = first value
        const float2 f = __half22float2(q);
        x[2 * i] -= f.x;
        x[2 * i + 1] -= f.y;
        w[i] = *reinterpret_cast<const uint32_t *>(&q);
      } else {
        const __nv_bfloat162 q = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
        const float2 f = __bfloat1622float2(q);
        x[2 * i] -= f.x;
        x[2 * i + 1] -= f.y;
        w[i] = *reinterpret_cast<const uint32_t *>(&q);
      }
    }
    uint16_t *dst = static_cast<uint16_t *>(p.base) + (size_t)pl * p.plane_stride + idx;
    if (VEC == 4) {
      uint2 u;
      u.x = w[0];
      u.y = w[VEC / 2 - 1];
      *reinterpret_cast<uint2 *>(dst) = u;
    } else {
      *reinterpret_cast<uint32_t *>(dst) = w[0];
    }
  }
}

template <int VEC>
__device__ __forceinline__ void zp_store_planes(const ZpPlanes &p, int64_t idx, const float (&v)[VEC],
                                                float inv = 1.f) {
  float x[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) x[i] = v[i] * inv;
  if (p.fp16) zp_store_planes_fmt<VEC, true>(p, idx, x);
  else zp_store_planes_fmt<VEC, false>(p, idx, x);
}

__device__ __forceinline__ float zp_plane_value(const ZpPlanes &p, uint16_t bits) {
  return p.fp16 ? __half2float(__ushort_as_half(bits)) : __uint_as_float((uint32_t)bits << 16);
}

// atomic max of a non-negative float (bit patterns of non-negative floats order like integers)
__device__ __forceinline__ void zp_atomic_absmax(float *addr, float v) {
  atomicMax(reinterpret_cast<unsigned int *>(addr), __float_as_uint(fabsf(v)));
}
