// bf16 "plane" storage of fp32 values: x = x0 + x1 + x2 with x0 = rn(x), x1 = rn(x - x0),
// x2 = rn(x - x0 - x1).  One plane keeps bf16 precision; three planes keep ~24 bits and are
// what the tensor-core contraction consumes when fp32 accuracy is asked for.
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

struct ZpPlanes {
  __nv_bfloat16 *base;     // plane 0
  int64_t plane_stride;    // elements between planes
  int64_t ld;              // row stride in elements (multiple of 8)
  int planes;              // 1 or 3
};

// writes VEC (2 or 4) consecutive values at element offset `idx` of every plane
template <int VEC>
__device__ __forceinline__ void zp_store_planes(const ZpPlanes &p, int64_t idx, const float (&v)[VEC]) {
  float x[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) x[i] = v[i];
  for (int pl = 0; pl < p.planes; ++pl) {
    __nv_bfloat16 h[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      h[i] = __float2bfloat16_rn(x[i]);
      x[i] -= __bfloat162float(h[i]);
    }
    __nv_bfloat16 *dst = p.base + (size_t)pl * p.plane_stride + idx;
    if (VEC == 4) {
      uint2 u;
      u.x = (uint32_t)__bfloat16_as_ushort(h[0]) | ((uint32_t)__bfloat16_as_ushort(h[1]) << 16);
      u.y = (uint32_t)__bfloat16_as_ushort(h[2]) | ((uint32_t)__bfloat16_as_ushort(h[VEC - 1]) << 16);
      *reinterpret_cast<uint2 *>(dst) = u;
    } else {
      uint32_t u = (uint32_t)__bfloat16_as_ushort(h[0]) | ((uint32_t)__bfloat16_as_ushort(h[VEC - 1]) << 16);
      *reinterpret_cast<uint32_t *>(dst) = u;
    }
  }
}

__device__ __forceinline__ float zp_load_planes(const ZpPlanes &p, int64_t idx) {
  float s = 0.f;
  for (int pl = p.planes - 1; pl >= 0; --pl)
    s += __bfloat162float(p.base[(size_t)pl * p.plane_stride + idx]);
  return s;
}
