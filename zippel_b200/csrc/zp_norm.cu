// LayerNorm followed by SiLU, forward and backward, for the hidden layers of the radial MLP
// (reference blocks/eso2_ref.py:170-180: Linear, LayerNorm, SiLU, Linear, LayerNorm, SiLU, Linear).
//
//   forward   z = (x - mean) * rstd;  u = z * gamma + beta;  y = u * sigmoid(u)
//   backward  du = dy * s * (1 + u * (1 - s)),  s = sigmoid(u)
//             dgamma = sum_rows du * z,  dbeta = sum_rows du
//             dz = du * gamma;  dx = rstd * (dz - mean(dz) - z * mean(dz * z))
//
// One warp owns a row (width <= 1024, a multiple of 4; lane i holds columns 4i..4i+3 of every
// 128-column group).  Rows are streamed once; mean and rstd are saved by the forward.  The
// parameter gradients are reduced in a fixed order: every lane sums its columns over the rows of
// its warp, the warps of a block are added in warp order through shared memory, each block writes
// one partial row, and a second kernel adds the partial rows in block order.
#include <algorithm>

#include "zp_common.cuh"
#include "zippel_b200.h"

namespace {

constexpr int kWarps = 8;
constexpr int kMaxGroups = 8;              // 128-column groups per row: width <= 1024
constexpr int kPartialBlocks = 296;        // blocks of the backward kernel = partial rows

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int G>
__global__ void __launch_bounds__(32 * kWarps)
ln_silu_fwd_kernel(int64_t rows, int width, const float *__restrict__ x,
                   const float *__restrict__ gamma, const float *__restrict__ beta, float eps,
                   float *__restrict__ y, float *__restrict__ mean_out,
                   float *__restrict__ rstd_out) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  float4 g[G], b[G];
#pragma unroll
  for (int i = 0; i < G; ++i) {
    const int c = 128 * i + 4 * lane;
    g[i] = c < width ? *reinterpret_cast<const float4 *>(gamma + c) : make_float4(0, 0, 0, 0);
    b[i] = c < width ? *reinterpret_cast<const float4 *>(beta + c) : make_float4(0, 0, 0, 0);
  }
  const float inv_w = 1.f / (float)width;
  for (int64_t r = (int64_t)blockIdx.x * kWarps + warp; r < rows; r += (int64_t)gridDim.x * kWarps) {
    const float *xr = x + (size_t)r * width;
    float4 v[G];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const int c = 128 * i + 4 * lane;
      v[i] = c < width ? *reinterpret_cast<const float4 *>(xr + c) : make_float4(0, 0, 0, 0);
      s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = warp_sum(s) * inv_w;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const int c = 128 * i + 4 * lane;
      if (c < width) {
        const float a0 = v[i].x - mean, a1 = v[i].y - mean, a2 = v[i].z - mean, a3 = v[i].w - mean;
        q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
      }
    }
    const float rstd = rsqrtf(warp_sum(q) * inv_w + eps);
    float *yr = y + (size_t)r * width;
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const int c = 128 * i + 4 * lane;
      if (c < width) {
        float4 o;
        float u;
        u = (v[i].x - mean) * rstd * g[i].x + b[i].x; o.x = u / (1.f + expf(-u));
        u = (v[i].y - mean) * rstd * g[i].y + b[i].y; o.y = u / (1.f + expf(-u));
        u = (v[i].z - mean) * rstd * g[i].z + b[i].z; o.z = u / (1.f + expf(-u));
        u = (v[i].w - mean) * rstd * g[i].w + b[i].w; o.w = u / (1.f + expf(-u));
        *reinterpret_cast<float4 *>(yr + c) = o;
      }
    }
    if (lane == 0) { mean_out[r] = mean; rstd_out[r] = rstd; }
  }
}

__device__ __forceinline__ void bwd_elem(float xv, float mean, float rstd, float g, float b,
                                         float dyv, float &z, float &du) {
  z = (xv - mean) * rstd;
  const float u = z * g + b;
  const float s = 1.f / (1.f + expf(-u));
  du = dyv * s * (1.f + u * (1.f - s));
}

template <int G>
__global__ void __launch_bounds__(32 * kWarps)
ln_silu_bwd_kernel(int64_t rows, int width, const float *__restrict__ x,
                   const float *__restrict__ gamma, const float *__restrict__ beta,
                   const float *__restrict__ mean_in, const float *__restrict__ rstd_in,
                   const float *__restrict__ dy, float *__restrict__ dx,
                   float *__restrict__ partial) {           // [gridDim.x][2][width]
  extern __shared__ float red[];                              // [kWarps][2][width]
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  float4 g[G], b[G], dg[G], db[G];
#pragma unroll
  for (int i = 0; i < G; ++i) {
    const int c = 128 * i + 4 * lane;
    g[i] = c < width ? *reinterpret_cast<const float4 *>(gamma + c) : make_float4(0, 0, 0, 0);
    b[i] = c < width ? *reinterpret_cast<const float4 *>(beta + c) : make_float4(0, 0, 0, 0);
    dg[i] = make_float4(0, 0, 0, 0);
    db[i] = make_float4(0, 0, 0, 0);
  }
  const float inv_w = 1.f / (float)width;
  for (int64_t r = (int64_t)blockIdx.x * kWarps + warp; r < rows; r += (int64_t)gridDim.x * kWarps) {
    const float *xr = x + (size_t)r * width, *dyr = dy + (size_t)r * width;
    const float mean = mean_in[r], rstd = rstd_in[r];
    float4 z[G], dz[G];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const int c = 128 * i + 4 * lane;
      z[i] = make_float4(0, 0, 0, 0);
      dz[i] = make_float4(0, 0, 0, 0);
      if (c < width) {
        const float4 xv = *reinterpret_cast<const float4 *>(xr + c);
        const float4 dv = *reinterpret_cast<const float4 *>(dyr + c);
        float du;
        bwd_elem(xv.x, mean, rstd, g[i].x, b[i].x, dv.x, z[i].x, du);
        dg[i].x += du * z[i].x; db[i].x += du; dz[i].x = du * g[i].x;
        bwd_elem(xv.y, mean, rstd, g[i].y, b[i].y, dv.y, z[i].y, du);
        dg[i].y += du * z[i].y; db[i].y += du; dz[i].y = du * g[i].y;
        bwd_elem(xv.z, mean, rstd, g[i].z, b[i].z, dv.z, z[i].z, du);
        dg[i].z += du * z[i].z; db[i].z += du; dz[i].z = du * g[i].z;
        bwd_elem(xv.w, mean, rstd, g[i].w, b[i].w, dv.w, z[i].w, du);
        dg[i].w += du * z[i].w; db[i].w += du; dz[i].w = du * g[i].w;
        s1 += (dz[i].x + dz[i].y) + (dz[i].z + dz[i].w);
        s2 += (dz[i].x * z[i].x + dz[i].y * z[i].y) + (dz[i].z * z[i].z + dz[i].w * z[i].w);
      }
    }
    const float m1 = warp_sum(s1) * inv_w, m2 = warp_sum(s2) * inv_w;
    float *dxr = dx + (size_t)r * width;
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const int c = 128 * i + 4 * lane;
      if (c < width) {
        float4 o;
        o.x = rstd * (dz[i].x - m1 - z[i].x * m2);
        o.y = rstd * (dz[i].y - m1 - z[i].y * m2);
        o.z = rstd * (dz[i].z - m1 - z[i].z * m2);
        o.w = rstd * (dz[i].w - m1 - z[i].w * m2);
        *reinterpret_cast<float4 *>(dxr + c) = o;
      }
    }
  }
  // block partial of (dgamma, dbeta): warps added in warp order
#pragma unroll
  for (int i = 0; i < G; ++i) {
    const int c = 128 * i + 4 * lane;
    if (c < width) {
      *reinterpret_cast<float4 *>(red + (size_t)(warp * 2 + 0) * width + c) = dg[i];
      *reinterpret_cast<float4 *>(red + (size_t)(warp * 2 + 1) * width + c) = db[i];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * width; i += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) s += red[(size_t)w * 2 * width + i];
    partial[(size_t)blockIdx.x * 2 * width + i] = s;
  }
}

__global__ void ln_param_grad_kernel(int blocks, int width, const float *__restrict__ partial,
                                     float *__restrict__ dgamma, float *__restrict__ dbeta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * width) return;
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += partial[(size_t)b * 2 * width + i];
  if (i < width) dgamma[i] = s;
  else dbeta[i - width] = s;
}

int check_shape(int64_t rows, int width) {
  if (rows < 0 || width < 4 || width > 128 * kMaxGroups || (width % 4)) return ZP_ERR_UNSUPPORTED;
  return ZP_OK;
}

#define ZP_DISPATCH_GROUPS(groups, CALL) \
  switch (groups) {                      \
    case 1: { CALL(1); break; }          \
    case 2: { CALL(2); break; }          \
    case 3: case 4: { CALL(4); break; }  \
    default: { CALL(8); break; }         \
  }

}  // namespace

extern "C" {

size_t zp_layernorm_work_bytes(int width) {
  return sizeof(float) * (size_t)kPartialBlocks * 2 * (size_t)(width > 0 ? width : 0);
}

int zp_layernorm_silu_forward(int64_t rows, int width, const float *x, const float *gamma,
                              const float *beta, float eps, float *y, float *mean, float *rstd,
                              void *stream) {
  int rc = check_shape(rows, width);
  if (rc) return rc;
  if (rows == 0) return ZP_OK;
  if (!x || !gamma || !beta || !y || !mean || !rstd) return ZP_ERR_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int groups = (width + 127) / 128;
  const unsigned grid = (unsigned)std::min<int64_t>(zp_ceil_div(rows, kWarps), 148 * 8);
#define CALL(G)                                                                              \
  ln_silu_fwd_kernel<G><<<grid, 32 * kWarps, 0, st>>>(rows, width, x, gamma, beta, eps, y, \
                                                      mean, rstd)
  ZP_DISPATCH_GROUPS(groups, CALL);
#undef CALL
  ZP_LAUNCH_CHECK("ln_silu_fwd_kernel");
  return ZP_OK;
}

int zp_layernorm_silu_backward(int64_t rows, int width, const float *x, const float *gamma,
                               const float *beta, const float *mean, const float *rstd,
                               const float *dy, float *dx, float *dgamma, float *dbeta,
                               void *work, size_t work_bytes, void *stream) {
  int rc = check_shape(rows, width);
  if (rc) return rc;
  if (!dgamma || !dbeta) return ZP_ERR_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (rows == 0) {
    ZP_CUDA(cudaMemsetAsync(dgamma, 0, sizeof(float) * width, st));
    ZP_CUDA(cudaMemsetAsync(dbeta, 0, sizeof(float) * width, st));
    return ZP_OK;
  }
  if (!x || !gamma || !beta || !mean || !rstd || !dy || !dx || !work) return ZP_ERR_INVALID_ARG;
  if (work_bytes < zp_layernorm_work_bytes(width)) return ZP_ERR_WORKSPACE;
  const int groups = (width + 127) / 128;
  const int blocks = (int)std::min<int64_t>(zp_ceil_div(rows, kWarps), kPartialBlocks);
  const size_t smem = sizeof(float) * kWarps * 2 * (size_t)width;     // <= 64 KB
  float *partial = static_cast<float *>(work);
#define CALL(G)                                                                                 \
  do {                                                                                          \
    static ZpSmemOptIn opt_in;                                                                  \
    if (int rc_ = zp_ensure_smem(ln_silu_bwd_kernel<G>, 65536, opt_in)) return rc_;             \
    ln_silu_bwd_kernel<G><<<blocks, 32 * kWarps, smem, st>>>(rows, width, x, gamma, beta, mean, \
                                                             rstd, dy, dx, partial);           \
  } while (0)
  ZP_DISPATCH_GROUPS(groups, CALL);
#undef CALL
  ZP_LAUNCH_CHECK("ln_silu_bwd_kernel");
  ln_param_grad_kernel<<<(unsigned)zp_ceil_div(2 * width, 128), 128, 0, st>>>(blocks, width, partial,
                                                                              dgamma, dbeta);
  ZP_LAUNCH_CHECK("ln_param_grad_kernel");
  return ZP_OK;
}

}  // extern "C"
