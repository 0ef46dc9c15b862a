// Dense pieces of the SO(2) convolution on CUDA cores: a strided fp32 GEMM, the gate
// activation and its VJP, weight folding, and column sums for the bias gradients.
//
// Weight folding.  For m > 0 the reference applies one Linear to the real and the imaginary
// rows and recombines the halves of its output (blocks/eso2_ref.py:282-291):
//     out_re = Wa x_re - Wb x_im,   out_im = Wb x_re + Wa x_im,   W = [Wa ; Wb].
// With the m'-major row order (real rows, then imaginary rows) that is ONE product with
//     W_fold = [ Wa  -Wb ]
//              [ Wb   Wa ]            of shape [2 km Cout, 2 km Cin],
// the same number of multiply-adds as the reference's two-row form, and no recombination.
// Every m-block of conv1 and conv2 is therefore a plain  Y[E, out] = X[E, in] W_fold^T.
#include <cuda_bf16.h>

#include "zp_common.cuh"

namespace {

// fp32 -> up to three bf16 terms whose sum reproduces the value to ~2^-24
__global__ void split_planes_kernel(int64_t rows, int64_t cols, const float *__restrict__ in,
                                    int64_t ld_in, __nv_bfloat16 *__restrict__ out, int64_t ld_out,
                                    int64_t plane_stride, int planes) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * ld_out) return;
  const int64_t r = idx / ld_out, c = idx % ld_out;
  float x = c < cols ? in[r * ld_in + c] : 0.f;
  for (int p = 0; p < planes; ++p) {
    const __nv_bfloat16 h = __float2bfloat16_rn(x);
    out[(size_t)p * plane_stride + idx] = h;
    x -= __bfloat162float(h);
  }
}

// ------------------------------------------------------------------------------------------
// strided SIMT GEMM, 128x128x16 tiles, 8x8 outputs per thread
// ------------------------------------------------------------------------------------------
constexpr int BM = 128, BN = 128, BK = 16, TM = 8, TN = 8;

__global__ void __launch_bounds__(256)
gemm_kernel(int64_t M, int64_t N, int64_t K, const float *__restrict__ A, int64_t am, int64_t ak,
            const float *__restrict__ B, int64_t bk, int64_t bn, const float *__restrict__ bias,
            float *__restrict__ C, int64_t ldc, int splits, int64_t k_per_split) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  const int split = blockIdx.z;
  const int64_t k_beg = split * k_per_split;
  const int64_t k_end = min(K, k_beg + k_per_split);
  const int tx = tid % 16, ty = tid / 16;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // loader index order follows the contiguous axis of each operand
  const bool a_kfast = (ak == 1), b_kfast = (bk == 1);
  for (int64_t k0 = k_beg; k0 < k_end; k0 += BK) {
#pragma unroll
    for (int it = 0; it < (BM * BK) / 256; ++it) {
      const int idx = it * 256 + tid;
      const int mm = a_kfast ? idx / BK : idx % BM;
      const int kk = a_kfast ? idx % BK : idx / BM;
      const int64_t gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < k_end) ? A[gm * am + gk * ak] : 0.f;
    }
#pragma unroll
    for (int it = 0; it < (BN * BK) / 256; ++it) {
      const int idx = it * 256 + tid;
      const int nn = b_kfast ? idx / BK : idx % BN;
      const int kk = b_kfast ? idx % BK : idx / BN;
      const int64_t gn = n0 + nn, gk = k0 + kk;
      Bs[kk][nn] = (gn < N && gk < k_end) ? B[gk * bk + gn * bn] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  float *out = C;
  int64_t ld = ldc;
  if (splits > 1) {            // partial results land in scratch [splits][M][N]
    out = C + (size_t)split * M * N;
    ld = N;
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int64_t gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int64_t gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (splits == 1 && bias) v += bias[gn];
      out[gm * ld + gn] = v;
    }
  }
}

__global__ void split_reduce_kernel(int64_t M, int64_t N, int splits,
                                    const float *__restrict__ part,
                                    const float *__restrict__ bias, float *__restrict__ C,
                                    int64_t ldc) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= M * N) return;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += part[(size_t)k * M * N + i];
  const int64_t m = i / N, n = i % N;
  if (bias) s += bias[n];
  C[m * ldc + n] = s;
}

// ------------------------------------------------------------------------------------------
// gate activation (blocks/eso2_ref.py:295-301): conv1 output row h1[e] = [gate (lmax*H) | y (Km*H)]
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void gate_fwd_kernel(const __grid_constant__ ZpTables t, int64_t E,
                                const float *__restrict__ h1, float *__restrict__ ht) {
  const int H4 = t.H / 4;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = E * t.Km * H4;
  if (idx >= total) return;
  const int h = (int)(idx % H4) * 4;
  const int r = (int)((idx / H4) % t.Km);
  const int64_t e = idx / ((int64_t)H4 * t.Km);
  const float *row = h1 + (size_t)e * t.w1_cols;
  const float4 x = *reinterpret_cast<const float4 *>(row + t.n_gate + r * t.H + h);
  float4 o;
  if (r == 0) {
    o.x = x.x * sigmoidf(x.x); o.y = x.y * sigmoidf(x.y);
    o.z = x.z * sigmoidf(x.z); o.w = x.w * sigmoidf(x.w);
  } else {
    const float4 g = *reinterpret_cast<const float4 *>(row + (t.row_l[r] - 1) * t.H + h);
    o.x = x.x * sigmoidf(g.x); o.y = x.y * sigmoidf(g.y);
    o.z = x.z * sigmoidf(g.z); o.w = x.w * sigmoidf(g.w);
  }
  *reinterpret_cast<float4 *>(ht + ((size_t)e * t.Km + r) * t.H + h) = o;
}

// one thread per (edge, hidden-channel quad): walks the Km rows, accumulates the lmax gate grads
__global__ void gate_bwd_kernel(const __grid_constant__ ZpTables t, int64_t E,
                                const float *__restrict__ h1, const float *__restrict__ dht,
                                float *__restrict__ dh1) {
  const int H4 = t.H / 4;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= E * H4) return;
  const int h = (int)(idx % H4) * 4;
  const int64_t e = idx / H4;
  const float *row = h1 + (size_t)e * t.w1_cols;
  float *drow = dh1 + (size_t)e * t.w1_cols;
  const float *dt = dht + (size_t)e * t.Km * t.H;
  float sg[ZP_MAX_L][4], dg[ZP_MAX_L][4];
#pragma unroll
  for (int l = 0; l < ZP_MAX_L; ++l) {
    if (l < t.lmax) {
      const float4 g = *reinterpret_cast<const float4 *>(row + l * t.H + h);
      sg[l][0] = sigmoidf(g.x); sg[l][1] = sigmoidf(g.y);
      sg[l][2] = sigmoidf(g.z); sg[l][3] = sigmoidf(g.w);
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) dg[l][v] = 0.f;
  }
  for (int r = 0; r < t.Km; ++r) {
    const float4 x4 = *reinterpret_cast<const float4 *>(row + t.n_gate + r * t.H + h);
    const float4 d4 = *reinterpret_cast<const float4 *>(dt + r * t.H + h);
    const float x[4] = {x4.x, x4.y, x4.z, x4.w}, d[4] = {d4.x, d4.y, d4.z, d4.w};
    float o[4];
    if (r == 0) {
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const float s = sigmoidf(x[v]);
        o[v] = d[v] * (s + x[v] * s * (1.f - s));
      }
    } else {
      const int l = t.row_l[r] - 1;
#pragma unroll
      for (int ll = 0; ll < ZP_MAX_L; ++ll) {
        if (ll == l) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            o[v] = d[v] * sg[ll][v];
            dg[ll][v] = fmaf(d[v], x[v], dg[ll][v]);
          }
        }
      }
    }
    *reinterpret_cast<float4 *>(drow + t.n_gate + r * t.H + h) = make_float4(o[0], o[1], o[2], o[3]);
  }
#pragma unroll
  for (int l = 0; l < ZP_MAX_L; ++l) {
    if (l < t.lmax) {
      float o[4];
#pragma unroll
      for (int v = 0; v < 4; ++v) o[v] = dg[l][v] * sg[l][v] * (1.f - sg[l][v]);
      *reinterpret_cast<float4 *>(drow + l * t.H + h) = make_float4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ------------------------------------------------------------------------------------------
// weight folding and its transpose
// ------------------------------------------------------------------------------------------
// fold:   dst [2*half, 2*kin] from src [2*half, kin]  (Wa = rows [0, half), Wb = rows [half, 2 half))
__global__ void fold_kernel(int half, int kin, const float *__restrict__ w,
                            float *__restrict__ f) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)2 * half * 2 * kin;
  if (idx >= total) return;
  const int col = (int)(idx % (2 * kin)), row = (int)(idx / (2 * kin));
  const bool lower = row >= half, right = col >= kin;
  const int o = lower ? row - half : row, c = right ? col - kin : col;
  // [ Wa -Wb ; Wb Wa ]
  const bool use_b = lower != right;
  float v = w[(size_t)(use_b ? half + o : o) * kin + c];
  if (!lower && right) v = -v;
  f[idx] = v;
}

// unfold: dWa = F[0,0] + F[1,1],  dWb = F[1,0] - F[0,1]
__global__ void unfold_kernel(int half, int kin, const float *__restrict__ f,
                              float *__restrict__ gw) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)2 * half * kin;
  if (idx >= total) return;
  const int c = (int)(idx % kin), row = (int)(idx / kin);
  const int ld = 2 * kin;
  if (row < half) {
    gw[idx] = f[(size_t)row * ld + c] + f[(size_t)(half + row) * ld + kin + c];
  } else {
    const int o = row - half;
    gw[idx] = f[(size_t)(half + o) * ld + c] - f[(size_t)o * ld + kin + c];
  }
}

// column sums in two fixed-order stages
constexpr int kColRowsPerBlock = 256;
__global__ void colsum_part_kernel(int64_t rows, int64_t cols, const float *__restrict__ a,
                                   int64_t lda, float *__restrict__ part) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  const int64_t r0 = (int64_t)blockIdx.y * kColRowsPerBlock;
  const int64_t r1 = min(rows, r0 + kColRowsPerBlock);
  float s = 0.f;
  for (int64_t r = r0; r < r1; ++r) s += a[r * lda + c];
  part[(size_t)blockIdx.y * cols + c] = s;
}
__global__ void colsum_final_kernel(int64_t nparts, int64_t cols, const float *__restrict__ part,
                                    float *__restrict__ out) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int64_t p = 0; p < nparts; ++p) s += part[(size_t)p * cols + c];
  out[c] = s;
}

}  // namespace

int zp_launch_gemm(int64_t M, int64_t N, int64_t K, const float *A, int64_t am, int64_t ak,
                   const float *B, int64_t bk, int64_t bn, const float *bias, float *C,
                   int64_t ldc, int splits, float *scratch, cudaStream_t st) {
  if (M == 0 || N == 0) return ZP_OK;
  if ((am != 1 && ak != 1) || (bk != 1 && bn != 1)) return ZP_ERR_INVALID_ARG;
  if (splits < 1) splits = 1;
  if (splits > 1 && !scratch) return ZP_ERR_INVALID_ARG;
  int64_t kps = zp_ceil_div(zp_ceil_div(K, splits), BK) * BK;
  if (kps == 0) kps = BK;
  const dim3 grid((unsigned)zp_ceil_div(N, BN), (unsigned)zp_ceil_div(M, BM), splits);
  gemm_kernel<<<grid, 256, 0, st>>>(M, N, K, A, am, ak, B, bk, bn, bias,
                                    splits > 1 ? scratch : C, ldc, splits, kps);
  ZP_LAUNCH_CHECK("gemm_kernel");
  if (splits > 1) {
    split_reduce_kernel<<<(unsigned)zp_ceil_div(M * N, 256), 256, 0, st>>>(M, N, splits, scratch,
                                                                           bias, C, ldc);
    ZP_LAUNCH_CHECK("split_reduce_kernel");
  }
  return ZP_OK;
}

int zp_launch_split_planes(int64_t rows, int64_t cols, const float *in, int64_t ld_in, void *out,
                           int64_t ld_out, int64_t plane_stride, int planes, cudaStream_t st) {
  if (rows == 0 || ld_out == 0) return ZP_OK;
  split_planes_kernel<<<(unsigned)zp_ceil_div(rows * ld_out, 256), 256, 0, st>>>(
      rows, cols, in, ld_in, (__nv_bfloat16 *)out, ld_out, plane_stride, planes);
  ZP_LAUNCH_CHECK("split_planes_kernel");
  return ZP_OK;
}

int zp_launch_gate_fwd(const zp_plan *p, int64_t E, const float *h1, float *ht, cudaStream_t st) {
  if (E == 0) return ZP_OK;
  const int64_t total = E * p->t.Km * (p->t.H / 4);
  gate_fwd_kernel<<<(unsigned)zp_ceil_div(total, 256), 256, 0, st>>>(p->t, E, h1, ht);
  ZP_LAUNCH_CHECK("gate_fwd_kernel");
  return ZP_OK;
}

int zp_launch_gate_bwd(const zp_plan *p, int64_t E, const float *h1, const float *dht, float *dh1,
                       cudaStream_t st) {
  if (E == 0) return ZP_OK;
  const int64_t total = E * (p->t.H / 4);
  gate_bwd_kernel<<<(unsigned)zp_ceil_div(total, 128), 128, 0, st>>>(p->t, E, h1, dht, dh1);
  ZP_LAUNCH_CHECK("gate_bwd_kernel");
  return ZP_OK;
}

int zp_launch_fold_weights(const zp_plan *p, const zp_weights *w, float *packed, cudaStream_t st) {
  // m = 0 blocks are used as they are
  ZP_CUDA(cudaMemcpyAsync(packed + p->c1_woff[0], w->c1_w0,
                          sizeof(float) * (size_t)p->c1_out[0] * p->c1_in[0],
                          cudaMemcpyDeviceToDevice, st));
  ZP_CUDA(cudaMemcpyAsync(packed + p->c2_woff[0], w->c2_w0,
                          sizeof(float) * (size_t)p->c2_out[0] * p->c2_in[0],
                          cudaMemcpyDeviceToDevice, st));
  for (int m = 1; m < p->n_blocks; ++m) {
    for (int conv = 0; conv < 2; ++conv) {
      const int out = conv ? p->c2_out[m] : p->c1_out[m], in = conv ? p->c2_in[m] : p->c1_in[m];
      const float *srcw = conv ? w->c2_wm[m - 1] : w->c1_wm[m - 1];
      float *dstw = packed + (conv ? p->c2_woff[m] : p->c1_woff[m]);
      const int64_t total = (int64_t)out * in;
      fold_kernel<<<(unsigned)zp_ceil_div(total, 256), 256, 0, st>>>(out / 2, in / 2, srcw, dstw);
      ZP_LAUNCH_CHECK("fold_kernel");
    }
  }
  return ZP_OK;
}

int zp_launch_unfold_wgrad(const zp_plan *p, const float *pg, const zp_weight_grads *gw,
                           cudaStream_t st) {
  ZP_CUDA(cudaMemcpyAsync(gw->c1_w0, pg + p->c1_woff[0],
                          sizeof(float) * (size_t)p->c1_out[0] * p->c1_in[0],
                          cudaMemcpyDeviceToDevice, st));
  ZP_CUDA(cudaMemcpyAsync(gw->c2_w0, pg + p->c2_woff[0],
                          sizeof(float) * (size_t)p->c2_out[0] * p->c2_in[0],
                          cudaMemcpyDeviceToDevice, st));
  for (int m = 1; m < p->n_blocks; ++m) {
    for (int conv = 0; conv < 2; ++conv) {
      const int out = conv ? p->c2_out[m] : p->c1_out[m], in = conv ? p->c2_in[m] : p->c1_in[m];
      const float *f = pg + (conv ? p->c2_woff[m] : p->c1_woff[m]);
      float *g = conv ? gw->c2_wm[m - 1] : gw->c1_wm[m - 1];
      const int64_t total = (int64_t)out * (in / 2);
      unfold_kernel<<<(unsigned)zp_ceil_div(total, 256), 256, 0, st>>>(out / 2, in / 2, f, g);
      ZP_LAUNCH_CHECK("unfold_kernel");
    }
  }
  return ZP_OK;
}

int zp_launch_colsum(int64_t rows, int64_t cols, const float *a, int64_t lda, float *out,
                     float *scratch, cudaStream_t st) {
  if (cols == 0) return ZP_OK;
  const int64_t nparts = rows > 0 ? zp_ceil_div(rows, kColRowsPerBlock) : 0;
  if (nparts > 0) {
    const dim3 grid((unsigned)zp_ceil_div(cols, 128), (unsigned)nparts);
    colsum_part_kernel<<<grid, 128, 0, st>>>(rows, cols, a, lda, scratch);
    ZP_LAUNCH_CHECK("colsum_part_kernel");
  }
  colsum_final_kernel<<<(unsigned)zp_ceil_div(cols, 128), 128, 0, st>>>(nparts, cols, scratch, out);
  ZP_LAUNCH_CHECK("colsum_final_kernel");
  return ZP_OK;
}
