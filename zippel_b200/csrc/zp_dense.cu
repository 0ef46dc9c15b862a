// Elementwise and layout pieces around the SO(2) contraction: the gate activation and its VJP,
// weight folding into bf16 planes (and the transpose of that for the weight gradients), and
// column sums for the bias gradients.  The contraction itself runs on the tensor cores.
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
// gate activation (blocks/eso2_ref.py:295-301): conv1 output row h1[e] = [gate (lmax*H) | y (Km*H)]
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void gate_fwd_kernel(const __grid_constant__ ZpTables t, int64_t E,
                                const float *__restrict__ h1, const ZpPlanes ht) {
  const int H4 = t.H / 4;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = E * t.Km * H4;
  if (idx >= total) return;
  const int h = (int)(idx % H4) * 4;
  const int r = (int)((idx / H4) % t.Km);
  const int64_t e = idx / ((int64_t)H4 * t.Km);
  const float *row = h1 + (size_t)e * t.w1_cols;
  const float4 x = *reinterpret_cast<const float4 *>(row + t.n_gate + r * t.H + h);
  float o[4];
  if (r == 0) {
    o[0] = x.x * sigmoidf(x.x); o[1] = x.y * sigmoidf(x.y);
    o[2] = x.z * sigmoidf(x.z); o[3] = x.w * sigmoidf(x.w);
  } else {
    const float4 g = *reinterpret_cast<const float4 *>(row + (t.row_l[r] - 1) * t.H + h);
    o[0] = x.x * sigmoidf(g.x); o[1] = x.y * sigmoidf(g.y);
    o[2] = x.z * sigmoidf(g.z); o[3] = x.w * sigmoidf(g.w);
  }
  zp_store_planes<4>(ht, e * ht.ld + (int64_t)r * t.H + h, o);
}

// one thread per (edge, hidden-channel quad): walks the Km rows, accumulates the lmax gate grads
__global__ void gate_bwd_kernel(const __grid_constant__ ZpTables t, int64_t E,
                                const float *__restrict__ h1, const float *__restrict__ dht,
                                const ZpPlanes dh1) {
  const int H4 = t.H / 4;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= E * H4) return;
  const int h = (int)(idx % H4) * 4;
  const int64_t e = idx / H4;
  const float *row = h1 + (size_t)e * t.w1_cols;
  const int64_t drow = e * dh1.ld;
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
    zp_store_planes<4>(dh1, drow + t.n_gate + r * t.H + h, o);
  }
#pragma unroll
  for (int l = 0; l < ZP_MAX_L; ++l) {
    if (l < t.lmax) {
      float o[4];
#pragma unroll
      for (int v = 0; v < 4; ++v) o[v] = dg[l][v] * sg[l][v] * (1.f - sg[l][v]);
      zp_store_planes<4>(dh1, drow + l * t.H + h, o);
    }
  }
}

// ------------------------------------------------------------------------------------------
// weight folding and its transpose
// ------------------------------------------------------------------------------------------
// fold: writes W_fold [out, in] and its transpose [in, out] as bf16 planes.
//   m = 0 (folded == 0): W_fold = W.   m > 0: W = [Wa ; Wb] (rows), W_fold = [Wa -Wb ; Wb Wa].
__global__ void fold_planes_kernel(int out, int in, int folded, const float *__restrict__ w,
                                   __nv_bfloat16 *__restrict__ wp, __nv_bfloat16 *__restrict__ wtp,
                                   int planes) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total = (int64_t)out * in;
  if (idx >= total) return;
  const int col = (int)(idx % in), row = (int)(idx / in);
  float v;
  if (!folded) {
    v = w[idx];
  } else {
    const int half = out / 2, kin = in / 2;
    const bool lower = row >= half, right = col >= kin;
    const int o = lower ? row - half : row, c = right ? col - kin : col;
    v = w[(size_t)((lower != right) ? half + o : o) * kin + c];
    if (!lower && right) v = -v;
  }
  for (int p = 0; p < planes; ++p) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    wp[(size_t)p * total + idx] = h;
    wtp[(size_t)p * total + (size_t)col * out + row] = h;
    v -= __bfloat162float(h);
  }
}

// Sums the `splits` partial folded gradients in order and maps them back to the reference
// layout: m = 0 copies; m > 0: dWa = F[0,0] + F[1,1], dWb = F[1,0] - F[0,1].
__global__ void unfold_kernel(int out, int in, int folded, int splits, int64_t split_stride,
                              const float *__restrict__ f, float *__restrict__ gw) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int kin = folded ? in / 2 : in, half = out / 2;
  const int64_t total = (int64_t)out * kin;
  if (idx >= total) return;
  const int c = (int)(idx % kin), row = (int)(idx / kin);
  float acc = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float *fs = f + (size_t)s * split_stride;
    if (!folded) acc += fs[idx];
    else if (row < half) acc += fs[(size_t)row * in + c] + fs[(size_t)(half + row) * in + kin + c];
    else acc += fs[(size_t)row * in + c] - fs[(size_t)(row - half) * in + kin + c];
  }
  gw[idx] = acc;
}

// column sums in two fixed-order stages.  Stage one: a block of 32 x 8 threads sums 128 rows of
// 256 columns; a thread owns 8 consecutive columns (one 16-byte load per row and plane) and every
// eighth row, the eight row groups are then added in order through shared memory.
constexpr int kColRowsPerBlock = 128;
__global__ void __launch_bounds__(256)
colsum_part_kernel(int64_t rows, int64_t cols, const ZpPlanes a, float *__restrict__ part) {
  __shared__ float red[8][32][9];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const int64_t c0 = ((int64_t)blockIdx.x * 32 + tx) * 8;
  const int64_t r0 = (int64_t)blockIdx.y * kColRowsPerBlock;
  const int64_t r1 = min(rows, r0 + kColRowsPerBlock);
  float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c0 < cols) {
    for (int64_t r = r0 + ty; r < r1; r += 8) {
      for (int pl = a.planes - 1; pl >= 0; --pl) {
        const uint4 v = *reinterpret_cast<const uint4 *>(a.base + (size_t)pl * a.plane_stride +
                                                         r * a.ld + c0);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          s[2 * k] += __uint_as_float(w[k] << 16);
          s[2 * k + 1] += __uint_as_float(w[k] & 0xffff0000u);
        }
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) red[ty][tx][k] = s[k];
  __syncthreads();
  if (ty == 0 && c0 < cols) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float acc = 0.f;
      for (int g = 0; g < 8; ++g) acc += red[g][tx][k];
      if (c0 + k < cols) part[(size_t)blockIdx.y * cols + c0 + k] = acc;
    }
  }
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

int zp_launch_split_planes(int64_t rows, int64_t cols, const float *in, int64_t ld_in, void *out,
                           int64_t ld_out, int64_t plane_stride, int planes, cudaStream_t st) {
  if (rows == 0 || ld_out == 0) return ZP_OK;
  split_planes_kernel<<<(unsigned)zp_ceil_div(rows * ld_out, 256), 256, 0, st>>>(
      rows, cols, in, ld_in, (__nv_bfloat16 *)out, ld_out, plane_stride, planes);
  ZP_LAUNCH_CHECK("split_planes_kernel");
  return ZP_OK;
}

int zp_launch_gate_fwd(const zp_plan *p, int64_t E, const float *h1, const ZpPlanes &ht,
                       cudaStream_t st) {
  if (E == 0) return ZP_OK;
  const int64_t total = E * p->t.Km * (p->t.H / 4);
  gate_fwd_kernel<<<(unsigned)zp_ceil_div(total, 256), 256, 0, st>>>(p->t, E, h1, ht);
  ZP_LAUNCH_CHECK("gate_fwd_kernel");
  return ZP_OK;
}

int zp_launch_gate_bwd(const zp_plan *p, int64_t E, const float *h1, const float *dht,
                       const ZpPlanes &dh1, cudaStream_t st) {
  if (E == 0) return ZP_OK;
  const int64_t total = E * (p->t.H / 4);
  gate_bwd_kernel<<<(unsigned)zp_ceil_div(total, 128), 128, 0, st>>>(p->t, E, h1, dht, dh1);
  ZP_LAUNCH_CHECK("gate_bwd_kernel");
  return ZP_OK;
}

static const float *block_weight(const zp_weights *w, int conv, int m) {
  if (m == 0) return conv ? w->c2_w0 : w->c1_w0;
  return conv ? w->c2_wm[m - 1] : w->c1_wm[m - 1];
}

int zp_launch_fold_weights(const zp_plan *p, const zp_weights *w, void *packed, cudaStream_t st) {
  __nv_bfloat16 *base = static_cast<__nv_bfloat16 *>(packed);
  for (int conv = 0; conv < 2; ++conv) {
    for (int m = 0; m < p->n_blocks; ++m) {
      const int out = conv ? p->c2_out[m] : p->c1_out[m], in = conv ? p->c2_in[m] : p->c1_in[m];
      const int64_t total = (int64_t)out * in;
      __nv_bfloat16 *wp = base + (conv ? p->c2_woff[m] : p->c1_woff[m]);
      fold_planes_kernel<<<(unsigned)zp_ceil_div(total, 256), 256, 0, st>>>(
          out, in, m > 0, block_weight(w, conv, m), wp, wp + (size_t)p->planes * total, p->planes);
      ZP_LAUNCH_CHECK("fold_planes_kernel");
    }
  }
  return ZP_OK;
}

int zp_launch_unfold_wgrad(const zp_plan *p, const float *partials, int64_t split_stride,
                           const int *splits_c1, const int *splits_c2, const zp_weight_grads *gw,
                           cudaStream_t st) {
  for (int conv = 0; conv < 2; ++conv) {
    for (int m = 0; m < p->n_blocks; ++m) {
      const int out = conv ? p->c2_out[m] : p->c1_out[m], in = conv ? p->c2_in[m] : p->c1_in[m];
      const float *f = partials + (conv ? p->c2_goff[m] : p->c1_goff[m]);
      float *g = m == 0 ? (conv ? gw->c2_w0 : gw->c1_w0)
                        : (conv ? gw->c2_wm[m - 1] : gw->c1_wm[m - 1]);
      const int64_t total = (int64_t)out * (m > 0 ? in / 2 : in);
      unfold_kernel<<<(unsigned)zp_ceil_div(total, 256), 256, 0, st>>>(
          out, in, m > 0, (conv ? splits_c2 : splits_c1)[m], split_stride, f, g);
      ZP_LAUNCH_CHECK("unfold_kernel");
    }
  }
  return ZP_OK;
}

int zp_launch_colsum(int64_t rows, int64_t cols, const ZpPlanes &a, float *out, float *scratch,
                     cudaStream_t st) {
  if (cols == 0) return ZP_OK;
  const int64_t nparts = rows > 0 ? zp_ceil_div(rows, kColRowsPerBlock) : 0;
  if (nparts > 0) {
    const dim3 grid((unsigned)zp_ceil_div(cols, 256), (unsigned)nparts), block(32, 8);
    colsum_part_kernel<<<grid, block, 0, st>>>(rows, cols, a, scratch);
    ZP_LAUNCH_CHECK("colsum_part_kernel");
  }
  colsum_final_kernel<<<(unsigned)zp_ceil_div(cols, 128), 128, 0, st>>>(nparts, cols, scratch, out);
  ZP_LAUNCH_CHECK("colsum_final_kernel");
  return ZP_OK;
}
