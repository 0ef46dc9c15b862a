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

// fp32 matrix -> planes (bf16, or fp16 with the tensor's scale), zero padding up to ld_out.
// threadIdx.x walks the quads of a row, threadIdx.y / blockIdx.x the rows (no division anywhere).
__global__ void split_planes_kernel(int64_t rows, int64_t cols, const float *__restrict__ in,
                                    int64_t ld_in, const ZpPlanes out) {
  const int64_t c = 4 * ((int64_t)blockIdx.y * blockDim.x + threadIdx.x);
  if (c >= out.ld) return;
  const bool vec = (ld_in & 3) == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 && c + 3 < cols;
  const float inv = zp_inv_scale(out);
  for (int64_t r = (int64_t)blockIdx.x * blockDim.y + threadIdx.y; r < rows;
       r += (int64_t)gridDim.x * blockDim.y) {
    float v[4];
    if (vec) {
      const float4 q = *reinterpret_cast<const float4 *>(in + r * ld_in + c);
      v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = c + k < cols ? in[r * ld_in + c + k] : 0.f;
    }
    zp_store_planes<4>(out, r * out.ld + c, v, inv);
  }
}

// max |x| over a strided matrix into *out (which the caller zeroed), and the scale derived from
// products of such maxima
__global__ void absmax_kernel(int64_t rows, int64_t cols, const float *__restrict__ in, int64_t ld,
                              float *out) {
  float m = 0.f;
  const int64_t n = rows * cols;
  if (ld == cols && (n & 3) == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0) {
    const float4 *in4 = reinterpret_cast<const float4 *>(in);     // contiguous: 16-byte loads
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n / 4;
         i += (int64_t)gridDim.x * blockDim.x) {
      const float4 v = in4[i];
      m = fmaxf(fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
    }
  } else {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
      m = fmaxf(m, fabsf(in[(i / cols) * ld + i % cols]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0.f) zp_atomic_absmax(out, m);
}

// largest node index the edge list names (the caller zeroed *out)
__global__ void max_index_kernel(int64_t E, const int32_t *__restrict__ src,
                                 const int32_t *__restrict__ dst, int *out) {
  int m = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < E;
       i += (int64_t)gridDim.x * blockDim.x)
    m = max(m, max(src[i], dst[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0) atomicMax(out, m);
}

// max |x| over rows [r0, r1) of a contiguous [*, cols] matrix (cols a multiple of 4, 16-byte
// aligned rows), the row numbers read from device memory:
//   r0 = first ? *first : 0,   r1 = max(min_rows, last ? *last + 1 : 0)
__global__ void absmax_row_range_kernel(const float *__restrict__ in, int64_t cols,
                                        const int32_t *first, const int32_t *last,
                                        int64_t min_rows, float *out) {
  const int64_t r0 = first ? *first : 0;
  int64_t r1 = last ? (int64_t)*last + 1 : 0;
  if (r1 < min_rows) r1 = min_rows;
  float m = 0.f;
  const float4 *in4 = reinterpret_cast<const float4 *>(in + r0 * cols);
  const int64_t n4 = (r1 > r0 ? r1 - r0 : 0) * cols / 4;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float4 v = in4[i];
    m = fmaxf(fmaxf(m, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0.f) zp_atomic_absmax(out, m);
}

// scale[0] = power of two mapping  factor * a * b * max(offset_c, c_factor * c * d)  to 2^15;
// null pointers count as 1, the max term is left out when c is null
__global__ void scale_kernel(float factor, const float *a, const float *b, const float *c,
                             const float *d, float c_factor, float offset_c, float *scale) {
  float bound = factor * (a ? *a : 1.f) * (b ? *b : 1.f);
  if (c) bound *= fmaxf(offset_c, c_factor * *c * (d ? *d : 1.f));
  *scale = zp_scale_for_bound(bound);
}

// ------------------------------------------------------------------------------------------
// gate activation (blocks/eso2_ref.py:295-301): conv1 output row h1[e] = [gate (lmax*H) | y (Km*H)]
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }

// One thread per (edge, pair of rows, hidden-channel quad): both rows' loads are issued before
// either is used, which doubles the bytes a thread keeps in flight.  With `gate_max` set it also records the largest
// sigmoid'(gate) it sees: max|dht| * rows(l) * max|h1| * that value bounds the gate part of the
// backward's dh1, which fixes the scale of its fp16 planes before they are written (the bound
// follows the gates into saturation, where a constant 1/4 would be orders of magnitude loose).
constexpr int kGateEdges = 8;
constexpr int kGateSub = 4;            // groups of kGateEdges edges per block of gate_fwd
__global__ void gate_fwd_kernel(const __grid_constant__ ZpTables t, int64_t E,
                                const float *__restrict__ h1, const ZpPlanes ht,
                                float *gate_max) {
  // blockIdx.x counts groups of kGateEdges edges; the items of a group are indexed with 32-bit
  // arithmetic (a 64-bit division per thread would cost more than the rest of the kernel)
  const int H4 = t.H / 4;
  const int per_edge = ((t.Km + 1) / 2) * H4;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;            // within the group
  const int le = item / per_edge, rem = item - le * per_edge;
  const int rp = rem / H4;
  const int h = (rem - rp * H4) * 4;
  float seen = 0.f;
  bool probe = false;
  const float inv = zp_inv_scale(ht);
  // a block walks kGateSub groups of kGateEdges edges: fewer, longer-lived blocks
#pragma unroll 2
  for (int sub = 0; sub < kGateSub; ++sub) {
    const int64_t e0 = ((int64_t)blockIdx.x * kGateSub + sub) * kGateEdges + le;
    const bool in_range = le < kGateEdges && e0 < E;
    const int64_t e = in_range ? e0 : 0;            // out-of-range threads recompute edge 0
    const float *row = h1 + (size_t)e * t.w1_cols;
    float4 x[2], g[2];
    int rk[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int r = 2 * rp + k;
      rk[k] = r < t.Km ? r : -1;
      const int rr = r < t.Km ? r : 0;               // a missing second row re-reads row 0
      x[k] = *reinterpret_cast<const float4 *>(row + t.n_gate + rr * t.H + h);
      g[k] = rr == 0 ? x[k] : *reinterpret_cast<const float4 *>(row + (t.row_l[rr] - 1) * t.H + h);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int r = rk[k];
      // row 0: x * sigmoid(x) (g holds x there); other rows: x * sigmoid(gate of the row's degree)
      const float s0 = sigmoidf(g[k].x), s1 = sigmoidf(g[k].y), s2 = sigmoidf(g[k].z), s3 = sigmoidf(g[k].w);
      const float o[4] = {x[k].x * s0, x[k].y * s1, x[k].z * s2, x[k].w * s3};
      // every gate l is used by the m = 0 row r = l: those rows alone probe sigmoid'
      if (gate_max != nullptr && r >= 1 && r <= t.lmax) {
        probe = true;
        seen = fmaxf(seen, fmaxf(fmaxf(s0 * (1.f - s0), s1 * (1.f - s1)),
                                 fmaxf(s2 * (1.f - s2), s3 * (1.f - s3))));
      }
      if (in_range && r >= 0) zp_store_planes<4>(ht, e * ht.ld + (int64_t)r * t.H + h, o, inv);
    }
  }
  if (__any_sync(0xffffffffu, probe)) {
#pragma unroll
    for (int k = 16; k > 0; k >>= 1) seen = fmaxf(seen, __shfl_xor_sync(0xffffffffu, seen, k));
    // one address for the whole grid: only warps that would raise the maximum touch it atomically
    if ((threadIdx.x & 31) == 0 && seen > *reinterpret_cast<volatile float *>(gate_max))
      zp_atomic_absmax(gate_max, seen);
  }
}

// one thread per (edge, hidden-channel quad): walks the Km rows, accumulates the lmax gate grads.
// The scale of the fp16 planes is fixed beforehand from max |dht| and the forward's gate bound:
//   |dh1 row| <= 1.1 max|dht|  (sigmoid <= 1, silu' <= 1.1),
//   |dh1 gate_l| = sigmoid'(g_l) |sum_rows dht h1| <= max|dht| * rows(l) * max|h1| * max sigmoid'.
template <int LM>
__global__ void __launch_bounds__(128, 6) gate_bwd_kernel(const __grid_constant__ ZpTables t, int64_t E,
                                const float *__restrict__ h1, const float *__restrict__ dht,
                                const ZpPlanes dh1) {
  const int H4 = t.H / 4;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;            // within a group of edges
  const int le = item / H4;
  const int64_t e0 = (int64_t)blockIdx.x * kGateEdges + le;
  const bool in_range = le < kGateEdges && e0 < E;
  const int64_t e = in_range ? e0 : 0;            // out-of-range threads recompute edge 0
  const int h = (item - le * H4) * 4;
  const float *row = h1 + (size_t)e * t.w1_cols;
  const int64_t drow = e * dh1.ld;
  const float inv = zp_inv_scale(dh1);
  const float *dt = dht + (size_t)e * t.Km * t.H;
  constexpr int NL = LM > 0 ? LM : 1;        // gates: one per degree 1..lmax
  float sg[NL][4], dg[NL][4];
#pragma unroll
  for (int l = 0; l < NL; ++l) {
    if (l < LM) {
      const float4 g = *reinterpret_cast<const float4 *>(row + l * t.H + h);
      sg[l][0] = sigmoidf(g.x); sg[l][1] = sigmoidf(g.y);
      sg[l][2] = sigmoidf(g.z); sg[l][3] = sigmoidf(g.w);
    }
#pragma unroll
    for (int v = 0; v < 4; ++v) dg[l][v] = 0.f;
  }
#pragma unroll 4
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
      for (int ll = 0; ll < NL; ++ll) {
        if (ll == l) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            o[v] = d[v] * sg[ll][v];
            dg[ll][v] = fmaf(d[v], x[v], dg[ll][v]);
          }
        }
      }
    }
    if (in_range) zp_store_planes<4>(dh1, drow + t.n_gate + r * t.H + h, o, inv);
  }
#pragma unroll
  for (int l = 0; l < NL; ++l) {
    if (l < LM) {
      float o[4];
#pragma unroll
      for (int v = 0; v < 4; ++v) o[v] = dg[l][v] * sg[l][v] * (1.f - sg[l][v]);
      if (in_range) zp_store_planes<4>(dh1, drow + l * t.H + h, o, inv);
    }
  }
}

// ------------------------------------------------------------------------------------------
// weight folding and its transpose
// ------------------------------------------------------------------------------------------
// All weight blocks of both convolutions in one launch each (blockIdx.y = block).
struct FoldDesc {
  int n;
  int out[2 * (ZP_MAX_L + 1)], in[2 * (ZP_MAX_L + 1)], folded[2 * (ZP_MAX_L + 1)];
  int slot[2 * (ZP_MAX_L + 1)];                 // index of the block's {max, scale} pair
  const float *w[2 * (ZP_MAX_L + 1)];
  int64_t woff[2 * (ZP_MAX_L + 1)];
};

__global__ void weight_absmax_kernel(const FoldDesc d, float *scales) {
  const int b = blockIdx.y;
  const int64_t total = (int64_t)d.out[b] * (d.folded[b] ? d.in[b] / 2 : d.in[b]);
  float m = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(d.w[b][i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m > 0.f) zp_atomic_absmax(scales + 2 * d.slot[b], m);
}

__global__ void weight_scale_kernel(const FoldDesc d, float *scales) {
  const int b = threadIdx.x;
  if (b < d.n) scales[2 * d.slot[b] + 1] = zp_scale_for_bound(scales[2 * d.slot[b]]);
}

// fold: writes W_fold [out, in] and its transpose [in, out] as 16-bit planes.
//   m = 0 (folded == 0): W_fold = W.   m > 0: W = [Wa ; Wb] (rows), W_fold = [Wa -Wb ; Wb Wa].
__global__ void __launch_bounds__(256)
fold_planes_kernel(const FoldDesc d, uint16_t *__restrict__ packed, int planes, int fp16,
                   const float *__restrict__ scales) {
  // 32 x 32 tiles: the planes of W_fold go out row-major as they are formed; the transpose is
  // written from a shared copy of the tile so that both stores run along the fastest axis.
  __shared__ uint16_t tile[3][32][34];
  const int b = blockIdx.y;
  const int out = d.out[b], in = d.in[b];
  const int64_t total = (int64_t)out * in;
  uint16_t *wp = packed + d.woff[b], *wtp = wp + (size_t)planes * total;
  const float inv = fp16 ? 1.f / scales[2 * d.slot[b] + 1] : 1.f;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;          // 32 x 8
  const int tiles_c = (in + 31) / 32, tiles = ((out + 31) / 32) * tiles_c;
  for (int tl = blockIdx.x; tl < tiles; tl += gridDim.x) {
    const int r0 = (tl / tiles_c) * 32, c0 = (tl % tiles_c) * 32;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int row = r0 + ty + 8 * k, col = c0 + tx;
      if (row < out && col < in) {
        float v;
        if (!d.folded[b]) {
          v = d.w[b][(size_t)row * in + col];
        } else {
          const int half = out / 2, kin = in / 2;
          const bool lower = row >= half, right = col >= kin;
          const int o = lower ? row - half : row, c = right ? col - kin : col;
          v = d.w[b][(size_t)((lower != right) ? half + o : o) * kin + c];
          if (!lower && right) v = -v;
        }
        v *= inv;
        for (int p = 0; p < planes; ++p) {
          uint16_t h;
          if (fp16) {
            const __half q = __float2half_rn(v);
            h = __half_as_ushort(q);
            v -= __half2float(q);
          } else {
            const __nv_bfloat16 q = __float2bfloat16_rn(v);
            h = __bfloat16_as_ushort(q);
            v -= __bfloat162float(q);
          }
          wp[(size_t)p * total + (size_t)row * in + col] = h;
          tile[p][ty + 8 * k][tx] = h;
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int col = c0 + ty + 8 * k, row = r0 + tx;
      if (row < out && col < in)
        for (int p = 0; p < planes; ++p)
          wtp[(size_t)p * total + (size_t)col * out + row] = tile[p][tx][ty + 8 * k];
    }
    __syncthreads();
  }
}

// Sums the `splits` partial folded gradients in order and maps them back to the reference
// layout: m = 0 copies; m > 0: dWa = F[0,0] + F[1,1], dWb = F[1,0] - F[0,1].  All weight blocks
// of both convolutions in one launch (blockIdx.y = block).
struct UnfoldDesc {
  int n;
  int out[2 * (ZP_MAX_L + 1)], in[2 * (ZP_MAX_L + 1)], folded[2 * (ZP_MAX_L + 1)];
  int splits[2 * (ZP_MAX_L + 1)];
  int64_t foff[2 * (ZP_MAX_L + 1)];             // offset of the block's folded gradient
  float *gw[2 * (ZP_MAX_L + 1)];
};
__global__ void unfold_kernel(const UnfoldDesc d, int64_t split_stride, const float *__restrict__ f) {
  const int b = blockIdx.y;
  const int out = d.out[b], in = d.in[b], folded = d.folded[b];
  const int kin = folded ? in / 2 : in, half = out / 2;
  const int64_t total = (int64_t)out * kin;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(idx % kin), row = (int)(idx / kin);
    float acc = 0.f;
    for (int s = 0; s < d.splits[b]; ++s) {
      const float *fs = f + d.foff[b] + (size_t)s * split_stride;
      if (!folded) acc += fs[idx];
      else if (row < half) acc += fs[(size_t)row * in + c] + fs[(size_t)(half + row) * in + kin + c];
      else acc += fs[(size_t)row * in + c] - fs[(size_t)(row - half) * in + kin + c];
    }
    d.gw[b][idx] = acc;
  }
}

// column sums in two fixed-order stages.  Stage one: a block of 32 x 8 threads sums 128 rows of
// 256 columns; a thread owns 8 consecutive columns (one 16-byte load per row and plane) and every
// eighth row, the eight row groups are then added in order through shared memory.
constexpr int kColRowsPerBlock = 512;    // scratch is sized for 128 (more partials than are used)
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
        const uint4 v = *reinterpret_cast<const uint4 *>(
            static_cast<const uint16_t *>(a.base) + (size_t)pl * a.plane_stride + r * a.ld + c0);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          s[2 * k] += zp_plane_value(a, (uint16_t)(w[k] & 0xffffu));
          s[2 * k + 1] += zp_plane_value(a, (uint16_t)(w[k] >> 16));
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
      if (c0 + k < cols) part[(size_t)blockIdx.y * cols + c0 + k] = acc * zp_scale(a);
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

// scale of conv1's activated output from an a-priori bound (one block):
//   |h1| <= max_m(in_m * A * max|W_m|) + max|b|,  A = 2^15 * a1_scale >= max|a1|
struct BoundDesc {
  int n;
  int in[ZP_MAX_L + 1];
  int n_bias;
};
__global__ void __launch_bounds__(256)
conv1_bound_kernel(const BoundDesc d, const float *a1_scale, const float *wscales,
                   const float *__restrict__ bias, float *ht_scale) {
  __shared__ float red[8];
  float m = 0.f;
  for (int i = threadIdx.x; i < d.n_bias; i += blockDim.x) m = fmaxf(m, fabsf(bias[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float bmax = 0.f;
    for (int i = 0; i < 8; ++i) bmax = fmaxf(bmax, red[i]);
    const float a = 32768.f * *a1_scale;
    float bound = 0.f;
    for (int b = 0; b < d.n; ++b) bound = fmaxf(bound, (float)d.in[b] * a * wscales[2 * b]);
    *ht_scale = zp_scale_for_bound(1.001f * (bound + bmax));
  }
}

}  // namespace

int zp_launch_conv1_bound(const zp_plan *p, const float *a1_scale, const float *wscales,
                          const float *bias, float *ht_scale, cudaStream_t st) {
  BoundDesc d;
  d.n = p->n_blocks;
  for (int m = 0; m < p->n_blocks; ++m) d.in[m] = p->c1_in[m];
  d.n_bias = p->c1_out[0];
  conv1_bound_kernel<<<1, 256, 0, st>>>(d, a1_scale, wscales, bias, ht_scale);
  ZP_LAUNCH_CHECK("conv1_bound_kernel");
  return ZP_OK;
}

int zp_launch_split_planes(int64_t rows, int64_t cols, const float *in, int64_t ld_in,
                           const ZpPlanes &out, cudaStream_t st) {
  if (rows == 0 || out.ld == 0) return ZP_OK;
  const int quads = (int)(out.ld / 4);
  int bx = 32;
  while (bx < quads && bx < 256) bx <<= 1;
  const int by = 256 / bx;
  int64_t gx = zp_ceil_div(rows, by);
  if (gx > 148 * 32) gx = 148 * 32;
  const dim3 grid((unsigned)gx, (unsigned)zp_ceil_div(quads, bx)), block(bx, by);
  split_planes_kernel<<<grid, block, 0, st>>>(rows, cols, in, ld_in, out);
  ZP_LAUNCH_CHECK("split_planes_kernel");
  return ZP_OK;
}

int zp_launch_absmax(int64_t rows, int64_t cols, const float *in, int64_t ld, float *out,
                     cudaStream_t st) {
  ZP_CUDA(cudaMemsetAsync(out, 0, sizeof(float), st));
  if (rows * cols == 0) return ZP_OK;
  int64_t blocks = zp_ceil_div(rows * cols, 256 * 8);
  if (blocks > 1184) blocks = 1184;
  absmax_kernel<<<(unsigned)blocks, 256, 0, st>>>(rows, cols, in, ld, out);
  ZP_LAUNCH_CHECK("absmax_kernel");
  return ZP_OK;
}

int zp_launch_max_index(int64_t E, const int32_t *src, const int32_t *dst, int *out,
                        cudaStream_t st) {
  ZP_CUDA(cudaMemsetAsync(out, 0, sizeof(int), st));
  if (E == 0) return ZP_OK;
  int64_t blocks = zp_ceil_div(E, 256 * 4);
  if (blocks > 592) blocks = 592;
  max_index_kernel<<<(unsigned)blocks, 256, 0, st>>>(E, src, dst, out);
  ZP_LAUNCH_CHECK("max_index_kernel");
  return ZP_OK;
}

int zp_launch_absmax_row_range(const float *in, int64_t cols, const int32_t *first,
                               const int32_t *last, int64_t min_rows, float *out,
                               cudaStream_t st) {
  ZP_CUDA(cudaMemsetAsync(out, 0, sizeof(float), st));
  if (cols == 0 || (cols & 3)) return cols ? ZP_ERR_INVALID_ARG : ZP_OK;
  absmax_row_range_kernel<<<1184, 256, 0, st>>>(in, cols, first, last, min_rows, out);
  ZP_LAUNCH_CHECK("absmax_row_range_kernel");
  return ZP_OK;
}

int zp_launch_scale(float factor, const float *a, const float *b, const float *c, float offset_c,
                    float *scale, cudaStream_t st, const float *d, float c_factor) {
  scale_kernel<<<1, 1, 0, st>>>(factor, a, b, c, d, c_factor, offset_c, scale);
  ZP_LAUNCH_CHECK("scale_kernel");
  return ZP_OK;
}

int zp_launch_gate_fwd(const zp_plan *p, int64_t E, const float *h1, const ZpPlanes &ht,
                       float *gate_max, cudaStream_t st) {
  if (gate_max) ZP_CUDA(cudaMemsetAsync(gate_max, 0, sizeof(float), st));
  if (E == 0) return ZP_OK;
  const int per_group = kGateEdges * ((p->t.Km + 1) / 2) * (p->t.H / 4);
  const dim3 grid((unsigned)zp_ceil_div(E, kGateEdges * kGateSub),
                  (unsigned)zp_ceil_div(per_group, 256));
  gate_fwd_kernel<<<grid, 256, 0, st>>>(p->t, E, h1, ht, gate_max);
  ZP_LAUNCH_CHECK("gate_fwd_kernel");
  return ZP_OK;
}

int zp_launch_gate_bwd(const zp_plan *p, int64_t E, const float *h1, const float *dht,
                       const ZpPlanes &dh1, cudaStream_t st) {
  if (E == 0) return ZP_OK;
  const int per_group = kGateEdges * (p->t.H / 4);
  const dim3 grid((unsigned)zp_ceil_div(E, kGateEdges), (unsigned)zp_ceil_div(per_group, 128));
#define CALL(LM) gate_bwd_kernel<LM><<<grid, 128, 0, st>>>(p->t, E, h1, dht, dh1)
  ZP_DISPATCH_LMAX(p->t.lmax, CALL)
#undef CALL
  ZP_LAUNCH_CHECK("gate_bwd_kernel");
  return ZP_OK;
}

static const float *block_weight(const zp_weights *w, int conv, int m) {
  if (m == 0) return conv ? w->c2_w0 : w->c1_w0;
  return conv ? w->c2_wm[m - 1] : w->c1_wm[m - 1];
}

int zp_launch_fold_weights(const zp_plan *p, const zp_weights *w, void *packed, float *scales,
                           cudaStream_t st) {
  FoldDesc d;
  d.n = 0;
  for (int conv = 0; conv < 2; ++conv)
    for (int m = 0; m < p->n_blocks; ++m) {
      const int b = d.n++;
      d.out[b] = conv ? p->c2_out[m] : p->c1_out[m];
      d.in[b] = conv ? p->c2_in[m] : p->c1_in[m];
      d.folded[b] = m > 0;
      d.slot[b] = conv * (ZP_MAX_L + 1) + m;
      d.w[b] = block_weight(w, conv, m);
      d.woff[b] = conv ? p->c2_woff[m] : p->c1_woff[m];
    }
  if (p->fp16) {       // one power-of-two scale per weight block from its largest magnitude
    ZP_CUDA(cudaMemsetAsync(scales, 0, sizeof(float) * 4 * (ZP_MAX_L + 1), st));
    weight_absmax_kernel<<<dim3(148, d.n), 256, 0, st>>>(d, scales);
    ZP_LAUNCH_CHECK("weight_absmax_kernel");
    weight_scale_kernel<<<1, 32, 0, st>>>(d, scales);
    ZP_LAUNCH_CHECK("weight_scale_kernel");
  }
  fold_planes_kernel<<<dim3(296, d.n), 256, 0, st>>>(d, static_cast<uint16_t *>(packed), p->planes,
                                                     p->fp16, scales);
  ZP_LAUNCH_CHECK("fold_planes_kernel");
  return ZP_OK;
}

int zp_launch_unfold_wgrad(const zp_plan *p, const float *partials, int64_t split_stride,
                           const int *splits_c1, const int *splits_c2, const zp_weight_grads *gw,
                           cudaStream_t st) {
  UnfoldDesc d;
  d.n = 0;
  for (int conv = 0; conv < 2; ++conv) {
    for (int m = 0; m < p->n_blocks; ++m) {
      const int b = d.n++;
      d.out[b] = conv ? p->c2_out[m] : p->c1_out[m];
      d.in[b] = conv ? p->c2_in[m] : p->c1_in[m];
      d.folded[b] = m > 0;
      d.splits[b] = (conv ? splits_c2 : splits_c1)[m];
      d.foff[b] = conv ? p->c2_goff[m] : p->c1_goff[m];
      d.gw[b] = m == 0 ? (conv ? gw->c2_w0 : gw->c1_w0)
                       : (conv ? gw->c2_wm[m - 1] : gw->c1_wm[m - 1]);
    }
  }
  unfold_kernel<<<dim3(148, d.n), 256, 0, st>>>(d, split_stride, partials);
  ZP_LAUNCH_CHECK("unfold_kernel");
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
