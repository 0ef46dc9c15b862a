// Per-edge front end of the block: geometry, Gaussian distance basis, element embeddings,
// envelope, and the re-ordering of the per-edge inputs into the destination-sorted order, in one
// pass; and its VJP (position and embedding gradients) with fixed-order node sums.
//
//   forward (reference blocks/eso2_ref.py:320-327, :164-168, :242-246)
//     v      = pos[dst] - pos[src] + shift                     edge_vec [E,3]
//     d      = sqrt(max(|v|^2, 1e-24))
//     x_edge = [ exp(coeff * (d - offset_b)^2)  |  emb[Z[src]]  |  emb[Z[dst]] ]      [E, NB + 2 EC]
//     env    = 1 + s^p (a + s (b + c s)) for s = d / cutoff < 1, else 0
//     cos/sin gamma rows copied to the sorted order
//   backward
//     d_d    = sum_b gx[b] gauss_b 2 coeff (d - offset_b)  +  g_env env'(s) / cutoff
//     g_v    = g_edge_vec + d_d v / d                          (0 through the clamp)
//     g_pos[n] = sum_{e into n} g_v[e] - sum_{e out of n} g_v[e]          (CSR order, no atomics)
//     g_emb[z] = sum over atoms n of element z, in index order, of
//                ( sum_{e out of n} gx[e, src part] + sum_{e into n} gx[e, dst part] )
//
// One warp per edge in the per-edge kernels (lanes run over basis functions / channels).
#include "zp_common.cuh"
#include "zippel_b200.h"

namespace {

constexpr int kWarps = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float ipow(float s, int p) {
  float r = 1.f;
  for (int i = 0; i < p; ++i) r *= s;
  return r;
}

struct EnvCoef {
  float a, b, c;
  int p;
};
__host__ __device__ inline EnvCoef env_coef(int p) {
  EnvCoef k;
  k.p = p;
  k.a = -(float)((p + 1) * (p + 2)) / 2.f;
  k.b = (float)(p * (p + 2));
  k.c = -(float)(p * (p + 1)) / 2.f;
  return k;
}

__global__ void __launch_bounds__(32 * kWarps)
edge_features_fwd_kernel(int64_t E, zp_front_config cfg, const float *__restrict__ pos,
                         const float *__restrict__ shifts, const int64_t *__restrict__ z,
                         const float *__restrict__ emb, const float *__restrict__ offsets,
                         const float *__restrict__ cos_g, const float *__restrict__ sin_g,
                         const int32_t *__restrict__ perm, const int32_t *__restrict__ src,
                         const int32_t *__restrict__ dst, float *__restrict__ edge_vec,
                         float *__restrict__ dist_out, float *__restrict__ x_edge,
                         float *__restrict__ env_out, float *__restrict__ cos_s,
                         float *__restrict__ sin_s) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t e = (int64_t)blockIdx.x * kWarps + warp;
  if (e >= E) return;
  const int64_t o = perm[e], i = src[e], j = dst[e];
  const float vx = pos[3 * j] - pos[3 * i] + shifts[3 * o];
  const float vy = pos[3 * j + 1] - pos[3 * i + 1] + shifts[3 * o + 1];
  const float vz = pos[3 * j + 2] - pos[3 * i + 2] + shifts[3 * o + 2];
  const float d = sqrtf(fmaxf((vx * vx + vy * vy) + vz * vz, 1e-24f));
  const int NB = cfg.num_basis, EC = cfg.edge_channels, W = NB + 2 * EC;
  float *row = x_edge + (size_t)e * W;
  for (int b = lane; b < NB; b += 32) {
    const float t = d - offsets[b];
    row[b] = expf(cfg.gauss_coeff * t * t);
  }
  // element numbers come from the caller: one outside the table never becomes an address (it is
  // clamped to the nearest row; the Python layer rejects such input before it gets here, as
  // nn.Embedding does in the reference)
  const int64_t zi = min(max(z[i], (int64_t)0), (int64_t)cfg.n_elements - 1);
  const int64_t zj = min(max(z[j], (int64_t)0), (int64_t)cfg.n_elements - 1);
  const float4 *es = reinterpret_cast<const float4 *>(emb + (size_t)zi * EC);
  const float4 *ed = reinterpret_cast<const float4 *>(emb + (size_t)zj * EC);
  for (int c = lane; c < EC / 4; c += 32) {
    const float4 a = es[c], b = ed[c];
    float *ps = row + NB + 4 * c, *pd = row + NB + EC + 4 * c;
    ps[0] = a.x; ps[1] = a.y; ps[2] = a.z; ps[3] = a.w;        // NB need not be a multiple of 4
    pd[0] = b.x; pd[1] = b.y; pd[2] = b.z; pd[3] = b.w;
  }
  const int nl = cfg.lmax + 1;
  for (int k = lane; k < nl; k += 32) {
    cos_s[e * nl + k] = cos_g[o * nl + k];
    sin_s[e * nl + k] = sin_g[o * nl + k];
  }
  if (lane == 0) {
    edge_vec[3 * e] = vx; edge_vec[3 * e + 1] = vy; edge_vec[3 * e + 2] = vz;
    dist_out[e] = d;
    const EnvCoef k = env_coef(cfg.envelope_exponent);
    const float s = d / cfg.cutoff;
    env_out[e] = s < 1.f ? 1.f + ipow(s, k.p) * (k.a + s * (k.b + k.c * s)) : 0.f;
  }
}

// g_v[e] = g_edge_vec[e] + d_d v / d
__global__ void __launch_bounds__(32 * kWarps)
edge_features_bwd_edge_kernel(int64_t E, zp_front_config cfg, const float *__restrict__ edge_vec,
                              const float *__restrict__ dist, const float *__restrict__ offsets,
                              const float *__restrict__ x_edge, const float *__restrict__ gx,
                              const float *__restrict__ g_env, const float *__restrict__ g_vec_in,
                              float *__restrict__ g_vec) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t e = (int64_t)blockIdx.x * kWarps + warp;
  if (e >= E) return;
  const int NB = cfg.num_basis, W = NB + 2 * cfg.edge_channels;
  const float d = dist[e];
  float acc = 0.f;
  if (gx) {
    const float *xr = x_edge + (size_t)e * W, *gr = gx + (size_t)e * W;
    for (int b = lane; b < NB; b += 32)
      acc += gr[b] * xr[b] * (2.f * cfg.gauss_coeff * (d - offsets[b]));
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    if (g_env) {
      const EnvCoef k = env_coef(cfg.envelope_exponent);
      const float s = d / cfg.cutoff;
      if (s < 1.f) {
        // d/ds [ s^p (a + b s + c s^2) ] = s^(p-1) (p a + (p+1) b s + (p+2) c s^2)
        const float ds = ipow(s, k.p - 1) * (k.p * k.a + s * ((k.p + 1) * k.b + (k.p + 2) * k.c * s));
        acc += g_env[e] * ds / cfg.cutoff;
      }
    }
    const float vx = edge_vec[3 * e], vy = edge_vec[3 * e + 1], vz = edge_vec[3 * e + 2];
    const bool clamped = (vx * vx + vy * vy) + vz * vz < 1e-24f;
    const float f = clamped ? 0.f : acc / d;
    g_vec[3 * e] = (g_vec_in ? g_vec_in[3 * e] : 0.f) + f * vx;
    g_vec[3 * e + 1] = (g_vec_in ? g_vec_in[3 * e + 1] : 0.f) + f * vy;
    g_vec[3 * e + 2] = (g_vec_in ? g_vec_in[3 * e + 2] : 0.f) + f * vz;
  }
}

// one block per atom: position gradient (threads 0..2) and the atom's embedding-gradient row
__global__ void __launch_bounds__(128)
edge_features_bwd_node_kernel(int64_t N, zp_front_config cfg, const float *__restrict__ g_vec,
                              const float *__restrict__ gx, const int32_t *__restrict__ row_ptr,
                              const int32_t *__restrict__ perm_src,
                              const int32_t *__restrict__ row_ptr_src, float *__restrict__ g_pos,
                              float *__restrict__ node_emb) {
  const int64_t n = blockIdx.x;
  const int beg = row_ptr[n], end = row_ptr[n + 1];
  const int sbeg = row_ptr_src[n], send = row_ptr_src[n + 1];
  if (threadIdx.x < 3) {
    float acc = 0.f;
    for (int e = beg; e < end; ++e) acc += g_vec[3 * (int64_t)e + threadIdx.x];
    for (int k = sbeg; k < send; ++k) acc -= g_vec[3 * (int64_t)perm_src[k] + threadIdx.x];
    g_pos[3 * n + threadIdx.x] = acc;
  }
  if (node_emb) {
    const int NB = cfg.num_basis, EC = cfg.edge_channels, W = NB + 2 * EC;
    for (int c = threadIdx.x; c < EC; c += blockDim.x) {
      float acc = 0.f;
      if (gx) {
        for (int k = sbeg; k < send; ++k) acc += gx[(size_t)perm_src[k] * W + NB + c];
        for (int e = beg; e < end; ++e) acc += gx[(size_t)e * W + NB + EC + c];
      }
      node_emb[(size_t)n * EC + c] = acc;
    }
  }
}

// one block per (element, slice of the atoms): rows of the slice's atoms of that element, in
// index order, into partial[slice][element]; the slices are then added in slice order.  Atoms are
// scanned in chunks of blockDim.x: every thread tests one atom, then all threads walk the chunk's
// flags in shared memory, so the serial part never waits on global memory for the element test.
constexpr int kElemSlices = 8;           // the rows of one element are a serial chain of loads
__global__ void __launch_bounds__(128)
edge_features_bwd_elem_kernel(int64_t N, int EC, const int64_t *__restrict__ z,
                              const float *__restrict__ node_emb, float *__restrict__ partial) {
  __shared__ unsigned char mine[128];
  __shared__ int any;
  const int64_t elem = blockIdx.x;
  const int64_t per = (N + kElemSlices - 1) / kElemSlices;
  const int64_t lo = blockIdx.y * per, hi = min(N, lo + per);
  float *g_emb = partial + (size_t)blockIdx.y * gridDim.x * EC;
  float acc[8];                                   // channels c = threadIdx.x + k * blockDim.x
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  for (int64_t n0 = lo; n0 < hi; n0 += blockDim.x) {
    if (threadIdx.x == 0) any = 0;
    __syncthreads();
    const int64_t n = n0 + threadIdx.x;
    const bool hit = n < hi && z[n] == elem;
    mine[threadIdx.x] = hit;
    if (hit) any = 1;
    __syncthreads();
    if (any) {
      const int cnt = (int)min((int64_t)blockDim.x, hi - n0);
      for (int t = 0; t < cnt; ++t)
        if (mine[t]) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c < EC) acc[k] += node_emb[(size_t)(n0 + t) * EC + c];
          }
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int c = threadIdx.x + k * blockDim.x;
    if (c < EC) g_emb[(size_t)elem * EC + c] = acc[k];
  }
}

__global__ void edge_features_elem_sum_kernel(int64_t total, const float *__restrict__ partial,
                                             float *__restrict__ g_emb) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float s = 0.f;
  for (int k = 0; k < kElemSlices; ++k) s += partial[(size_t)k * total + i];
  g_emb[i] = s;
}

int check_cfg(const zp_front_config *cfg) {
  if (!cfg) return ZP_ERR_INVALID_ARG;
  if (cfg->num_basis < 1 || cfg->edge_channels < 4 || (cfg->edge_channels % 4) ||
      cfg->n_elements < 1 || cfg->lmax < 0 || cfg->lmax > ZP_MAX_L || !(cfg->cutoff > 0.f) ||
      cfg->edge_channels > 1024 || cfg->envelope_exponent < 1 || cfg->envelope_exponent > 16)
    return ZP_ERR_UNSUPPORTED;
  return ZP_OK;
}

}  // namespace

extern "C" {

size_t zp_edge_features_work_bytes(const zp_front_config *cfg, int64_t n_nodes, int64_t n_edges) {
  if (check_cfg(cfg) || n_nodes < 0 || n_edges < 0) return 0;
  return zp_align_up(sizeof(float) * 3 * (size_t)n_edges, 256) +
         zp_align_up(sizeof(float) * (size_t)n_nodes * cfg->edge_channels, 256) +
         zp_align_up(sizeof(float) * (size_t)kElemSlices * cfg->n_elements * cfg->edge_channels, 256) +
         256;
}

int zp_edge_features_forward(const zp_front_config *cfg, int64_t N, int64_t E, const float *pos,
                             const float *shifts, const int64_t *atomic_numbers, const float *emb,
                             const float *gauss_offsets, const float *cos_g, const float *sin_g,
                             const int32_t *perm, const int32_t *src, const int32_t *dst,
                             float *edge_vec, float *dist, float *x_edge, float *env,
                             float *cos_sorted, float *sin_sorted, void *stream) {
  int rc = check_cfg(cfg);
  if (rc) return rc;
  if (N < 0 || E < 0) return ZP_ERR_INVALID_ARG;
  if (E == 0) return ZP_OK;
  if (!pos || !shifts || !atomic_numbers || !emb || !gauss_offsets || !cos_g || !sin_g || !perm ||
      !src || !dst || !edge_vec || !dist || !x_edge || !env || !cos_sorted || !sin_sorted)
    return ZP_ERR_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(emb) & 15) return ZP_ERR_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  edge_features_fwd_kernel<<<(unsigned)zp_ceil_div(E, kWarps), 32 * kWarps, 0, st>>>(
      E, *cfg, pos, shifts, atomic_numbers, emb, gauss_offsets, cos_g, sin_g, perm, src, dst,
      edge_vec, dist, x_edge, env, cos_sorted, sin_sorted);
  ZP_LAUNCH_CHECK("edge_features_fwd_kernel");
  return ZP_OK;
}

int zp_edge_features_backward(const zp_front_config *cfg, int64_t N, int64_t E,
                              const float *edge_vec, const float *dist, const float *x_edge,
                              const float *gauss_offsets, const int64_t *atomic_numbers,
                              const float *grad_edge_vec, const float *grad_x_edge,
                              const float *grad_env, const int32_t *row_ptr,
                              const int32_t *perm_src, const int32_t *row_ptr_src,
                              float *grad_pos, float *grad_emb, void *work, size_t work_bytes,
                              void *stream) {
  int rc = check_cfg(cfg);
  if (rc) return rc;
  if (N < 0 || E < 0 || !grad_pos) return ZP_ERR_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (N == 0) return E == 0 ? ZP_OK : ZP_ERR_INVALID_ARG;
  if (!atomic_numbers || !row_ptr || !row_ptr_src || !work) return ZP_ERR_INVALID_ARG;
  if (E && (!edge_vec || !dist || !x_edge || !gauss_offsets || !perm_src)) return ZP_ERR_INVALID_ARG;
  if (work_bytes < zp_edge_features_work_bytes(cfg, N, E)) return ZP_ERR_WORKSPACE;
  float *g_vec = static_cast<float *>(work);
  float *node_emb = reinterpret_cast<float *>(static_cast<unsigned char *>(work) +
                                              zp_align_up(sizeof(float) * 3 * (size_t)E, 256));
  if (E) {
    edge_features_bwd_edge_kernel<<<(unsigned)zp_ceil_div(E, kWarps), 32 * kWarps, 0, st>>>(
        E, *cfg, edge_vec, dist, gauss_offsets, x_edge, grad_x_edge, grad_env, grad_edge_vec, g_vec);
    ZP_LAUNCH_CHECK("edge_features_bwd_edge_kernel");
  }
  edge_features_bwd_node_kernel<<<(unsigned)N, 128, 0, st>>>(
      N, *cfg, g_vec, grad_x_edge, row_ptr, perm_src, row_ptr_src, grad_pos,
      grad_emb ? node_emb : nullptr);
  ZP_LAUNCH_CHECK("edge_features_bwd_node_kernel");
  if (grad_emb) {
    float *partial = reinterpret_cast<float *>(
        reinterpret_cast<unsigned char *>(node_emb) +
        zp_align_up(sizeof(float) * (size_t)N * cfg->edge_channels, 256));
    const int64_t total = (int64_t)cfg->n_elements * cfg->edge_channels;
    edge_features_bwd_elem_kernel<<<dim3((unsigned)cfg->n_elements, kElemSlices), 128, 0, st>>>(
        N, cfg->edge_channels, atomic_numbers, node_emb, partial);
    ZP_LAUNCH_CHECK("edge_features_bwd_elem_kernel");
    edge_features_elem_sum_kernel<<<(unsigned)zp_ceil_div(total, 256), 256, 0, st>>>(total, partial,
                                                                                  grad_emb);
    ZP_LAUNCH_CHECK("edge_features_elem_sum_kernel");
  }
  return ZP_OK;
}

}  // extern "C"
