// Gather / rotate / scatter kernels around the SO(2) contraction.
//
//   rotate_in            a[e, r, c2] = radial[e, .] * sum_j rot[e, r, j] * [x_src ; x_dst][l_r^2 + j, c2]
//   rotate_back_scatter  node_out[n, l^2 + j, c] = sum_{e -> n} env_e * sum_r rot[e, r, j] * y[e, r, c]
//   rotate_grad_out      the VJP of rotate_back_scatter (needs y), one edge per warp group
//   rotate_in_bwd        the VJP of rotate_in, one edge per warp group, per-edge node contributions
//   node_reduce          fixed-order sums of those contributions per destination / source node
//
// They take over blocks/eso2_ref.py:334-335 (gather + rotate in, with the radial gain of
// :269-271, :284-285 applied while the row is in registers) and :343-349 (envelope, rotate
// back, index_add_).  The rotation is block diagonal in the degree l, so each thread keeps
// one degree's 2l+1 input rows of its channel group in registers and forms only the rows with
// |m| <= mmax.  Channels are the fastest axis everywhere: a thread owns VEC consecutive
// channels and moves them with one vector load/store.  No atomics: every output element is
// produced by exactly one thread, in an order fixed by the CSR offsets.
#include <algorithm>

#include "zp_common.cuh"
#include "zp_planes.cuh"

namespace {

template <int VEC> struct Vec;
template <> struct Vec<4> { using type = float4; };
template <> struct Vec<2> { using type = float2; };
template <> struct Vec<1> { using type = float; };

template <int VEC>
__device__ __forceinline__ void vload(float (&r)[VEC], const float *p) {
  using V = typename Vec<VEC>::type;
  const V v = *reinterpret_cast<const V *>(p);
  const float *s = reinterpret_cast<const float *>(&v);
#pragma unroll
  for (int i = 0; i < VEC; ++i) r[i] = s[i];
}
template <int VEC>
__device__ __forceinline__ void vstore(float *p, const float (&r)[VEC]) {
  using V = typename Vec<VEC>::type;
  V v;
  float *s = reinterpret_cast<float *>(&v);
#pragma unroll
  for (int i = 0; i < VEC; ++i) s[i] = r[i];
  *reinterpret_cast<V *>(p) = v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------------------
// rotate_in: one (edge, channel quad) per thread
// ------------------------------------------------------------------------------------------

constexpr int kRotInThreads = 256;
constexpr int kRotInMaxEdges = 32;

template <int L, int LMAX>
struct RotIn {
  static __device__ __forceinline__ void run(const ZpTables &t, const float *xrow,
                                             const float *rot_s, const float *rad_e,
                                             const ZpPlanes &a1, int64_t a_row, int c2, float inv) {
    RotIn<L - 1, LMAX>::run(t, xrow, rot_s, rad_e, a1, a_row, c2, inv);
    constexpr int n = 2 * L + 1;
    const int C2 = 2 * t.C;
    float u[n][4];
#pragma unroll
    for (int j = 0; j < n; ++j) vload<4>(u[j], xrow + (size_t)(L * L + j) * t.C);
    const int mm = t.mmax < L ? t.mmax : L;
    // a real loop over the rows |m| <= mmax of this degree: one copy of the body per degree keeps
    // the kernel's code inside the instruction cache
    // the radial gain of the NEXT row is requested before this row's sums are formed
    float g_next[4];
    vload<4>(g_next, rad_e + t.rad_off[mm] + (L - mm) * C2 + c2);
#pragma unroll 1
    for (int i = L - mm; i <= L + mm; ++i) {
      {
        const int r = t.row_of[L][i];
        const float *rr = rot_s + t.rot_off[r];
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, g[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) g[v] = g_next[v];
        if (i < L + mm) {
          const int an = i + 1 > L ? i + 1 - L : L - i - 1;
          vload<4>(g_next, rad_e + t.rad_off[an] + (L - an) * C2 + c2);
        }
#pragma unroll
        for (int j = 0; j < n; ++j) {
          const float w = rr[j];
#pragma unroll
          for (int v = 0; v < 4; ++v) acc[v] = fmaf(w, u[j][v], acc[v]);
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[v] *= g[v];
        zp_store_planes<4>(a1, a_row + (int64_t)r * C2 + c2, acc, inv);
      }
    }
  }
};
template <int LMAX>
struct RotIn<-1, LMAX> {
  static __device__ __forceinline__ void run(const ZpTables &, const float *, const float *,
                                             const float *, const ZpPlanes &, int64_t, int, float) {}
};

template <int LMAX>
__global__ void __launch_bounds__(kRotInThreads, (LMAX <= 4 ? 4 : 3))
rotate_in_kernel(const __grid_constant__ ZpTables t, int64_t E, int epb,
                 const float *__restrict__ x, const int32_t *__restrict__ src,
                 const int32_t *__restrict__ dst, const float *__restrict__ rot,
                 const float *__restrict__ radial, const ZpPlanes a1) {
  extern __shared__ float rot_s[];                       // [epb][nnz_pad]
  const int Q = t.C / 2;                                 // channel quads of the 2C-wide message
  const int64_t e0 = (int64_t)blockIdx.x * epb;
  const int n_e = (int)min((int64_t)epb, E - e0);
  for (int i = threadIdx.x; i < n_e * t.nnz_pad; i += blockDim.x)
    rot_s[i] = rot[e0 * t.nnz_pad + i];
  __syncthreads();
  const int le = threadIdx.x / Q, q = threadIdx.x % Q;
  if (le >= n_e) return;
  const int64_t e = e0 + le;
  const int c2 = 4 * q;
  const bool second = c2 >= t.C;
  const int64_t node = second ? dst[e] : src[e];
  const float *xrow = x + (size_t)node * t.K * t.C + (second ? c2 - t.C : c2);
  RotIn<LMAX, LMAX>::run(t, xrow, rot_s + le * t.nnz_pad, radial + (size_t)e * t.R,
                         a1, e * a1.ld, c2, zp_inv_scale(a1));
}

// ------------------------------------------------------------------------------------------
// per-destination-node kernel (forward scatter)
// ------------------------------------------------------------------------------------------


// stage one edge's packed rotation in this node slot's shared buffer
__device__ __forceinline__ void stage_rot(const ZpTables &t, const float *rot_e, float *buf,
                                          int tid, int nthreads) {
  for (int i = tid; i < t.nnz_pad; i += nthreads) buf[i] = rot_e[i];
}

template <int L, int LMAX, int VEC>
struct RotBack {
  // y_e: the edge's rows [Km][row_stride], this lane's channels start at c
  static __device__ __forceinline__ void run(const ZpTables &t, const float *y_e, int row_stride,
                                             const float *rot_s, float env,
                                             float (&acc)[(LMAX + 1) * (LMAX + 1)][VEC], int c) {
    RotBack<L - 1, LMAX, VEC>::run(t, y_e, row_stride, rot_s, env, acc, c);
    constexpr int n = 2 * L + 1;
    const int mm = t.mmax < L ? t.mmax : L;
#pragma unroll
    for (int i = 0; i < n; ++i) {
      const int am = i > L ? i - L : L - i;
      if (am <= mm) {
        const int r = t.row_of[L][i];
        const float *rr = rot_s + t.rot_off[r];
        float yv[VEC];
        vload<VEC>(yv, y_e + (size_t)r * row_stride + c);
#pragma unroll
        for (int v = 0; v < VEC; ++v) yv[v] *= env;
#pragma unroll
        for (int j = 0; j < n; ++j) {
          const float w = rr[j];
#pragma unroll
          for (int v = 0; v < VEC; ++v) acc[L * L + j][v] = fmaf(w, yv[v], acc[L * L + j][v]);
        }
      }
    }
  }
};
template <int LMAX, int VEC>
struct RotBack<-1, LMAX, VEC> {
  static __device__ __forceinline__ void run(const ZpTables &, const float *, int, const float *,
                                             float, float (&)[(LMAX + 1) * (LMAX + 1)][VEC],
                                             int) {}
};

// One block (four warps) owns 32 x VEC channels of one destination node.  The node's edges are
// dealt round-robin to the warps (warp w takes edges w, w + 4, ... of the CSR segment), which cuts
// the serial chain per node by four; the four partial sums are then added in warp order through
// shared memory, so the result does not depend on timing.
// Each warp keeps the rows of its NEXT edge in flight while it rotates the current one: every lane
// copies its own channels of the Km rows into a two-stage shared buffer with cp.async (16 or 8
// bytes per row), so the memory latency is paid once per edge, not once per row.
constexpr int kBackWarps = 4;

template <int BYTES>
__device__ __forceinline__ void cp_async(float *smem_dst, const float *gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  if (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int LMAX, int VEC>
__global__ void __launch_bounds__(32 * kBackWarps, (LMAX >= 5 && VEC == 2 ? 3 : 1))
rotate_back_scatter_kernel(const __grid_constant__ ZpTables t, int64_t N,
                           const float *__restrict__ y, const float *__restrict__ env,
                           const float *__restrict__ rot, const int32_t *__restrict__ row_ptr,
                           float *__restrict__ node_out) {
  constexpr int K = (LMAX + 1) * (LMAX + 1);
  constexpr int W = 32 * VEC;              // channels of this block
  // rot [4][nnz_pad] | y stages [4 warps][2][Km][W], reused as partial [4][K][W] at the end
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  float *rot_s = smem + warp * t.nnz_pad;
  float *region = smem + kBackWarps * t.nnz_pad;
  float *ybuf = region + (size_t)warp * 2 * t.Km * W;
  float *part = region;
  const int64_t n = blockIdx.x;
  const int c0 = blockIdx.y * W;
  const int c = c0 + lane * VEC;
  const bool active = c < t.C;
  float acc[K][VEC];
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[k][v] = 0.f;
  const int e_beg = row_ptr[n], e_end = row_ptr[n + 1];
  // the next edge's packed rotation is fetched into registers while the current one is used
  float nxt[8];
  auto fetch = [&](int e) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = lane + 32 * i;
      nxt[i] = (e < e_end && k < t.nnz_pad) ? rot[(size_t)e * t.nnz_pad + k] : 0.f;
    }
  };
  auto stage_rows = [&](int e, int stage) {          // this lane's channels of edge e's Km rows
    if (e < e_end && active) {
      const float *src = y + (size_t)e * t.Km * t.C + c;
      float *dst = ybuf + (size_t)stage * t.Km * W + lane * VEC;
      for (int r = 0; r < t.Km; ++r) cp_async<4 * VEC>(dst + r * W, src + (size_t)r * t.C);
    }
    cp_async_commit();
  };
  fetch(e_beg + warp);
  stage_rows(e_beg + warp, 0);
  int stage = 0;
  for (int e = e_beg + warp; e < e_end; e += kBackWarps, stage ^= 1) {
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (lane + 32 * i < t.nnz_pad) rot_s[lane + 32 * i] = nxt[i];
    const float env_e = env[e];
    fetch(e + kBackWarps);
    stage_rows(e + kBackWarps, stage ^ 1);
    cp_async_wait<1>();                  // everything but the group just committed has landed
    __syncwarp();
    if (active)
      RotBack<LMAX, LMAX, VEC>::run(t, ybuf + (size_t)stage * t.Km * W, W, rot_s, env_e, acc,
                                    lane * VEC);
  }
  cp_async_wait<0>();
  __syncthreads();                       // all warps are done with their stages: reuse as partials
#pragma unroll
  for (int k = 0; k < K; ++k)
#pragma unroll
    for (int v = 0; v < VEC; ++v) part[(warp * K + k) * W + lane * VEC + v] = acc[k][v];
  __syncthreads();
  for (int i = threadIdx.x; i < K * W; i += blockDim.x) {
    const int k = i / W, cc = i % W;
    if (c0 + cc < t.C) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kBackWarps; ++w) s += part[(w * K + k) * W + cc];
      node_out[((size_t)n * K + k) * t.C + c0 + cc] = s;
    }
  }
}

// ------------------------------------------------------------------------------------------
// per-edge backward kernels: W warps cover one edge's channel groups.  rotate_grad_out runs eight
// warps per block and loads rows as it goes; rotate_in_bwd runs four warps per block and first puts
// every row it will read in flight with cp.async (one commit group per degree).  Channel
// reductions (the 2l+1 rotation-gradient entries of a row) use a halving exchange.
// ------------------------------------------------------------------------------------------
constexpr int kEdgeThreads = 256;

template <int N>
struct Pow2Ceil {
  static constexpr int v = N <= 1 ? 1 : N <= 2 ? 2 : N <= 4 ? 4 : N <= 8 ? 8 : N <= 16 ? 16 : 32;
};

// Sums each of p[0..N) over the 32 lanes.  Halving exchange: at every step a lane hands half of
// its values to the partner lane and adds the partner's other half to its own, so the step
// costs half as many shuffles as the one before (about Pow2Ceil<N> shuffles in all, against
// 5 N for one butterfly per value).  Afterwards the lane holds the total of element `idx`;
// lanes that differ only in their low log2(32 / Pow2Ceil<N>) bits hold the same element.
// The summation tree is fixed.
template <int N>
__device__ __forceinline__ float warp_sum_scatter(const float (&p)[N], int lane, int &idx) {
  constexpr int NP = Pow2Ceil<N>::v;
  static_assert(N <= 32, "at most one value per lane");
  float q[NP];
#pragma unroll
  for (int j = 0; j < NP; ++j) q[j] = j < N ? p[j] : 0.f;
  idx = 0;
  int mask = 16;
#pragma unroll
  for (int h = NP / 2; h >= 1; h >>= 1) {
    const bool up = (lane & mask) != 0;
#pragma unroll
    for (int j = 0; j < h; ++j) {
      const float send = up ? q[j] : q[j + h];
      const float keep = up ? q[j + h] : q[j];
      q[j] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
    }
    idx += up ? h : 0;
    mask >>= 1;
  }
  for (; mask >= 1; mask >>= 1) q[0] += __shfl_xor_sync(0xffffffffu, q[0], mask);
  return q[0];
}
// lanes that publish the result of warp_sum_scatter<N>: one per element
template <int N>
__device__ __forceinline__ bool warp_sum_owner(int lane, int idx) {
  return (lane & (32 / Pow2Ceil<N>::v - 1)) == 0 && idx < N;
}

// ---- VJP of rotate_back_scatter, one edge per warp group ----------------------------------
//   t[r]        = sum_j rot[r, j] g[dst, l^2 + j]        (g = grad of node_out)
//   dy[e, r]    = env_e * t[r]                            (written as bf16 planes)
//   grad_env[e] = sum_{r, c} y[e, r, c] t[r, c]
//   grad_rot[e, r, j] = env_e * sum_c y[e, r, c] g[dst, l^2 + j, c]
template <int L, int LMAX>
struct GradOutE {
  static __device__ __forceinline__ void run(const ZpTables &t, const float *g_row, const float *y_e,
                                             const ZpPlanes &dy, int64_t dy_row, const float *rot_s,
                                             float *part_s, float env, float &genv, int c,
                                             bool active, int lane, float inv) {
    GradOutE<L - 1, LMAX>::run(t, g_row, y_e, dy, dy_row, rot_s, part_s, env, genv, c, active, lane,
                               inv);
    constexpr int n = 2 * L + 1;
    const int mm = t.mmax < L ? t.mmax : L;
    float g[n][4];
#pragma unroll
    for (int j = 0; j < n; ++j) {
#pragma unroll
      for (int v = 0; v < 4; ++v) g[j][v] = 0.f;
      if (active) vload<4>(g[j], g_row + (size_t)(L * L + j) * t.C);
    }
    // a real loop over the rows |m| <= mmax of this degree (one copy of the body per degree: the
    // unrolled form spent more time waiting for instructions than for data)
    // the NEXT row of y is requested before this row's sums and reductions
    float y_next[4] = {0.f, 0.f, 0.f, 0.f};
    if (active) vload<4>(y_next, y_e + (size_t)t.row_of[L][L - mm] * t.C + c);
#pragma unroll 1
    for (int i = L - mm; i <= L + mm; ++i) {
      {
        const int r = t.row_of[L][i];
        const float *rr = rot_s + t.rot_off[r];
        float yv[4], tv[4] = {0.f, 0.f, 0.f, 0.f}, part[n];
#pragma unroll
        for (int v = 0; v < 4; ++v) yv[v] = y_next[v];
        if (active && i < L + mm) vload<4>(y_next, y_e + (size_t)t.row_of[L][i + 1] * t.C + c);
#pragma unroll
        for (int j = 0; j < n; ++j) {
          const float w = rr[j];
          float s = 0.f;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            tv[v] = fmaf(w, g[j][v], tv[v]);
            s = fmaf(yv[v], g[j][v], s);
          }
          part[j] = s;
        }
        int idx;
        const float tot = warp_sum_scatter<n>(part, lane, idx);
        if (warp_sum_owner<n>(lane, idx)) part_s[t.rot_off[r] + idx] = tot;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          genv = fmaf(yv[v], tv[v], genv);
          tv[v] *= env;
        }
        if (active) zp_store_planes<4>(dy, dy_row + (int64_t)r * t.C + c, tv, inv);
      }
    }
  }
};
template <int LMAX>
struct GradOutE<-1, LMAX> {
  static __device__ __forceinline__ void run(const ZpTables &, const float *, const float *,
                                             const ZpPlanes &, int64_t, const float *, float *,
                                             float, float &, int, bool, int, float) {}
};

// shared memory: rot [epb][nnz_pad] | partial [8 warps][nnz_pad] | genv [8]
template <int LMAX>
__global__ void __launch_bounds__(kEdgeThreads, 3)
rotate_grad_out_kernel(const __grid_constant__ ZpTables t, int64_t E, int W,
                       const float *__restrict__ g_out, const float *__restrict__ y,
                       const float *__restrict__ env, const float *__restrict__ rot,
                       const int32_t *__restrict__ dst, const ZpPlanes dy,
                       float *__restrict__ grad_env, float *__restrict__ grad_rot) {
  extern __shared__ float smem[];
  const int epb = 8 / W;
  float *rot_s = smem;
  float *part_all = smem + epb * t.nnz_pad;
  float *genv_s = part_all + 8 * t.nnz_pad;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int slot = warp / W, wsub = warp % W;
  const int64_t e0 = (int64_t)blockIdx.x * epb;
  const int n_e = (int)min((int64_t)epb, E - e0);
  for (int i = threadIdx.x; i < n_e * t.nnz_pad; i += blockDim.x) rot_s[i] = rot[e0 * t.nnz_pad + i];
  __syncthreads();
  const bool edge_ok = slot < n_e;
  const int64_t e = e0 + (edge_ok ? slot : 0);
  const int c = (wsub * 32 + lane) * 4;
  const bool active = edge_ok && c < t.C;
  float genv = 0.f;
  if (edge_ok) {
    const float *g_row = g_out + (size_t)dst[e] * t.K * t.C + c;
    GradOutE<LMAX, LMAX>::run(t, g_row, y + (size_t)e * t.Km * t.C, dy, e * dy.ld,
                              rot_s + slot * t.nnz_pad, part_all + warp * t.nnz_pad, env[e], genv,
                              c, active, lane, zp_inv_scale(dy));
    genv = warp_sum(genv);
    if (lane == 0) genv_s[warp] = genv;
  }
  __syncthreads();
  // fixed-order sum over the W warps of each edge
  for (int i = threadIdx.x; i < n_e * t.nnz_pad; i += blockDim.x) {
    const int s = i / t.nnz_pad, k = i % t.nnz_pad;
    float acc = 0.f;
    if (k < t.nnz)
      for (int w = 0; w < W; ++w) acc += part_all[(s * W + w) * t.nnz_pad + k];
    grad_rot[(e0 + s) * t.nnz_pad + k] = acc * env[e0 + s];
  }
  if (threadIdx.x < n_e) {
    float acc = 0.f;
    for (int w = 0; w < W; ++w) acc += genv_s[threadIdx.x * W + w];
    grad_env[e0 + threadIdx.x] = acc;
  }
}

// ---- VJP of rotate_in, one edge per warp group over the 2C message channels --------------------
//   a[r]   = sum_j rot[r, j] u[l^2 + j]            (recomputed; u = x_src | x_dst half)
//   ga[r]  = da[e, r] * radial
//   grad_radial[e, col] = sum over the +m / -m rows sharing the column of  da[r] * a[r]
//   du[e, half, l^2 + j] = sum_r rot[r, j] ga[r]   (summed per node afterwards)
//   grad_rot[e, r, j] += sum_c2 ga[r, c2] u[l^2 + j, c2]
template <int L, int LMAX>
struct RotInBwdE {
  // stage: this warp's [Km + radial rows][128] buffer, filled by StageInBwd in level order
  static __device__ __forceinline__ void run(const ZpTables &t, const float *xrow,
                                             const float *stage, const float *rad_e,
                                             float *grad_e, const ZpPlanes &gp, int64_t gp_row,
                                             float gp_inv, const float *rot_s, float *part_s,
                                             float *du_row, int c2, bool active, int lane) {
    RotInBwdE<L - 1, LMAX>::run(t, xrow, stage, rad_e, grad_e, gp, gp_row, gp_inv, rot_s, part_s,
                                du_row, c2, active, lane);
    constexpr int n = 2 * L + 1;
    const int C2 = 2 * t.C;
    const int mm = t.mmax < L ? t.mmax : L;
    float u[n][4], du[n][4];
#pragma unroll
    for (int j = 0; j < n; ++j) {
#pragma unroll
      for (int v = 0; v < 4; ++v) { u[j][v] = 0.f; du[j][v] = 0.f; }
      if (active) vload<4>(u[j], xrow + (size_t)(L * L + j) * t.C);
    }
    cp_async_wait<LMAX - L>();             // the rows of levels 0..L have landed
    // a real loop over |m| (one copy of the body per degree keeps the code in the instruction cache)
    // the radial gains of the NEXT |m| are requested before this |m|'s rows are worked on
    float rad_next[4] = {0.f, 0.f, 0.f, 0.f};
    if (active) vload<4>(rad_next, rad_e + t.rad_off[0] + L * C2 + c2);
#pragma unroll 1
    for (int am = 0; am <= mm; ++am) {
      {
        float gr[4] = {0.f, 0.f, 0.f, 0.f}, rad[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) rad[v] = rad_next[v];
        const int col = t.rad_off[am] + (L - am) * C2 + c2;
        if (active && am < mm)
          vload<4>(rad_next, rad_e + t.rad_off[am + 1] + (L - am - 1) * C2 + c2);
#pragma unroll
        for (int sgn = 0; sgn < 2; ++sgn) {
          if (sgn == 1 && am == 0) continue;
          const int i = sgn == 0 ? L + am : L - am;
          const int r = t.row_of[L][i];
          const float *rr = rot_s + t.rot_off[r];
          float a[4] = {0.f, 0.f, 0.f, 0.f}, da[4] = {0.f, 0.f, 0.f, 0.f}, ga[4], part[n];
          if (active) vload<4>(da, stage + (size_t)r * 128 + lane * 4);
#pragma unroll
          for (int j = 0; j < n; ++j)
#pragma unroll
            for (int v = 0; v < 4; ++v) a[v] = fmaf(rr[j], u[j][v], a[v]);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            gr[v] = fmaf(da[v], a[v], gr[v]);
            ga[v] = da[v] * rad[v];
          }
#pragma unroll
          for (int j = 0; j < n; ++j) {
            float s = 0.f;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              du[j][v] = fmaf(rr[j], ga[v], du[j][v]);
              s = fmaf(ga[v], u[j][v], s);
            }
            part[j] = s;
          }
          int idx;
          const float tot = warp_sum_scatter<n>(part, lane, idx);
          if (warp_sum_owner<n>(lane, idx)) part_s[t.rot_off[r] + idx] = tot;
        }
        if (active) {              // fp32 rows, or operand planes for the radial layer's VJP
          if (gp.planes) zp_store_planes<4>(gp, gp_row + col, gr, gp_inv);
          else vstore<4>(grad_e + col, gr);
        }
      }
    }
    if (active && du_row) {              // no du_both: the caller wants no gradient of x_node
#pragma unroll
      for (int j = 0; j < n; ++j) vstore<4>(du_row + (size_t)(L * L + j) * t.C, du[j]);
    }
  }
};
template <int LMAX>
struct RotInBwdE<-1, LMAX> {
  static __device__ __forceinline__ void run(const ZpTables &, const float *, const float *,
                                             const float *, float *, const ZpPlanes &, int64_t,
                                             float, const float *, float *, float *, int, bool,
                                             int) {}
};

// Puts the gradient rows of the edge in flight at once: each lane copies its own four channels of
// the Km rows into the warp's shared buffer with cp.async, one commit group per degree, so
// RotInBwdE waits once per degree instead of once per row (the radial rows are loaded directly).
template <int L, int LMAX>
struct StageInBwd {
  static __device__ __forceinline__ void run(const ZpTables &t, const float *da_e,
                                             const float *rad_e, float *stage, int c2, int lane,
                                             bool active) {
    StageInBwd<L - 1, LMAX>::run(t, da_e, rad_e, stage, c2, lane, active);
    constexpr int n = 2 * L + 1;
    const int C2 = 2 * t.C;
    const int mm = t.mmax < L ? t.mmax : L;
    if (active) {
#pragma unroll
      for (int i = 0; i < n; ++i) {
        const int am = i > L ? i - L : L - i;
        if (am <= mm) {
          const int r = t.row_of[L][i];
          cp_async<16>(stage + (size_t)r * 128 + lane * 4, da_e + (size_t)r * C2 + c2);
        }
      }
    }
    cp_async_commit();
  }
};
template <int LMAX>
struct StageInBwd<-1, LMAX> {
  static __device__ __forceinline__ void run(const ZpTables &, const float *, const float *, float *,
                                             int, int, bool) {}
};

// du_both [E][2][K][C]: half 0 = contribution to the source node, half 1 = to the destination.
// Blocks of `nw` warps, W warps per edge; shared memory: rot [nw / W][nnz_pad] |
// partial [nw][nnz_pad] | stage [nw][Km][128].
template <int LMAX>
__global__ void __launch_bounds__(128, (LMAX <= 4 ? 4 : 3))
rotate_in_bwd_kernel(const __grid_constant__ ZpTables t, int64_t E, int W,
                     const float *__restrict__ da1, const float *__restrict__ radial,
                     const float *__restrict__ x, const int32_t *__restrict__ src,
                     const int32_t *__restrict__ dst, const float *__restrict__ rot,
                     float *__restrict__ grad_radial, const ZpPlanes grad_radial_planes,
                     float *__restrict__ du_both, float *__restrict__ grad_rot) {
  extern __shared__ __align__(16) float smem[];
  const int nw = blockDim.x / 32;
  const int epb = nw / W;
  const int stage_rows = t.Km;
  float *rot_s = smem;
  float *part_all = smem + epb * t.nnz_pad;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  float *stage = part_all + nw * t.nnz_pad + (size_t)warp * stage_rows * 128;
  const int slot = warp / W, wsub = warp % W;
  const int64_t e0 = (int64_t)blockIdx.x * epb;
  const int n_e = (int)min((int64_t)epb, E - e0);
  const bool edge_ok = slot < n_e;
  const int64_t e = e0 + (edge_ok ? slot : 0);
  const int c2 = (wsub * 32 + lane) * 4;
  const bool active = edge_ok && c2 < 2 * t.C;
  StageInBwd<LMAX, LMAX>::run(t, da1 + (size_t)e * t.Km * 2 * t.C, radial + (size_t)e * t.R, stage,
                              c2, lane, active);
  for (int i = threadIdx.x; i < n_e * t.nnz_pad; i += blockDim.x) rot_s[i] = rot[e0 * t.nnz_pad + i];
  __syncthreads();
  if (edge_ok) {
    const int half = c2 >= t.C ? 1 : 0;
    const int c = c2 - half * t.C;
    const int64_t node = half ? dst[e] : src[e];
    const float *xrow = x + (size_t)node * t.K * t.C + c;
    float *du_row = du_both ? du_both + ((size_t)e * 2 + half) * t.K * t.C + c : nullptr;
    RotInBwdE<LMAX, LMAX>::run(t, xrow, stage, radial + (size_t)e * t.R,
                               grad_radial + (size_t)e * t.R, grad_radial_planes,
                               e * grad_radial_planes.ld, zp_inv_scale(grad_radial_planes),
                               rot_s + slot * t.nnz_pad, part_all + warp * t.nnz_pad, du_row, c2,
                               active, lane);
  }
  cp_async_wait<0>();
  __syncthreads();
  for (int i = threadIdx.x; i < n_e * t.nnz_pad; i += blockDim.x) {
    const int s = i / t.nnz_pad, k = i % t.nnz_pad;
    if (k >= t.nnz) continue;
    float acc = 0.f;
    for (int w = 0; w < W; ++w) acc += part_all[(s * W + w) * t.nnz_pad + k];
    grad_rot[(e0 + s) * t.nnz_pad + k] += acc;
  }
}

// grad_x[n] = sum over edges INTO n of du_both[e][1]  +  sum over edges OUT OF n of du_both[e][0],
// both in fixed (sorted) order.
__global__ void __launch_bounds__(128)
node_reduce_kernel(int64_t N, int KC4, const float4 *__restrict__ du_both,
                   const int32_t *__restrict__ row_ptr, const int32_t *__restrict__ perm_src,
                   const int32_t *__restrict__ row_ptr_src, float4 *__restrict__ grad_x) {
  const int64_t n = blockIdx.x;
  if (n >= N) return;
  const int beg = row_ptr[n], end = row_ptr[n + 1];
  const int sbeg = row_ptr_src[n], send = row_ptr_src[n + 1];
  for (int i = threadIdx.x; i < KC4; i += blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int e = beg; e < end; ++e) {
      const float4 v = du_both[((size_t)e * 2 + 1) * KC4 + i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    for (int k = sbeg; k < send; ++k) {
      const float4 v = du_both[((size_t)perm_src[k] * 2) * KC4 + i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    grad_x[(size_t)n * KC4 + i] = acc;
  }
}

// Final sums after the rotate-back epilogue of conv2.  The epilogue leaves, per m' row r, the
// partial sums of a node's edges: head[n] for the run that starts at the node's first edge and
// cont[b] for the run that enters 32-edge block b from the block before.  One block per node adds,
// per output row (l, j), the rows r of that degree in table order and, within a row, head first and
// then the continuation blocks in ascending order: a fixed order, so results repeat bit for bit.
__global__ void __launch_bounds__(128)
node_sum_kernel(const __grid_constant__ ZpTables t, int64_t N, const float *__restrict__ head,
                const float *__restrict__ cont, const int32_t *__restrict__ row_ptr,
                float *__restrict__ node_out) {
  const int64_t n = blockIdx.x;
  const int C4 = t.C / 4;
  const int beg = row_ptr[n], end = row_ptr[n + 1];
  const int b_first = beg >> 5, b_last = end > beg ? (end - 1) >> 5 : b_first;
  const size_t slab = (size_t)t.nnz * t.C;
  const float *hn = head + (size_t)n * slab;
  for (int i = threadIdx.x; i < t.K * C4; i += blockDim.x) {
    const int k = i / C4, c = (i - k * C4) * 4;
    int l = 0;
    while ((l + 1) * (l + 1) <= k) ++l;
    const int j = k - l * l;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (end > beg) {
      const int mm = t.mmax < l ? t.mmax : l;
      for (int q = l - mm; q <= l + mm; ++q) {
        const size_t o = (size_t)(t.rot_off[t.row_of[l][q]] + j) * t.C + c;
        float4 v = *reinterpret_cast<const float4 *>(hn + o);
        for (int b = b_first + 1; b <= b_last; ++b) {
          const float4 w = *reinterpret_cast<const float4 *>(cont + (size_t)b * slab + o);
          v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    *reinterpret_cast<float4 *>(node_out + ((size_t)n * t.K + k) * t.C + c) = acc;
  }
}

}  // namespace

int zp_launch_node_sum(const zp_plan *p, int64_t N, const float *head, const float *cont,
                       const int32_t *row_ptr, float *node_out, cudaStream_t st) {
  if (N == 0) return ZP_OK;
  node_sum_kernel<<<(unsigned)N, 128, 0, st>>>(p->t, N, head, cont, row_ptr, node_out);
  ZP_LAUNCH_CHECK("node_sum_kernel");
  return ZP_OK;
}

int zp_launch_rotate_in(const zp_plan *p, int64_t E, const float *x, const int32_t *src,
                        const int32_t *dst, const float *rot, const float *radial,
                        const ZpPlanes &a1, cudaStream_t st) {
  if (E == 0) return ZP_OK;
  const ZpTables &t = p->t;
  const int Q = t.C / 2;
  if (Q < 1 || Q > kRotInThreads) return ZP_ERR_UNSUPPORTED;
  int epb = kRotInThreads / Q;
  if (epb > kRotInMaxEdges) epb = kRotInMaxEdges;
  const dim3 grid((unsigned)zp_ceil_div(E, epb)), block(epb * Q);
  const size_t smem = (size_t)epb * t.nnz_pad * sizeof(float);
#define CALL(LM) \
  rotate_in_kernel<LM><<<grid, block, smem, st>>>(t, E, epb, x, src, dst, rot, radial, a1)
  ZP_DISPATCH_LMAX(t.lmax, CALL)
#undef CALL
  ZP_LAUNCH_CHECK("rotate_in_kernel");
  return ZP_OK;
}

int zp_launch_rotate_back_scatter(const zp_plan *p, int64_t N, const float *y, const float *env,
                                  const float *rot, const int32_t *row_ptr, float *node_out,
                                  cudaStream_t st) {
  if (N == 0) return ZP_OK;
  const ZpTables &t = p->t;
  const int vec = t.lmax <= 4 ? 4 : 2;     // K x VEC accumulators must fit in registers
  const dim3 grid((unsigned)N, (unsigned)zp_ceil_div(t.C, 32 * vec));
  const size_t rows = std::max<size_t>((size_t)t.K, 2 * (size_t)t.Km);   // partials | two y stages
  const size_t smem = (size_t)kBackWarps * (t.nnz_pad + rows * 32 * vec) * sizeof(float);
#define CALL(LM)                                                                               \
  {                                                                                            \
    auto kern = vec == 4 ? rotate_back_scatter_kernel<LM, 4> : rotate_back_scatter_kernel<LM, 2>; \
    static ZpSmemOptIn opt_in;             /* per instantiation and device */                    \
    if (int rc_ = zp_ensure_smem(kern, smem, opt_in)) return rc_;                              \
    kern<<<grid, 32 * kBackWarps, smem, st>>>(t, N, y, env, rot, row_ptr, node_out);           \
  }
  ZP_DISPATCH_LMAX(t.lmax, CALL)
#undef CALL
  ZP_LAUNCH_CHECK("rotate_back_scatter_kernel");
  return ZP_OK;
}

// warps per edge for `quads` channel quads (1, 2 or 4), or 0 if unsupported
static int warps_per_edge(int quads) {
  const int w = (quads + 31) / 32;
  return w <= 1 ? 1 : w == 2 ? 2 : w <= 4 ? 4 : 0;
}

int zp_launch_rotate_grad_out(const zp_plan *p, int64_t E, const float *g, const float *y,
                              const float *env, const float *rot, const int32_t *dst,
                              const ZpPlanes &dy, float *grad_env, float *grad_rot,
                              cudaStream_t st) {
  if (E == 0) return ZP_OK;
  const ZpTables &t = p->t;
  const int W = warps_per_edge(t.C / 4);
  if (!W) return ZP_ERR_UNSUPPORTED;
  const int epb = 8 / W;
  const dim3 grid((unsigned)zp_ceil_div(E, epb));
  const size_t smem = ((size_t)(epb + 8) * t.nnz_pad + 8) * sizeof(float);
#define CALL(LM)                                                                              \
  rotate_grad_out_kernel<LM><<<grid, kEdgeThreads, smem, st>>>(t, E, W, g, y, env, rot, dst, dy, \
                                                               grad_env, grad_rot)
  ZP_DISPATCH_LMAX(t.lmax, CALL)
#undef CALL
  ZP_LAUNCH_CHECK("rotate_grad_out_kernel");
  return ZP_OK;
}

int zp_launch_rotate_in_bwd(const zp_plan *p, int64_t E, const float *da1, const float *radial,
                            const float *x, const int32_t *src, const int32_t *dst,
                            const float *rot, float *grad_radial, float *du_both, float *grad_rot,
                            cudaStream_t st, const ZpPlanes *grad_radial_planes) {
  ZpPlanes gp{nullptr, 0, 0, 0, 0, nullptr};
  if (grad_radial_planes) gp = *grad_radial_planes;
  if (E == 0) return ZP_OK;
  const ZpTables &t = p->t;
  const int W = warps_per_edge(t.C / 2);
  if (!W) return ZP_ERR_UNSUPPORTED;
  const int nw = 4;                          // warps per block
  const int epb = nw / W;
  const dim3 grid((unsigned)zp_ceil_div(E, epb));
  const size_t stage_rows = (size_t)t.Km;
  const size_t smem = ((size_t)(epb + nw) * t.nnz_pad + (size_t)nw * stage_rows * 128) * sizeof(float);
#define CALL(LM)                                                                               \
  {                                                                                            \
    static ZpSmemOptIn opt_in;               /* per instantiation and device */                  \
    if (int rc_ = zp_ensure_smem(rotate_in_bwd_kernel<LM>, smem, opt_in)) return rc_;          \
    rotate_in_bwd_kernel<LM><<<grid, 32 * nw, smem, st>>>(t, E, W, da1, radial, x, src, dst,   \
                                                          rot, grad_radial, gp, du_both,       \
                                                          grad_rot);                           \
  }
  ZP_DISPATCH_LMAX(t.lmax, CALL)
#undef CALL
  ZP_LAUNCH_CHECK("rotate_in_bwd_kernel");
  return ZP_OK;
}

int zp_launch_node_reduce(const zp_plan *p, int64_t N, const float *du_both,
                          const int32_t *row_ptr, const int32_t *perm_src,
                          const int32_t *row_ptr_src, float *grad_x, cudaStream_t st) {
  if (N == 0) return ZP_OK;
  const int KC4 = p->t.K * p->t.C / 4;
  node_reduce_kernel<<<(unsigned)N, 128, 0, st>>>(N, KC4, (const float4 *)du_both, row_ptr,
                                                  perm_src, row_ptr_src, (float4 *)grad_x);
  ZP_LAUNCH_CHECK("node_reduce_kernel");
  return ZP_OK;
}
