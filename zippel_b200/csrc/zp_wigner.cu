// Per-edge rational Wigner-D rotation and its VJP with respect to the edge vector.
//
// Follows the construction of the reference's blocks/wigner.py:60-160: normalise the edge,
// cos/sin(k beta) from Chebyshev polynomials of y, cos/sin(k alpha) by de Moivre from
// (z, x) / sqrt(x^2 + z^2), then per degree l
//     D_l = Xa(-gamma) J_l Xb(-beta) J_l Xc(-alpha)
// with X(theta) carrying cos on the diagonal and signed sin on the anti-diagonal.  Only the
// rows with |m| <= mmax are formed and they are written straight into the packed m'-major
// layout (the reference's `to_m @ wigner`, blocks/eso2_ref.py:330-331).
//
// One thread per edge, arithmetic in fp64 (a few thousand flops per edge, far below the cost
// of the SO(2) contraction), result rounded once to fp32.  The sparse X factors are applied
// as two-term updates; only the product with J in the middle is dense.
#include "zp_common.cuh"

namespace {

constexpr double kS2Floor = 1e-12;   // blocks/wigner.py:57

template <int LMAX>
struct Frame {
  double v[3];
  double n2_raw, inv_norm, xh, yh, zh, s2_raw, s2, inv_r, r, ca1, sa1;
  double cb[LMAX + 1], sb[LMAX + 1], u[LMAX + 1], ca[LMAX + 1], sa[LMAX + 1];
};

template <int LMAX>
__device__ __forceinline__ void frame_forward(Frame<LMAX> &f, const float *ev) {
  f.v[0] = ev[0]; f.v[1] = ev[1]; f.v[2] = ev[2];
  f.n2_raw = f.v[0] * f.v[0] + f.v[1] * f.v[1] + f.v[2] * f.v[2];
  f.inv_norm = rsqrt(fmax(f.n2_raw, kS2Floor));
  f.xh = f.v[0] * f.inv_norm; f.yh = f.v[1] * f.inv_norm; f.zh = f.v[2] * f.inv_norm;
  f.s2_raw = f.xh * f.xh + f.zh * f.zh;
  f.s2 = fmax(f.s2_raw, kS2Floor);
  f.inv_r = rsqrt(f.s2);
  f.r = f.s2 * f.inv_r;
  f.cb[0] = 1.0; f.u[0] = 1.0; f.sb[0] = 0.0; f.ca[0] = 1.0; f.sa[0] = 0.0;
  f.ca1 = f.zh * f.inv_r; f.sa1 = f.xh * f.inv_r;
  if constexpr (LMAX >= 1) {
    f.cb[1] = f.yh; f.u[1] = 2.0 * f.yh; f.ca[1] = f.ca1; f.sa[1] = f.sa1;
  }
#pragma unroll
  for (int k = 2; k <= LMAX; ++k) {
    f.cb[k] = 2.0 * f.yh * f.cb[k - 1] - f.cb[k - 2];
    f.u[k] = 2.0 * f.yh * f.u[k - 1] - f.u[k - 2];
    f.ca[k] = f.ca1 * f.ca[k - 1] - f.sa1 * f.sa[k - 1];
    f.sa[k] = f.sa1 * f.ca[k - 1] + f.ca1 * f.sa[k - 1];
  }
#pragma unroll
  for (int k = 1; k <= LMAX; ++k) f.sb[k] = f.r * f.u[k - 1];
}

// signed anti-diagonal entry of X(-theta) on row i of the degree-L block (0 on the centre row)
template <int L>
__device__ __forceinline__ double anti(const double *sn, int i) {
  const int f = L - i;
  return f > 0 ? -sn[f] : (f < 0 ? sn[-f] : 0.0);
}

template <int L, int LMAX>
__device__ __forceinline__ void block_forward(const ZpTables &t, const double *__restrict__ J,
                                              const Frame<LMAX> &f, const double *cg,
                                              const double *sg, float *rot_e) {
  constexpr int n = 2 * L + 1;
  const int mm = t.mmax < L ? t.mmax : L;
#pragma unroll 1
  for (int j = 0; j < n; ++j) {
    // column j of  Xb J Xc
    const int dj = j > L ? j - L : L - j;
    const double c1 = f.ca[dj];
    const double s1 = j > L ? -f.sa[dj] : (j < L ? f.sa[dj] : 0.0);   // Xc[n-1-j, j]
    double P[n], Nn[n];
#pragma unroll
    for (int i = 0; i < n; ++i) P[i] = J[i * n + j] * c1 + J[i * n + (n - 1 - j)] * s1;
#pragma unroll
    for (int i = 0; i < n; ++i) {
      const int di = i > L ? i - L : L - i;
      Nn[i] = f.cb[di] * P[i] + anti<L>(f.sb, i) * P[n - 1 - i];
    }
    // rows |m| <= mm of J (Xb J Xc), then the Xa mix of row i with its partner n-1-i
    double M[n];
#pragma unroll
    for (int i = 0; i < n; ++i) {
      M[i] = 0.0;
      const int di = i > L ? i - L : L - i;
      if (di <= mm) {
        double acc = 0.0;
#pragma unroll
        for (int k = 0; k < n; ++k) acc += J[i * n + k] * Nn[k];
        M[i] = acc;
      }
    }
#pragma unroll
    for (int i = 0; i < n; ++i) {
      const int di = i > L ? i - L : L - i;
      if (di <= mm) {
        const double d = cg[di] * M[i] + anti<L>(sg, i) * M[n - 1 - i];
        rot_e[t.rot_off[t.row_of[L][i]] + j] = (float)d;
      }
    }
  }
}

template <int L, int LMAX>
struct ForEachL {
  static __device__ __forceinline__ void fwd(const ZpTables &t, const double *J,
                                             const Frame<LMAX> &f, const double *cg,
                                             const double *sg, float *rot_e) {
    ForEachL<L - 1, LMAX>::fwd(t, J, f, cg, sg, rot_e);
    block_forward<L, LMAX>(t, J + t.jd_off[L], f, cg, sg, rot_e);
  }
  static __device__ __forceinline__ void bwd(const ZpTables &t, const double *J,
                                             const Frame<LMAX> &f, const double *cg,
                                             const double *sg, const float *g_e, double *dcb,
                                             double *dsb, double *dca, double *dsa);
};
template <int LMAX>
struct ForEachL<-1, LMAX> {
  static __device__ __forceinline__ void fwd(const ZpTables &, const double *,
                                             const Frame<LMAX> &, const double *, const double *,
                                             float *) {}
  static __device__ __forceinline__ void bwd(const ZpTables &, const double *,
                                             const Frame<LMAX> &, const double *, const double *,
                                             const float *, double *, double *, double *,
                                             double *) {}
};

// Reverse of block_forward: accumulates the cotangents of cos/sin(k beta), cos/sin(k alpha).
template <int L, int LMAX>
__device__ __forceinline__ void block_backward(const ZpTables &t, const double *__restrict__ J,
                                               const Frame<LMAX> &f, const double *cg,
                                               const double *sg, const float *g_e, double *dcb,
                                               double *dsb, double *dca, double *dsa) {
  constexpr int n = 2 * L + 1;
  const int mm = t.mmax < L ? t.mmax : L;
#pragma unroll 1
  for (int j = 0; j < n; ++j) {
    const int dj = j > L ? j - L : L - j;
    const double c1 = f.ca[dj];
    const double s1 = j > L ? -f.sa[dj] : (j < L ? f.sa[dj] : 0.0);
    double P[n];
#pragma unroll
    for (int i = 0; i < n; ++i) P[i] = J[i * n + j] * c1 + J[i * n + (n - 1 - j)] * s1;
    // G = dL/dD column j (zero outside the kept rows);  dM = Xa^T G
    double G[n], dM[n];
#pragma unroll
    for (int i = 0; i < n; ++i) {
      const int di = i > L ? i - L : L - i;
      G[i] = di <= mm ? (double)g_e[t.rot_off[t.row_of[L][i]] + j] : 0.0;
    }
#pragma unroll
    for (int k = 0; k < n; ++k) {
      const int dk = k > L ? k - L : L - k;
      // Xa[n-1-k, k] is the anti-diagonal entry of row n-1-k
      dM[k] = dk <= mm ? cg[dk] * G[k] + anti<L>(sg, n - 1 - k) * G[n - 1 - k] : 0.0;
    }
    // dN = J^T dM (J symmetric in exact arithmetic; transpose written out regardless)
    double dN[n];
#pragma unroll
    for (int k = 0; k < n; ++k) {
      double acc = 0.0;
#pragma unroll
      for (int i = 0; i < n; ++i) {
        const int di = i > L ? i - L : L - i;
        if (di <= mm) acc += J[i * n + k] * dM[i];
      }
      dN[k] = acc;
    }
    // N = Xb P:  cotangents of the beta harmonics, and dP = Xb^T dN
    double dP[n];
#pragma unroll
    for (int i = 0; i < n; ++i) {
      const int di = i > L ? i - L : L - i;
      dcb[di] += dN[i] * P[i];
      if (i < L) dsb[di] -= dN[i] * P[n - 1 - i];
      if (i > L) dsb[di] += dN[i] * P[n - 1 - i];
      dP[i] = f.cb[di] * dN[i] + anti<L>(f.sb, n - 1 - i) * dN[n - 1 - i];
    }
    // P = J Xc:  column j of Xc holds cos at row j and the signed sin at row n-1-j
    double acc_c = 0.0, acc_s = 0.0;
#pragma unroll
    for (int i = 0; i < n; ++i) {
      acc_c += J[i * n + j] * dP[i];
      acc_s += J[i * n + (n - 1 - j)] * dP[i];
    }
    dca[dj] += acc_c;
    if (j > L) dsa[dj] -= acc_s;
    if (j < L) dsa[dj] += acc_s;
  }
}

template <int L, int LMAX>
__device__ __forceinline__ void ForEachL<L, LMAX>::bwd(const ZpTables &t, const double *J,
                                                       const Frame<LMAX> &f, const double *cg,
                                                       const double *sg, const float *g_e,
                                                       double *dcb, double *dsb, double *dca,
                                                       double *dsa) {
  ForEachL<L - 1, LMAX>::bwd(t, J, f, cg, sg, g_e, dcb, dsb, dca, dsa);
  block_backward<L, LMAX>(t, J + t.jd_off[L], f, cg, sg, g_e, dcb, dsb, dca, dsa);
}

template <int LMAX>
__global__ void __launch_bounds__(128)
wigner_fwd_kernel(const __grid_constant__ ZpTables t, const double *__restrict__ J, int64_t E,
                  const float *__restrict__ ev, const float *__restrict__ cgam,
                  const float *__restrict__ sgam, float *__restrict__ rot) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  Frame<LMAX> f;
  frame_forward<LMAX>(f, ev + 3 * e);
  double cg[LMAX + 1], sg[LMAX + 1];
#pragma unroll
  for (int k = 0; k <= LMAX; ++k) {
    cg[k] = cgam[e * (LMAX + 1) + k];
    sg[k] = sgam[e * (LMAX + 1) + k];
  }
  float *rot_e = rot + e * t.nnz_pad;
  for (int p = t.nnz; p < t.nnz_pad; ++p) rot_e[p] = 0.f;
  ForEachL<LMAX, LMAX>::fwd(t, J, f, cg, sg, rot_e);
}

template <int LMAX>
__global__ void __launch_bounds__(128)
wigner_bwd_kernel(const __grid_constant__ ZpTables t, const double *__restrict__ J, int64_t E,
                  const float *__restrict__ ev, const float *__restrict__ cgam,
                  const float *__restrict__ sgam, const float *__restrict__ grot,
                  float *__restrict__ gev) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  Frame<LMAX> f;
  frame_forward<LMAX>(f, ev + 3 * e);
  double cg[LMAX + 1], sg[LMAX + 1];
  double dcb[LMAX + 1], dsb[LMAX + 1], dca[LMAX + 1], dsa[LMAX + 1], du[LMAX + 1];
#pragma unroll
  for (int k = 0; k <= LMAX; ++k) {
    cg[k] = cgam[e * (LMAX + 1) + k];
    sg[k] = sgam[e * (LMAX + 1) + k];
    dcb[k] = dsb[k] = dca[k] = dsa[k] = du[k] = 0.0;
  }
  ForEachL<LMAX, LMAX>::bwd(t, J, f, cg, sg, grot + e * t.nnz_pad, dcb, dsb, dca, dsa);

  // sin(k beta) = r * U_{k-1}(y)
  double dr = 0.0, dy = 0.0;
#pragma unroll
  for (int k = 1; k <= LMAX; ++k) {
    dr += dsb[k] * f.u[k - 1];
    du[k - 1] += dsb[k] * f.r;
  }
  // Chebyshev recursions, reversed
#pragma unroll
  for (int k = LMAX; k >= 2; --k) {
    dy += 2.0 * (f.cb[k - 1] * dcb[k] + f.u[k - 1] * du[k]);
    dcb[k - 1] += 2.0 * f.yh * dcb[k]; dcb[k - 2] -= dcb[k];
    du[k - 1] += 2.0 * f.yh * du[k];   du[k - 2] -= du[k];
  }
  double dca1 = 0.0, dsa1 = 0.0;
  if constexpr (LMAX >= 1) dy += dcb[1] + 2.0 * du[1];
  // de Moivre recursion, reversed
#pragma unroll
  for (int k = LMAX; k >= 2; --k) {
    dca1 += dca[k] * f.ca[k - 1] + dsa[k] * f.sa[k - 1];
    dsa1 += -dca[k] * f.sa[k - 1] + dsa[k] * f.ca[k - 1];
    dca[k - 1] += dca[k] * f.ca1 + dsa[k] * f.sa1;
    dsa[k - 1] += -dca[k] * f.sa1 + dsa[k] * f.ca1;
  }
  if constexpr (LMAX >= 1) { dca1 += dca[1]; dsa1 += dsa[1]; }

  double dz = dca1 * f.inv_r, dx = dsa1 * f.inv_r;
  const double dinv_r = dca1 * f.zh + dsa1 * f.xh + dr * f.s2;
  double ds2 = dr * f.inv_r - 0.5 * dinv_r * f.inv_r / f.s2;
  if (!(f.s2_raw >= kS2Floor)) ds2 = 0.0;             // clamp_min passes no gradient below the floor
  dx += 2.0 * f.xh * ds2;
  dz += 2.0 * f.zh * ds2;
  const double dinv_norm = dx * f.v[0] + dy * f.v[1] + dz * f.v[2];
  double dn2 = -0.5 * dinv_norm * f.inv_norm / fmax(f.n2_raw, kS2Floor);
  if (!(f.n2_raw >= kS2Floor)) dn2 = 0.0;
  gev[3 * e + 0] = (float)(dx * f.inv_norm + 2.0 * f.v[0] * dn2);
  gev[3 * e + 1] = (float)(dy * f.inv_norm + 2.0 * f.v[1] * dn2);
  gev[3 * e + 2] = (float)(dz * f.inv_norm + 2.0 * f.v[2] * dn2);
}

}  // namespace

int zp_launch_wigner_fwd(const zp_plan *p, int64_t E, const float *ev, const float *cg,
                         const float *sg, float *rot, cudaStream_t st) {
  if (E == 0) return ZP_OK;
  const dim3 grid((unsigned)zp_ceil_div(E, 128)), block(128);
#define CALL(LM) wigner_fwd_kernel<LM><<<grid, block, 0, st>>>(p->t, p->jd_dev, E, ev, cg, sg, rot)
  ZP_DISPATCH_LMAX(p->t.lmax, CALL)
#undef CALL
  ZP_LAUNCH_CHECK("wigner_fwd_kernel");
  return ZP_OK;
}

int zp_launch_wigner_bwd(const zp_plan *p, int64_t E, const float *ev, const float *cg,
                         const float *sg, const float *grot, float *gev, cudaStream_t st) {
  if (E == 0) return ZP_OK;
  const dim3 grid((unsigned)zp_ceil_div(E, 128)), block(128);
#define CALL(LM) \
  wigner_bwd_kernel<LM><<<grid, block, 0, st>>>(p->t, p->jd_dev, E, ev, cg, sg, grot, gev)
  ZP_DISPATCH_LMAX(p->t.lmax, CALL)
#undef CALL
  ZP_LAUNCH_CHECK("wigner_bwd_kernel");
  return ZP_OK;
}
