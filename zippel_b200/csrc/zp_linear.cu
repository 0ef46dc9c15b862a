// A dense layer  y = x W^T + b  and its VJP on the tensor-core contraction engine, with the
// plan's operand format (fp32-accurate or bf16).  Used for the widest layer of the radial MLP
// (edge_channels -> R, the reference's rad_func[6], blocks/eso2_ref.py:169-182), which as an fp32
// library GEMM costs more than the whole SO(2) forward.
//
// No transposed copies are made: W [N, K] as stored is the K-major B operand of the forward, the
// MN-major B operand of the input gradient (contraction over N), and x / dy as stored are the
// MN-major operands of the weight gradient (contraction over the M rows).
#include "zp_common.cuh"

namespace {

struct LinWork {
  float *scales;          // {max x, s_x, max w, s_w, max dy, s_dy}
  ZpPlanes x, w, dy;
  float *partials;        // weight-gradient partial sums [splits][N*K]
  float *colsum;          // bias-gradient partials
  size_t bytes;
};

constexpr int kLinSplits = 8;

LinWork carve_lin(const zp_plan *p, int64_t M, int64_t K, int64_t N, void *base) {
  LinWork w;
  size_t off = 0;
  auto take = [&](size_t nbytes) {
    char *ptr = base ? static_cast<char *>(base) + off : nullptr;
    off += zp_align_up(nbytes, 256);
    return ptr;
  };
  auto planes = [&](int64_t rows, int64_t cols, float *scale) {
    ZpPlanes pl;
    pl.ld = (cols + 7) / 8 * 8;
    pl.planes = p->planes;
    pl.fp16 = p->fp16;
    pl.scale = p->fp16 ? scale : nullptr;
    pl.plane_stride = (int64_t)zp_align_up((size_t)rows * pl.ld, 128);
    pl.base = take((size_t)pl.planes * pl.plane_stride * 2);
    return pl;
  };
  w.scales = reinterpret_cast<float *>(take(8 * sizeof(float)));
  w.x = planes(M, K, w.scales + 1);
  w.w = planes(N, K, w.scales + 3);
  w.dy = planes(M, N, w.scales + 5);
  w.partials = reinterpret_cast<float *>(take(sizeof(float) * kLinSplits * N * K));
  w.colsum = reinterpret_cast<float *>(take(sizeof(float) * (size_t)zp_ceil_div(M > 0 ? M : 1, 128) * N));
  w.bytes = off;
  return w;
}

__global__ void sum_partials_kernel(int64_t n, int splits, const float *__restrict__ part,
                                    float *__restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += part[(size_t)k * n + i];
  out[i] = s;
}

int split_scaled(const zp_plan *p, int64_t rows, int64_t cols, const float *in, const ZpPlanes &pl,
                 float *max_slot, cudaStream_t st) {
  int rc;
  if (p->fp16) {
    if ((rc = zp_launch_absmax(rows, cols, in, cols, max_slot, st))) return rc;
    if ((rc = zp_launch_scale(1.f, max_slot, nullptr, nullptr, 0.f, max_slot + 1, st))) return rc;
  }
  return zp_launch_split_planes(rows, cols, in, cols, pl, st);
}

}  // namespace

// The three products of a dense layer's VJP with every operand already in plane form.
//   dx[M, K] = dy[M, N] W[N, K]        (contraction over N: W as stored is the MN-major operand)
//   dw[N, K] = dy^T x                  (contraction over the M rows, both operands MN-major,
//                                       split over CTAs into `partials`, summed in order)
//   db[N]    = column sums of dy
int zp_linear_backward_planes(const zp_plan *plan, int64_t M, int64_t K, int64_t N,
                              const ZpPlanes &x, const ZpPlanes &w, const ZpPlanes &dy, float *dx,
                              float *dw, float *db, float *partials, int max_splits,
                              float *colsum_scratch, cudaStream_t st) {
  int rc;
  if (dx) {
    const ZpGemmTc g{M, K, N, plan->planes, dy.base, dy.ld, dy.plane_stride, 0,
                     w.base, w.ld, w.plane_stride, 1, nullptr, dx, K, plan->status_dev,
                     0, 1, 0, 0, plan->fp16, dy.scale, w.scale, nullptr};
    if ((rc = zp_launch_gemm_tc(g, st))) return rc;
  }
  if (!dw) return db ? zp_launch_colsum(M, N, dy, db, colsum_scratch, st) : ZP_OK;
  ZpGemmTc g{N, K, M, plan->planes, dy.base, dy.ld, dy.plane_stride, 1,
             x.base, x.ld, x.plane_stride, 1, nullptr, partials, K, plan->status_dev,
             0, 1, N * K, 0, plan->fp16, dy.scale, x.scale, nullptr};
  g.ksplit = zp_gemm_tc_pick_splits(g, max_splits);
  const int splits = zp_gemm_tc_splits(g);
  if ((rc = zp_launch_gemm_tc(g, st))) return rc;
  sum_partials_kernel<<<(unsigned)zp_ceil_div(N * K, 256), 256, 0, st>>>(N * K, splits, partials, dw);
  ZP_LAUNCH_CHECK("sum_partials_kernel");
  if (db) return zp_launch_colsum(M, N, dy, db, colsum_scratch, st);
  return ZP_OK;
}

namespace {

int check(const zp_plan *p, int64_t M, int64_t K, int64_t N) {
  if (!p || M < 0 || K <= 0 || N <= 0) return ZP_ERR_INVALID_ARG;
  if (K % 8 || N % 8) return ZP_ERR_UNSUPPORTED;
  return ZP_OK;
}

}  // namespace

extern "C" {

size_t zp_linear_work_bytes(const zp_plan *plan, int64_t M, int64_t K, int64_t N) {
  if (check(plan, M, K, N)) return 0;
  return carve_lin(plan, M, K, N, nullptr).bytes;
}

int zp_linear_forward(const zp_plan *plan, int64_t M, int64_t K, int64_t N, const float *x,
                      const float *w, const float *bias, float *y, void *work, size_t work_bytes,
                      void *stream) {
  int rc = check(plan, M, K, N);
  if (rc) return rc;
  if (M == 0) return ZP_OK;
  if (!x || !w || !y || !work) return ZP_ERR_INVALID_ARG;
  const LinWork lw = carve_lin(plan, M, K, N, work);
  if (work_bytes < lw.bytes) return ZP_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if ((rc = split_scaled(plan, M, K, x, lw.x, lw.scales + 0, st))) return rc;
  if ((rc = split_scaled(plan, N, K, w, lw.w, lw.scales + 2, st))) return rc;
  const ZpGemmTc g{M, N, K, plan->planes, lw.x.base, lw.x.ld, lw.x.plane_stride, 0,
                   lw.w.base, lw.w.ld, lw.w.plane_stride, 0, bias, y, N, plan->status_dev,
                   0, 1, 0, 0, plan->fp16, lw.x.scale, lw.w.scale, nullptr};
  return zp_launch_gemm_tc(g, st);
}

int zp_linear_backward(const zp_plan *plan, int64_t M, int64_t K, int64_t N, const float *x,
                       const float *w, const float *dy, float *dx, float *dw, float *db,
                       void *work, size_t work_bytes, void *stream) {
  int rc = check(plan, M, K, N);
  if (rc) return rc;
  if (!w || !work || (!dw && !dx) || (M && (!x || !dy))) return ZP_ERR_INVALID_ARG;
  const LinWork lw = carve_lin(plan, M, K, N, work);
  if (work_bytes < lw.bytes) return ZP_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (M == 0) {
    if (dw) ZP_CUDA(cudaMemsetAsync(dw, 0, sizeof(float) * N * K, st));
    if (db) ZP_CUDA(cudaMemsetAsync(db, 0, sizeof(float) * N, st));
    return ZP_OK;
  }
  // dw == NULL: frozen parameters, only the input gradient (and db if given) is formed
  if (dw && (rc = split_scaled(plan, M, K, x, lw.x, lw.scales + 0, st))) return rc;
  if (dx && (rc = split_scaled(plan, N, K, w, lw.w, lw.scales + 2, st))) return rc;
  if ((rc = split_scaled(plan, M, N, dy, lw.dy, lw.scales + 4, st))) return rc;
  return zp_linear_backward_planes(plan, M, K, N, lw.x, lw.w, lw.dy, dx, dw, db, lw.partials,
                                   kLinSplits, lw.colsum, st);
}

int zp_linear_backward_saved(const zp_plan *plan, int64_t M, int64_t K, int64_t N, const float *dy,
                             float *dx, float *dw, float *db, void *work, size_t work_bytes,
                             void *stream) {
  int rc = check(plan, M, K, N);
  if (rc) return rc;
  if (!work || (!dw && !dx) || (M && !dy)) return ZP_ERR_INVALID_ARG;
  const LinWork lw = carve_lin(plan, M, K, N, work);
  if (work_bytes < lw.bytes) return ZP_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (M == 0) {
    if (dw) ZP_CUDA(cudaMemsetAsync(dw, 0, sizeof(float) * N * K, st));
    if (db) ZP_CUDA(cudaMemsetAsync(db, 0, sizeof(float) * N, st));
    return ZP_OK;
  }
  // the planes of x and w and their scales are where zp_linear_forward left them
  if ((rc = split_scaled(plan, M, N, dy, lw.dy, lw.scales + 4, st))) return rc;
  return zp_linear_backward_planes(plan, M, K, N, lw.x, lw.w, lw.dy, dx, dw, db, lw.partials,
                                   kLinSplits, lw.colsum, st);
}

}  // extern "C"
