// Shared declarations of the zippel_b200 kernels: layout tables, the plan, launch helpers.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "zippel_b200.h"
#include "zp_planes.cuh"

#define ZP_MAX_L 6                              // largest supported lmax
#define ZP_MAX_KM ((ZP_MAX_L + 1) * (ZP_MAX_L + 1))
#define ZP_MAX_N (2 * ZP_MAX_L + 1)

// Index tables of one (lmax, mmax) layout, passed to kernels by value.
//   m'-major rows: m = 0 for l = 0..lmax, then for |m| = 1..mmax the +m rows (l = m..lmax)
//   followed by the -m rows.  Row r belongs to degree row_l[r]; its 2l+1 rotation entries sit
//   at rot_off[r] in the packed per-edge rotation.
struct ZpTables {
  int lmax, mmax, K, Km, nnz, nnz_pad;
  int C, H;
  int n_gate;                                   // lmax * H
  int w1_cols;                                  // n_gate + Km * H
  int R;                                        // 2C * sum_m km
  int8_t row_l[ZP_MAX_KM];
  int8_t row_m[ZP_MAX_KM];                      // signed m
  int16_t rot_off[ZP_MAX_KM];
  int8_t row_of[ZP_MAX_L + 1][ZP_MAX_N];        // m' row of (l, i = m + l), or -1
  int16_t m_row0[ZP_MAX_L + 1];                 // first m' row of m-block m
  int16_t m_rows[ZP_MAX_L + 1];                 // rows in m-block m (km or 2 km)
  int32_t rad_off[ZP_MAX_L + 1];                // first radial column of m-block m
  int16_t jd_off[ZP_MAX_L + 1];                 // offset of J_l in the packed J array
};

struct ZpTimer;

struct zp_plan {
  ZpTimer *timer;                               // null unless timing is enabled
  zp_config cfg;
  ZpTables t;
  int device;
  double *jd_dev;                               // packed J_l, fp64
  int *status_dev;                              // device status word (0 = ok)
  // per-m GEMM shapes of the folded SO(2) weights
  int n_blocks;                                 // mmax + 1
  int c1_in[ZP_MAX_L + 1], c1_out[ZP_MAX_L + 1], c2_in[ZP_MAX_L + 1], c2_out[ZP_MAX_L + 1];
  int planes;                                   // 16-bit planes per operand: 3 bf16, 2 fp16 or 1 bf16
  int fp16;                                     // planes are fp16 with per-tensor scales
  int64_t c1_woff[ZP_MAX_L + 1], c2_woff[ZP_MAX_L + 1];   // bf16 offsets of the folded planes
  int64_t w_elems;                              // bf16 elements of all folded planes
  int64_t c1_goff[ZP_MAX_L + 1], c2_goff[ZP_MAX_L + 1];   // fp32 offsets of the folded gradients
  int64_t g_elems;                              // fp32 elements of one set of folded gradients
  // Two more streams for launches that do not depend on each other (the per-m products of one
  // convolution, input- and weight-gradient products): run side by side, the last partial wave
  // of one persistent kernel is filled by the next kernel's CTAs.  Forked from and joined back
  // into the caller's stream inside every call; `lane_lock` serialises the enqueueing of calls
  // that share the plan.
  cudaStream_t aux_stream[2];
  cudaEvent_t ev_fork, ev_join[2];
  void *lane_lock;                              // std::mutex
};

// thread-local text of the last CUDA error
void zp_set_cuda_error(cudaError_t e, const char *where);

#define ZP_CUDA(call)                                   \
  do {                                                  \
    cudaError_t e_ = (call);                            \
    if (e_ != cudaSuccess) {                            \
      zp_set_cuda_error(e_, #call);                     \
      return ZP_ERR_CUDA;                               \
    }                                                   \
  } while (0)

// kernel launches issued by this thread (each launch is followed by one ZP_LAUNCH_CHECK)
int64_t &zp_launch_counter();

#define ZP_LAUNCH_CHECK(name)                           \
  do {                                                  \
    ++zp_launch_counter();                              \
    cudaError_t e_ = cudaGetLastError();                \
    if (e_ != cudaSuccess) {                            \
      zp_set_cuda_error(e_, name);                      \
      return ZP_ERR_CUDA;                               \
    }                                                   \
  } while (0)

// A kernel's raised dynamic shared-memory limit is an attribute of the function ON a device, so
// "already raised" is remembered per device ordinal (one ZpSmemOptIn per call site, under a lock:
// plans on several devices and several host threads may share the process).
struct ZpSmemOptIn {
  std::mutex lock;
  size_t allowed[64];
  ZpSmemOptIn() { for (size_t &a : allowed) a = 48 * 1024; }
};
template <typename Kernel>
int zp_ensure_smem(Kernel kernel, size_t bytes, ZpSmemOptIn &state) {
  int dev = 0;
  ZP_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return ZP_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> hold(state.lock);
  if (bytes > state.allowed[dev]) {
    ZP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    state.allowed[dev] = bytes;
  }
  return ZP_OK;
}

static inline int64_t zp_ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline size_t zp_align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

#define ZP_DISPATCH_LMAX(lmax, CALL)          \
  switch (lmax) {                             \
    case 0: { CALL(0); break; }               \
    case 1: { CALL(1); break; }               \
    case 2: { CALL(2); break; }               \
    case 3: { CALL(3); break; }               \
    case 4: { CALL(4); break; }               \
    case 5: { CALL(5); break; }               \
    case 6: { CALL(6); break; }               \
    default: return ZP_ERR_UNSUPPORTED;       \
  }

// ---- kernels (each in its own translation unit) --------------------------------------------
int zp_launch_wigner_fwd(const zp_plan *p, int64_t E, const float *ev, const float *cg,
                         const float *sg, float *rot, cudaStream_t st);
int zp_launch_wigner_bwd(const zp_plan *p, int64_t E, const float *ev, const float *cg,
                         const float *sg, const float *grot, float *gev, cudaStream_t st);

int zp_launch_rotate_in(const zp_plan *p, int64_t E, const float *x, const int32_t *src,
                        const int32_t *dst, const float *rot, const float *radial,
                        const ZpPlanes &a1, cudaStream_t st);
int zp_launch_rotate_back_scatter(const zp_plan *p, int64_t N, const float *y, const float *env,
                                  const float *rot, const int32_t *row_ptr, float *node_out,
                                  cudaStream_t st);
int zp_launch_rotate_grad_out(const zp_plan *p, int64_t E, const float *g, const float *y,
                              const float *env, const float *rot, const int32_t *dst,
                              const ZpPlanes &dy, float *grad_env, float *grad_rot,
                              cudaStream_t st);
// du_both [E][2][K][C]: per-edge contributions to grad_x of the source (0) and destination (1)
// grad_radial goes out as fp32 rows [E, R], or (grad_radial_planes given) as operand planes
int zp_launch_rotate_in_bwd(const zp_plan *p, int64_t E, const float *da1, const float *radial,
                            const float *x, const int32_t *src, const int32_t *dst,
                            const float *rot, float *grad_radial, float *du_both, float *grad_rot,
                            cudaStream_t st, const ZpPlanes *grad_radial_planes = nullptr);
// node_out[n, l^2 + j, c] = sum over the m' rows r of degree l, in table order, of
//   head[n][rot_off[r] + j][c] + the continuation partials of the 32-edge blocks n's edges reach
int zp_launch_node_sum(const zp_plan *p, int64_t N, const float *head, const float *cont,
                       const int32_t *row_ptr, float *node_out, cudaStream_t st);
int zp_launch_node_reduce(const zp_plan *p, int64_t N, const float *du_both,
                          const int32_t *row_ptr, const int32_t *perm_src,
                          const int32_t *row_ptr_src, float *grad_x, cudaStream_t st);

int zp_launch_gate_fwd(const zp_plan *p, int64_t E, const float *h1, const ZpPlanes &ht,
                       float *gate_max, cudaStream_t st);
// gate_max (device scalar, may be null): largest sigmoid'(gate) seen by the forward
int zp_launch_gate_bwd(const zp_plan *p, int64_t E, const float *h1, const float *dht,
                       const ZpPlanes &dh1, cudaStream_t st);

// Work the contraction's epilogue does on a finished 32-row x 32-column block of the result
// while it is still on chip (staged in shared memory), besides or instead of storing it.
//   ZP_EPI_GATE         conv1 of the SO(2) block: column n is hidden channel (n % width) of m' row
//                       row_first + n / width; the block goes through the gate activation
//                       (blocks/eso2_ref.py:295-301: SiLU for row 0, x * sigmoid(gate[l-1]) for the
//                       others, the raw gate scalars read from `gate`) and is written as 16-bit
//                       operand planes for conv2.
//   ZP_EPI_ROTATE_BACK  conv2: column n is channel (n % width) of m' row row_first + n / width;
//                       every edge's value is scaled by its envelope, expanded by the edge's
//                       packed rotation row into the 2l+1 outputs of its degree and summed over
//                       the consecutive edges of a destination node (the edges are destination
//                       sorted).  A node's first run of edges inside a 32-row block goes to
//                       head[node], a run that continues from the previous block to cont[block];
//                       zp_launch_node_sum adds them up in a fixed order.
// Requires K-major operands, one accumulation chunk and no K split.
enum { ZP_EPI_NONE = 0, ZP_EPI_GATE = 1, ZP_EPI_ROTATE_BACK = 2 };
struct ZpEpilogue {
  int mode;
  int store_c;                                  // also store the fp32 result to C
  int width;                                    // channels per m' row (H or C)
  int row_first;                                // m' row of column 0
  int8_t row_l[ZP_MAX_KM];                      // degree of each m' row
  int16_t rot_off[ZP_MAX_KM];                   // offset of the row's entries in a packed rotation
  // gate
  const float *gate;                            // [M, ld_gate] raw gate scalars, block l-1 at column (l-1)*width
  int64_t ld_gate;
  ZpPlanes out;                                 // activated rows: element (e, n) at e*out.ld + n
  float *slope_max;                             // running max of sigmoid'(gate), or null
  // rotate back
  const float *rot, *env;                       // [M, nnz_pad], [M]
  const int32_t *row_ptr;                       // [n_nodes + 1] offsets of the nodes' edges
  const int32_t *block_node;                    // [ceil(M/32)] node of edge 32 b (zp_launch_block_nodes)
  int n_nodes, nnz, nnz_pad;
  float *head, *cont;                           // [n_nodes][nnz][width], [ceil(M/32)][nnz][width]
};

// Tensor-core product over bf16 planes: C[M,N] = sum_pairs A_pa * B_pb^T (+ bias), fp32 out.
// K-major operand: X[p*plane + r*ld + k]; MN-major (x_mn = 1): X[p*plane + k*ld + r].
struct ZpGemmTc {
  int64_t M, N, K;
  int planes;                                   // 1 (bf16) or 3 (fp32 carried as three bf16)
  const void *A; int64_t lda, a_plane; int a_mn;
  const void *B; int64_t ldb, b_plane; int b_mn;
  const float *bias;
  float *C; int64_t ldc;
  int *status;                                  // device word, set on a device-side timeout
  int variant;                                  // tile-shape choice for the 3-plane K-major case
  int ksplit;                                   // requested split of K over CTAs (>= 1)
  int64_t split_stride;                         // elements between the partial outputs of splits
  int kc_elems;                                 // K per TMEM accumulation chunk (0 = 2048)
  int fp16;                                     // planes are fp16 (planes must be 2), else bf16
  const float *scale_a, *scale_b;               // device scalars multiplied into the result
  float *absmax_out;                            // device scalar updated with max |C| (or null)
  const ZpEpilogue *epi;                        // fused epilogue (null = store C)
  int64_t wait_limit_ns;                        // bound of the device-side waits (0 = 2 s)
  int unarmed;                                  // self-test: no operand is ever loaded
};
int zp_launch_gemm_tc(const ZpGemmTc &g, cudaStream_t st);
// block_node[b] = node of the first edge of 32-edge block b, for ZpEpilogue::block_node
int zp_launch_block_nodes(int64_t E, int64_t N, const int32_t *row_ptr, int32_t *block_node,
                          cudaStream_t st);
// whether zp_launch_gemm_tc accepts a fused epilogue for this problem
bool zp_gemm_tc_fusable(const ZpGemmTc &g);
// number of partial outputs the launch above will write for this problem (<= g.ksplit)
int zp_gemm_tc_splits(const ZpGemmTc &g);
// K split (<= max_splits) that fills the device's CTAs (or CTA pairs) most evenly for this problem
int zp_gemm_tc_pick_splits(const ZpGemmTc &g, int max_splits);
// fp32 [rows, cols] (row stride ld_in) -> planes [rows, out.ld], zero padded
int zp_launch_split_planes(int64_t rows, int64_t cols, const float *in, int64_t ld_in,
                           const ZpPlanes &out, cudaStream_t st);
// *out = max |in| (device scalar)
int zp_launch_absmax(int64_t rows, int64_t cols, const float *in, int64_t ld, float *out,
                     cudaStream_t st);
// *out = largest node index in src / dst (device scalar)
int zp_launch_max_index(int64_t E, const int32_t *src, const int32_t *dst, int *out,
                        cudaStream_t st);
// *out = max |in| over rows [first ? *first : 0, max(min_rows, last ? *last + 1 : 0)) of a
// contiguous [*, cols] matrix; first / last are device pointers to row numbers
int zp_launch_absmax_row_range(const float *in, int64_t cols, const int32_t *first,
                               const int32_t *last, int64_t min_rows, float *out,
                               cudaStream_t st);
// *scale = power of two mapping factor*a*b*max(offset_c, c_factor*c*d) to 2^15 (device scalars;
// null = 1; without c the max term is left out)
int zp_launch_scale(float factor, const float *a, const float *b, const float *c, float offset_c,
                    float *scale, cudaStream_t st, const float *d = nullptr, float c_factor = 1.f);

// Folded SO(2) weights as bf16 planes: per block W_fold [P][out][in] followed by its transpose
// [P][in][out], at element offset c{1,2}_woff[m] of `packed`.
// `scales`: per block (conv * (ZP_MAX_L+1) + m) two floats {max |W|, scale}; used for fp16 planes
int zp_launch_fold_weights(const zp_plan *p, const zp_weights *w, void *packed, float *scales,
                           cudaStream_t st);
// partials: per split s the folded fp32 gradients at partials + s*split_stride + c{1,2}_goff[m]
int zp_launch_unfold_wgrad(const zp_plan *p, const float *partials, int64_t split_stride,
                           const int *splits_c1, const int *splits_c2, const zp_weight_grads *gw,
                           cudaStream_t st);
// *ht_scale = fp16-plane scale of conv1's activated output from an a-priori bound:
//   |h1| <= max_m(in_m * max|a1| * max|W1_m|) + max|b1|,  |gate_act(h1)| <= |h1|
// (a1_scale maps the bound of a1 to 2^15; wscales: {max, scale} pairs per weight block)
int zp_launch_conv1_bound(const zp_plan *p, const float *a1_scale, const float *wscales,
                          const float *bias, float *ht_scale, cudaStream_t st);
// VJP of y = x W^T + b with all operands as planes; `partials`: max_splits * N * K floats,
// `colsum_scratch`: ceil(M / 128) * N floats (only when db is wanted)
int zp_linear_backward_planes(const zp_plan *plan, int64_t M, int64_t K, int64_t N,
                              const ZpPlanes &x, const ZpPlanes &w, const ZpPlanes &dy, float *dx,
                              float *dw, float *db, float *partials, int max_splits,
                              float *colsum_scratch, cudaStream_t st);
int zp_launch_colsum(int64_t rows, int64_t cols, const ZpPlanes &a, float *out, float *scratch,
                     cudaStream_t st);
