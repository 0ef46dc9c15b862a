// C ABI of zippel_b200: plan/tables, workspace carving, and the forward / backward drivers
// that sequence the kernels on the caller's stream.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include <cuda_bf16.h>

#include "zp_common.cuh"

// Event pairs recorded around kernel classes while timing is on.
struct ZpTimer {
  struct Span { int cls; cudaEvent_t a, b; int64_t launches; };
  std::vector<Span> spans;      // pool; `used` of them hold live records
  size_t used = 0;
  Span *open(int cls, cudaStream_t st) {
    if (used == spans.size()) {
      Span s{cls, nullptr, nullptr, 0};
      if (cudaEventCreate(&s.a) != cudaSuccess || cudaEventCreate(&s.b) != cudaSuccess) return nullptr;
      spans.push_back(s);
    }
    Span *s = &spans[used++];
    s->cls = cls;
    s->launches = zp_launch_counter();
    cudaEventRecord(s->a, st);
    return s;
  }
  static void close(Span *s, cudaStream_t st) {
    if (!s) return;
    cudaEventRecord(s->b, st);
    s->launches = zp_launch_counter() - s->launches;
  }
};

namespace {

thread_local char g_cuda_error[512] = "";
thread_local int64_t g_launches = 0;

// brackets one expression with a timing span when the plan has a timer
#define ZP_TIMED(cls, expr)                                                      \
  do {                                                                           \
    ZpTimer::Span *span_ = plan->timer ? plan->timer->open(cls, st) : nullptr;   \
    rc = (expr);                                                                 \
    ZpTimer::close(span_, st);                                                   \
    if (rc) return rc;                                                           \
  } while (0)

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Workspace carving; every region starts 256-byte aligned.
//   forward:  rot | a1 planes | h1 | ht planes | y | folded weight planes | head, cont partials
//   backward: dy planes | dht | dh1 planes | da1 | du_src | grot | wgrad partials | scratch
// mode 0 / 1: forward that keeps what a backward reads (1: plus the backward's own regions);
// mode 2: forward alone with fused epilogues -- of h1 only the gate scalars exist, y does not.
struct Workspace {
  float *rot, *h1, *y, *dht, *da1, *du_src, *grot, *wgrad, *scratch, *scales, *head, *cont;
  float *radial, *rad_partials;          // radial layer inside the call: its output, dW partials
  int64_t ld_h1;
  int32_t *block_node;
  ZpPlanes a1, ht, dy, dh1;
  ZpPlanes hr, rw, gr;                   // planes of the layer's input, weight, output gradient
  uint16_t *wfold;
  size_t bytes;
};

// slots of the device-side scale array (fp16-plane precision): raw maxima, derived scales, and
// per weight block {max |W|, scale} from kScWeights on
enum { kScX = 0, kScRad, kScG, kScH1, kScDht, kScA1, kScHt, kScDy, kScDh1, kScGate,
       kScMaxNode /* an int */,
       // the radial layer run inside the call: {max, scale} of its input and of its weight, max
       // of conv1's input gradient, scale of the planes of grad_radial
       kScHr, kScHrScale, kScRw, kScRwScale, kScDa1, kScGrScale,
       kScWeights = 24,
       kScCount = kScWeights + 4 * (ZP_MAX_L + 1) };

constexpr int kMaxWgradSplits = 8;
constexpr int kChunkK = 2048;          // contraction length of one TMEM accumulation chunk

int64_t round8(int64_t x) { return (x + 7) / 8 * 8; }

// The fused epilogues (gate activation in conv1, rotation back + segmented sums in conv2) need
// one- or two-plane operands and contractions that fit one accumulation chunk.  They are opt-in
// (ZP_FUSED_EPILOGUE=1 in the environment): they keep conv1's pre-activation rows and conv2's
// output out of HBM and shrink the inference workspace, but the eight epilogue warps of a CTA
// cannot hide the latency of that extra work, and on B200 the contractions then wait for their
// epilogues (measured: forward 6.6 ms against 3.2 ms with the stand-alone kernels at 60 000 edges).
bool fused_enabled() {
  static int on = -1;
  if (on < 0) {
    const char *e = getenv("ZP_FUSED_EPILOGUE");
    on = (e && e[0] == '1') ? 1 : 0;
  }
  return on == 1;
}
bool can_fuse(const zp_plan *p, int conv) {
  if (!fused_enabled() || p->planes == 3) return false;
  if ((conv ? p->t.C : p->t.H) % 4) return false;
  for (int m = 0; m < p->n_blocks; ++m)
    if ((conv ? p->c2_in[m] : p->c1_in[m]) > kChunkK) return false;
  return true;
}

constexpr int kRadialSplits = 8;         // K splits of the radial layer's weight gradient

// ec > 0: the last layer of the radial MLP (ec -> R) runs inside the call
Workspace carve(const zp_plan *p, int64_t N, int64_t E, int mode, void *base, int ec = 0) {
  const ZpTables &t = p->t;
  Workspace w;
  std::memset(&w, 0, sizeof(w));
  size_t off = 0;
  auto take = [&](size_t nbytes) {
    char *ptr = base ? static_cast<char *>(base) + off : nullptr;
    off += zp_align_up(nbytes, 256);
    return ptr;
  };
  auto takef = [&](size_t elems) { return reinterpret_cast<float *>(take(elems * sizeof(float))); };
  auto takep_rows = [&](int64_t rows, int64_t cols) {
    ZpPlanes pl;
    pl.ld = round8(cols);
    pl.planes = p->planes;
    pl.fp16 = p->fp16;
    pl.scale = nullptr;
    pl.plane_stride = (int64_t)zp_align_up((size_t)rows * pl.ld, 128);
    pl.base = take((size_t)pl.planes * pl.plane_stride * 2);
    return pl;
  };
  auto takep = [&](int64_t cols) { return takep_rows(E, cols); };
  const size_t e = (size_t)E;
  const bool lean = mode == 2 && can_fuse(p, 0) && can_fuse(p, 1);
  w.rot = takef(e * t.nnz_pad);
  w.a1 = takep((int64_t)t.Km * 2 * t.C);
  w.ld_h1 = lean ? t.n_gate : t.w1_cols;
  w.h1 = takef(e * w.ld_h1);
  w.ht = takep((int64_t)t.Km * t.H);
  if (!lean) w.y = takef(e * t.Km * t.C);
  w.wfold = reinterpret_cast<uint16_t *>(take((size_t)p->w_elems * 2));
  w.scales = takef(kScCount);
  if (ec > 0) {
    w.radial = takef(e * t.R);
    w.hr = takep(ec);
    w.rw = takep_rows(t.R, ec);
  }
  // the partial sums of the rotate-back epilogue live only inside the forward: the backward's own
  // regions start at the same offset and reuse the space
  const size_t off_fwd = off;
  if (can_fuse(p, 1)) {
    w.head = takef((size_t)N * t.nnz * t.C);
    w.cont = takef((size_t)zp_ceil_div(E, 32) * t.nnz * t.C);
    w.block_node = reinterpret_cast<int32_t *>(take((size_t)zp_ceil_div(E, 32) * sizeof(int32_t)));
  }
  const size_t end_fwd = off;
  if (mode == 1) {
    off = off_fwd;
    w.dy = takep((int64_t)t.Km * t.C);
    w.dht = takef(e * t.Km * t.H);
    w.dh1 = takep(t.w1_cols);
    w.da1 = takef(e * t.Km * 2 * t.C);
    w.du_src = takef(e * 2 * t.K * t.C);
    w.grot = takef(e * t.nnz_pad);
    w.wgrad = takef((size_t)kMaxWgradSplits * p->g_elems);
    // column-sum partials (bias gradients; the widest user is the radial layer's R columns)
    w.scratch = takef((size_t)zp_ceil_div(E > 0 ? E : 1, 128) *
                      (size_t)(ec > 0 && t.R > t.w1_cols ? t.R : t.w1_cols));
    if (ec > 0) {
      w.gr = takep(t.R);
      w.rad_partials = takef((size_t)kRadialSplits * t.R * ec);
    }
  }
  if (p->fp16 && base) {
    w.a1.scale = w.scales + kScA1;
    w.ht.scale = w.scales + kScHt;
    w.dy.scale = w.scales + kScDy;
    w.dh1.scale = w.scales + kScDh1;
    w.hr.scale = w.scales + kScHrScale;
    w.rw.scale = w.scales + kScRwScale;
    w.gr.scale = w.scales + kScGrScale;
  }
  w.bytes = off > end_fwd ? off : end_fwd;
  return w;
}

// ZP_STREAMS=0 in the environment keeps every launch on the caller's stream.
bool lanes_enabled() {
  static int on = -1;
  if (on < 0) {
    const char *e = getenv("ZP_STREAMS");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

// The caller's stream plus the plan's two side streams for one forward / backward call.
struct Lanes {
  const zp_plan *p;
  cudaStream_t main;
  bool on;
  std::unique_lock<std::mutex> hold;
  Lanes(const zp_plan *plan, cudaStream_t st)
      : p(plan), main(st), on(lanes_enabled() && !plan->timer && plan->aux_stream[0]) {
    if (on) hold = std::unique_lock<std::mutex>(*static_cast<std::mutex *>(plan->lane_lock));
  }
  cudaStream_t pick(int i) const { return (!on || i % 3 == 0) ? main : p->aux_stream[i % 3 - 1]; }
  // side streams continue from what the caller's stream has been given so far
  int fork() {
    if (!on) return ZP_OK;
    ZP_CUDA(cudaEventRecord(p->ev_fork, main));
    for (int i = 0; i < 2; ++i) ZP_CUDA(cudaStreamWaitEvent(p->aux_stream[i], p->ev_fork, 0));
    return ZP_OK;
  }
  // the caller's stream continues after everything the side streams have been given
  int join() {
    if (!on) return ZP_OK;
    for (int i = 0; i < 2; ++i) {
      ZP_CUDA(cudaEventRecord(p->ev_join[i], p->aux_stream[i]));
      ZP_CUDA(cudaStreamWaitEvent(main, p->ev_join[i], 0));
    }
    return ZP_OK;
  }
};

const float *wscale(const zp_plan *p, const Workspace &w, int conv, int m) {
  return p->fp16 ? w.scales + kScWeights + (conv * (ZP_MAX_L + 1) + m) * 2 + 1 : nullptr;
}

// operand views of one m-block inside a plane buffer (column offset `col`)
ZpPlanes sub(const ZpPlanes &p, int64_t col) {
  ZpPlanes q = p;
  q.base = static_cast<uint16_t *>(p.base) + col;
  return q;
}

}  // namespace

int64_t &zp_launch_counter() { return g_launches; }

void zp_set_cuda_error(cudaError_t e, const char *where) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e),
                cudaGetErrorString(e));
}

extern "C" {

const char *zp_status_string(int status) {
  switch (status) {
    case ZP_OK: return "ok";
    case ZP_ERR_INVALID_ARG: return "invalid argument";
    case ZP_ERR_UNSUPPORTED: return "unsupported configuration";
    case ZP_ERR_WORKSPACE: return "workspace too small";
    case ZP_ERR_CUDA: return "CUDA runtime error";
    case ZP_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
    case ZP_ERR_NO_DEVICE_CODE: return "no device code for this GPU (library is built for sm_100a)";
    case ZP_ERR_TOO_LARGE: return "problem exceeds a fixed capacity of this entry point";
    default: return "unknown status";
  }
}

const char *zp_last_cuda_error(void) { return g_cuda_error; }

int zp_device_supported(void) {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
    return 0;
  return major == 10;
}

int zp_plan_create(const zp_config *cfg, const double *jd_host, zp_plan **plan_out) {
  if (!cfg || !jd_host || !plan_out) return ZP_ERR_INVALID_ARG;
  const int L = cfg->lmax, MM = cfg->mmax, C = cfg->sphere_channels, H = cfg->hidden_channels;
  if (L < 0 || L > ZP_MAX_L || MM < 0 || MM > L) return ZP_ERR_UNSUPPORTED;
  if (C <= 0 || H <= 0 || C % 8 || H % 8 || C > 512) return ZP_ERR_UNSUPPORTED;
  if (cfg->precision < 0 || cfg->precision > 2) return ZP_ERR_UNSUPPORTED;
  if (!zp_device_supported()) return ZP_ERR_NO_DEVICE_CODE;

  zp_plan *p = new (std::nothrow) zp_plan;
  if (!p) return ZP_ERR_INVALID_ARG;
  std::memset(p, 0, sizeof(*p));
  p->cfg = *cfg;
  ZpTables &t = p->t;
  t.lmax = L; t.mmax = MM; t.C = C; t.H = H;
  t.K = (L + 1) * (L + 1);
  std::memset(t.row_of, -1, sizeof(t.row_of));
  int r = 0, off = 0, rad = 0, jo = 0;
  for (int m = 0; m <= MM; ++m) {
    t.m_row0[m] = (int16_t)r;
    t.rad_off[m] = rad;
    const int km = L + 1 - m;
    rad += km * 2 * C;
    for (int sgn = 1; sgn >= (m == 0 ? 1 : -1); sgn -= 2) {
      for (int l = m; l <= L; ++l) {
        t.row_l[r] = (int8_t)l;
        t.row_m[r] = (int8_t)(sgn * m);
        t.rot_off[r] = (int16_t)off;
        t.row_of[l][l + sgn * m] = (int8_t)r;
        off += 2 * l + 1;
        ++r;
      }
    }
    t.m_rows[m] = (int16_t)(r - t.m_row0[m]);
  }
  t.Km = r;
  t.nnz = off;
  t.nnz_pad = (off + 3) / 4 * 4;
  t.R = rad;
  t.n_gate = L * H;
  t.w1_cols = t.n_gate + t.Km * H;
  for (int l = 0; l <= L; ++l) {
    t.jd_off[l] = (int16_t)jo;
    jo += (2 * l + 1) * (2 * l + 1);
  }

  p->n_blocks = MM + 1;
  p->planes = cfg->precision == 0 ? 3 : cfg->precision == 2 ? 2 : 1;
  p->fp16 = cfg->precision == 2;
  int64_t woff = 0, goff = 0;
  for (int conv = 0; conv < 2; ++conv) {
    for (int m = 0; m <= MM; ++m) {
      const int km = L + 1 - m;
      const int cin = conv ? H : 2 * C, cout = conv ? C : H;
      const int in = (m == 0 ? 1 : 2) * km * cin;
      const int out = (m == 0 ? 1 : 2) * km * cout + ((m == 0 && conv == 0) ? t.n_gate : 0);
      (conv ? p->c2_in : p->c1_in)[m] = in;
      (conv ? p->c2_out : p->c1_out)[m] = out;
      (conv ? p->c2_woff : p->c1_woff)[m] = woff;
      (conv ? p->c2_goff : p->c1_goff)[m] = goff;
      woff += (int64_t)zp_align_up((size_t)2 * p->planes * in * out, 64);
      goff += (int64_t)zp_align_up((size_t)in * out, 64);
    }
  }
  p->w_elems = woff;
  p->g_elems = goff;

  p->lane_lock = new (std::nothrow) std::mutex;
  if (!p->lane_lock ||
      cudaStreamCreateWithFlags(&p->aux_stream[0], cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&p->aux_stream[1], cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&p->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&p->ev_join[0], cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&p->ev_join[1], cudaEventDisableTiming) != cudaSuccess) {
    zp_set_cuda_error(cudaGetLastError(), "zp_plan_create (streams)");
    zp_plan_destroy(p);
    return ZP_ERR_CUDA;
  }
  if (cudaGetDevice(&p->device) != cudaSuccess ||
      cudaMalloc(&p->status_dev, sizeof(int)) != cudaSuccess ||
      cudaMemset(p->status_dev, 0, sizeof(int)) != cudaSuccess ||
      cudaMalloc(&p->jd_dev, sizeof(double) * jo) != cudaSuccess ||
      cudaMemcpy(p->jd_dev, jd_host, sizeof(double) * jo, cudaMemcpyHostToDevice) !=
          cudaSuccess) {
    zp_set_cuda_error(cudaGetLastError(), "zp_plan_create");
    zp_plan_destroy(p);
    return ZP_ERR_CUDA;
  }
  *plan_out = p;
  return ZP_OK;
}

const char *zp_kernel_class_name(int cls) {
  static const char *names[ZP_N_KERNEL_CLASSES] = {
      "fold_weights", "wigner_fwd", "rotate_in", "gemm_fwd", "gate_fwd", "rotate_back_scatter",
      "rotate_grad_out", "gemm_dgrad", "gemm_wgrad", "bias_grad", "gate_bwd", "rotate_in_bwd",
      "src_reduce", "wigner_bwd"};
  return cls >= 0 && cls < ZP_N_KERNEL_CLASSES ? names[cls] : "?";
}

int zp_timing_enable(zp_plan *plan, int on) {
  if (!plan) return ZP_ERR_INVALID_ARG;
  if (on && !plan->timer) plan->timer = new (std::nothrow) ZpTimer;
  if (!on && plan->timer) {
    for (auto &s : plan->timer->spans) { cudaEventDestroy(s.a); cudaEventDestroy(s.b); }
    delete plan->timer;
    plan->timer = nullptr;
  }
  return ZP_OK;
}

int zp_timing_read(zp_plan *plan, float *ms, int64_t *launches) {
  if (!plan || !plan->timer || !ms || !launches) return ZP_ERR_INVALID_ARG;
  ZpTimer *t = plan->timer;
  for (size_t i = 0; i < t->used; ++i) {
    ZpTimer::Span &s = t->spans[i];
    ZP_CUDA(cudaEventSynchronize(s.b));
    float v = 0.f;
    ZP_CUDA(cudaEventElapsedTime(&v, s.a, s.b));
    ms[s.cls] += v;
    launches[s.cls] += s.launches;
  }
  t->used = 0;
  return ZP_OK;
}

int zp_plan_destroy(zp_plan *plan) {
  if (!plan) return ZP_OK;
  zp_timing_enable(plan, 0);
  if (plan->jd_dev) cudaFree(plan->jd_dev);
  if (plan->status_dev) cudaFree(plan->status_dev);
  for (int i = 0; i < 2; ++i) {
    if (plan->aux_stream[i]) cudaStreamDestroy(plan->aux_stream[i]);
    if (plan->ev_join[i]) cudaEventDestroy(plan->ev_join[i]);
  }
  if (plan->ev_fork) cudaEventDestroy(plan->ev_fork);
  delete static_cast<std::mutex *>(plan->lane_lock);
  delete plan;
  return ZP_OK;
}

int zp_plan_sizes(const zp_plan *plan, zp_sizes *out) {
  if (!plan || !out) return ZP_ERR_INVALID_ARG;
  const ZpTables &t = plan->t;
  out->K = t.K; out->Km = t.Km; out->nnz = t.nnz; out->nnz_pad = t.nnz_pad;
  out->R = t.R; out->n_gate = t.n_gate; out->w1_cols = t.w1_cols;
  return ZP_OK;
}

int zp_plan_tables(const zp_plan *plan, int32_t *row_l, int32_t *row_m, int32_t *rot_off,
                   int32_t *gate_idx) {
  if (!plan) return ZP_ERR_INVALID_ARG;
  const ZpTables &t = plan->t;
  for (int r = 0; r < t.Km; ++r) {
    if (row_l) row_l[r] = t.row_l[r];
    if (row_m) row_m[r] = t.row_m[r];
    if (rot_off) rot_off[r] = t.rot_off[r];
    if (gate_idx) gate_idx[r] = r == 0 ? -1 : t.row_l[r] - 1;
  }
  return ZP_OK;
}

int zp_plan_device_status(zp_plan *plan, int *status_out) {
  if (!plan || !status_out) return ZP_ERR_INVALID_ARG;
  ZP_CUDA(cudaMemcpy(status_out, plan->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status_out) ZP_CUDA(cudaMemset(plan->status_dev, 0, sizeof(int)));
  return ZP_OK;
}

int zp_split_planes(int64_t rows, int64_t cols, const float *in, int64_t ld_in, void *out,
                    int64_t ld_out, int64_t plane_stride, int planes, void *stream) {
  if (rows < 0 || cols < 0 || cols > ld_out || planes < 1 || planes > 3 || !in || !out || ld_out % 2)
    return ZP_ERR_INVALID_ARG;
  const ZpPlanes pl{out, plane_stride, ld_out, planes, planes == 2, nullptr};
  return zp_launch_split_planes(rows, cols, in, ld_in, pl, (cudaStream_t)stream);
}

int zp_gemm_planes(zp_plan *plan, int64_t M, int64_t N, int64_t K, int planes, const void *A,
                   int64_t lda, int64_t a_plane, int a_mn, const void *B, int64_t ldb,
                   int64_t b_plane, int b_mn, const float *bias, float *C, int64_t ldc,
                   int variant, int ksplit, int64_t split_stride, int kc_elems, int *splits_out,
                   void *stream) {
  if (!plan || !A || !B || !C || M < 0 || N < 0 || K <= 0) return ZP_ERR_INVALID_ARG;
  const int fp16 = planes == 2;
  ZpGemmTc g{M, N, K, planes, A, lda, a_plane, a_mn, B, ldb, b_plane, b_mn, bias, C, ldc,
             plan->status_dev, variant, ksplit, split_stride, kc_elems, fp16, nullptr, nullptr,
             nullptr};
  if (splits_out) *splits_out = zp_gemm_tc_splits(g);
  return zp_launch_gemm_tc(g, (cudaStream_t)stream);
}

int zp_selftest_bounded_wait(zp_plan *plan, void *scratch, size_t scratch_bytes, int64_t limit_ns,
                             void *stream) {
  // a 128 x 32 x 64 one-plane product whose producer never loads: the MMA warp's first wait
  // runs out, raises the CTA's abort flag and the status word, and every warp leaves normally
  constexpr int64_t M = 128, N = 32, K = 64;
  const size_t need = (size_t)(M * K + N * K) * 2 + (size_t)M * N * 4;
  if (!plan || !scratch || limit_ns <= 0 || (reinterpret_cast<uintptr_t>(scratch) & 255))
    return ZP_ERR_INVALID_ARG;
  if (scratch_bytes < need) return ZP_ERR_WORKSPACE;
  char *base = static_cast<char *>(scratch);
  ZP_CUDA(cudaMemsetAsync(base, 0, need, (cudaStream_t)stream));
  ZpGemmTc g{M, N, K, 1, base, K, M * K, 0, base + M * K * 2, K, N * K, 0, nullptr,
             reinterpret_cast<float *>(base + (M * K + N * K) * 2), N, plan->status_dev,
             2 /* one-SM kernel */, 1, 0, 0, 0, nullptr, nullptr, nullptr, nullptr, limit_ns, 1};
  return zp_launch_gemm_tc(g, (cudaStream_t)stream);
}

int zp_wigner_forward(const zp_plan *plan, int64_t n_edges, const float *edge_vec,
                      const float *cos_g, const float *sin_g, float *rot, void *stream) {
  if (!plan || n_edges < 0) return ZP_ERR_INVALID_ARG;
  if (n_edges && (!edge_vec || !cos_g || !sin_g || !rot)) return ZP_ERR_INVALID_ARG;
  return zp_launch_wigner_fwd(plan, n_edges, edge_vec, cos_g, sin_g, rot, (cudaStream_t)stream);
}

int zp_wigner_backward(const zp_plan *plan, int64_t n_edges, const float *edge_vec,
                       const float *cos_g, const float *sin_g, const float *grad_rot,
                       float *grad_edge_vec, void *stream) {
  if (!plan || n_edges < 0) return ZP_ERR_INVALID_ARG;
  if (n_edges && (!edge_vec || !cos_g || !sin_g || !grad_rot || !grad_edge_vec))
    return ZP_ERR_INVALID_ARG;
  return zp_launch_wigner_bwd(plan, n_edges, edge_vec, cos_g, sin_g, grad_rot, grad_edge_vec,
                              (cudaStream_t)stream);
}

size_t zp_workspace_bytes(const zp_plan *plan, int64_t n_nodes, int64_t n_edges,
                          int with_backward) {
  if (!plan || n_nodes < 0 || n_edges < 0 || with_backward < 0 || with_backward > 2) return 0;
  return carve(plan, n_nodes, n_edges, with_backward, nullptr).bytes;
}

static int check_weights(const zp_plan *p, const zp_weights *w) {
  if (!w || !w->c1_w0 || !w->c1_b0 || !w->c2_w0 || !w->c2_b0) return ZP_ERR_INVALID_ARG;
  if (p->n_blocks > 1 && (!w->c1_wm || !w->c2_wm)) return ZP_ERR_INVALID_ARG;
  for (int m = 1; m < p->n_blocks; ++m)
    if (!w->c1_wm[m - 1] || !w->c2_wm[m - 1]) return ZP_ERR_INVALID_ARG;
  return ZP_OK;
}

// The last dense layer of the radial MLP (blocks/eso2_ref.py:169-182, rad_func[6]), when the call
// runs it itself: radial[E, R] = h[E, ec] w[R, ec]^T + b.
struct RadialLayer {
  const float *h, *w, *b;
  int ec;
  float *grad_h, *grad_w, *grad_b;       // backward only
};

static int check_radial_layer(const zp_plan *plan, const RadialLayer *rl, int64_t E, bool backward) {
  if (!rl->w || !rl->b || (E && !rl->h)) return ZP_ERR_INVALID_ARG;
  if (rl->ec <= 0 || rl->ec % 8 || plan->t.R % 8) return ZP_ERR_UNSUPPORTED;
  if (!aligned16(rl->h) || !aligned16(rl->w)) return ZP_ERR_INVALID_ARG;
  // the layer's parameter gradients are wanted together or not at all (frozen parameters)
  if (backward && ((!rl->grad_w != !rl->grad_b) || (E && !rl->grad_h))) return ZP_ERR_INVALID_ARG;
  return ZP_OK;
}

// keep != 0: everything a following zp_eso2_backward reads is left in the workspace
static int eso2_forward(const zp_plan *plan, int64_t N, int64_t E, const float *x_node,
                        const float *edge_vec, const float *cos_g, const float *sin_g,
                        const float *radial, const float *env, const int32_t *src,
                        const int32_t *dst, const int32_t *row_ptr, const zp_weights *w,
                        float *node_out, void *workspace, size_t workspace_bytes, void *stream,
                        int keep, const RadialLayer *rl = nullptr) {
  if (!plan || N < 0 || E < 0) return ZP_ERR_INVALID_ARG;
  if (N == 0) return E == 0 ? ZP_OK : ZP_ERR_INVALID_ARG;
  if (!x_node || !row_ptr || !node_out || !workspace) return ZP_ERR_INVALID_ARG;
  if (E && (!edge_vec || !cos_g || !sin_g || (!radial && !rl) || !env || !src || !dst))
    return ZP_ERR_INVALID_ARG;
  if (!aligned16(x_node) || !aligned16(node_out) || !aligned16(radial) || !aligned16(workspace))
    return ZP_ERR_INVALID_ARG;
  int rc = check_weights(plan, w);
  if (rc) return rc;
  if (rl && (rc = check_radial_layer(plan, rl, E, false))) return rc;
  const Workspace ws = carve(plan, N, E, keep ? 0 : 2, workspace, rl ? rl->ec : 0);
  if (workspace_bytes < ws.bytes) return ZP_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  Lanes lanes(plan, st);
  const ZpTables &t = plan->t;
  const bool fuse1 = can_fuse(plan, 0), fuse2 = can_fuse(plan, 1);
  const bool lean = !keep && fuse1 && fuse2;          // h1 rows and y are never written

  if (rl && E > 0) {
    // the radial layer: its input and weight as planes, its output into the workspace; the
    // largest output magnitude (which scales the rotated message) falls out of the epilogue
    const int ec = rl->ec;
    if (plan->fp16) {
      ZP_TIMED(ZP_K_FOLD, zp_launch_absmax(E, ec, rl->h, ec, ws.scales + kScHr, st));
      ZP_TIMED(ZP_K_FOLD, zp_launch_scale(1.f, ws.scales + kScHr, nullptr, nullptr, 0.f,
                                          ws.scales + kScHrScale, st));
      ZP_TIMED(ZP_K_FOLD, zp_launch_absmax(t.R, ec, rl->w, ec, ws.scales + kScRw, st));
      ZP_TIMED(ZP_K_FOLD, zp_launch_scale(1.f, ws.scales + kScRw, nullptr, nullptr, 0.f,
                                          ws.scales + kScRwScale, st));
      ZP_CUDA(cudaMemsetAsync(ws.scales + kScRad, 0, sizeof(float), st));
    }
    ZP_TIMED(ZP_K_FOLD, zp_launch_split_planes(E, ec, rl->h, ec, ws.hr, st));
    ZP_TIMED(ZP_K_FOLD, zp_launch_split_planes(t.R, ec, rl->w, ec, ws.rw, st));
    const ZpGemmTc g{E, t.R, ec, plan->planes, ws.hr.base, ws.hr.ld, ws.hr.plane_stride, 0,
                     ws.rw.base, ws.rw.ld, ws.rw.plane_stride, 0, rl->b, ws.radial, t.R,
                     plan->status_dev, 0, 1, 0, 0, plan->fp16, ws.hr.scale, ws.rw.scale,
                     plan->fp16 ? ws.scales + kScRad : nullptr};
    ZP_TIMED(ZP_K_GEMM_FWD, zp_launch_gemm_tc(g, st));
    radial = ws.radial;
  }
  if (plan->fp16) {
    // magnitude bounds -> power-of-two scales, all on the device:  |rot row . x| <= sqrt(2l+1) max|x|
    // over every row the edges can name: a caller that asks for the rows of a node range passes
    // that range's row count as N while its edges gather from the whole array
    int *max_node = reinterpret_cast<int *>(ws.scales + kScMaxNode);
    ZP_TIMED(ZP_K_FOLD, zp_launch_max_index(E, src, dst, max_node, st));
    ZP_TIMED(ZP_K_FOLD, zp_launch_absmax_row_range(x_node, (int64_t)t.K * t.C, nullptr, max_node, N,
                                                   ws.scales + kScX, st));
    if (!rl || E == 0)
      ZP_TIMED(ZP_K_FOLD, zp_launch_absmax(E, t.R, radial, t.R, ws.scales + kScRad, st));
    ZP_TIMED(ZP_K_FOLD, zp_launch_scale(3.7f, ws.scales + kScX, ws.scales + kScRad, nullptr, 0.f,
                                        ws.scales + kScA1, st));
    ZP_CUDA(cudaMemsetAsync(ws.scales + kScH1, 0, sizeof(float), st));
  }
  ZP_TIMED(ZP_K_FOLD, zp_launch_fold_weights(plan, w, ws.wfold, ws.scales + kScWeights, st));
  ZP_TIMED(ZP_K_WIGNER_FWD, zp_launch_wigner_fwd(plan, E, edge_vec, cos_g, sin_g, ws.rot, st));
  ZP_TIMED(ZP_K_ROTATE_IN,
           zp_launch_rotate_in(plan, E, x_node, src, dst, ws.rot, radial, ws.a1, st));
  const int P = plan->planes;
  const int64_t ldy = (int64_t)t.Km * t.C;

  // tables of the fused epilogues
  ZpEpilogue epi;
  std::memset(&epi, 0, sizeof(epi));
  std::memcpy(epi.row_l, t.row_l, sizeof(epi.row_l));
  std::memcpy(epi.rot_off, t.rot_off, sizeof(epi.rot_off));

  // ---- conv1 (+ gate) ----
  if (fuse1 && E > 0) {
    // The gate activation runs in the epilogue of conv1.  Its fp16 planes need their scale before
    // the values exist, so the scale comes from a bound: |gate_act(h1)| <= |h1| <= in * max|a1| *
    // max|W| + max|b| (two planes keep 22 bits of everything within 2^19 of the bound).  The gate
    // scalars (the first n_gate columns of the m = 0 block) are formed first, by a launch of
    // their own; the other launches read them back from h1.
    if (plan->fp16)
      ZP_TIMED(ZP_K_GATE_FWD, zp_launch_conv1_bound(plan, ws.scales + kScA1, ws.scales + kScWeights,
                                                    w->c1_b0, ws.scales + kScHt, st));
    float *slope = plan->fp16 ? ws.scales + kScGate : nullptr;
    if (slope) ZP_CUDA(cudaMemsetAsync(slope, 0, sizeof(float), st));
    epi.mode = ZP_EPI_GATE;
    epi.store_c = lean ? 0 : 1;
    epi.width = t.H;
    epi.gate = ws.h1;
    epi.ld_gate = ws.ld_h1;
    epi.slope_max = slope;
    for (int m = 0; m < plan->n_blocks; ++m) {
      const int in = plan->c1_in[m], out = plan->c1_out[m];
      const ZpPlanes A = sub(ws.a1, (int64_t)t.m_row0[m] * 2 * t.C);
      const int gate_cols = m == 0 ? t.n_gate : 0;
      if (gate_cols) {
        const ZpGemmTc g{E, gate_cols, in, P, A.base, A.ld, A.plane_stride, 0,
                         ws.wfold + plan->c1_woff[m], in, (int64_t)out * in, 0,
                         w->c1_b0, ws.h1, ws.ld_h1, plan->status_dev, 0, 1, 0, 0,
                         plan->fp16, A.scale, wscale(plan, ws, 0, m),
                         plan->fp16 ? ws.scales + kScH1 : nullptr, nullptr};
        ZP_TIMED(ZP_K_GEMM_FWD, zp_launch_gemm_tc(g, st));
      }
      if (m == 0 && (rc = lanes.fork())) return rc;      // the other launches read the gates
      epi.row_first = t.m_row0[m];
      epi.out = sub(ws.ht, (int64_t)t.m_row0[m] * t.H);
      // lean: the fp32 rows are never stored (C is not dereferenced)
      float *Cc = ws.h1 + (lean ? 0 : t.n_gate + (size_t)t.m_row0[m] * t.H);
      const ZpGemmTc g{E, out - gate_cols, in, P, A.base, A.ld, A.plane_stride, 0,
                       ws.wfold + plan->c1_woff[m] + (int64_t)gate_cols * in, in,
                       (int64_t)out * in, 0, m == 0 ? w->c1_b0 + gate_cols : nullptr, Cc,
                       ws.ld_h1, plan->status_dev, 0, 1, 0, 0, plan->fp16, A.scale,
                       wscale(plan, ws, 0, m), plan->fp16 ? ws.scales + kScH1 : nullptr, &epi};
      ZP_TIMED(ZP_K_GEMM_FWD, zp_launch_gemm_tc(g, lanes.pick(m)));
    }
    if ((rc = lanes.join())) return rc;
  } else {
    // the per-m products are independent: side by side on the plan's streams
    if ((rc = lanes.fork())) return rc;
    for (int m = 0; m < plan->n_blocks && E > 0; ++m) {
      const int in = plan->c1_in[m], out = plan->c1_out[m];
      const ZpPlanes A = sub(ws.a1, (int64_t)t.m_row0[m] * 2 * t.C);
      float *Cc = ws.h1 + (m == 0 ? 0 : t.n_gate + (size_t)t.m_row0[m] * t.H);
      const ZpGemmTc g{E, out, in, P, A.base, A.ld, A.plane_stride, 0,
                       ws.wfold + plan->c1_woff[m], in, (int64_t)out * in, 0,
                       m == 0 ? w->c1_b0 : nullptr, Cc, t.w1_cols, plan->status_dev, 0, 1, 0, 0,
                       plan->fp16, A.scale, wscale(plan, ws, 0, m),
                       plan->fp16 ? ws.scales + kScH1 : nullptr, nullptr};
      ZP_TIMED(ZP_K_GEMM_FWD, zp_launch_gemm_tc(g, lanes.pick(m)));
    }
    if ((rc = lanes.join())) return rc;
    if (plan->fp16)      // |gate(h1)| <= |h1|
      ZP_TIMED(ZP_K_GATE_FWD, zp_launch_scale(1.f, ws.scales + kScH1, nullptr, nullptr, 0.f,
                                              ws.scales + kScHt, st));
    ZP_TIMED(ZP_K_GATE_FWD, zp_launch_gate_fwd(plan, E, ws.h1, ws.ht,
                                               plan->fp16 ? ws.scales + kScGate : nullptr, st));
  }

  // ---- conv2 (+ envelope, rotation back, segmented sums) ----
  if (fuse2) {
    epi.mode = ZP_EPI_ROTATE_BACK;
    epi.store_c = lean ? 0 : 1;
    epi.width = t.C;
    epi.rot = ws.rot;
    epi.env = env;
    epi.row_ptr = row_ptr;
    epi.n_nodes = (int)N;
    epi.nnz = t.nnz;
    epi.nnz_pad = t.nnz_pad;
    epi.head = ws.head;
    epi.cont = ws.cont;
    epi.block_node = ws.block_node;
    ZP_TIMED(ZP_K_ROTATE_BACK, zp_launch_block_nodes(E, N, row_ptr, ws.block_node, st));
  }
  if ((rc = lanes.fork())) return rc;
  for (int m = 0; m < plan->n_blocks && E > 0; ++m) {
    const int in = plan->c2_in[m], out = plan->c2_out[m];
    const ZpPlanes A = sub(ws.ht, (int64_t)t.m_row0[m] * t.H);
    float *Cc = lean ? ws.h1 : ws.y + (size_t)t.m_row0[m] * t.C;     // lean: never dereferenced
    epi.row_first = t.m_row0[m];
    const ZpGemmTc g{E, out, in, P, A.base, A.ld, A.plane_stride, 0,
                     ws.wfold + plan->c2_woff[m], in, (int64_t)out * in, 0,
                     m == 0 ? w->c2_b0 : nullptr, Cc, ldy, plan->status_dev, 0, 1, 0, 0,
                     plan->fp16, A.scale, wscale(plan, ws, 1, m), nullptr,
                     fuse2 ? &epi : nullptr};
    ZP_TIMED(ZP_K_GEMM_FWD, zp_launch_gemm_tc(g, lanes.pick(m)));
  }
  if ((rc = lanes.join())) return rc;
  if (fuse2)
    ZP_TIMED(ZP_K_ROTATE_BACK,
             zp_launch_node_sum(plan, N, ws.head, ws.cont, row_ptr, node_out, st));
  else
    ZP_TIMED(ZP_K_ROTATE_BACK,
             zp_launch_rotate_back_scatter(plan, N, ws.y, env, ws.rot, row_ptr, node_out, st));
  return ZP_OK;
}

int zp_eso2_forward(const zp_plan *plan, int64_t N, int64_t E, const float *x_node,
                    const float *edge_vec, const float *cos_g, const float *sin_g,
                    const float *radial, const float *env, const int32_t *src,
                    const int32_t *dst, const int32_t *row_ptr, const zp_weights *w,
                    float *node_out, void *workspace, size_t workspace_bytes, void *stream) {
  return eso2_forward(plan, N, E, x_node, edge_vec, cos_g, sin_g, radial, env, src, dst, row_ptr,
                      w, node_out, workspace, workspace_bytes, stream, 1);
}

int zp_eso2_forward_inference(const zp_plan *plan, int64_t N, int64_t E, const float *x_node,
                              const float *edge_vec, const float *cos_g, const float *sin_g,
                              const float *radial, const float *env, const int32_t *src,
                              const int32_t *dst, const int32_t *row_ptr, const zp_weights *w,
                              float *node_out, void *workspace, size_t workspace_bytes,
                              void *stream) {
  return eso2_forward(plan, N, E, x_node, edge_vec, cos_g, sin_g, radial, env, src, dst, row_ptr,
                      w, node_out, workspace, workspace_bytes, stream, 0);
}

static int eso2_backward(const zp_plan *plan, int64_t N, int64_t E, const float *grad_node_out,
                         const float *x_node, const float *edge_vec, const float *cos_g,
                         const float *sin_g, const float *radial, const float *env,
                         const int32_t *src, const int32_t *dst, const int32_t *row_ptr,
                         const int32_t *perm_src, const int32_t *row_ptr_src, const zp_weights *w,
                         float *grad_x_node, float *grad_edge_vec, float *grad_radial,
                         float *grad_env, const zp_weight_grads *gw, void *workspace,
                         size_t workspace_bytes, void *stream, const RadialLayer *rl) {
  if (!plan || N < 0 || E < 0) return ZP_ERR_INVALID_ARG;
  if (N == 0) return E == 0 ? ZP_OK : ZP_ERR_INVALID_ARG;
  if (!grad_node_out || !x_node || !row_ptr || !row_ptr_src || !workspace)
    return ZP_ERR_INVALID_ARG;
  // gw == NULL: the parameters are frozen (an MD / inference force evaluation): no weight-gradient
  // product, no bias column sum, no unfolding
  const bool want_w = gw != nullptr;
  if (E && (!edge_vec || !cos_g || !sin_g || (!radial && !rl) || !env || !src || !dst || !perm_src ||
            !grad_edge_vec || (!grad_radial && !rl) || !grad_env))
    return ZP_ERR_INVALID_ARG;
  if (want_w) {
    if (!gw->c1_w0 || !gw->c1_b0 || !gw->c2_w0 || !gw->c2_b0) return ZP_ERR_INVALID_ARG;
    for (int m = 1; m < plan->n_blocks; ++m)
      if (!gw->c1_wm || !gw->c2_wm || !gw->c1_wm[m - 1] || !gw->c2_wm[m - 1])
        return ZP_ERR_INVALID_ARG;
  }
  if (!aligned16(grad_node_out) || !aligned16(grad_x_node) || !aligned16(grad_radial) ||
      !aligned16(workspace))   /* a null grad_radial (radial layer inside the call) is aligned */
    return ZP_ERR_INVALID_ARG;
  int rc = check_weights(plan, w);
  if (rc) return rc;
  if (rl && (rc = check_radial_layer(plan, rl, E, true))) return rc;
  // (the node count only sizes regions that live inside the forward)
  const Workspace ws = carve(plan, 0, E, 1, workspace, rl ? rl->ec : 0);
  if (workspace_bytes < ws.bytes) return ZP_ERR_WORKSPACE;
  if (rl) radial = ws.radial;            // left there by the forward
  // grad_x_node == NULL: the embeddings are an input without a gradient (E and dE/dpos of one
  // block): the per-edge contributions are neither written nor summed
  float *du_out = grad_x_node ? ws.du_src : nullptr;
  cudaStream_t st = (cudaStream_t)stream;
  Lanes lanes(plan, st);
  const ZpTables &t = plan->t;
  const int P = plan->planes;
  const int64_t lda = (int64_t)t.Km * 2 * t.C, ldh = (int64_t)t.Km * t.H;
  int splits_c1[ZP_MAX_L + 1], splits_c2[ZP_MAX_L + 1];
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, plan->device);

  if (plan->fp16) {
    // only rows dst[0] .. dst[E-1] (the edges are destination-sorted): the rows the kernels read,
    // and the only ones a caller that holds a node range's rows alone has
    if (E > 0)
      ZP_TIMED(ZP_K_ROTATE_GRAD_OUT,
               zp_launch_absmax_row_range(grad_node_out, (int64_t)t.K * t.C, dst, dst + (E - 1), 0,
                                          ws.scales + kScG, st));
    else
      ZP_CUDA(cudaMemsetAsync(ws.scales + kScG, 0, sizeof(float), st));
    ZP_TIMED(ZP_K_ROTATE_GRAD_OUT, zp_launch_scale(3.7f, ws.scales + kScG, nullptr, nullptr, 0.f,
                                                   ws.scales + kScDy, st));
  }
  ZP_TIMED(ZP_K_ROTATE_GRAD_OUT,
           zp_launch_rotate_grad_out(plan, E, grad_node_out, ws.y, env, ws.rot, dst, ws.dy,
                                     grad_env, ws.grot, st));
  // One conv at a time: input gradient dX = dY W_fold (K-major against the transposed planes),
  // weight gradient dW_fold = dY^T X with both operands MN-major (the contraction runs over
  // edges), bias gradient = column sums of dY.
  for (int conv = 1; conv >= 0; --conv) {
    const ZpPlanes &dYp = conv ? ws.dy : ws.dh1;
    const ZpPlanes &Xp = conv ? ws.ht : ws.a1;
    float *dX = conv ? ws.dht : ws.da1;
    const int64_t ldx = conv ? ldh : lda;
    const int cin = conv ? t.H : 2 * t.C, cout = conv ? t.C : t.H;
    if (conv == 0) {
      if (plan->fp16 && rl) ZP_CUDA(cudaMemsetAsync(ws.scales + kScDa1, 0, sizeof(float), st));
      if (plan->fp16)        // |dh1| <= 1.1 max|dht| max(1, rows * max sigmoid' * max|h1|)
        ZP_TIMED(ZP_K_GATE_BWD,
                 zp_launch_scale(1.1f, ws.scales + kScDht, nullptr, ws.scales + kScGate, 1.f,
                                 ws.scales + kScDh1, st, ws.scales + kScH1,
                                 (float)(2 * t.mmax + 1)));
      ZP_TIMED(ZP_K_GATE_BWD, zp_launch_gate_bwd(plan, E, ws.h1, ws.dht, ws.dh1, st));
    } else if (plan->fp16) {
      ZP_CUDA(cudaMemsetAsync(ws.scales + kScDht, 0, sizeof(float), st));
    }
    // the input- and weight-gradient products of the blocks and the bias column sums only read
    // dY, X and the weights: side by side on the plan's streams
    if ((rc = lanes.fork())) return rc;
    for (int m = 0; m < plan->n_blocks; ++m) {
      const int in = conv ? plan->c2_in[m] : plan->c1_in[m];
      const int out = conv ? plan->c2_out[m] : plan->c1_out[m];
      const int64_t ycol = (conv == 0 && m > 0 ? t.n_gate : 0) + (m == 0 ? 0 : (int64_t)t.m_row0[m] * cout);
      const int64_t xcol = (int64_t)t.m_row0[m] * cin;
      const ZpPlanes dYm = sub(dYp, ycol), Xm = sub(Xp, xcol);
      const uint16_t *Wt = ws.wfold + (conv ? plan->c2_woff[m] : plan->c1_woff[m]) +
                                (int64_t)P * out * in;
      float *G = ws.wgrad + (conv ? plan->c2_goff[m] : plan->c1_goff[m]);
      int &nsplit = (conv ? splits_c2 : splits_c1)[m];
      nsplit = 1;
      if (E == 0) {
        if (want_w)
          ZP_CUDA(cudaMemsetAsync(G, 0, sizeof(float) * (size_t)out * in, lanes.pick(2 * m + 1)));
        continue;
      }
      const ZpGemmTc gd{E, in, out, P, dYm.base, dYm.ld, dYm.plane_stride, 0,
                        Wt, out, (int64_t)out * in, 0, nullptr, dX + xcol, ldx,
                        plan->status_dev, 0, 1, 0, 0, plan->fp16, dYm.scale,
                        wscale(plan, ws, conv, m),
                        // max |dht|; max |da1| when the radial layer's gradient needs it
                        !plan->fp16 ? nullptr : conv ? ws.scales + kScDht
                                                     : rl ? ws.scales + kScDa1 : nullptr};
      ZP_TIMED(ZP_K_GEMM_DGRAD, zp_launch_gemm_tc(gd, lanes.pick(want_w ? 2 * m : m)));
      if (!want_w) continue;
      ZpGemmTc gw_{out, in, E, P, dYm.base, dYm.ld, dYm.plane_stride, 1,
                   Xm.base, Xm.ld, Xm.plane_stride, 1, nullptr, G, in,
                   plan->status_dev, 0, 1, plan->g_elems, 0, plan->fp16, dYm.scale, Xm.scale,
                   nullptr};
      gw_.ksplit = zp_gemm_tc_pick_splits(gw_, kMaxWgradSplits);
      nsplit = zp_gemm_tc_splits(gw_);
      ZP_TIMED(ZP_K_GEMM_WGRAD, zp_launch_gemm_tc(gw_, lanes.pick(2 * m + 1)));
    }
    if (want_w)
      ZP_TIMED(ZP_K_BIAS_GRAD,
               zp_launch_colsum(E, conv ? plan->c2_out[0] : plan->c1_out[0], dYp,
                                conv ? gw->c2_b0 : gw->c1_b0, ws.scratch, lanes.pick(2)));
    if ((rc = lanes.join())) return rc;
  }
  if (rl) {
    // grad_radial leaves the kernel as operand planes for the layer's VJP; their scale comes from
    // |grad_radial| <= 2 max|da1| max|rot . x| <= 2 * 3.7 max|da1| max|x|
    if (plan->fp16)
      ZP_TIMED(ZP_K_ROTATE_IN_BWD, zp_launch_scale(7.4f, ws.scales + kScDa1, ws.scales + kScX, nullptr,
                                                   0.f, ws.scales + kScGrScale, st));
    ZP_TIMED(ZP_K_ROTATE_IN_BWD,
             zp_launch_rotate_in_bwd(plan, E, ws.da1, radial, x_node, src, dst, ws.rot,
                                     nullptr, du_out, ws.grot, st, &ws.gr));
    if (E > 0) {
      ZP_TIMED(ZP_K_GEMM_WGRAD,
               zp_linear_backward_planes(plan, E, rl->ec, t.R, ws.hr, ws.rw, ws.gr, rl->grad_h,
                                         rl->grad_w, rl->grad_b, ws.rad_partials, kRadialSplits,
                                         ws.scratch, st));
    } else if (rl->grad_w) {
      ZP_CUDA(cudaMemsetAsync(rl->grad_w, 0, sizeof(float) * (size_t)t.R * rl->ec, st));
      ZP_CUDA(cudaMemsetAsync(rl->grad_b, 0, sizeof(float) * (size_t)t.R, st));
    }
  } else {
    ZP_TIMED(ZP_K_ROTATE_IN_BWD,
             zp_launch_rotate_in_bwd(plan, E, ws.da1, radial, x_node, src, dst, ws.rot,
                                     grad_radial, du_out, ws.grot, st));
  }
  if (grad_x_node)
    ZP_TIMED(ZP_K_SRC_REDUCE,
             zp_launch_node_reduce(plan, N, ws.du_src, row_ptr, perm_src, row_ptr_src,
                                   grad_x_node, st));
  ZP_TIMED(ZP_K_WIGNER_BWD,
           zp_launch_wigner_bwd(plan, E, edge_vec, cos_g, sin_g, ws.grot, grad_edge_vec, st));
  if (want_w)
    ZP_TIMED(ZP_K_FOLD, zp_launch_unfold_wgrad(plan, ws.wgrad, plan->g_elems, splits_c1, splits_c2,
                                               gw, st));
  return ZP_OK;
}

int zp_eso2_backward(const zp_plan *plan, int64_t N, int64_t E, const float *grad_node_out,
                     const float *x_node, const float *edge_vec, const float *cos_g,
                     const float *sin_g, const float *radial, const float *env,
                     const int32_t *src, const int32_t *dst, const int32_t *row_ptr,
                     const int32_t *perm_src, const int32_t *row_ptr_src, const zp_weights *w,
                     float *grad_x_node, float *grad_edge_vec, float *grad_radial,
                     float *grad_env, const zp_weight_grads *gw, void *workspace,
                     size_t workspace_bytes, void *stream) {
  return eso2_backward(plan, N, E, grad_node_out, x_node, edge_vec, cos_g, sin_g, radial, env, src,
                       dst, row_ptr, perm_src, row_ptr_src, w, grad_x_node, grad_edge_vec,
                       grad_radial, grad_env, gw, workspace, workspace_bytes, stream, nullptr);
}

size_t zp_workspace_bytes_radial(const zp_plan *plan, int64_t n_nodes, int64_t n_edges,
                                 int edge_channels, int with_backward) {
  if (!plan || n_nodes < 0 || n_edges < 0 || with_backward < 0 || with_backward > 2 ||
      edge_channels <= 0 || edge_channels % 8)
    return 0;
  return carve(plan, n_nodes, n_edges, with_backward, nullptr, edge_channels).bytes;
}

int zp_eso2_forward_radial(const zp_plan *plan, int64_t N, int64_t E, const float *x_node,
                           const float *edge_vec, const float *cos_g, const float *sin_g,
                           const float *h_rad, const float *rad_w, const float *rad_b,
                           int edge_channels, const float *env, const int32_t *src,
                           const int32_t *dst, const int32_t *row_ptr, const zp_weights *w,
                           float *node_out, void *workspace, size_t workspace_bytes,
                           int keep_for_backward, void *stream) {
  const RadialLayer rl{h_rad, rad_w, rad_b, edge_channels, nullptr, nullptr, nullptr};
  return eso2_forward(plan, N, E, x_node, edge_vec, cos_g, sin_g, nullptr, env, src, dst, row_ptr,
                      w, node_out, workspace, workspace_bytes, stream, keep_for_backward, &rl);
}

int zp_eso2_backward_radial(const zp_plan *plan, int64_t N, int64_t E, const float *grad_node_out,
                            const float *x_node, const float *edge_vec, const float *cos_g,
                            const float *sin_g, const float *h_rad, const float *rad_w,
                            const float *rad_b, int edge_channels, const float *env,
                            const int32_t *src, const int32_t *dst, const int32_t *row_ptr,
                            const int32_t *perm_src, const int32_t *row_ptr_src,
                            const zp_weights *w, float *grad_x_node, float *grad_edge_vec,
                            float *grad_h_rad, float *grad_rad_w, float *grad_rad_b,
                            float *grad_env, const zp_weight_grads *gw, void *workspace,
                            size_t workspace_bytes, void *stream) {
  const RadialLayer rl{h_rad, rad_w, rad_b, edge_channels, grad_h_rad, grad_rad_w, grad_rad_b};
  return eso2_backward(plan, N, E, grad_node_out, x_node, edge_vec, cos_g, sin_g, nullptr, env, src,
                       dst, row_ptr, perm_src, row_ptr_src, w, grad_x_node, grad_edge_vec, nullptr,
                       grad_env, gw, workspace, workspace_bytes, stream, &rl);
}

}  // extern "C"
