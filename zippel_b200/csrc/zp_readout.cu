// The block's energy head and its VJP (reference blocks/eso2_ref.py:351-362):
//
//   inv[n, 0*C + c] = node_out[n, 0, c]                         (l = 0 is already invariant)
//   inv[n, l*C + c] = sum_m node_out[n, l^2 + m, c]^2           (squared norm of each degree)
//   hid = inv W0^T + b0 ;  e_n = b1 + sum_c W1[c] silu(hid[n, c]) ;  E = sum_n e_n
//
// and, given dE:  the gradients of W0, b0, W1, b1 and of node_out -- the upstream gradient of the
// edge convolution's backward in the force pass.  The hidden layer runs on the tensor-core
// contraction engine (zp_linear_forward / zp_linear_backward); everything else is streaming
// kernels.  Every sum over nodes has a fixed order (strided partial sums, then one ordered pass),
// so E and the parameter gradients repeat bit for bit.
#include "zp_common.cuh"
#include "zippel_b200.h"

namespace {

constexpr int kSumBlocks = 64;           // partial sums over nodes: node n goes to block n % 64

__device__ __forceinline__ float sigmoid_fast(float x) { return 1.f / (1.f + __expf(-x)); }

__global__ void __launch_bounds__(128)
node_invariants_kernel(const __grid_constant__ ZpTables t, int64_t N,
                       const float *__restrict__ node_out, float *__restrict__ inv) {
  const int64_t n = blockIdx.x;
  const float *row = node_out + (size_t)n * t.K * t.C;
  float *out = inv + (size_t)n * (t.lmax + 1) * t.C;
  for (int i = threadIdx.x; i < (t.lmax + 1) * t.C; i += blockDim.x) {
    const int l = i / t.C, c = i - l * t.C;
    float s;
    if (l == 0) {
      s = row[c];
    } else {
      s = 0.f;
      for (int k = l * l; k < (l + 1) * (l + 1); ++k) {
        const float v = row[(size_t)k * t.C + c];
        s = fmaf(v, v, s);
      }
    }
    out[i] = s;
  }
}

// grad_node_out from the gradient of the invariants
__global__ void __launch_bounds__(128)
node_invariants_bwd_kernel(const __grid_constant__ ZpTables t, int64_t N,
                           const float *__restrict__ node_out, const float *__restrict__ g_inv,
                           float *__restrict__ grad_node_out) {
  const int64_t n = blockIdx.x;
  const float *row = node_out + (size_t)n * t.K * t.C;
  const float *gi = g_inv + (size_t)n * (t.lmax + 1) * t.C;
  float *out = grad_node_out + (size_t)n * t.K * t.C;
  for (int i = threadIdx.x; i < t.K * t.C; i += blockDim.x) {
    const int k = i / t.C, c = i - k * t.C;
    int l = 0;
    while ((l + 1) * (l + 1) <= k) ++l;
    out[i] = l == 0 ? gi[c] : 2.f * row[i] * gi[l * t.C + c];
  }
}

// one warp per node: e_n = b1 + sum_c W1[c] silu(hid[n, c])
__global__ void __launch_bounds__(256)
head_fwd_kernel(int64_t N, int C, const float *__restrict__ hid, const float *__restrict__ w1,
                const float *__restrict__ b1, float *__restrict__ e_node) {
  const int64_t n = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (n >= N) return;
  float s = 0.f;
  for (int c = lane; c < C; c += 32) {
    const float h = hid[(size_t)n * C + c];
    s = fmaf(w1[c], h * sigmoid_fast(h), s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) e_node[n] = s + b1[0];
}

// out[0] = sum of v[0..n) in a fixed order: thread i adds v[i], v[i + 1024], ...; the 1024
// partial sums are then added pairwise in a fixed tree
__global__ void __launch_bounds__(1024) ordered_sum_kernel(int64_t n, const float *__restrict__ v,
                                                           float *__restrict__ out) {
  __shared__ float part[1024];
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += 1024) s += v[i];
  part[threadIdx.x] = s;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) part[threadIdx.x] += part[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = part[0];
}

// g_hid[n, c] = dE * W1[c] * silu'(hid[n, c]);  block b also sums silu(hid[n, c]) over its nodes
// n = b, b + 64, ... (in that order) into partial[b][c]
__global__ void __launch_bounds__(128)
head_bwd_kernel(int64_t N, int C, const float *__restrict__ hid, const float *__restrict__ w1,
                const float *__restrict__ grad_e, float *__restrict__ g_hid,
                float *__restrict__ partial) {
  const float ge = grad_e[0];
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float w = w1[c];
    float acc = 0.f;
    for (int64_t n = blockIdx.x; n < N; n += kSumBlocks) {
      const float h = hid[(size_t)n * C + c];
      const float s = sigmoid_fast(h);
      acc += h * s;
      g_hid[(size_t)n * C + c] = ge * w * (s + h * s * (1.f - s));
    }
    partial[(size_t)blockIdx.x * C + c] = acc;
  }
}

__global__ void head_param_grad_kernel(int64_t N, int C, const float *__restrict__ partial,
                                       const float *__restrict__ grad_e, float *__restrict__ grad_w1,
                                       float *__restrict__ grad_b1) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const float ge = grad_e[0];
  if (c < C) {
    float s = 0.f;
    for (int b = 0; b < kSumBlocks; ++b) s += partial[(size_t)b * C + c];
    grad_w1[c] = ge * s;
  }
  if (c == 0) grad_b1[0] = ge * (float)N;
}

struct ReadoutWork {
  float *inv, *hid, *e_node, *g_hid, *g_inv, *partial;
  void *linear;
  size_t linear_bytes, bytes;
};

ReadoutWork carve_readout(const zp_plan *p, int64_t N, void *base) {
  ReadoutWork w;
  size_t off = 0;
  auto take = [&](size_t nbytes) {
    char *ptr = base ? static_cast<char *>(base) + off : nullptr;
    off += zp_align_up(nbytes, 256);
    return ptr;
  };
  const size_t n = (size_t)N, C = (size_t)p->t.C, W = (size_t)(p->t.lmax + 1) * C;
  w.inv = reinterpret_cast<float *>(take(n * W * 4));
  w.hid = reinterpret_cast<float *>(take(n * C * 4));
  w.e_node = reinterpret_cast<float *>(take((n ? n : 1) * 4));
  w.g_hid = reinterpret_cast<float *>(take(n * C * 4));
  w.g_inv = reinterpret_cast<float *>(take(n * W * 4));
  w.partial = reinterpret_cast<float *>(take((size_t)kSumBlocks * C * 4));
  w.linear_bytes = zp_linear_work_bytes(p, N, (int64_t)W, (int64_t)C);
  w.linear = take(w.linear_bytes);
  w.bytes = off;
  return w;
}

}  // namespace

extern "C" {

size_t zp_readout_work_bytes(const zp_plan *plan, int64_t n_nodes) {
  if (!plan || n_nodes < 0) return 0;
  return carve_readout(plan, n_nodes, nullptr).bytes;
}

int zp_readout_forward(const zp_plan *plan, int64_t N, const float *node_out, const float *w0,
                       const float *b0, const float *w1, const float *b1, float *energy, void *work,
                       size_t work_bytes, void *stream) {
  if (!plan || N < 0 || !energy || !work || !w0 || !b0 || !w1 || !b1 || (N && !node_out))
    return ZP_ERR_INVALID_ARG;
  const ReadoutWork rw = carve_readout(plan, N, work);
  if (work_bytes < rw.bytes) return ZP_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const ZpTables &t = plan->t;
  if (N == 0) {
    ZP_CUDA(cudaMemsetAsync(energy, 0, sizeof(float), st));
    return ZP_OK;
  }
  node_invariants_kernel<<<(unsigned)N, 128, 0, st>>>(t, N, node_out, rw.inv);
  ZP_LAUNCH_CHECK("node_invariants_kernel");
  int rc = zp_linear_forward(plan, N, (int64_t)(t.lmax + 1) * t.C, t.C, rw.inv, w0, b0, rw.hid,
                             rw.linear, rw.linear_bytes, stream);
  if (rc) return rc;
  head_fwd_kernel<<<(unsigned)zp_ceil_div(N * 32, 256), 256, 0, st>>>(N, t.C, rw.hid, w1, b1, rw.e_node);
  ZP_LAUNCH_CHECK("head_fwd_kernel");
  ordered_sum_kernel<<<1, 1024, 0, st>>>(N, rw.e_node, energy);
  ZP_LAUNCH_CHECK("ordered_sum_kernel");
  return ZP_OK;
}

int zp_readout_backward(const zp_plan *plan, int64_t N, const float *node_out, const float *w0,
                        const float *b0, const float *w1, const float *b1, const float *grad_energy,
                        float *grad_node_out, float *grad_w0, float *grad_b0, float *grad_w1,
                        float *grad_b1, void *work, size_t work_bytes, void *stream) {
  (void)b0; (void)b1;
  if (!plan || N < 0 || !grad_energy || !work || !w0 || !w1 || !grad_w0 || !grad_b0 || !grad_w1 ||
      !grad_b1 || (N && (!node_out || !grad_node_out)))
    return ZP_ERR_INVALID_ARG;
  const ReadoutWork rw = carve_readout(plan, N, work);
  if (work_bytes < rw.bytes) return ZP_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const ZpTables &t = plan->t;
  const int64_t W = (int64_t)(t.lmax + 1) * t.C;
  if (N == 0) {
    ZP_CUDA(cudaMemsetAsync(grad_w0, 0, sizeof(float) * W * t.C, st));
    ZP_CUDA(cudaMemsetAsync(grad_b0, 0, sizeof(float) * t.C, st));
    ZP_CUDA(cudaMemsetAsync(grad_w1, 0, sizeof(float) * t.C, st));
    ZP_CUDA(cudaMemsetAsync(grad_b1, 0, sizeof(float), st));
    return ZP_OK;
  }
  head_bwd_kernel<<<kSumBlocks, 128, 0, st>>>(N, t.C, rw.hid, w1, grad_energy, rw.g_hid, rw.partial);
  ZP_LAUNCH_CHECK("head_bwd_kernel");
  head_param_grad_kernel<<<(unsigned)zp_ceil_div(t.C, 128), 128, 0, st>>>(N, t.C, rw.partial,
                                                                          grad_energy, grad_w1, grad_b1);
  ZP_LAUNCH_CHECK("head_param_grad_kernel");
  // the hidden layer's operand planes are still in the work buffer the forward used
  int rc = zp_linear_backward_saved(plan, N, W, t.C, rw.g_hid, rw.g_inv, grad_w0, grad_b0,
                                    rw.linear, rw.linear_bytes, stream);
  if (rc) return rc;
  node_invariants_bwd_kernel<<<(unsigned)N, 128, 0, st>>>(t, N, node_out, rw.g_inv, grad_node_out);
  ZP_LAUNCH_CHECK("node_invariants_bwd_kernel");
  return ZP_OK;
}

}  // extern "C"
