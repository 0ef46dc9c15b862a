// Destination-sorted edge order, CSR offsets and the source-sorted view, built on the device.
//
// The required order is the total order (dst, src, original position); the source view orders
// sorted-edge ids by (src, sorted id).  Both are total orders without ties, so any algorithm
// gives the same arrays bit for bit: bucket the edges by node with atomics (arbitrary order
// inside a bucket), then rank every element inside its bucket by counting the keys below it.
// Buckets are the in-/out-neighbourhoods (tens of edges), so the quadratic rank is cheap.
#include <mutex>

#include "zp_common.cuh"

// Scratch of zp_csr_build_static: one fixed array per GPU that loads the library.  In host code
// this name is only a handle for cudaGetSymbolAddress, never a pointer a kernel can be given.
static __device__ __align__(256) unsigned char g_csr_static_scratch[ZP_CSR_STATIC_BYTES];

namespace {

constexpr int kScanBlock = 1024;

// Node indices come from the caller.  One outside [0, N) is never used as an address: the edge
// is left out, the flag word is raised, and zp_csr_status reports it (the arrays of such a call
// are not a valid sort).
__global__ void count_kernel(int64_t E, int64_t N, const int64_t *__restrict__ key,
                             const int64_t *__restrict__ other, int32_t *counts, int32_t *flag) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= E) return;
  const int64_t k = key[i];
  if ((uint64_t)k >= (uint64_t)N || (uint64_t)other[i] >= (uint64_t)N) {
    *flag = 1;
    return;
  }
  atomicAdd(&counts[k], 1);
}
// keys written by rank_dst_kernel, or the 0 a slot without a valid edge was cleared to: in range
// by construction (the test keeps a broken invariant from becoming a wild access)
__global__ void count32_kernel(int64_t E, int64_t N, const int32_t *__restrict__ key,
                               int32_t *counts) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < E && (uint32_t)key[i] < (uint64_t)N) atomicAdd(&counts[key[i]], 1);
}

// exclusive scan of n ints in three steps: per-block scan, scan of block totals, add back
__global__ void scan_block_kernel(int64_t n, const int32_t *__restrict__ in, int32_t *out,
                                  int32_t *block_sums) {
  __shared__ int32_t s[kScanBlock];
  const int64_t i = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
  s[threadIdx.x] = i < n ? in[i] : 0;
  __syncthreads();
  for (int off = 1; off < kScanBlock; off <<= 1) {
    const int32_t v = threadIdx.x >= off ? s[threadIdx.x - off] : 0;
    __syncthreads();
    s[threadIdx.x] += v;
    __syncthreads();
  }
  if (i < n) out[i] = s[threadIdx.x] - in[i];          // exclusive
  if (threadIdx.x == kScanBlock - 1) block_sums[blockIdx.x] = s[threadIdx.x];
}
// block_sums [nb + 1]: exclusive prefix of the block totals, the grand total in slot nb
__global__ void scan_sums_kernel(int64_t nb, int32_t *block_sums) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int32_t run = 0;
    for (int64_t b = 0; b < nb; ++b) {
      const int32_t v = block_sums[b];
      block_sums[b] = run;
      run += v;
    }
    block_sums[nb] = run;
  }
}
// out[n] = the number of elements COUNTED (edges that were left out for an invalid node index are
// not among them), so that no offset range ever covers a slot nothing was written to
__global__ void scan_add_kernel(int64_t n, int64_t nb, int32_t *out,
                                const int32_t *__restrict__ block_sums) {
  const int64_t i = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
  if (i < n) out[i] += block_sums[blockIdx.x];
  if (i == n) out[n] = block_sums[nb];
}

__global__ void bucket_kernel(int64_t E, int64_t N, const int64_t *__restrict__ key,
                              const int64_t *__restrict__ other,
                              const int32_t *__restrict__ row_ptr, int32_t *cursor,
                              int32_t *tmp) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= E) return;
  const int64_t k = key[i];
  if ((uint64_t)k >= (uint64_t)N || (uint64_t)other[i] >= (uint64_t)N) return;   // flagged above
  tmp[row_ptr[k] + atomicAdd(&cursor[k], 1)] = (int32_t)i;
}
__global__ void bucket32_kernel(int64_t E, int64_t N, const int32_t *__restrict__ key,
                                const int32_t *__restrict__ row_ptr, int32_t *cursor,
                                int32_t *tmp) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= E) return;
  const int32_t k = key[i];
  if ((uint32_t)k >= (uint64_t)N) return;
  tmp[row_ptr[k] + atomicAdd(&cursor[k], 1)] = (int32_t)i;
}

// One warp per destination node: order its edges by (src, original position).
__global__ void rank_dst_kernel(int64_t N, int64_t E, const int64_t *__restrict__ src64,
                                const int32_t *__restrict__ row_ptr,
                                const int32_t *__restrict__ tmp, int32_t *perm,
                                int32_t *src_sorted, int32_t *dst_sorted) {
  const int64_t n = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (n >= N) return;
  const int beg = row_ptr[n], end = row_ptr[n + 1];
  for (int i = beg + lane; i < end; i += 32) {
    // every slot of a bucket was filled by bucket_kernel with an edge id; the range test only
    // keeps a broken invariant from turning into a wild read
    const int32_t id = tmp[i];
    if ((uint32_t)id >= (uint64_t)E) continue;
    const int64_t s = src64[id];
    int rank = 0;
    for (int j = beg; j < end; ++j) {
      const int32_t jd = tmp[j];
      if ((uint32_t)jd >= (uint64_t)E) continue;
      const int64_t sj = src64[jd];
      rank += (sj < s) || (sj == s && jd < id);
    }
    perm[beg + rank] = id;
    src_sorted[beg + rank] = (int32_t)s;
    dst_sorted[beg + rank] = (int32_t)n;
  }
}

// One warp per source node: order the sorted-edge ids of its outgoing edges increasingly.
__global__ void rank_src_kernel(int64_t N, const int32_t *__restrict__ row_ptr_src,
                                const int32_t *__restrict__ tmp, int32_t *perm_src) {
  const int64_t n = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
  const int lane = threadIdx.x % 32;
  if (n >= N) return;
  const int beg = row_ptr_src[n], end = row_ptr_src[n + 1];
  for (int i = beg + lane; i < end; i += 32) {
    const int32_t id = tmp[i];
    int rank = 0;
    for (int j = beg; j < end; ++j) rank += tmp[j] < id;
    perm_src[beg + rank] = id;          // ids are positions 0 .. E-1 written by bucket32_kernel
  }
}

struct CsrWork {
  int32_t *flag, *counts, *cursor, *tmp, *block_sums;
  size_t bytes;
};

CsrWork carve_csr(int64_t E, int64_t N, void *base) {
  CsrWork w;
  size_t off = 0;
  auto take = [&](size_t n) {
    int32_t *p = base ? reinterpret_cast<int32_t *>(static_cast<char *>(base) + off) : nullptr;
    off += zp_align_up(n * sizeof(int32_t), 256);
    return p;
  };
  w.flag = take(1);
  w.counts = take((size_t)N + 1);
  w.cursor = take((size_t)N + 1);
  w.tmp = take((size_t)(E > 0 ? E : 1));
  w.block_sums = take((size_t)zp_ceil_div(N + 1, kScanBlock) + 1);
  w.bytes = off;
  return w;
}

int exclusive_scan(int64_t n, const int32_t *in, int32_t *out, int32_t *block_sums,
                   cudaStream_t st) {
  const int64_t nb = zp_ceil_div(n + 1, kScanBlock);
  scan_block_kernel<<<(unsigned)nb, kScanBlock, 0, st>>>(n, in, out, block_sums);
  ZP_LAUNCH_CHECK("scan_block_kernel");
  scan_sums_kernel<<<1, 32, 0, st>>>(nb, block_sums);
  ZP_LAUNCH_CHECK("scan_sums_kernel");
  scan_add_kernel<<<(unsigned)nb, kScanBlock, 0, st>>>(n, nb, out, block_sums);
  ZP_LAUNCH_CHECK("scan_add_kernel");
  return ZP_OK;
}

}  // namespace

extern "C" {

size_t zp_csr_work_bytes(int64_t n_edges, int64_t n_nodes) {
  if (n_edges < 0 || n_nodes < 0) return 0;
  return carve_csr(n_edges, n_nodes, nullptr).bytes;
}

int zp_csr_build(const int64_t *edge_index, int64_t E, int64_t N, int32_t *perm,
                 int32_t *src_sorted, int32_t *dst_sorted, int32_t *row_ptr, int32_t *perm_src,
                 int32_t *row_ptr_src, void *work, size_t work_bytes, void *stream) {
  if (E < 0 || N < 0 || E > INT32_MAX || N >= INT32_MAX) return ZP_ERR_INVALID_ARG;
  if (!row_ptr || !row_ptr_src || !work) return ZP_ERR_INVALID_ARG;
  if (E && (!edge_index || !perm || !src_sorted || !dst_sorted || !perm_src))
    return ZP_ERR_INVALID_ARG;
  const CsrWork w = carve_csr(E, N, work);
  if (work_bytes < w.bytes) return ZP_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t *src64 = edge_index, *dst64 = edge_index + E;
  const unsigned eb = (unsigned)zp_ceil_div(E > 0 ? E : 1, 256);
  const unsigned nbw = (unsigned)zp_ceil_div((N > 0 ? N : 1) * 32, 256);
  int rc;

  // destination view
  ZP_CUDA(cudaMemsetAsync(w.flag, 0, sizeof(int32_t), st));
  if (E) {
    // The slots an invalid edge leaves empty (the last ones, past row_ptr[N]) read as edges
    // 0 -> 0 at position 0: a caller that launches per-edge kernels over all E slots without
    // looking at the flag (a recorded graph replay) still indexes inside its arrays.
    ZP_CUDA(cudaMemsetAsync(src_sorted, 0, sizeof(int32_t) * E, st));
    ZP_CUDA(cudaMemsetAsync(dst_sorted, 0, sizeof(int32_t) * E, st));
    ZP_CUDA(cudaMemsetAsync(perm, 0, sizeof(int32_t) * E, st));
    ZP_CUDA(cudaMemsetAsync(perm_src, 0, sizeof(int32_t) * E, st));
  }
  ZP_CUDA(cudaMemsetAsync(w.counts, 0, sizeof(int32_t) * (N + 1), st));
  ZP_CUDA(cudaMemsetAsync(w.cursor, 0, sizeof(int32_t) * (N + 1), st));
  if (E) {
    count_kernel<<<eb, 256, 0, st>>>(E, N, dst64, src64, w.counts, w.flag);
    ZP_LAUNCH_CHECK("count_kernel");
  }
  if ((rc = exclusive_scan(N, w.counts, row_ptr, w.block_sums, st))) return rc;
  if (E) {
    bucket_kernel<<<eb, 256, 0, st>>>(E, N, dst64, src64, row_ptr, w.cursor, w.tmp);
    ZP_LAUNCH_CHECK("bucket_kernel");
    rank_dst_kernel<<<nbw, 256, 0, st>>>(N, E, src64, row_ptr, w.tmp, perm, src_sorted, dst_sorted);
    ZP_LAUNCH_CHECK("rank_dst_kernel");
  }

  // source view over sorted-edge ids
  ZP_CUDA(cudaMemsetAsync(w.counts, 0, sizeof(int32_t) * (N + 1), st));
  ZP_CUDA(cudaMemsetAsync(w.cursor, 0, sizeof(int32_t) * (N + 1), st));
  if (E) {
    count32_kernel<<<eb, 256, 0, st>>>(E, N, src_sorted, w.counts);
    ZP_LAUNCH_CHECK("count32_kernel");
  }
  if ((rc = exclusive_scan(N, w.counts, row_ptr_src, w.block_sums, st))) return rc;
  if (E) {
    bucket32_kernel<<<eb, 256, 0, st>>>(E, N, src_sorted, row_ptr_src, w.cursor, w.tmp);
    ZP_LAUNCH_CHECK("bucket32_kernel");
    rank_src_kernel<<<nbw, 256, 0, st>>>(N, row_ptr_src, w.tmp, perm_src);
    ZP_LAUNCH_CHECK("rank_src_kernel");
  }
  return ZP_OK;
}

int zp_csr_status(const void *work, void *stream, int *status_out) {
  if (!work || !status_out) return ZP_ERR_INVALID_ARG;
  int32_t flag = 0;
  cudaStream_t st = (cudaStream_t)stream;
  ZP_CUDA(cudaMemcpyAsync(&flag, carve_csr(0, 0, const_cast<void *>(work)).flag, sizeof(flag),
                          cudaMemcpyDeviceToHost, st));
  ZP_CUDA(cudaStreamSynchronize(st));
  *status_out = flag ? ZP_ERR_INVALID_ARG : ZP_OK;
  return ZP_OK;
}

// The sort without a caller-provided work buffer and without any allocation: the scratch is the
// file-scope device array above.  Its device address is looked up once per device (first call on
// that device, with that device current) and cached; the sort itself is zp_csr_build unchanged,
// which clears the counters it needs at the start of every call.
static int static_scratch(void **out) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static void *scratch_of_device[kMaxDevices] = {nullptr};
  int dev = -1;
  ZP_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return ZP_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (!scratch_of_device[dev]) {
    void *ptr = nullptr;
    ZP_CUDA(cudaGetSymbolAddress(&ptr, g_csr_static_scratch));
    scratch_of_device[dev] = ptr;
  }
  *out = scratch_of_device[dev];
  return ZP_OK;
}

int zp_csr_build_static(const int64_t *edge_index, int64_t E, int64_t N, int32_t *perm,
                        int32_t *src_sorted, int32_t *dst_sorted, int32_t *row_ptr,
                        int32_t *perm_src, int32_t *row_ptr_src, void *stream) {
  if (E < 0 || N < 0) return ZP_ERR_INVALID_ARG;
  if (E > ZP_CSR_STATIC_MAX_EDGES || N > ZP_CSR_STATIC_MAX_NODES ||
      carve_csr(E, N, nullptr).bytes > (size_t)ZP_CSR_STATIC_BYTES)
    return ZP_ERR_TOO_LARGE;
  void *scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc) return rc;
  return zp_csr_build(edge_index, E, N, perm, src_sorted, dst_sorted, row_ptr, perm_src,
                      row_ptr_src, scratch, (size_t)ZP_CSR_STATIC_BYTES, stream);
}

int zp_csr_static_status(void *stream, int *status_out) {
  void *scratch = nullptr;
  const int rc = static_scratch(&scratch);
  if (rc) return rc;
  return zp_csr_status(scratch, stream, status_out);
}

}  // extern "C"
