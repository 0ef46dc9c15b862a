// Periodic neighbour list with the per-destination cap, built on the device.
//
// The graph front end of the block: all directed edges src -> dst with
//     d2 = |pos[dst] - pos[src] + shift|^2 < cutoff^2,   shift = image * box,
// in a cubic periodic box, without the self pair at zero shift, keeping per destination the
// `max_neighbors` edges of smallest (d2, src, shift_x, shift_y, shift_z).  The reference builds
// its edge lists on the host with an external neighbour-list package and applies no cap
// (fixtures/make_fixtures.py:13-15, 78-100); the cap and the order are defined by this library.
//
// Output order is (dst, src, shift_x, shift_y, shift_z), i.e. already the destination-sorted form,
// with row_ptr.  Everything is a function of exact fp64 arithmetic written without contraction
//     dx = (pos[dst].x - pos[src].x) + shift_x;   d2 = (dx*dx + dy*dy) + dz*dz
// and of total orders without ties, so the arrays are reproducible bit for bit and equal to the
// host statement of the same rule.
//
// Method: uniform cells of edge >= cutoff / w (w = 1 unless the box is smaller than the cutoff);
// one warp per destination walks the (2w+1)^3 cells around it in unwrapped cell coordinates; the
// unwrapped coordinate gives both the wrapped cell and the periodic image, so every
// (source, image) pair is visited exactly once.  Pass 1 counts, a scan gives row_ptr, pass 2
// collects the hits in shared memory, selects by a bitonic sort on (d2, src, image) when the cap
// binds, orders the survivors by (src, image) and writes them.
#include <algorithm>
#include <cmath>

#include "zp_common.cuh"
#include "zippel_b200.h"

namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kHitCap = ZP_NEIGHBORS_MAX_HITS;     // hits held per destination in shared memory
constexpr int kScanBlock = 1024;

struct Grid {
  double box, cell, cutoff2;
  int nc;          // cells per dimension
  int w;           // search half-width in cells
  int reach;       // largest |image| component that can occur
};

struct Hit {
  double d2;
  unsigned long long tie;      // src << 32 | image code (ascending = ascending shift tuple)
};

__device__ __forceinline__ bool hit_less(const Hit &a, const Hit &b) {
  return a.d2 < b.d2 || (a.d2 == b.d2 && a.tie < b.tie);
}

// Positions may lie outside [0, box): o = floor(p / box) is the atom's own image offset and
// p - o * box its wrapped coordinate, used only to pick the cell.  Distances are always taken
// between the positions as given.
__device__ __forceinline__ int own_image(double p, const Grid &g) { return (int)floor(p / g.box); }
__device__ __forceinline__ int cell_coord(double p, const Grid &g) {
  const double pw = p - floor(p / g.box) * g.box;
  int c = (int)floor(pw / g.cell);
  return c < 0 ? 0 : (c >= g.nc ? g.nc - 1 : c);
}

__device__ __forceinline__ int floor_div(int a, int n) {
  int q = a / n;
  if ((a % n) < 0) --q;
  return q;
}

// Image code.  The shift of a hit is (o_src - o_dst - k) * box with k the image found in wrapped
// coordinates (|k| <= reach) and o the atoms' own offsets.  For one (dst, src) pair the offsets
// are fixed, so ordering by -k orders by shift: the code holds -k only, and the writer adds the
// offsets back.
__device__ __forceinline__ unsigned image_code(int nkx, int nky, int nkz, int reach) {
  const unsigned s = 2u * reach + 1u;
  return ((unsigned)(nkx + reach) * s + (unsigned)(nky + reach)) * s + (unsigned)(nkz + reach);
}

__global__ void cell_count_kernel(int64_t N, const double *__restrict__ pos, Grid g,
                                  int32_t *__restrict__ atom_cell, int32_t *cell_count,
                                  int32_t *flags) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N) return;
  const double x = pos[3 * i], y = pos[3 * i + 1], z = pos[3 * i + 2];
  const double far = 1.0e6 * g.box;
  if (!(fabs(x) < far && fabs(y) < far && fabs(z) < far))
    atomicOr(flags, 1);                               // not finite, or absurdly far from the box
  const int c = (cell_coord(x, g) * g.nc + cell_coord(y, g)) * g.nc + cell_coord(z, g);
  atom_cell[i] = c;
  atomicAdd(&cell_count[c], 1);
}

__global__ void cell_fill_kernel(int64_t N, const int32_t *__restrict__ atom_cell,
                                 const int32_t *__restrict__ cell_start, int32_t *cell_cursor,
                                 int32_t *__restrict__ cell_atoms) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N) return;
  const int c = atom_cell[i];
  cell_atoms[cell_start[c] + atomicAdd(&cell_cursor[c], 1)] = (int32_t)i;
}

// exclusive scan of n ints (n + 1 outputs, the last is the total): block scans, serial scan of
// the block totals, add back
__global__ void scan_block_kernel(int64_t n, const int32_t *__restrict__ in, int32_t *out,
                                  int32_t *block_sums) {
  __shared__ int32_t s[kScanBlock];
  const int64_t i = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
  const int32_t mine = i < n ? in[i] : 0;
  s[threadIdx.x] = mine;
  __syncthreads();
  for (int off = 1; off < kScanBlock; off <<= 1) {
    const int32_t v = threadIdx.x >= off ? s[threadIdx.x - off] : 0;
    __syncthreads();
    s[threadIdx.x] += v;
    __syncthreads();
  }
  if (i <= n) out[i] = s[threadIdx.x] - mine;
  if (threadIdx.x == kScanBlock - 1) block_sums[blockIdx.x] = s[threadIdx.x];
}
__global__ void scan_sums_kernel(int64_t nb, int32_t *block_sums) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int32_t run = 0;
    for (int64_t b = 0; b < nb; ++b) {
      const int32_t v = block_sums[b];
      block_sums[b] = run;
      run += v;
    }
  }
}
__global__ void scan_add_kernel(int64_t n, int32_t *out, const int32_t *__restrict__ block_sums) {
  const int64_t i = (int64_t)blockIdx.x * kScanBlock + threadIdx.x;
  if (i <= n) out[i] += block_sums[blockIdx.x];
}

int exclusive_scan(int64_t n, const int32_t *in, int32_t *out, int32_t *block_sums,
                   cudaStream_t st) {
  const int64_t nb = zp_ceil_div(n + 1, kScanBlock);
  scan_block_kernel<<<(unsigned)nb, kScanBlock, 0, st>>>(n, in, out, block_sums);
  ZP_LAUNCH_CHECK("scan_block_kernel");
  scan_sums_kernel<<<1, 32, 0, st>>>(nb, block_sums);
  ZP_LAUNCH_CHECK("scan_sums_kernel");
  scan_add_kernel<<<(unsigned)nb, kScanBlock, 0, st>>>(n, out, block_sums);
  ZP_LAUNCH_CHECK("scan_add_kernel");
  return ZP_OK;
}

// Calls f(hit, src, -kx, -ky, -kz, d2) on all 32 lanes together for every batch of candidate
// (source, image) pairs around destination j; `hit` marks the lanes whose candidate lies within
// the cutoff, k is its image in wrapped coordinates.
template <typename F>
__device__ __forceinline__ void for_each_hit(const Grid &g, const double *__restrict__ pos,
                                             const int32_t *__restrict__ cell_start,
                                             const int32_t *__restrict__ cell_atoms, int64_t j,
                                             int lane, F &&f) {
  const double xj = pos[3 * j], yj = pos[3 * j + 1], zj = pos[3 * j + 2];
  const int cx = cell_coord(xj, g), cy = cell_coord(yj, g), cz = cell_coord(zj, g);
  const int ojx = own_image(xj, g), ojy = own_image(yj, g), ojz = own_image(zj, g);
  for (int ux = cx - g.w; ux <= cx + g.w; ++ux) {
    const int kx = floor_div(ux, g.nc), wx = ux - kx * g.nc;
    for (int uy = cy - g.w; uy <= cy + g.w; ++uy) {
      const int ky = floor_div(uy, g.nc), wy = uy - ky * g.nc;
      for (int uz = cz - g.w; uz <= cz + g.w; ++uz) {
        const int kz = floor_div(uz, g.nc), wz = uz - kz * g.nc;
        const int c = (wx * g.nc + wy) * g.nc + wz;
        const int beg = cell_start[c], end = cell_start[c + 1];
        for (int a0 = beg; a0 < end; a0 += 32) {
          const int a = a0 + lane;
          bool hit = false;
          int i = 0, mx = 0, my = 0, mz = 0;
          double d2 = 0.0;
          if (a < end) {
            i = cell_atoms[a];
            const double xi = pos[3 * (int64_t)i], yi = pos[3 * (int64_t)i + 1],
                         zi = pos[3 * (int64_t)i + 2];
            // the source's wrapped copy sits k boxes away in wrapped coordinates:
            // pos[j] - (pos[i] - o_i box + k box) stays as (pos[j] - pos[i]) + (o_i - o_j - k) box
            // once the destination's own offset o_j is taken out of the search origin
            mx = own_image(xi, g) - ojx - kx;
            my = own_image(yi, g) - ojy - ky;
            mz = own_image(zi, g) - ojz - kz;
            const double dx = __dadd_rn(__dsub_rn(xj, xi), __dmul_rn((double)mx, g.box));
            const double dy = __dadd_rn(__dsub_rn(yj, yi), __dmul_rn((double)my, g.box));
            const double dz = __dadd_rn(__dsub_rn(zj, zi), __dmul_rn((double)mz, g.box));
            d2 = __dadd_rn(__dadd_rn(__dmul_rn(dx, dx), __dmul_rn(dy, dy)), __dmul_rn(dz, dz));
            hit = d2 < g.cutoff2 && !(i == j && mx == 0 && my == 0 && mz == 0);
          }
          f(hit, i, -kx, -ky, -kz, d2);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(32 * kWarpsPerBlock)
count_kernel(int64_t N, const double *__restrict__ pos, Grid g,
             const int32_t *__restrict__ cell_start, const int32_t *__restrict__ cell_atoms,
             int cap, int32_t *__restrict__ counts, int32_t *flags) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int64_t j = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
  if (j >= N) return;
  int n = 0;
  for_each_hit(g, pos, cell_start, cell_atoms, j, lane,
               [&](bool hit, int, int, int, int, double) {
                 n += __popc(__ballot_sync(0xffffffffu, hit));
               });
  if (lane == 0) {
    if (cap <= 0 && n > kHitCap) atomicOr(flags, 2);       // uncapped list too long for pass 2
    counts[j] = cap > 0 && n > cap ? cap : n;
  }
}

// bitonic sort of the first n2 (a power of two) entries of h by `less`, one warp
template <typename Less>
__device__ __forceinline__ void warp_bitonic(Hit *h, int n2, int lane, Less less) {
  for (int k = 2; k <= n2; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = lane; i < n2; i += 32) {
        const int p = i ^ j;
        if (p > i) {
          const Hit a = h[i], b = h[p];
          const bool up = (i & k) == 0;
          if (up ? less(b, a) : less(a, b)) { h[i] = b; h[p] = a; }
        }
      }
      __syncwarp();
    }
  }
}

__device__ __forceinline__ int pow2_at_least(int n) {
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}

__global__ void __launch_bounds__(32 * kWarpsPerBlock)
fill_kernel(int64_t N, const double *__restrict__ pos, Grid g,
            const int32_t *__restrict__ cell_start, const int32_t *__restrict__ cell_atoms,
            int cap, const int32_t *__restrict__ row_ptr, int64_t E,
            int64_t *__restrict__ edge_index, double *__restrict__ shifts, int32_t *flags) {
  extern __shared__ unsigned char smem_raw[];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  Hit *h = reinterpret_cast<Hit *>(smem_raw) + (size_t)warp * kHitCap;
  const int64_t j = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
  if (j >= N) return;
  const Hit inf{INFINITY, ~0ull};
  int n = 0;                      // hits held (warp-uniform)
  bool overflow = false;
  for_each_hit(g, pos, cell_start, cell_atoms, j, lane,
               [&](bool hit, int i, int nkx, int nky, int nkz, double d2) {
                 const unsigned m = __ballot_sync(0xffffffffu, hit);
                 const int add = __popc(m);
                 if (n + add > kHitCap) {
                   if (cap > 0) {          // keep the best `cap` so far, drop the rest
                     const int n2 = pow2_at_least(n);
                     for (int t = n + lane; t < n2; t += 32) h[t] = inf;
                     __syncwarp();
                     warp_bitonic(h, n2, lane, hit_less);
                     n = n < cap ? n : cap;
                   } else {
                     overflow = true;
                   }
                 }
                 if (hit && !overflow) {
                   const int slot = n + __popc(m & ((1u << lane) - 1u));
                   h[slot].d2 = d2;
                   h[slot].tie = ((unsigned long long)(unsigned)i << 32) |
                                 image_code(nkx, nky, nkz, g.reach);
                 }
                 if (!overflow) n += add;
                 __syncwarp();
               });
  if (overflow) {
    if (lane == 0) atomicOr(flags, 2);
    return;
  }
  if (cap > 0 && n > cap) {
    const int n2 = pow2_at_least(n);
    for (int t = n + lane; t < n2; t += 32) h[t] = inf;
    __syncwarp();
    warp_bitonic(h, n2, lane, hit_less);
    n = cap;
  }
  // survivors in (src, image) order
  {
    const int n2 = pow2_at_least(n);
    for (int t = n + lane; t < n2; t += 32) h[t] = inf;
    __syncwarp();
    warp_bitonic(h, n2, lane, [](const Hit &a, const Hit &b) { return a.tie < b.tie; });
  }
  const int64_t base = row_ptr[j];
  if (lane == 0 && row_ptr[j + 1] - base != n) atomicOr(flags, 4);     // passes disagree
  const unsigned s = 2u * g.reach + 1u;
  const int ojx = own_image(pos[3 * j], g), ojy = own_image(pos[3 * j + 1], g),
            ojz = own_image(pos[3 * j + 2], g);
  for (int t = lane; t < n; t += 32) {
    const unsigned long long tie = h[t].tie;
    const unsigned code = (unsigned)(tie & 0xffffffffu);
    const int64_t i = (int64_t)(tie >> 32);
    const int nkz = (int)(code % s) - g.reach, nky = (int)((code / s) % s) - g.reach,
              nkx = (int)(code / (s * s)) - g.reach;
    edge_index[base + t] = i;
    edge_index[E + base + t] = j;
    shifts[3 * (base + t)] = (double)(own_image(pos[3 * i], g) - ojx + nkx) * g.box;
    shifts[3 * (base + t) + 1] = (double)(own_image(pos[3 * i + 1], g) - ojy + nky) * g.box;
    shifts[3 * (base + t) + 2] = (double)(own_image(pos[3 * i + 2], g) - ojz + nkz) * g.box;
  }
}

struct NbWork {
  int32_t *flags, *cell_count, *cell_start, *cell_cursor, *atom_cell, *cell_atoms, *counts,
      *block_sums;
  size_t bytes;
};

int make_grid(double box, double cutoff, Grid *g) {
  if (!(box > 0.0) || !(cutoff > 0.0) || !std::isfinite(box) || !std::isfinite(cutoff))
    return ZP_ERR_INVALID_ARG;
  // cells a hair wider than the cutoff, so that a last-bit rounding of a cell coordinate can
  // never put a pair within the cutoff more than w cells apart
  int nc = (int)std::floor(box / (cutoff * (1.0 + 1e-9)));
  if (nc < 1) nc = 1;
  if (nc > 256) nc = 256;
  g->box = box;
  g->nc = nc;
  g->cell = box / nc;
  g->cutoff2 = cutoff * cutoff;
  g->w = (int)std::ceil(cutoff * (1.0 + 1e-9) / g->cell);
  if (g->w < 1) g->w = 1;
  g->reach = (int)std::ceil(cutoff / box);
  if (g->reach < 1) g->reach = 1;
  if (g->reach > 8) return ZP_ERR_UNSUPPORTED;         // box far smaller than the cutoff
  return ZP_OK;
}

NbWork carve_nb(int64_t N, const Grid &g, void *base) {
  NbWork w;
  size_t off = 0;
  auto take = [&](size_t n) {
    int32_t *p = base ? reinterpret_cast<int32_t *>(static_cast<unsigned char *>(base) + off)
                      : nullptr;
    off += zp_align_up(n * sizeof(int32_t), 256);
    return p;
  };
  const size_t cells = (size_t)g.nc * g.nc * g.nc;
  w.flags = take(4);
  w.cell_count = take(cells + 1);
  w.cell_start = take(cells + 1);
  w.cell_cursor = take(cells + 1);
  w.atom_cell = take((size_t)N);
  w.cell_atoms = take((size_t)N);
  w.counts = take((size_t)N + 1);
  w.block_sums = take((size_t)zp_ceil_div((int64_t)std::max<size_t>(cells, (size_t)N) + 2, kScanBlock) + 1);
  w.bytes = off;
  return w;
}

}  // namespace

extern "C" {

size_t zp_neighbors_work_bytes(int64_t n_atoms, double box, double cutoff) {
  Grid g;
  if (n_atoms < 0 || make_grid(box, cutoff, &g)) return 0;
  return carve_nb(n_atoms, g, nullptr).bytes;
}

int zp_neighbors_count(const double *pos, int64_t N, double box, double cutoff, int max_neighbors,
                       int32_t *row_ptr, int32_t *flags_out, void *work, size_t work_bytes,
                       void *stream) {
  Grid g;
  int rc = make_grid(box, cutoff, &g);
  if (rc) return rc;
  if (N < 0 || N > 2000000000ll || !row_ptr || !flags_out || !work || (N && !pos))
    return ZP_ERR_INVALID_ARG;
  if (max_neighbors > ZP_NEIGHBORS_MAX_CAP) return ZP_ERR_TOO_LARGE;
  const NbWork w = carve_nb(N, g, work);
  if (work_bytes < w.bytes) return ZP_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const size_t cells = (size_t)g.nc * g.nc * g.nc;
  ZP_CUDA(cudaMemsetAsync(w.flags, 0, 4 * sizeof(int32_t), st));
  ZP_CUDA(cudaMemsetAsync(w.cell_count, 0, (cells + 1) * sizeof(int32_t), st));
  ZP_CUDA(cudaMemsetAsync(w.cell_cursor, 0, (cells + 1) * sizeof(int32_t), st));
  if (N > 0) {
    cell_count_kernel<<<(unsigned)zp_ceil_div(N, 256), 256, 0, st>>>(N, pos, g, w.atom_cell,
                                                                     w.cell_count, w.flags);
    ZP_LAUNCH_CHECK("cell_count_kernel");
  }
  if ((rc = exclusive_scan((int64_t)cells, w.cell_count, w.cell_start, w.block_sums, st))) return rc;
  if (N > 0) {
    cell_fill_kernel<<<(unsigned)zp_ceil_div(N, 256), 256, 0, st>>>(N, w.atom_cell, w.cell_start,
                                                                    w.cell_cursor, w.cell_atoms);
    ZP_LAUNCH_CHECK("cell_fill_kernel");
    count_kernel<<<(unsigned)zp_ceil_div(N, kWarpsPerBlock), 32 * kWarpsPerBlock, 0, st>>>(
        N, pos, g, w.cell_start, w.cell_atoms, max_neighbors, w.counts, w.flags);
    ZP_LAUNCH_CHECK("count_kernel");
  }
  if ((rc = exclusive_scan(N, w.counts, row_ptr, w.block_sums, st))) return rc;
  ZP_CUDA(cudaMemcpyAsync(flags_out, w.flags, sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
  return ZP_OK;
}

int zp_neighbors_fill(const double *pos, int64_t N, double box, double cutoff, int max_neighbors,
                      const int32_t *row_ptr, int64_t E, int64_t *edge_index, double *shifts,
                      int32_t *flags_out, void *work, size_t work_bytes, void *stream) {
  Grid g;
  int rc = make_grid(box, cutoff, &g);
  if (rc) return rc;
  if (N < 0 || E < 0 || !row_ptr || !flags_out || !work || (N && !pos) ||
      (E && (!edge_index || !shifts)))
    return ZP_ERR_INVALID_ARG;
  if (max_neighbors > ZP_NEIGHBORS_MAX_CAP) return ZP_ERR_TOO_LARGE;
  const NbWork w = carve_nb(N, g, work);
  if (work_bytes < w.bytes) return ZP_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  if (N > 0) {
    const size_t smem = sizeof(Hit) * kHitCap * kWarpsPerBlock;
    static ZpSmemOptIn opt_in;
    if (int rc_ = zp_ensure_smem(fill_kernel, smem, opt_in)) return rc_;
    fill_kernel<<<(unsigned)zp_ceil_div(N, kWarpsPerBlock), 32 * kWarpsPerBlock, smem, st>>>(
        N, pos, g, w.cell_start, w.cell_atoms, max_neighbors, row_ptr, E, edge_index, shifts,
        w.flags);
    ZP_LAUNCH_CHECK("fill_kernel");
  }
  ZP_CUDA(cudaMemcpyAsync(flags_out, w.flags, sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
  return ZP_OK;
}

}  // extern "C"
