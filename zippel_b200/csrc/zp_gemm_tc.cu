// The SO(2) contraction on the Blackwell tensor cores (tcgen05 + TMEM + TMA), sm_100a only.
//
//     C[M, N] (fp32) = sum over plane pairs (pa, pb) of  A_pa[M, K] * B_pb[N, K]^T   (+ bias[n])
//
// Operands are bf16 "planes".  With one plane per operand this is a plain bf16 GEMM with fp32
// accumulation.  With three planes an fp32 value x is carried as x = x0 + x1 + x2 (each a
// bf16, x0 = rn(x), x1 = rn(x - x0), x2 = rn(x - x0 - x1)), and the six products
//     A0B0, A0B1, A1B0, A1B1, A0B2, A2B0
// (everything down to 2^-16 of the leading term) reproduce the fp32 product to ~2^-22 while
// staying on the bf16 pipe and keeping fp32's exponent range.  All planes of a k-block are
// loaded once and reused by the six MMAs.
//
// Accumulation accuracy.  The tensor core adds each k = 16 step into the fp32 accumulator with
// truncation, a bias of about 3e-8 of the accumulator per step (measured: relative error
// ~1e-9 * K for one product, 6.5e-9 * K when all six share an accumulator).  Two measures keep
// that below the fp32 budget: (1) the leading product A0B0 has its own TMEM accumulator and the
// five small products share a second one, whose truncation is 2^-8 smaller in absolute terms;
// (2) the contraction is cut into chunks of at most `kc` k-blocks, each accumulated in TMEM
// from zero and then added to C in fp32 by the epilogue (first chunk stores, later chunks
// add), so the bias never grows beyond one chunk's length.  Long contractions (the weight
// gradients, which run over all edges) can also be split over CTAs: split s writes its own
// partial matrix C + s * split_stride, reduced afterwards in a fixed order.
//
// Structure: persistent CTAs (one per SM), 320 threads.
//   warp 0      TMA producer: one elected lane streams A/B plane tiles into a ring of stages
//   warp 1      allocates TMEM, then one elected lane issues tcgen05.mma and commits
//   warps 2..9  epilogue: tcgen05.ld the 128 x BN accumulator into registers, release TMEM,
//               then scale, add bias and store fp32 rows
// With one plane two TMEM accumulators (2 x 256 columns) let the epilogue of one tile overlap
// the main loop of the next; with three planes the 512 columns hold the leading and the small
// accumulator of one tile.  Tiles are ordered n-fastest so CTAs running side by side share one A row block
// (read from HBM once, then L2) while the weights stay L2 resident.
//
// Operand layouts in global memory (element strides, all multiples of 8 so TMA rows are 16-byte
// aligned):  K-major   X[p*plane + r*ld + k]   (rows r = m or n, contraction index fastest)
//            MN-major  X[p*plane + k*ld + r]   (used by the weight-gradient products, whose
//                                               contraction runs over edges)
// Shared-memory tiles use the 128-byte (BK = 64) or 64-byte (BK = 32) swizzle that TMA writes
// and the matrix descriptors name.  Every mbarrier wait is bounded: after ~2 s it records
// ZP_ERR_DEVICE_TIMEOUT in the status word, raises the CTA's abort flag and the CTA drains.
#include <cstdlib>
#include <mutex>

#include <cuda.h>
#include <cuda_bf16.h>

#include "zp_common.cuh"

namespace {

constexpr int BM = 128;
constexpr int kTmemBuf = 256;          // TMEM columns per accumulator buffer
constexpr int kThreads = 320;            // producer warp, MMA warp, eight epilogue warps
constexpr uint64_t kWaitLimitNs = 2000000000ull;   // default bound of every device-side wait

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .pred px;\n"
      "elect.sync _|px, 0xFFFFFFFF;\n"
      "@px mov.s32 %0, 1;\n"
      "}\n"
      : "+r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the CTA is aborting (this wait or another one timed out).
// The clock is only looked at every 1024 failed polls (the first look starts the interval), so a
// wait that is satisfied quickly never pays for reading the global timer.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          int *status, uint64_t limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ff) == 0) {
      if (*abort_flag) return false;
      const uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        *abort_flag = 1;
        atomicExch(status, (int)ZP_ERR_DEVICE_TIMEOUT);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0),
        "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor.
//   K-major tile  [rows][BK] with a BK*2-byte swizzle: 8-row groups are 8*BK*2 bytes apart (SBO).
//   MN-major tile [BK][64] with the 128-byte swizzle: 8 k-rows are 1024 bytes apart (SBO) and the
//   next 64 elements along M/N start `lbo_bytes` later (LBO).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fff);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;                       // descriptor version of this architecture
  d |= (uint64_t)layout_type << 61;             // 2 = 128-byte swizzle, 4 = 64-byte swizzle
  return d;
}

struct GemmParams {
  int M, N, K;
  int BN;                 // tile width, multiple of 16, <= 256
  int num_m, num_n, num_k;
  int ksplit, kb_per_split, kc;   // CTAs-level split of K; k-blocks per TMEM accumulation chunk
  int a_mn, b_mn;         // operand is MN-major
  int fp16;               // operand planes are fp16 (else bf16)
  const float *scale_a, *scale_b;   // device scalars multiplying the result (null = 1)
  float *absmax_out;      // device scalar: running max |C| of what this launch stores (or null)
  const float *bias;
  float *C;
  int64_t ldc, split_stride;
  int tma_store;          // epilogue goes through TMA stores (map_c is valid)
  int *status;
  uint64_t wait_limit_ns; // bound of every mbarrier wait
  int unarmed;            // self-test: the producers load nothing, so the first wait runs out
  ZpEpilogue epi;         // work of the fused epilogues (mode 0: none)
};

// plane pairs; for three planes pair 0 is the leading product, pairs 1..5 the small ones
template <int P> struct Pairs;
template <> struct Pairs<1> {
  static constexpr int n = 1;
  __device__ static constexpr int a(int) { return 0; }
  __device__ static constexpr int b(int) { return 0; }
};
template <> struct Pairs<2> {
  static constexpr int n = 3;          // fp16 pair: h0 h0 | h0 h1, h1 h0
  __device__ static constexpr int a(int i) { return i == 2 ? 1 : 0; }
  __device__ static constexpr int b(int i) { return i == 1 ? 1 : 0; }
};
template <> struct Pairs<3> {
  static constexpr int n = 6;
  __device__ static constexpr int a(int i) { return i == 0 ? 0 : i == 1 ? 2 : i == 2 ? 0 : i == 3 ? 1 : i == 4 ? 1 : 0; }
  __device__ static constexpr int b(int i) { return i == 0 ? 0 : i == 1 ? 0 : i == 2 ? 2 : i == 3 ? 1 : i == 4 ? 0 : 1; }
};

// ---- epilogue through TMA stores ------------------------------------------------------------
// In TMEM a lane owns a row, so storing straight from the registers sends every lane of an
// instruction to a different output row: 32 separate 16-byte pieces per instruction, and the
// epilogue of a 128 x 256 tile costs ~8 000 store wavefronts.  Instead each epilogue warp writes
// 32 x 32 blocks into its own 4 KB of shared memory (128-byte rows under the 128-byte swizzle, the
// layout the tensor map names) and one lane hands the block to the TMA unit, which writes full
// lines and clips rows / columns beyond the matrix.  Later K chunks of a tile use the reducing
// store (add) after the previous store of that tile has completed.
constexpr int kEpiBlockBytes = 32 * 32 * 4;
constexpr int kEpiBytes = 8 * kEpiBlockBytes;                 // eight epilogue warps

__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, const void *src, int c0, int c1,
                                             int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap *map, const void *src, int c0,
                                                  int c1, int c2) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
      :
      : "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() {            // shared source may be overwritten
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_read_but_one() {    // all but the newest group were read
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_all() {             // the writes themselves are done
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// v[b][j]: value at row `row0 + lane`, column `n0 + col_lo + 32 b + j` (scaled, no bias yet).
// EB = 2: the warp alternates between two block buffers, so one block's store is still being read
// out of shared memory while the next block is staged (products with a short contraction are
// bound by their output stores, and one 4 KB block per warp in flight does not cover the latency).
template <int EB>
__device__ __forceinline__ void epilogue_store_tma(const GemmParams &p, const CUtensorMap *map_c,
                                                   float (&v)[4][32], uint8_t *stage0, int lane,
                                                   int row0, int n0, int col_lo, int col_hi,
                                                   int split, const float *bias, bool first,
                                                   float &seen_max, uint32_t &blocks_done) {
  if (row0 >= p.M) return;                        // warp-uniform: nothing of this slice exists
  const bool row_ok = row0 + lane < p.M;
  if (!first) {                                   // the tile's previous store must have landed
    if (lane == 0) bulk_wait_all();
    __syncwarp();
  }
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int cc = col_lo + 32 * b;
    if (cc >= col_hi) continue;                   // warp-uniform
    const int n = n0 + cc;
    if (n >= p.N) continue;
    uint8_t *stage = stage0 + (EB == 2 ? (blocks_done & 1) * kEpiBlockBytes : 0);
    ++blocks_done;
    if (lane == 0) {                              // the block buffer is free again
      if (EB == 2) bulk_wait_read_but_one();
      else bulk_wait_read();
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float4 o = make_float4(v[b][4 * k], v[b][4 * k + 1], v[b][4 * k + 2], v[b][4 * k + 3]);
      if (first && bias) {
        const int c = n + 4 * k;
        o.x += c < p.N ? bias[c] : 0.f;
        o.y += c + 1 < p.N ? bias[c + 1] : 0.f;
        o.z += c + 2 < p.N ? bias[c + 2] : 0.f;
        o.w += c + 3 < p.N ? bias[c + 3] : 0.f;
      }
      if (row_ok) {
        const int c = n + 4 * k;
        float m = c < p.N ? fabsf(o.x) : 0.f;
        m = fmaxf(m, c + 1 < p.N ? fabsf(o.y) : 0.f);
        m = fmaxf(m, c + 2 < p.N ? fabsf(o.z) : 0.f);
        m = fmaxf(m, c + 3 < p.N ? fabsf(o.w) : 0.f);
        seen_max = fmaxf(seen_max, m);
      }
      // 128-byte swizzle: 16-byte chunk k of row r sits at chunk k ^ (r & 7)
      *reinterpret_cast<float4 *>(stage + lane * 128 + ((k ^ (lane & 7)) << 4)) = o;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) {
      if (first) tma_store_3d(map_c, stage, n, row0, split);
      else tma_reduce_add_3d(map_c, stage, n, row0, split);
      bulk_commit();
    }
  }
}


// ---- fused epilogues ------------------------------------------------------------------------
// A finished 32 x 32 block of the result sits in the warp's shared-memory stage in the layout
// above (row = edge, 16-byte chunk k of row r at chunk k ^ (r & 7)).  The fused epilogues read
// it back in a second assignment of lanes and consume it there, so the values never have to come
// back from HBM: the gate activation walks it row-wise (eight lanes share a row, coalesced
// loads of the gate scalars and 8-byte plane stores), the rotation back walks it column-wise
// (a lane owns one channel and runs over the block's edges in order).
__device__ __forceinline__ float fast_sigmoid(float x) { return 1.f / (1.f + __expf(-x)); }

__device__ __forceinline__ void gate_block(const ZpEpilogue &f, const uint8_t *stage, int lane,
                                           int row0, int n, int M, int N, float inv,
                                           float &slope_max) {
  // Pass 1: request the gate scalars of all eight row groups (independent loads, one memory round
  // trip for the block).  Pass 2: activate and store.
  const int k = lane & 7, col = n + 4 * k;
  const int rq = col / f.width;
  const int r = f.row_first + rq, h = col - rq * f.width;
  const bool col_ok = col < N;
  const bool gated = r != 0;                      // row 0 (l = 0): x * sigmoid(x)
  const float *gcol = f.gate + (gated ? (f.row_l[r] - 1) * f.width + h : 0);
  float4 g[8];
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int row = row0 + it * 4 + (lane >> 3);
    g[it] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (gated && col_ok && row < M)
      g[it] = *reinterpret_cast<const float4 *>(gcol + (size_t)row * f.ld_gate);
  }
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int rr = it * 4 + (lane >> 3);
    const int row = row0 + rr;
    if (row < M && col_ok) {
      const float4 x = *reinterpret_cast<const float4 *>(stage + rr * 128 + ((k ^ (rr & 7)) << 4));
      const float4 q = gated ? g[it] : x;
      const float s0 = fast_sigmoid(q.x), s1 = fast_sigmoid(q.y), s2 = fast_sigmoid(q.z),
                  s3 = fast_sigmoid(q.w);
      const float o[4] = {x.x * s0, x.y * s1, x.z * s2, x.w * s3};
      if (gated)
        slope_max = fmaxf(slope_max, fmaxf(fmaxf(s0 * (1.f - s0), s1 * (1.f - s1)),
                                           fmaxf(s2 * (1.f - s2), s3 * (1.f - s3))));
      zp_store_planes<4>(f.out, (int64_t)row * f.out.ld + col, o, inv);
    }
  }
}

// row_ptr[idx] for the rotate-back epilogue: lane d of the warp holds row_ptr[node0 + d] (fetched
// once per tile), anything further away comes from memory.  idx is warp-uniform.
__device__ __forceinline__ int row_ptr_at(const ZpEpilogue &f, int idx, int node0, int rp_l) {
  const int d = idx - node0;
  return (d >= 0 && d < 32) ? __shfl_sync(0xffffffffu, rp_l, d) : f.row_ptr[idx];
}

constexpr int kMaxNj = 2 * ZP_MAX_L + 1;

// node: the node of edge row0 (from find_node)
__device__ __forceinline__ void rotate_back_block(const ZpEpilogue &f, const uint8_t *stage, int lane,
                                                  int row0, int n, int M, int N, int node,
                                                  const int node0, const int rp_l) {
  const int col = n + lane;
  const bool col_ok = col < N;
  const int cq = col_ok ? col : n;               // lanes beyond the matrix shadow column n
  const int rq = cq / f.width;
  const int r = f.row_first + rq, c = cq - rq * f.width;
  const int off = f.rot_off[r];
  const int nj = 2 * f.row_l[r] + 1;
  const int njmax = __reduce_max_sync(0xffffffffu, nj);
  const int row_end = min(row0 + 32, M);
  const size_t slab = (size_t)f.nnz * f.width;
  // Usual case: the block's 32 columns lie in one m' row, so every lane needs the same rotation
  // entries.  Lane i then fetches the envelope and the row's 2l+1 entries of EDGE row0 + i (all
  // requests in flight together: one memory round trip per block) and the edge loop broadcasts
  // them with shuffles.  Otherwise every lane reads its own row's entries edge by edge.
  const bool one_row = __all_sync(0xffffffffu, r == __shfl_sync(0xffffffffu, r, 0));
  float env_l = 0.f, rot_l[kMaxNj];
#pragma unroll
  for (int j = 0; j < kMaxNj; ++j) rot_l[j] = 0.f;
  if (one_row && row0 + lane < row_end) {
    const int ei = row0 + lane;
    env_l = f.env[ei];
    const float *re = f.rot + (size_t)ei * f.nnz_pad + off;
#pragma unroll
    for (int j = 0; j < kMaxNj; ++j)
      if (j < nj) rot_l[j] = re[j];
  }
  int e = row0;
  while (e < row_end) {
    int next = row_ptr_at(f, node + 1, node0, rp_l);
    while (node + 1 < f.n_nodes && next <= e) {  // nodes without edges
      ++node;
      next = row_ptr_at(f, node + 1, node0, rp_l);
    }
    const bool is_head = row_ptr_at(f, node, node0, rp_l) == e;
    int stop = min(next, row_end);
    if (stop <= e) stop = row_end;               // offsets that do not cover the edges: never spin
    float acc[kMaxNj];
#pragma unroll
    for (int j = 0; j < kMaxNj; ++j) acc[j] = 0.f;
    if (one_row) {
#pragma unroll 4
      for (; e < stop; ++e) {
        const int i = e - row0;
        const float yv = __shfl_sync(0xffffffffu, env_l, i) *
                         *reinterpret_cast<const float *>(stage + i * 128 + (((lane >> 2) ^ (i & 7)) << 4) +
                                                          ((lane & 3) << 2));
#pragma unroll
        for (int j = 0; j < kMaxNj; ++j) {
          if (j >= njmax) break;                 // warp-uniform
          acc[j] = fmaf(__shfl_sync(0xffffffffu, rot_l[j], i), yv, acc[j]);
        }
      }
    } else {
#pragma unroll 2
      for (; e < stop; ++e) {
        const int i = e - row0;
        const float yv = f.env[e] * *reinterpret_cast<const float *>(
                                        stage + i * 128 + (((lane >> 2) ^ (i & 7)) << 4) + ((lane & 3) << 2));
        const float *re = f.rot + (size_t)e * f.nnz_pad + off;
#pragma unroll
        for (int j = 0; j < kMaxNj; ++j) {
          if (j >= njmax) break;                 // warp-uniform
          if (j < nj) acc[j] = fmaf(re[j], yv, acc[j]);
        }
      }
    }
    float *out = (is_head ? f.head + (size_t)node * slab : f.cont + (size_t)(row0 >> 5) * slab) +
                 (size_t)off * f.width + c;
    if (col_ok) {
#pragma unroll
      for (int j = 0; j < kMaxNj; ++j)
        if (j < nj) out[(size_t)j * f.width] = acc[j];
    }
  }
}

// v[b][j]: value at row `row0 + lane`, column `n0 + col_lo + 32 b + j` (scaled, no bias yet).
template <int EPI>
__device__ __forceinline__ void epilogue_fused(const GemmParams &p, const CUtensorMap *map_c,
                                               float (&v)[4][32], uint8_t *stage, int lane, int row0,
                                               int n0, int col_lo, int col_hi, const float *bias,
                                               float &seen_max, float &slope_max, int node,
                                               int rp_l) {
  if (row0 >= p.M) return;
  const bool row_ok = row0 + lane < p.M;
  const float inv = EPI == ZP_EPI_GATE ? zp_inv_scale(p.epi.out) : 1.f;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const int cc = col_lo + 32 * b;
    if (cc >= col_hi) continue;                   // warp-uniform
    const int n = n0 + cc;
    if (n >= p.N) continue;
    if (p.epi.store_c && lane == 0) bulk_wait_read();   // the TMA store of the previous block
    __syncwarp();                                 // ... and every lane's reads of it are done
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float4 o = make_float4(v[b][4 * k], v[b][4 * k + 1], v[b][4 * k + 2], v[b][4 * k + 3]);
      const int c = n + 4 * k;
      if (bias) {
        o.x += c < p.N ? bias[c] : 0.f;
        o.y += c + 1 < p.N ? bias[c + 1] : 0.f;
        o.z += c + 2 < p.N ? bias[c + 2] : 0.f;
        o.w += c + 3 < p.N ? bias[c + 3] : 0.f;
      }
      if (row_ok) {
        float m = c < p.N ? fabsf(o.x) : 0.f;
        m = fmaxf(m, c + 1 < p.N ? fabsf(o.y) : 0.f);
        m = fmaxf(m, c + 2 < p.N ? fabsf(o.z) : 0.f);
        m = fmaxf(m, c + 3 < p.N ? fabsf(o.w) : 0.f);
        seen_max = fmaxf(seen_max, m);
      }
      *reinterpret_cast<float4 *>(stage + lane * 128 + ((k ^ (lane & 7)) << 4)) = o;
    }
    if (p.epi.store_c) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        tma_store_3d(map_c, stage, n, row0, 0);
        bulk_commit();
      }
    } else {
      __syncwarp();
    }
    if (EPI == ZP_EPI_GATE) gate_block(p.epi, stage, lane, row0, n, p.M, p.N, inv, slope_max);
    else rotate_back_block(p.epi, stage, lane, row0, n, p.M, p.N, node, node, rp_l);
  }
}

template <int P, int BK, int STAGES, int BN_CAP, int EB = 1>
struct SmemLayout {
  static constexpr int kEpiBytes = EB * ::kEpiBytes;
  static constexpr int kATile = BM * BK * 2;
  static constexpr int kBTile = BN_CAP * BK * 2;
  static constexpr int kStage = P * (kATile + kBTile);
  static constexpr int kTiles = STAGES * kStage;
  static constexpr int kBars = 8 * (2 * STAGES + 4);
  // barriers, TMEM slot and abort flag live in the first KB after the tiles; the epilogue's
  // store blocks (when the CTA's budget allows them) follow, 1 KB aligned; + 1 KB alignment slack
  static_assert(kBars + 16 <= 1024, "control words fit in one KB");
  static constexpr bool kTmaEpilogue = kTiles + 1024 + kEpiBytes + 1024 <= 232448;
  static constexpr int kEpiOffset = kTiles + 1024;
  static constexpr int kTotal = kTiles + 1024 + (kTmaEpilogue ? kEpiBytes : 0) + 1024;
};

// One unit of work of a CTA: an output tile, a K split, and its k-block range.
struct Work {
  int m0, n0, split, kb0, kb1;
};
__device__ __forceinline__ Work decode_work(const GemmParams &p, int w) {
  Work x;
  x.split = w % p.ksplit;
  const int tile = w / p.ksplit;
  x.m0 = (tile / p.num_n) * BM;
  x.n0 = (tile % p.num_n) * p.BN;
  x.kb0 = x.split * p.kb_per_split;
  x.kb1 = min(p.num_k, x.kb0 + p.kb_per_split);
  return x;
}

template <int P, int BK, int STAGES, int BN_CAP, int EPI, int EB = 1>
__device__ __forceinline__ void gemm_tc_body(const CUtensorMap &map_a, const CUtensorMap &map_b,
                                             const CUtensorMap &map_c, const GemmParams &p) {
  using L = SmemLayout<P, BK, STAGES, BN_CAP, EB>;
  constexpr int kAccBufs = P == 1 ? 2 : 1;      // accumulation units in flight in TMEM
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~(uintptr_t)1023);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + L::kTiles);
  uint64_t *empty = full + STAGES;
  uint64_t *tmem_full = empty + STAGES;
  uint64_t *tmem_empty = tmem_full + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int num_work = p.num_m * p.num_n * p.ksplit;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 8); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t a_bytes = BM * BK * 2;
  const uint32_t b_bytes = (uint32_t)p.BN * BK * 2;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (!p.unarmed && elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const Work x = decode_work(p, w);
        for (int kb = x.kb0; kb < x.kb1 && ok; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag, p.status, p.wait_limit_ns);
          if (!ok) break;
          uint8_t *st = smem + (size_t)s * L::kStage;
          mbar_expect_tx(&full[s], P * (a_bytes + b_bytes));
          const int k0 = kb * BK;
#pragma unroll
          for (int pl = 0; pl < P; ++pl) {
            uint8_t *ta = st + pl * L::kATile, *tb = st + P * L::kATile + pl * L::kBTile;
            if (!p.a_mn) {
              tma_load_3d(ta, &map_a, &full[s], k0, x.m0, pl);
            } else {                      // two 64-wide column blocks of [BK][64]
              tma_load_3d(ta, &map_a, &full[s], x.m0, k0, pl);
              tma_load_3d(ta + BK * 128, &map_a, &full[s], x.m0 + 64, k0, pl);
            }
            if (!p.b_mn) {
              tma_load_3d(tb, &map_b, &full[s], k0, x.n0, pl);
            } else {
              for (int nb = 0; nb < p.BN; nb += 64)
                tma_load_3d(tb + (nb / 64) * BK * 128, &map_b, &full[s], x.n0 + nb, k0, pl);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const uint32_t fmt = p.fp16 ? 0u : 1u;    // operand format field: 0 = f16, 1 = bf16
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.a_mn ? 1 : 0) << 15) |
                             ((uint32_t)(p.b_mn ? 1 : 0) << 16) | ((uint32_t)(p.BN >> 3) << 17) |
                             ((uint32_t)(BM >> 4) << 24);
      constexpr uint32_t kLayout = BK == 64 ? 2u : 4u;
      uint32_t it = 0, unit = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
        const Work x = decode_work(p, w);
        for (int c0 = x.kb0; c0 < x.kb1 && ok; c0 += p.kc, ++unit) {
          const int c1 = min(x.kb1, c0 + p.kc);
          const int buf = unit % kAccBufs;
          ok = mbar_wait(&tmem_empty[buf], ((unit / kAccBufs) & 1) ^ 1, abort_flag, p.status, p.wait_limit_ns);
          if (!ok) break;
          tcgen05_fence_after();
          // one plane: accumulator `buf`; three planes: leading product at column 0, small at 256
          const uint32_t d_main = tmem_base + (P == 1 ? (uint32_t)buf * kTmemBuf : 0u);
          const uint32_t d_small = tmem_base + kTmemBuf;
          for (int kb = c0; kb < c1 && ok; ++kb, ++it) {
            const int s = it % STAGES;
            ok = mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, p.status, p.wait_limit_ns);
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t sa = smem_u32(smem + (size_t)s * L::kStage);
            const uint32_t sb = sa + P * L::kATile;
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks) {
#pragma unroll
              for (int q = 0; q < Pairs<P>::n; ++q) {
                const uint32_t ta = sa + Pairs<P>::a(q) * L::kATile;
                const uint32_t tb = sb + Pairs<P>::b(q) * L::kBTile;
                // K-major: 32 bytes along the swizzled row per k-step of 16
                // MN-major: 16 k-rows of 128 bytes per k-step
                const uint64_t da = p.a_mn ? make_desc(ta + ks * 2048, BK * 128, 1024, 2u)
                                           : make_desc(ta + ks * 32, 16, 8 * BK * 2, kLayout);
                const uint64_t db = p.b_mn ? make_desc(tb + ks * 2048, BK * 128, 1024, 2u)
                                           : make_desc(tb + ks * 32, 16, 8 * BK * 2, kLayout);
                const bool first_step = kb == c0 && ks == 0;
                if (q == 0) umma_bf16(d_main, da, db, idesc, first_step ? 0u : 1u);
                else umma_bf16(d_small, da, db, idesc, (first_step && q == 1) ? 0u : 1u);
              }
            }
            tcgen05_commit(&empty[s]);          // stage reusable once these MMAs have read it
          }
          if (ok) tcgen05_commit(&tmem_full[buf]);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..9)
    // Eight warps: warp w reads TMEM lane quarter w % 4 (the only one it may access) and column
    // half (w - 2) / 4.  A warp first pulls its whole 32 x 128 slice of the accumulator(s) into
    // registers and releases TMEM, so the next tile's MMAs start while it scales and stores.
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    uint8_t *epi_stage = smem + L::kEpiOffset + (warp - 2) * kEpiBlockBytes * EB;
    uint32_t unit = 0, blocks_done = 0;
    bool ok = true;
    const float out_scale = (p.scale_a ? *p.scale_a : 1.f) * (p.scale_b ? *p.scale_b : 1.f);
    float seen_max = 0.f, slope_max = 0.f;
    const int col_lo = half * 128, col_hi = min(p.BN, col_lo + 128);
    for (int w = blockIdx.x; w < num_work && ok; w += gridDim.x) {
      const Work x = decode_work(p, w);
      const int row0 = x.m0 + q * 32;
      const int row = row0 + lane;
      float *crow = p.C + (size_t)x.split * p.split_stride + (size_t)row * p.ldc;
      const float *bias = x.split == 0 ? p.bias : nullptr;
      for (int c0 = x.kb0; c0 < x.kb1 && ok; c0 += p.kc, ++unit) {
        const int buf = unit % kAccBufs;
        const bool first = c0 == x.kb0;         // first chunk stores, later chunks add
        // the node of the warp's first edge and the offsets of the 32 nodes from there on,
        // fetched while the tile is still being formed
        int node = 0, rp_l = 0;
        if (EPI == ZP_EPI_ROTATE_BACK && row0 < p.M) {
          node = p.epi.block_node[row0 >> 5];
          rp_l = p.epi.row_ptr[min(node + lane, p.epi.n_nodes)];
        }
        ok = mbar_wait(&tmem_full[buf], (unit / kAccBufs) & 1, abort_flag, p.status, p.wait_limit_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) +
                               (P == 1 ? (uint32_t)buf * kTmemBuf : 0u);
        float v[4][32];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int cc = col_lo + 32 * b;
          if (cc < col_hi) {                    // warp-uniform
            // 16 columns at a time, the small-product accumulator added in place: the slice
            // itself (128 values per thread) leaves little room for staging registers
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              // both accumulators' loads are in flight together: one wait per 16 columns
              uint32_t r[16], r2[16];
              tmem_ld16(t_row + cc + 16 * h, r);
              if (P != 1) tmem_ld16(t_row + kTmemBuf + cc + 16 * h, r2);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float a = __uint_as_float(r[j]);
                if (P != 1) a += __uint_as_float(r2[j]);
                v[b][16 * h + j] = a * out_scale;
              }
            }
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[buf]);      // TMEM slice is in registers now

        if (EPI != ZP_EPI_NONE) {
          if (L::kTmaEpilogue)
            epilogue_fused<EPI>(p, &map_c, v, epi_stage, lane, row0, x.n0, col_lo, col_hi, bias,
                                seen_max, slope_max, node, rp_l);
        } else if (L::kTmaEpilogue && p.tma_store) {
          epilogue_store_tma<EB>(p, &map_c, v, epi_stage, lane, row0, x.n0, col_lo, col_hi, x.split,
                                 bias, first, seen_max, blocks_done);
        } else if (row < p.M) {
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const int cc = col_lo + 32 * b;
            if (cc >= col_hi) continue;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const int n = x.n0 + cc + j;
              if (cc + j < p.BN && n + 3 < p.N) {
                float4 o = make_float4(v[b][j], v[b][j + 1], v[b][j + 2], v[b][j + 3]);
                if (first) {
                  if (bias) {
                    const float4 bv = *reinterpret_cast<const float4 *>(bias + n);
                    o.x += bv.x; o.y += bv.y; o.z += bv.z; o.w += bv.w;
                  }
                } else {
                  const float4 old = *reinterpret_cast<const float4 *>(crow + n);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4 *>(crow + n) = o;
                seen_max = fmaxf(seen_max, fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)),
                                                 fmaxf(fabsf(o.z), fabsf(o.w))));
              } else if (cc + j < p.BN) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                  if (n + u < p.N) {
                    const float base = first ? (bias ? bias[n + u] : 0.f) : crow[n + u];
                    const float o = v[b][j + u] + base;
                    crow[n + u] = o;
                    seen_max = fmaxf(seen_max, fabsf(o));
                  }
              }
            }
          }
        }
      }
    }
    if (L::kTmaEpilogue && p.tma_store && lane == 0) bulk_wait_all();   // this warp's stores are done
    if (p.absmax_out) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) seen_max = fmaxf(seen_max, __shfl_xor_sync(0xffffffffu, seen_max, o));
      if (lane == 0 && seen_max > 0.f) zp_atomic_absmax(p.absmax_out, seen_max);
    }
    if (EPI == ZP_EPI_GATE && p.epi.slope_max) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) slope_max = fmaxf(slope_max, __shfl_xor_sync(0xffffffffu, slope_max, o));
      if (lane == 0 && slope_max > 0.f) zp_atomic_absmax(p.epi.slope_max, slope_max);
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u)
                 : "memory");
  }
}

template <int P, int BK, int STAGES, int BN_CAP, int EB = 1>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const __grid_constant__ GemmParams p) {
  gemm_tc_body<P, BK, STAGES, BN_CAP, ZP_EPI_NONE, EB>(map_a, map_b, map_c, p);
}
// the same contraction with a fused epilogue (the epilogue warps hold more live values)
template <int P, int BK, int STAGES, int BN_CAP, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_fused_kernel(const __grid_constant__ CUtensorMap map_a,
                     const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_c,
                     const __grid_constant__ GemmParams p) {
  gemm_tc_body<P, BK, STAGES, BN_CAP, EPI>(map_a, map_b, map_c, p);
}

// ---- CTA-pair variant ---------------------------------------------------------------------
//
// Two CTAs of a cluster (an SM pair) work on one 256 x BN tile with tcgen05.mma.cta_group::2:
// each CTA stages its own 128 rows of A and HALF of the B tile, and the pair's tensor cores read
// both halves, so a CTA pulls (128 + BN/2) operand rows per k-block from L2 instead of
// (128 + BN).  With two fp16 planes and three MMA passes per k-block the single-CTA kernel is
// limited by that operand feed; the pair is not.
//
// Roles per CTA are as above, except that only the even CTA of the pair (the leader) issues MMAs.
//   full[s]       leader's barrier; the leader's producer announces the bytes of BOTH CTAs and
//                 both producers' TMA loads complete on it (cta_group::2 loads)
//   empty[s]      one per CTA; the leader's tcgen05.commit releases the stage in both CTAs
//   tmem_full     one per CTA, signalled by the same kind of commit
//   tmem_empty    leader's barrier, 16 arrivals: the eight epilogue warps of each CTA
// TMEM holds rows 0..127 of the tile in the leader and rows 128..255 in its peer; each CTA's
// epilogue reads its own half.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release;\n"
               "barrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// load into this CTA's shared memory, completing on a barrier of the pair's leader
__device__ __forceinline__ void tma_load_3d_pair(void *dst, const CUtensorMap *map,
                                                 uint32_t bar_cluster_addr, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0),
        "r"(c1), "r"(c2)
      : "memory");
}
// arrive on the barrier at this offset in both CTAs of the pair once the MMAs issued so far finish
__device__ __forceinline__ void tcgen05_commit_pair(uint64_t *bar) {
  const uint16_t both = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;" ::"r"(smem_u32(bar)),
      "h"(both)
      : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

constexpr int BM2 = 256;               // rows of a pair's tile

template <int P, int BK, int STAGES>
struct SmemLayoutPair {
  static constexpr int kATile = BM * BK * 2;          // this CTA's 128 rows
  static constexpr int kBTile = 128 * BK * 2;         // this CTA's half of a <= 256-wide B tile
  static constexpr int kStage = P * (kATile + kBTile);
  static constexpr int kTiles = STAGES * kStage;
  static constexpr int kBars = 8 * (2 * STAGES + 4);
  static_assert(kBars + 16 <= 1024, "control words fit in one KB");
  static constexpr bool kTmaEpilogue = kTiles + 1024 + kEpiBytes + 1024 <= 232448;
  static constexpr int kEpiOffset = kTiles + 1024;
  static constexpr int kTotal = kTiles + 1024 + (kTmaEpilogue ? kEpiBytes : 0) + 1024;
};

__device__ __forceinline__ Work decode_work_pair(const GemmParams &p, int w) {
  Work x;
  x.split = w % p.ksplit;
  const int tile = w / p.ksplit;
  x.m0 = (tile / p.num_n) * BM2;
  x.n0 = (tile % p.num_n) * p.BN;
  x.kb0 = x.split * p.kb_per_split;
  x.kb1 = min(p.num_k, x.kb0 + p.kb_per_split);
  return x;
}

template <int P, int BK, int STAGES, int EPI>
__device__ __forceinline__ void gemm_tc_pair_body(const CUtensorMap &map_a, const CUtensorMap &map_b,
                                                  const CUtensorMap &map_c, const GemmParams &p) {
  using L = SmemLayoutPair<P, BK, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  // the dynamic shared window starts at the same offset in both CTAs, so does everything below
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~(uintptr_t)1023);
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + L::kTiles);
  uint64_t *empty = full + STAGES;
  uint64_t *tmem_full = empty + STAGES;
  uint64_t *tmem_empty = tmem_full + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_empty + 2);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_work = p.num_m * p.num_n * p.ksplit;
  const int half_n = p.BN >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], 16); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  cluster_sync_all();                   // both CTAs' barriers exist before anything signals them
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();                   // both allocations exist before the leader's first MMA
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const uint32_t a_bytes = BM * BK * 2;
  const uint32_t b_bytes = (uint32_t)half_n * BK * 2;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer (both CTAs)
    if (!p.unarmed && elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = pair; w < num_work && ok; w += num_pairs) {
        const Work x = decode_work_pair(p, w);
        const int m0 = x.m0 + (int)rank * BM, n0 = x.n0 + (int)rank * half_n;
        for (int kb = x.kb0; kb < x.kb1 && ok; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort_flag, p.status, p.wait_limit_ns);
          if (!ok) break;
          uint8_t *st = smem + (size_t)s * L::kStage;
          if (rank == 0) mbar_expect_tx(&full[s], 2 * P * (a_bytes + b_bytes));
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          const int k0 = kb * BK;
#pragma unroll
          for (int pl = 0; pl < P; ++pl) {
            uint8_t *ta = st + pl * L::kATile, *tb = st + P * L::kATile + pl * L::kBTile;
            if (!p.a_mn) {
              tma_load_3d_pair(ta, &map_a, bar, k0, m0, pl);
            } else {
              tma_load_3d_pair(ta, &map_a, bar, m0, k0, pl);
              tma_load_3d_pair(ta + BK * 128, &map_a, bar, m0 + 64, k0, pl);
            }
            if (!p.b_mn) {
              tma_load_3d_pair(tb, &map_b, bar, k0, n0, pl);
            } else {
              for (int nb = 0; nb < half_n; nb += 64)
                tma_load_3d_pair(tb + (nb / 64) * BK * 128, &map_b, bar, n0 + nb, k0, pl);
            }
          }
        }
      }
      // the leader's last stage releases must have landed here before this CTA may exit
      for (int j = 0; j < STAGES && ok; ++j, ++it)
        ok = mbar_wait(&empty[it % STAGES], ((it / STAGES) & 1) ^ 1, abort_flag, p.status, p.wait_limit_ns);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader only)
    if (rank == 0 && elect_one()) {
      const uint32_t fmt = p.fp16 ? 0u : 1u;
      const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(p.a_mn ? 1 : 0) << 15) |
                             ((uint32_t)(p.b_mn ? 1 : 0) << 16) | ((uint32_t)(p.BN >> 3) << 17) |
                             ((uint32_t)(BM2 >> 4) << 24);
      constexpr uint32_t kLayout = BK == 64 ? 2u : 4u;
      uint32_t it = 0, unit = 0;
      bool ok = true;
      for (int w = pair; w < num_work && ok; w += num_pairs) {
        const Work x = decode_work_pair(p, w);
        for (int c0 = x.kb0; c0 < x.kb1 && ok; c0 += p.kc, ++unit) {
          const int c1 = min(x.kb1, c0 + p.kc);
          // one plane: the two accumulator buffers alternate, so the next tile's MMAs run
          // while the epilogue drains this one
          const int buf = P == 1 ? (int)(unit & 1) : 0;
          const uint32_t round = P == 1 ? (unit >> 1) : unit;
          ok = mbar_wait(&tmem_empty[buf], (round & 1) ^ 1, abort_flag, p.status, p.wait_limit_ns);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t d_main = tmem_base + (uint32_t)buf * kTmemBuf;
          const uint32_t d_small = tmem_base + kTmemBuf;
          for (int kb = c0; kb < c1 && ok; ++kb, ++it) {
            const int s = it % STAGES;
            ok = mbar_wait(&full[s], (it / STAGES) & 1, abort_flag, p.status, p.wait_limit_ns);
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t sa = smem_u32(smem + (size_t)s * L::kStage);
            const uint32_t sb = sa + P * L::kATile;
#pragma unroll
            for (int ks = 0; ks < BK / 16; ++ks) {
#pragma unroll
              for (int q = 0; q < Pairs<P>::n; ++q) {
                const uint32_t ta = sa + Pairs<P>::a(q) * L::kATile;
                const uint32_t tb = sb + Pairs<P>::b(q) * L::kBTile;
                const uint64_t da = p.a_mn ? make_desc(ta + ks * 2048, BK * 128, 1024, 2u)
                                           : make_desc(ta + ks * 32, 16, 8 * BK * 2, kLayout);
                const uint64_t db = p.b_mn ? make_desc(tb + ks * 2048, BK * 128, 1024, 2u)
                                           : make_desc(tb + ks * 32, 16, 8 * BK * 2, kLayout);
                const bool first_step = kb == c0 && ks == 0;
                if (q == 0 || P == 1) umma_pair(d_main, da, db, idesc, first_step ? 0u : 1u);
                else umma_pair(d_small, da, db, idesc, (first_step && q == 1) ? 0u : 1u);
              }
            }
            tcgen05_commit_pair(&empty[s]);
          }
          if (ok) tcgen05_commit_pair(&tmem_full[buf]);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs)
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    uint8_t *epi_stage = smem + L::kEpiOffset + (warp - 2) * kEpiBlockBytes;
    uint32_t unit = 0, blocks_done = 0;
    bool ok = true;
    const float out_scale = (p.scale_a ? *p.scale_a : 1.f) * (p.scale_b ? *p.scale_b : 1.f);
    float seen_max = 0.f, slope_max = 0.f;
    const int col_lo = half * 128, col_hi = min(p.BN, col_lo + 128);
    const uint32_t release_bar0 = map_to_cta(smem_u32(&tmem_empty[0]), 0);
    const uint32_t release_bar1 = map_to_cta(smem_u32(&tmem_empty[1]), 0);
    for (int w = pair; w < num_work && ok; w += num_pairs) {
      const Work x = decode_work_pair(p, w);
      const int row0 = x.m0 + (int)rank * BM + q * 32;
      const int row = row0 + lane;
      float *crow = p.C + (size_t)x.split * p.split_stride + (size_t)row * p.ldc;
      const float *bias = x.split == 0 ? p.bias : nullptr;
      for (int c0 = x.kb0; c0 < x.kb1 && ok; c0 += p.kc, ++unit) {
        const bool first = c0 == x.kb0;
        const int buf = P == 1 ? (int)(unit & 1) : 0;
        const uint32_t round = P == 1 ? (unit >> 1) : unit;
        // the node of the warp's first edge and the offsets of the 32 nodes from there on,
        // fetched while the tile is still being formed
        int node = 0, rp_l = 0;
        if (EPI == ZP_EPI_ROTATE_BACK && row0 < p.M) {
          node = p.epi.block_node[row0 >> 5];
          rp_l = p.epi.row_ptr[min(node + lane, p.epi.n_nodes)];
        }
        ok = mbar_wait(&tmem_full[buf], round & 1, abort_flag, p.status, p.wait_limit_ns);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)buf * kTmemBuf;
        float v[4][32];
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const int cc = col_lo + 32 * b;
          if (cc < col_hi) {
            // 16 columns at a time, the small-product accumulator added in place: the slice
            // itself (128 values per thread) leaves little room for staging registers
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              // both accumulators' loads are in flight together: one wait per 16 columns
              uint32_t r[16], r2[16];
              tmem_ld16(t_row + cc + 16 * h, r);
              if (P != 1) tmem_ld16(t_row + kTmemBuf + cc + 16 * h, r2);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                float a = __uint_as_float(r[j]);
                if (P != 1) a += __uint_as_float(r2[j]);
                v[b][16 * h + j] = a * out_scale;
              }
            }
          }
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(buf ? release_bar1 : release_bar0);

        if (EPI != ZP_EPI_NONE) {
          if (L::kTmaEpilogue)
            epilogue_fused<EPI>(p, &map_c, v, epi_stage, lane, row0, x.n0, col_lo, col_hi, bias,
                                seen_max, slope_max, node, rp_l);
        } else if (L::kTmaEpilogue && p.tma_store) {
          epilogue_store_tma<1>(p, &map_c, v, epi_stage, lane, row0, x.n0, col_lo, col_hi, x.split,
                                bias, first, seen_max, blocks_done);
        } else if (row < p.M) {
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const int cc = col_lo + 32 * b;
            if (cc >= col_hi) continue;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const int n = x.n0 + cc + j;
              if (cc + j < p.BN && n + 3 < p.N) {
                float4 o = make_float4(v[b][j], v[b][j + 1], v[b][j + 2], v[b][j + 3]);
                if (first) {
                  if (bias) {
                    const float4 bv = *reinterpret_cast<const float4 *>(bias + n);
                    o.x += bv.x; o.y += bv.y; o.z += bv.z; o.w += bv.w;
                  }
                } else {
                  const float4 old = *reinterpret_cast<const float4 *>(crow + n);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4 *>(crow + n) = o;
                seen_max = fmaxf(seen_max, fmaxf(fmaxf(fabsf(o.x), fabsf(o.y)),
                                                 fmaxf(fabsf(o.z), fabsf(o.w))));
              } else if (cc + j < p.BN) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                  if (n + u < p.N) {
                    const float base = first ? (bias ? bias[n + u] : 0.f) : crow[n + u];
                    const float o = v[b][j + u] + base;
                    crow[n + u] = o;
                    seen_max = fmaxf(seen_max, fabsf(o));
                  }
              }
            }
          }
        }
      }
    }
    if (L::kTmaEpilogue && p.tma_store && lane == 0) bulk_wait_all();   // this warp's stores are done
    if (p.absmax_out) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) seen_max = fmaxf(seen_max, __shfl_xor_sync(0xffffffffu, seen_max, o));
      if (lane == 0 && seen_max > 0.f) zp_atomic_absmax(p.absmax_out, seen_max);
    }
    if (EPI == ZP_EPI_GATE && p.epi.slope_max) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) slope_max = fmaxf(slope_max, __shfl_xor_sync(0xffffffffu, slope_max, o));
      if (lane == 0 && slope_max > 0.f) zp_atomic_absmax(p.epi.slope_max, slope_max);
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();                   // neither CTA frees TMEM or exits while its peer still works
  if (warp == 1) {
    __syncwarp();
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u)
                 : "memory");
  }
}

template <int P, int BK, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_c,
                    const __grid_constant__ GemmParams p) {
  gemm_tc_pair_body<P, BK, STAGES, ZP_EPI_NONE>(map_a, map_b, map_c, p);
}
template <int P, int BK, int STAGES, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_pair_fused_kernel(const __grid_constant__ CUtensorMap map_a,
                          const __grid_constant__ CUtensorMap map_b,
                          const __grid_constant__ CUtensorMap map_c,
                          const __grid_constant__ GemmParams p) {
  gemm_tc_pair_body<P, BK, STAGES, EPI>(map_a, map_b, map_c, p);
}

// block_node[b] = the last node n with row_ptr[n] <= 32 b: the node of the first edge of 32-edge
// block b (row_ptr[0] = 0 and row_ptr[n_nodes] = E > 32 b)
__global__ void block_node_kernel(int64_t n_blocks, int n_nodes, const int32_t *__restrict__ row_ptr,
                                  int32_t *__restrict__ block_node) {
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= n_blocks) return;
  const int e = (int)(b * 32);
  int lo = 0, hi = n_nodes;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (row_ptr[mid] <= e) lo = mid; else hi = mid;
  }
  block_node[b] = lo;
}

// ---- host side ---------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 3-d map over (inner, outer, plane) of a bf16 operand
int make_map(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer, uint64_t planes,
             uint64_t ld, uint64_t plane_stride, uint32_t box_inner, uint32_t box_outer,
             CUtensorMapSwizzle swz, int fp16) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return ZP_ERR_CUDA;
  const cuuint64_t dims[3] = {inner, outer, planes};
  const cuuint64_t strides[2] = {ld * 2, plane_stride * 2};
  const cuuint32_t box[3] = {box_inner, box_outer, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void *>(base), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    zp_set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
    return ZP_ERR_CUDA;
  }
  return ZP_OK;
}

// Tile width: the multiple of `step` in [cap/2, cap] that wastes the fewest padded columns
// (ties: the widest); problems narrower than cap/2 get one tile.
// 3-d map over (column, row, split) of the fp32 output, 32 x 32 boxes under the 128-byte swizzle
int make_map_c(CUtensorMap *map, float *C, uint64_t N, uint64_t M, uint64_t splits, uint64_t ldc,
               uint64_t split_stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return ZP_ERR_CUDA;
  const cuuint64_t dims[3] = {N, M, splits};
  const cuuint64_t strides[2] = {ldc * 4, (splits > 1 ? split_stride : ldc * M) * 4};
  const cuuint32_t box[3] = {32, 32, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, C, dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    zp_set_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled (output)");
    return ZP_ERR_CUDA;
  }
  return ZP_OK;
}

int pick_bn(int64_t N, int cap, int step = 16) {
  if (N <= cap / 2) return (int)(zp_ceil_div(N, step) * step);
  int best = cap;
  int64_t best_pad = zp_ceil_div(N, cap) * cap;
  for (int bn = cap - step; bn >= cap / 2; bn -= step) {
    const int64_t pad = zp_ceil_div(N, bn) * bn;
    if (pad < best_pad) { best_pad = pad; best = bn; }
  }
  return best;
}

// The CTA-pair kernel serves the two-plane (fp16) and one-plane (bf16) formats unless the caller
// forces a kernel:
// variant 2 = single-CTA kernel, variant 3 = pair kernel.
bool pair_enabled() {
  static int on = -1;
  if (on < 0) {
    const char *e = getenv("ZP_GEMM_PAIR");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}
int device_sms() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}
// Expected utilisation of the tensor pipes for one kernel choice and K split: padded-tile waste
// times the evenness of the last wave, with the pair's lighter operand feed counted as a gain.
double launch_score(const ZpGemmTc &g, bool pair, int splits) {
  const int64_t units = pair ? device_sms() / 2 : device_sms();
  const int tm = pair ? 256 : BM;
  const int bn = pair ? pick_bn(g.N, 256, g.b_mn ? 128 : 32) : pick_bn(g.N, 256, g.b_mn ? 64 : 32);
  const int64_t tiles_m = zp_ceil_div(g.M, tm), tiles_n = zp_ceil_div(g.N, bn);
  const double pad = (double)(g.M * g.N) / (double)(tiles_m * tm * tiles_n * bn);
  const int64_t items = tiles_m * tiles_n * splits;
  const double wave = (double)items / (double)(zp_ceil_div(items, units) * units);
  // one plane (one MMA pass per k-block) leans on the operand feed harder than two planes do
  const double feed = !pair ? 1.0 : g.planes == 1 ? 1.25 : 1.12;
  return pad * wave * feed - 0.004 * splits;
}
bool use_pair(const ZpGemmTc &g) {
  if (g.planes != 2 && g.planes != 1) return false;
  if (g.variant == 2) return false;
  if (g.variant == 3) return true;
  if (!pair_enabled()) return false;
  // short contractions leave the pair's cross-SM hand-offs exposed on every tile
  if (g.K < 512) return false;
  int s = g.ksplit < 1 ? 1 : g.ksplit;
  return launch_score(g, true, s) >= launch_score(g, false, s);
}

int block_k(const ZpGemmTc &g) {
  if (use_pair(g)) return 64;
  return ((g.planes == 3 && g.variant != 1) || g.planes == 2) ? 32 : 64;
}

void split_plan(const ZpGemmTc &g, int bk, int *ksplit, int *kbs, int *num_k) {
  *num_k = (int)zp_ceil_div(g.K, bk);
  int req = g.ksplit < 1 ? 1 : g.ksplit;
  if (req > *num_k) req = *num_k;
  *kbs = (int)zp_ceil_div(*num_k, req);
  *ksplit = (int)zp_ceil_div(*num_k, *kbs);
}

// One-time set-up of a kernel is per device (the raised dynamic shared-memory limit is an
// attribute of the function ON a device): remembered per device ordinal under a lock, since a
// plan may be used from several host threads.
constexpr int kMaxDevices = 64;
struct PerDevice {
  std::mutex lock;
  int value[kMaxDevices];
  bool done[kMaxDevices];
  PerDevice() { for (int i = 0; i < kMaxDevices; ++i) { value[i] = 0; done[i] = false; } }
};

bool fused_mode_ok(const ZpGemmTc &g, int bk) {
  if (!g.epi || g.epi->mode == ZP_EPI_NONE) return true;
  if (g.a_mn || g.b_mn || (g.planes != 1 && g.planes != 2)) return false;
  int ksplit, kbs, num_k;
  split_plan(g, bk, &ksplit, &kbs, &num_k);
  const int kc_elems = g.kc_elems > 0 ? g.kc_elems : 2048;
  const int kc = kc_elems / bk < 1 ? 1 : kc_elems / bk;
  return ksplit == 1 && kbs <= kc && (g.epi->width % 4) == 0;
}

void fill_params(GemmParams &p, const ZpGemmTc &g, int bk) {
  p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K;
  split_plan(g, bk, &p.ksplit, &p.kb_per_split, &p.num_k);
  const int kc_elems = g.kc_elems > 0 ? g.kc_elems : 2048;
  p.kc = kc_elems / bk < 1 ? 1 : kc_elems / bk;
  p.a_mn = g.a_mn; p.b_mn = g.b_mn;
  p.fp16 = g.fp16; p.scale_a = g.scale_a; p.scale_b = g.scale_b; p.absmax_out = g.absmax_out;
  p.bias = g.bias; p.C = g.C; p.ldc = g.ldc; p.split_stride = g.split_stride; p.status = g.status;
  p.wait_limit_ns = g.wait_limit_ns > 0 ? (uint64_t)g.wait_limit_ns : kWaitLimitNs;
  p.unarmed = g.unarmed;
  if (g.epi) p.epi = *g.epi;
  else p.epi.mode = ZP_EPI_NONE;
}

template <int P, int BK, int STAGES, int BN_CAP, int EPI, int EB = 1>
int launch_e(const ZpGemmTc &g, cudaStream_t st) {
  using L = SmemLayout<P, BK, STAGES, BN_CAP, EB>;
  static_assert(EB == 1 || EPI == ZP_EPI_NONE, "two store buffers only in the plain epilogue");
  static_assert(L::kTotal <= 232448, "shared memory budget of one CTA");
  static_assert(EPI == ZP_EPI_NONE || L::kTmaEpilogue, "fused epilogues need the store stage");
  auto kernel = [] {
    if constexpr (EPI == ZP_EPI_NONE) return gemm_tc_kernel<P, BK, STAGES, BN_CAP, EB>;
    else return gemm_tc_fused_kernel<P, BK, STAGES, BN_CAP, EPI>;
  }();
  int dev = 0, sms = 148;
  ZP_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return ZP_ERR_UNSUPPORTED;
  static PerDevice configured;
  {
    std::lock_guard<std::mutex> hold(configured.lock);
    if (!configured.done[dev]) {
      ZP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      configured.done[dev] = true;
    }
  }
  GemmParams p;
  fill_params(p, g, BK);
  // whole 32-column store blocks; MN-major B tiles come in 64-wide blocks
  p.BN = pick_bn(g.N, BN_CAP, g.b_mn ? 64 : 32);
  p.num_m = (int)zp_ceil_div(g.M, BM);
  p.num_n = (int)zp_ceil_div(g.N, p.BN);
  const CUtensorMapSwizzle kswz = BK == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUtensorMap ma, mb;
  int rc;
  if (!g.a_mn) rc = make_map(&ma, g.A, g.K, g.M, P, g.lda, g.a_plane, BK, BM, kswz, g.fp16);
  else rc = make_map(&ma, g.A, g.M, g.K, P, g.lda, g.a_plane, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B, g.fp16);
  if (rc) return rc;
  if (!g.b_mn) rc = make_map(&mb, g.B, g.K, g.N, P, g.ldb, g.b_plane, BK, p.BN, kswz, g.fp16);
  else rc = make_map(&mb, g.B, g.N, g.K, P, g.ldb, g.b_plane, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B, g.fp16);
  if (rc) return rc;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  CUtensorMap mc;
  const int chunks = (int)zp_ceil_div(p.kb_per_split, p.kc);
  p.tma_store = EPI == ZP_EPI_NONE ? (L::kTmaEpilogue && !(g.absmax_out && chunks > 1))
                                   : p.epi.store_c;
  if (p.tma_store) {
    if ((rc = make_map_c(&mc, g.C, g.N, g.M, p.ksplit, g.ldc, g.split_stride))) return rc;
  } else {
    mc = ma;                                      // never read
  }
  const int work = p.num_m * p.num_n * p.ksplit;
  const int grid = work < sms ? work : sms;
  kernel<<<grid, kThreads, L::kTotal, st>>>(ma, mb, mc, p);
  ZP_LAUNCH_CHECK("gemm_tc_kernel");
  return ZP_OK;
}

template <int P, int BK, int STAGES, int BN_CAP>
int launch(const ZpGemmTc &g, cudaStream_t st) {
  const int mode = g.epi ? g.epi->mode : ZP_EPI_NONE;
  if constexpr (SmemLayout<P, BK, STAGES, BN_CAP>::kTmaEpilogue && (P == 1 || P == 2)) {
    if (mode == ZP_EPI_GATE) return launch_e<P, BK, STAGES, BN_CAP, ZP_EPI_GATE>(g, st);
    if (mode == ZP_EPI_ROTATE_BACK) return launch_e<P, BK, STAGES, BN_CAP, ZP_EPI_ROTATE_BACK>(g, st);
  }
  if (mode != ZP_EPI_NONE) return ZP_ERR_UNSUPPORTED;
  return launch_e<P, BK, STAGES, BN_CAP, ZP_EPI_NONE>(g, st);
}

template <int P, int BK, int STAGES, int EPI>
int launch_pair_e(const ZpGemmTc &g, cudaStream_t st) {
  using L = SmemLayoutPair<P, BK, STAGES>;
  static_assert(L::kTotal <= 232448, "shared memory budget of one CTA");
  static_assert(EPI == ZP_EPI_NONE || L::kTmaEpilogue, "fused epilogues need the store stage");
  auto kernel = [] {
    if constexpr (EPI == ZP_EPI_NONE) return gemm_tc_pair_kernel<P, BK, STAGES>;
    else return gemm_tc_pair_fused_kernel<P, BK, STAGES, EPI>;
  }();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = L::kTotal; cfg.stream = st;
  cfg.attrs = attr; cfg.numAttrs = 1;
  int dev = 0;
  ZP_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return ZP_ERR_UNSUPPORTED;
  static PerDevice pairs;               // co-resident CTA pairs of this kernel, per device
  int max_pairs;
  {
    std::lock_guard<std::mutex> hold(pairs.lock);
    if (!pairs.done[dev]) {
      ZP_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      int sms = 148, n = 0;
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      cfg.gridDim = dim3((unsigned)(sms / 2 * 2));
      ZP_CUDA(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
      pairs.value[dev] = n < sms / 2 ? n : sms / 2;
      pairs.done[dev] = true;
    }
    max_pairs = pairs.value[dev];
  }
  if (max_pairs < 1) return ZP_ERR_UNSUPPORTED;
  GemmParams p;
  fill_params(p, g, BK);
  // whole 32-column store blocks; each CTA's half of an MN-major tile comes in 64-wide blocks
  p.BN = pick_bn(g.N, 256, g.b_mn ? 128 : 32);
  p.num_m = (int)zp_ceil_div(g.M, BM2);
  p.num_n = (int)zp_ceil_div(g.N, p.BN);
  const CUtensorMapSwizzle kswz = BK == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUtensorMap ma, mb;
  int rc;
  if (!g.a_mn) rc = make_map(&ma, g.A, g.K, g.M, P, g.lda, g.a_plane, BK, BM, kswz, g.fp16);
  else rc = make_map(&ma, g.A, g.M, g.K, P, g.lda, g.a_plane, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B, g.fp16);
  if (rc) return rc;
  if (!g.b_mn) rc = make_map(&mb, g.B, g.K, g.N, P, g.ldb, g.b_plane, BK, p.BN / 2, kswz, g.fp16);
  else rc = make_map(&mb, g.B, g.N, g.K, P, g.ldb, g.b_plane, 64, BK, CU_TENSOR_MAP_SWIZZLE_128B, g.fp16);
  if (rc) return rc;
  CUtensorMap mc;
  const int chunks = (int)zp_ceil_div(p.kb_per_split, p.kc);
  p.tma_store = EPI == ZP_EPI_NONE ? (L::kTmaEpilogue && !(g.absmax_out && chunks > 1))
                                   : p.epi.store_c;
  if (p.tma_store) {
    if ((rc = make_map_c(&mc, g.C, g.N, g.M, p.ksplit, g.ldc, g.split_stride))) return rc;
  } else {
    mc = ma;                                      // never read
  }
  const int work = p.num_m * p.num_n * p.ksplit;
  cfg.gridDim = dim3((unsigned)(2 * (work < max_pairs ? work : max_pairs)));
  ZP_CUDA(cudaLaunchKernelEx(&cfg, kernel, ma, mb, mc, p));
  ZP_LAUNCH_CHECK("gemm_tc_pair_kernel");
  return ZP_OK;
}

template <int P, int BK, int STAGES>
int launch_pair(const ZpGemmTc &g, cudaStream_t st) {
  const int mode = g.epi ? g.epi->mode : ZP_EPI_NONE;
  if (mode == ZP_EPI_GATE) return launch_pair_e<P, BK, STAGES, ZP_EPI_GATE>(g, st);
  if (mode == ZP_EPI_ROTATE_BACK) return launch_pair_e<P, BK, STAGES, ZP_EPI_ROTATE_BACK>(g, st);
  return launch_pair_e<P, BK, STAGES, ZP_EPI_NONE>(g, st);
}

}  // namespace

int zp_gemm_tc_splits(const ZpGemmTc &g) {
  if (g.K <= 0) return 1;
  int ksplit, kbs, num_k;
  split_plan(g, block_k(g), &ksplit, &kbs, &num_k);
  return ksplit;
}

int zp_gemm_tc_pick_splits(const ZpGemmTc &g, int max_splits) {
  ZpGemmTc t = g;
  int best = 1;
  double best_score = -1.0;
  for (int s = 1; s <= max_splits; ++s) {
    t.ksplit = s;
    const double score = launch_score(t, use_pair(t), s);
    if (score > best_score) { best_score = score; best = s; }
  }
  return best;
}

int zp_launch_block_nodes(int64_t E, int64_t N, const int32_t *row_ptr, int32_t *block_node,
                          cudaStream_t st) {
  const int64_t nb = zp_ceil_div(E, 32);
  if (nb == 0 || N == 0) return ZP_OK;
  block_node_kernel<<<(unsigned)zp_ceil_div(nb, 256), 256, 0, st>>>(nb, (int)N, row_ptr, block_node);
  ZP_LAUNCH_CHECK("block_node_kernel");
  return ZP_OK;
}

bool zp_gemm_tc_fusable(const ZpGemmTc &g) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return false;
  return fused_mode_ok(g, block_k(g));
}

int zp_launch_gemm_tc(const ZpGemmTc &g, cudaStream_t st) {
  if (g.M <= 0 || g.N <= 0) return ZP_OK;
  if (g.K <= 0) return ZP_ERR_INVALID_ARG;
  if (g.fp16 != (g.planes == 2)) return ZP_ERR_UNSUPPORTED;   // fp16 planes come in pairs
  if (!fused_mode_ok(g, block_k(g))) return ZP_ERR_UNSUPPORTED;
  if ((g.lda % 8) || (g.ldb % 8) || (g.a_plane % 8) || (g.b_plane % 8) || (g.ldc % 4) ||
      (g.split_stride % 4))
    return ZP_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(g.A) | reinterpret_cast<uintptr_t>(g.B) |
       reinterpret_cast<uintptr_t>(g.C)) & 15)
    return ZP_ERR_INVALID_ARG;
  if (use_pair(g))
    return g.planes == 2 ? launch_pair<2, 64, 3>(g, st) : launch_pair<1, 64, 6>(g, st);
  if (g.a_mn || g.b_mn) {
    // MN-major tiles are [BK][64] blocks under the 128-byte swizzle
    if (g.planes == 3)
      return g.variant == 1 ? launch<3, 64, 2, 128>(g, st) : launch<3, 32, 3, 256>(g, st);
    if (g.planes == 2) return launch<2, 32, 4, 256>(g, st);
    if (g.planes == 1) return launch<1, 64, 4, 256>(g, st);
    return ZP_ERR_UNSUPPORTED;
  }
  // a contraction of at most four k-blocks is bound by its output stores: fewer operand stages,
  // two store buffers per epilogue warp
  const bool store_bound = !(g.epi && g.epi->mode) && g.ksplit <= 1;
  if (g.planes == 2) {
    if (store_bound && g.K <= 128) return launch_e<2, 32, 2, 256, ZP_EPI_NONE, 2>(g, st);
    return launch<2, 32, 4, 256>(g, st);
  }
  if (g.planes == 3)
    return g.variant == 1 ? launch<3, 64, 2, 128>(g, st) : launch<3, 32, 3, 256>(g, st);
  if (g.planes == 1) {
    if (store_bound && g.K <= 256) return launch_e<1, 64, 2, 256, ZP_EPI_NONE, 2>(g, st);
    return launch<1, 64, 4, 256>(g, st);
  }
  return ZP_ERR_UNSUPPORTED;
}
