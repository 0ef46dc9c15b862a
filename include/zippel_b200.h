/* zippel_b200 -- C ABI of the B200 (sm_100a) kernels for the eSEN SO(2) edge-convolution
 * block: gather, per-edge Wigner-D rotation, per-m SO(2) linear mixing, gate, inverse
 * rotation, deterministic segmented scatter, and the matching first-order VJP.
 *
 * The reference project has no native boundary: its GPU back end is a Python API
 * (codegen/compose.py:113-239 compile_program / allocate / run_program) that launches
 * run-time generated kernels.  Each entry point below names the reference code whose work
 * it takes over.
 *
 * Conventions
 *   - every function returns a zp_status (0 = ok); nothing throws across the boundary
 *   - unless said otherwise every pointer is DEVICE memory owned by the caller, fp32 values,
 *     int32 indices, row-major, 16-byte aligned
 *   - every launch goes to the cudaStream_t given as `stream` (an opaque pointer here)
 *   - edges are expected in destination-sorted order (see zp_csr_build); `row_ptr[n]` ..
 *     `row_ptr[n+1]` are the edges whose destination is node n
 *   - a zp_plan owns static tables only (layout indices, the J matrices); it may be shared
 *     by threads that use different streams and different workspaces
 */
#ifndef ZIPPEL_B200_H
#define ZIPPEL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum zp_status {
  ZP_OK = 0,
  ZP_ERR_INVALID_ARG = 1,      /* null pointer, negative size, misaligned pointer          */
  ZP_ERR_UNSUPPORTED = 2,      /* lmax/mmax/channel combination outside the built kernels  */
  ZP_ERR_WORKSPACE = 3,        /* workspace smaller than zp_workspace_bytes()              */
  ZP_ERR_CUDA = 4,             /* a CUDA runtime call failed; see zp_last_cuda_error()     */
  ZP_ERR_DEVICE_TIMEOUT = 5,   /* a bounded device-side wait gave up (status word set)     */
  ZP_ERR_NO_DEVICE_CODE = 6,   /* the library holds no code for this GPU (needs sm_100a)   */
  ZP_ERR_TOO_LARGE = 7         /* sizes exceed a fixed capacity of the entry point           */
} zp_status;

/* Mirrors the fields of the reference's BlockConfig (blocks/eso2_ref.py:51-76) that the
 * kernel path reads.  precision selects how the operands of the SO(2) contraction are carried:
 *   0  three bf16 terms per fp32 value (six tensor-core passes, ~24 bits, no range limits);
 *   1  one bf16 term (bf16 operands, fp32 accumulation);
 *   2  two fp16 terms and a per-tensor power-of-two scale derived on the device from
 *      magnitude bounds (three passes, 22 bits relative to each tensor's largest entries).  */
typedef struct zp_config {
  int32_t lmax;
  int32_t mmax;
  int32_t sphere_channels;   /* C  */
  int32_t hidden_channels;   /* H  */
  int32_t precision;
} zp_config;

/* Derived sizes, filled by zp_plan_sizes(). */
typedef struct zp_sizes {
  int32_t K;         /* (lmax+1)^2, rows of x_node / node_out                               */
  int32_t Km;        /* m'-major rows with |m| <= mmax                                      */
  int32_t nnz;       /* nonzeros of one edge's [Km, K] rotation (block diagonal in l)       */
  int32_t nnz_pad;   /* row stride of the packed rotation array (nnz rounded up to 4)       */
  int32_t R;         /* radial width: 2C * sum_m m_size[m]                                  */
  int32_t n_gate;    /* lmax * H gate scalars emitted by conv1's m = 0 head                 */
  int32_t w1_cols;   /* n_gate + Km*H: row width of conv1's output                          */
} zp_sizes;

typedef struct zp_plan zp_plan;

const char *zp_status_string(int status);
/* Text of the last CUDA error seen by this thread inside the library. */
const char *zp_last_cuda_error(void);
/* 1 if the current device can run the kernels in this library (compute capability 10.x). */
int zp_device_supported(void);

/* Layout tables (replaces Layout.make / to_m / gate_expand_index, blocks/eso2_ref.py:98-146,
 * with the rectangular [Km, K] selection for mmax < lmax).  `jd_host` is HOST memory: the
 * J_l matrices for l = 0..lmax, each (2l+1)^2 doubles row-major, concatenated.             */
int zp_plan_create(const zp_config *cfg, const double *jd_host, zp_plan **plan_out);
int zp_plan_destroy(zp_plan *plan);
int zp_plan_sizes(const zp_plan *plan, zp_sizes *out);
/* Host copies of the index tables, for callers and tests: row_l/row_m [Km] give (l, signed m)
 * of each m' row, rot_off [Km] the offset of that row's 2l+1 entries in a packed rotation,
 * gate_idx [Km] the gate scalar block (l-1) used by the row (-1 for row 0).                */
int zp_plan_tables(const zp_plan *plan, int32_t *row_l, int32_t *row_m, int32_t *rot_off,
                   int32_t *gate_idx);

/* Destination-sorted edge order and CSR offsets (the reference scatters with index_add_,
 * blocks/eso2_ref.py:346-349, and has no sorted form).  Stable sort of the E edges by
 * (dst, src, original position); `perm[i]` is the original position of sorted edge i.
 * Also builds the source-sorted view used by the backward scatter: `perm_src[i]` is the
 * SORTED-edge id of the i-th edge in (src, sorted id) order and `row_ptr_src` its offsets.
 * `work` needs zp_csr_work_bytes(E, N) bytes.                                              */
size_t zp_csr_work_bytes(int64_t n_edges, int64_t n_nodes);
/* Node indices outside [0, n_nodes) are never used as addresses: such an edge is left out and a
 * flag in `work` is raised (the reference's torch indexing raises on the same input).
 * zp_csr_status waits for `stream` (the one the build was given) and reads the flag:
 * *status_out = ZP_OK, or ZP_ERR_INVALID_ARG when the arrays of that call are not a valid sort.
 * Even then every entry stays inside its range: row_ptr[n_nodes] is the number of edges that were
 * kept, and the slots past it hold an edge 0 -> 0 at original position 0, so a caller that
 * launches per-edge work over all E slots without reading the flag (a recorded graph replay)
 * never indexes outside its arrays.                                                           */
int zp_csr_status(const void *work, void *stream, int *status_out);
int zp_csr_build(const int64_t *edge_index /* [2,E] int64: row 0 src, row 1 dst */,
                 int64_t n_edges, int64_t n_nodes,
                 int32_t *perm, int32_t *src_sorted, int32_t *dst_sorted, int32_t *row_ptr,
                 int32_t *perm_src, int32_t *row_ptr_src, void *work, size_t work_bytes,
                 void *stream);

/* zp_csr_build for callers that must not allocate device memory.  This entry point has no
 * counterpart in the reference.  A molecular-dynamics driver typically reserves all device
 * memory when it starts and then rebuilds its neighbour list every few steps from inside the
 * stepping loop; at that point it has no spare buffer to lend as `work`, and it does not want a
 * runtime allocation either, because an allocation stalls the whole device and can fail long
 * after start-up.  For such callers the scratch of the sort lives in a fixed array inside the
 * library: ZP_CSR_STATIC_BYTES of device memory on every GPU that loads the library, held
 * until the process exits.  Inputs and outputs are the caller's, exactly as for zp_csr_build,
 * and the results are identical.
 *   - Limits: n_edges <= ZP_CSR_STATIC_MAX_EDGES and n_nodes <= ZP_CSR_STATIC_MAX_NODES,
 *     otherwise ZP_ERR_TOO_LARGE and nothing is launched.
 *   - The first call on a device looks up the array's device address (no allocation); make
 *     that first call before starting any stream capture on that device.
 *   - All calls on a device share the one array.  Its counters are cleared at the start of
 *     every call, so stale contents never matter, but two calls that can run on the GPU at the
 *     same time (different streams, different host threads) race on it: serialise them.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.                        */
#define ZP_CSR_STATIC_MAX_EDGES 262144
#define ZP_CSR_STATIC_MAX_NODES 65536
#define ZP_CSR_STATIC_BYTES 1574144
int zp_csr_build_static(const int64_t *edge_index, int64_t n_edges, int64_t n_nodes,
                        int32_t *perm, int32_t *src_sorted, int32_t *dst_sorted,
                        int32_t *row_ptr, int32_t *perm_src, int32_t *row_ptr_src, void *stream);
/* zp_csr_status for the last zp_csr_build_static on the current device. */
int zp_csr_static_status(void *stream, int *status_out);

/* Packed rotation rot[e, rot_off[r] + j] = D_l(e)[row of (l, m_r), j], the nonzeros of
 * to_m @ wigner (replaces wigner_from_edge_vec, blocks/wigner.py:115-160, and the einsum at
 * blocks/eso2_ref.py:330-331).  edge_vec [E,3], cos_g/sin_g [E, lmax+1], rot [E, nnz_pad].  */
int zp_wigner_forward(const zp_plan *plan, int64_t n_edges, const float *edge_vec,
                      const float *cos_g, const float *sin_g, float *rot, void *stream);
/* VJP of the above w.r.t. edge_vec (autograd through blocks/wigner.py:60-160, including the
 * clamp_min masks).  grad_rot [E, nnz_pad] -> grad_edge_vec [E,3] (overwritten).            */
int zp_wigner_backward(const zp_plan *plan, int64_t n_edges, const float *edge_vec,
                       const float *cos_g, const float *sin_g, const float *grad_rot,
                       float *grad_edge_vec, void *stream);

/* SO(2) weights in the reference module's own layout (blocks/eso2_ref.py:184-202):
 * c1_w0 [n_gate + (lmax+1)H, (lmax+1)*2C] + bias, c1_wm[m-1] [2*km*H, km*2C],
 * c2_w0 [(lmax+1)C, (lmax+1)H] + bias, c2_wm[m-1] [2*km*C, km*H]; km = lmax+1-m.
 * The pointer arrays c1_wm / c2_wm are HOST arrays of mmax device pointers.                */
typedef struct zp_weights {
  const float *c1_w0;
  const float *c1_b0;
  const float *const *c1_wm;
  const float *c2_w0;
  const float *c2_b0;
  const float *const *c2_wm;
} zp_weights;

typedef struct zp_weight_grads {
  float *c1_w0;
  float *c1_b0;
  float *const *c1_wm;
  float *c2_w0;
  float *c2_b0;
  float *const *c2_wm;
} zp_weight_grads;

/* Bytes of scratch + saved activations for E edges / N nodes (N = the n_nodes given to the
 * forward call it serves; the backward's share does not depend on it).  with_backward = ZP_WS_FORWARD: zp_eso2_forward alone; ZP_WS_BACKWARD:
 * zp_eso2_forward and the zp_eso2_backward that follows it, which must get the same workspace;
 * ZP_WS_INFERENCE: zp_eso2_forward_inference.                                                */
#define ZP_WS_FORWARD 0
#define ZP_WS_BACKWARD 1
#define ZP_WS_INFERENCE 2
size_t zp_workspace_bytes(const zp_plan *plan, int64_t n_nodes, int64_t n_edges,
                          int with_backward);

/* node_out[n] = sum over edges e into n of  rot_e^T * env_e * conv2(gate(conv1(radial_e .
 * (rot_e [x_src ; x_dst])))).  Replaces blocks/eso2_ref.py:334-349 and the 55-kernel program
 * run by codegen/compose.py:218-239.  x_node, node_out [N, K, C]; edge_vec [E,3];
 * cos_g, sin_g [E, lmax+1]; radial [E, R]; env [E]; src, dst [E]; row_ptr [N+1].
 * node_out is overwritten (rows without incoming edges become zero).
 * Node ranges: to get rows n0..n1 only, pass n_nodes = n1 - n0, row_ptr + n0 and a node_out of
 * n1 - n0 rows with the edges into those nodes; src / dst keep the numbering of x_node, which
 * then has more than n_nodes rows (every row an edge names is read, no other).             */
int zp_eso2_forward(const zp_plan *plan, int64_t n_nodes, int64_t n_edges,
                    const float *x_node, const float *edge_vec, const float *cos_g,
                    const float *sin_g, const float *radial, const float *env,
                    const int32_t *src, const int32_t *dst, const int32_t *row_ptr,
                    const zp_weights *w, float *node_out, void *workspace,
                    size_t workspace_bytes, void *stream);

/* zp_eso2_forward for callers that will not ask for gradients (the reference under
 * torch.no_grad(): blocks/eso2_ref.py:334-349 with nothing saved for autograd).  Same arguments
 * and result; the workspace (ZP_WS_INFERENCE) is smaller because conv1's pre-activation rows and
 * conv2's output are consumed on chip by the epilogues of the contractions (gate activation;
 * envelope, rotation back and the per-node sums) and never written.  zp_eso2_backward cannot
 * follow this call.                                                                          */
int zp_eso2_forward_inference(const zp_plan *plan, int64_t n_nodes, int64_t n_edges,
                              const float *x_node, const float *edge_vec, const float *cos_g,
                              const float *sin_g, const float *radial, const float *env,
                              const int32_t *src, const int32_t *dst, const int32_t *row_ptr,
                              const zp_weights *w, float *node_out, void *workspace,
                              size_t workspace_bytes, void *stream);

/* First-order VJP of zp_eso2_forward (what torch.autograd.grad computes through
 * blocks/eso2_ref.py:334-349; IR rule zippel/vjp.py:88-153).  Needs the workspace of the
 * matching forward call.  Outputs (all overwritten): grad_x_node [N,K,C]; grad_edge_vec
 * [E,3] (through the rotation only); grad_radial [E,R]; grad_env [E]; weight gradients in
 * the reference layout.  perm_src / row_ptr_src: the source-sorted view from zp_csr_build.
 * grad_node_out is indexed by dst and read at rows dst[0] .. dst[E-1] only (the edges are
 * destination-sorted), so a caller holding the gradient of rows n0..n1 alone passes that
 * array's address minus n0 rows.
 * gw == NULL: the parameters are frozen (a force evaluation in an MD loop, autograd with
 * requires_grad = False on the weights): the weight-gradient products, the bias column sums and
 * the unfolding are not run, everything else is unchanged.  grad_x_node == NULL: the embeddings
 * are an input without a gradient (E and dE/dpos of one block, the reference's build_force,
 * blocks/eso2_ir.py:579-590): the per-edge contributions are neither written nor summed.       */
int zp_eso2_backward(const zp_plan *plan, int64_t n_nodes, int64_t n_edges,
                     const float *grad_node_out, const float *x_node, const float *edge_vec,
                     const float *cos_g, const float *sin_g, const float *radial,
                     const float *env, const int32_t *src, const int32_t *dst,
                     const int32_t *row_ptr, const int32_t *perm_src,
                     const int32_t *row_ptr_src, const zp_weights *w, float *grad_x_node,
                     float *grad_edge_vec, float *grad_radial, float *grad_env,
                     const zp_weight_grads *gw, void *workspace, size_t workspace_bytes,
                     void *stream);

/* The edge convolution with the LAST dense layer of the radial MLP inside the call
 * (rad_func[6] of blocks/eso2_ref.py:169-182, the layer blocks/eso2_ir.py:353-358, 423-429 split per
 * m): instead of radial [E, R] the caller passes the layer's input h_rad [E, edge_channels], its
 * weight rad_w [R, edge_channels] and bias rad_b [R].  The call forms radial in its workspace, takes
 * its largest magnitude from the product's epilogue instead of scanning it, and in the backward
 * hands the gradient of radial to the layer's VJP as operand planes, so neither radial nor its
 * gradient is read back for a magnitude scan or a format change; the backward returns
 * grad_h_rad [E, edge_channels], grad_rad_w and grad_rad_b instead of grad_radial.
 * edge_channels: a multiple of 8.  Workspace: zp_workspace_bytes_radial (modes as
 * zp_workspace_bytes).  keep_for_backward = 0 behaves like zp_eso2_forward_inference.
 * In the backward gw may be NULL as in zp_eso2_backward, and grad_rad_w / grad_rad_b may be NULL
 * together (frozen layer): only grad_h_rad is then formed from the gradient of radial.          */
size_t zp_workspace_bytes_radial(const zp_plan *plan, int64_t n_nodes, int64_t n_edges,
                                 int edge_channels, int with_backward);
int zp_eso2_forward_radial(const zp_plan *plan, int64_t n_nodes, int64_t n_edges,
                           const float *x_node, const float *edge_vec, const float *cos_g,
                           const float *sin_g, const float *h_rad, const float *rad_w,
                           const float *rad_b, int edge_channels, const float *env,
                           const int32_t *src, const int32_t *dst, const int32_t *row_ptr,
                           const zp_weights *w, float *node_out, void *workspace,
                           size_t workspace_bytes, int keep_for_backward, void *stream);
int zp_eso2_backward_radial(const zp_plan *plan, int64_t n_nodes, int64_t n_edges,
                            const float *grad_node_out, const float *x_node,
                            const float *edge_vec, const float *cos_g, const float *sin_g,
                            const float *h_rad, const float *rad_w, const float *rad_b,
                            int edge_channels, const float *env, const int32_t *src,
                            const int32_t *dst, const int32_t *row_ptr, const int32_t *perm_src,
                            const int32_t *row_ptr_src, const zp_weights *w, float *grad_x_node,
                            float *grad_edge_vec, float *grad_h_rad, float *grad_rad_w,
                            float *grad_rad_b, float *grad_env, const zp_weight_grads *gw,
                            void *workspace, size_t workspace_bytes, void *stream);

/* The contraction engine on its own (no reference counterpart: the reference calls
 * torch.nn.functional.linear, blocks/eso2_ref.py:272,286).  Exposed for tests and benchmarks.
 * zp_split_planes writes an fp32 matrix [rows, cols] (row stride ld_in) as `planes` 16-bit
 * matrices [rows, ld_out] that sum to it (1 or 3: bf16 terms; 2: fp16 terms, unscaled), plane p starting plane_stride elements after
 * plane p-1; columns cols..ld_out-1 are zero.  zp_gemm_planes computes, on the tensor cores,
 *   C[M, N] = sum over plane pairs  A_pa  B_pb^T  (+ bias[n]),   fp32 output, row stride ldc,
 * for K-major operands X[p*plane + r*ld + k] or, with a_mn / b_mn = 1, MN-major operands
 * X[p*plane + k*ld + r].  ld, plane strides: multiples of 8; ldc: multiple of 4.
 * The contraction is accumulated in TMEM in chunks of kc_elems (0 = 2048) and the chunks are
 * summed in fp32; ksplit > 1 additionally splits it over CTAs, split s writing its partial
 * matrix at C + s*split_stride (the number actually written is returned in *splits_out and
 * never exceeds ksplit; the caller sums them).  variant selects a tile shape (0 = default).  */
int zp_split_planes(int64_t rows, int64_t cols, const float *in, int64_t ld_in, void *out,
                    int64_t ld_out, int64_t plane_stride, int planes, void *stream);
int zp_gemm_planes(zp_plan *plan, int64_t M, int64_t N, int64_t K, int planes, const void *A,
                   int64_t lda, int64_t a_plane, int a_mn, const void *B, int64_t ldb,
                   int64_t b_plane, int b_mn, const float *bias, float *C, int64_t ldc,
                   int variant, int ksplit, int64_t split_stride, int kc_elems, int *splits_out,
                   void *stream);
/* A dense layer on the same engine, in the plan's operand format: y[M,N] = x[M,K] w[N,K]^T + bias,
 * and its VJP (dx may be null; db may be null; dw may be null if dx is not: frozen layer).  Takes over the fp32 library GEMMs of the widest
 * radial-MLP layer (rad_func[6], blocks/eso2_ref.py:169-182, 327).  K and N multiples of 8.
 * `work`: zp_linear_work_bytes(plan, M, K, N) bytes of device scratch, caller-owned.           */
size_t zp_linear_work_bytes(const zp_plan *plan, int64_t M, int64_t K, int64_t N);
int zp_linear_forward(const zp_plan *plan, int64_t M, int64_t K, int64_t N, const float *x,
                      const float *w, const float *bias, float *y, void *work, size_t work_bytes,
                      void *stream);
int zp_linear_backward(const zp_plan *plan, int64_t M, int64_t K, int64_t N, const float *x,
                       const float *w, const float *dy, float *dx, float *dw, float *db,
                       void *work, size_t work_bytes, void *stream);
/* zp_linear_backward for a caller that kept the `work` buffer of the matching zp_linear_forward
 * untouched: the 16-bit planes of x and w and their scales are still there, so neither is scanned
 * or re-formatted again (x and w themselves are not read).                                     */
int zp_linear_backward_saved(const zp_plan *plan, int64_t M, int64_t K, int64_t N, const float *dy,
                             float *dx, float *dw, float *db, void *work, size_t work_bytes,
                             void *stream);

/* LayerNorm followed by SiLU over rows of `width` floats (a multiple of 4, at most 1024), and the
 * VJP: the hidden layers of the radial MLP (nn.LayerNorm + nn.SiLU, rad_func[1..2] and
 * rad_func[4..5], blocks/eso2_ref.py:170-180) in one pass each way.  The forward saves mean[rows]
 * and rstd[rows] for the backward.  dgamma/dbeta are summed in a fixed order (bit-reproducible).
 * `work`: zp_layernorm_work_bytes(width) bytes of device scratch, caller-owned.                  */
size_t zp_layernorm_work_bytes(int width);
int zp_layernorm_silu_forward(int64_t rows, int width, const float *x, const float *gamma,
                              const float *beta, float eps, float *y, float *mean, float *rstd,
                              void *stream);
int zp_layernorm_silu_backward(int64_t rows, int width, const float *x, const float *gamma,
                               const float *beta, const float *mean, const float *rstd,
                               const float *dy, float *dx, float *dgamma, float *dbeta,
                               void *work, size_t work_bytes, void *stream);

/* The energy head after the node output and its VJP (readout, blocks/eso2_ref.py:351-362 and
 * :236-238): rotation invariants of node_out [N, K, C] (the l = 0 row, and per degree l >= 1 the
 * squared norm over m), Linear((lmax+1)C -> C) with weight w0 [C, (lmax+1)C] and bias b0 [C], SiLU,
 * Linear(C -> 1) with w1 [C] and b1 [1], summed over the nodes into *energy (device).  The
 * backward takes dE (*grad_energy, device) and returns the parameter gradients and
 * grad_node_out [N, K, C], which is the upstream gradient zp_eso2_backward wants in a force
 * pass.  The hidden layer runs on the contraction engine in the plan's operand format; all sums
 * over nodes have a fixed order.  `work`: zp_readout_work_bytes() bytes; the backward reads what
 * the forward left there, so both get the same buffer.                                          */
size_t zp_readout_work_bytes(const zp_plan *plan, int64_t n_nodes);
int zp_readout_forward(const zp_plan *plan, int64_t n_nodes, const float *node_out, const float *w0,
                       const float *b0, const float *w1, const float *b1, float *energy, void *work,
                       size_t work_bytes, void *stream);
int zp_readout_backward(const zp_plan *plan, int64_t n_nodes, const float *node_out,
                        const float *w0, const float *b0, const float *w1, const float *b1,
                        const float *grad_energy, float *grad_node_out, float *grad_w0,
                        float *grad_b0, float *grad_w1, float *grad_b1, void *work,
                        size_t work_bytes, void *stream);

/* Per-edge front end of the block in one pass, and its VJP: geometry (eso2_ref.py:320-321),
 * Gaussian distance basis (:164-168, 323), element embeddings of both atoms (:324-326), envelope
 * (:242-246, 343), and the copy of the roll-angle harmonics into the sorted edge order.  Inputs are
 * in the caller's edge order; `perm`, `src`, `dst`, `row_ptr`, `perm_src`, `row_ptr_src` come from
 * zp_csr_build; outputs are in the sorted order.  x_edge [E, num_basis + 2 edge_channels] is the
 * input of the radial MLP.  The backward takes the gradients of edge_vec (from
 * zp_eso2_backward), x_edge and env (any may be null = zero) and returns grad_pos [N,3] and
 * grad_emb [n_elements, edge_channels] (may be null), both summed in a fixed order.
 * edge_channels must be a multiple of 4.  `work`: zp_edge_features_work_bytes() bytes.          */
typedef struct zp_front_config {
  int32_t lmax;
  int32_t num_basis;
  int32_t edge_channels;
  int32_t n_elements;          /* rows of the embedding table                                  */
  int32_t envelope_exponent;   /* p of the polynomial envelope                                 */
  float cutoff;
  float gauss_coeff;           /* -0.5 / spacing^2 of the Gaussian basis                       */
} zp_front_config;
size_t zp_edge_features_work_bytes(const zp_front_config *cfg, int64_t n_nodes, int64_t n_edges);
int zp_edge_features_forward(const zp_front_config *cfg, int64_t n_nodes, int64_t n_edges,
                             const float *pos, const float *shifts, const int64_t *atomic_numbers,
                             const float *emb, const float *gauss_offsets, const float *cos_g,
                             const float *sin_g, const int32_t *perm, const int32_t *src,
                             const int32_t *dst, float *edge_vec, float *dist, float *x_edge,
                             float *env, float *cos_sorted, float *sin_sorted, void *stream);
int zp_edge_features_backward(const zp_front_config *cfg, int64_t n_nodes, int64_t n_edges,
                              const float *edge_vec, const float *dist, const float *x_edge,
                              const float *gauss_offsets, const int64_t *atomic_numbers,
                              const float *grad_edge_vec, const float *grad_x_edge,
                              const float *grad_env, const int32_t *row_ptr,
                              const int32_t *perm_src, const int32_t *row_ptr_src,
                              float *grad_pos, float *grad_emb, void *work, size_t work_bytes,
                              void *stream);

/* Periodic neighbour list with the per-destination cap, on the device (the graph front end; the
 * reference builds edge lists on the host with an external package and applies no cap,
 * fixtures/make_fixtures.py:13-15, 78-100).  Cubic periodic box of edge `box`; positions fp64 [N,3],
 * not necessarily inside [0, box) (shifts refer to the positions as given).
 * Edges src -> dst with d2 = |pos[dst] - pos[src] + shift|^2 < cutoff^2 (shift = image * box,
 * the zero-shift self pair excluded); per destination the max_neighbors smallest by
 * (d2, src, shift_x, shift_y, shift_z) are kept (max_neighbors <= 0: all, at most
 * ZP_NEIGHBORS_MAX_HITS per atom).  Output order is (dst, src, shift): destination-sorted, with
 * row_ptr.  Two calls, because the edge count is only known after the first:
 *   zp_neighbors_count  builds the cell list in `work`, writes row_ptr[N+1] (row_ptr[N] = E);
 *   zp_neighbors_fill   (same pos/box/cutoff/max_neighbors/work) writes edge_index [2,E] int64
 *                       (row 0 = src, row 1 = dst) and shifts [E,3] fp64.
 * *flags_out (device int) is 0 on success; bit 0: a position that is not finite, bit 1: more than
 * ZP_NEIGHBORS_MAX_HITS neighbours of one atom in an uncapped list, bit 2: the passes disagree.  */
#define ZP_NEIGHBORS_MAX_HITS 1024
#define ZP_NEIGHBORS_MAX_CAP 256
size_t zp_neighbors_work_bytes(int64_t n_atoms, double box, double cutoff);
int zp_neighbors_count(const double *pos, int64_t n_atoms, double box, double cutoff,
                       int max_neighbors, int32_t *row_ptr, int32_t *flags_out, void *work,
                       size_t work_bytes, void *stream);
int zp_neighbors_fill(const double *pos, int64_t n_atoms, double box, double cutoff,
                      int max_neighbors, const int32_t *row_ptr, int64_t n_edges,
                      int64_t *edge_index, double *shifts, int32_t *flags_out, void *work,
                      size_t work_bytes, void *stream);

/* Reads (synchronously) and clears the plan's device status word: ZP_OK, or
 * ZP_ERR_DEVICE_TIMEOUT if a bounded device-side wait gave up since the last read.          */
int zp_plan_device_status(zp_plan *plan, int *status_out);

/* Self-test of the bounded device-side waits (no reference counterpart).  Every wait inside the
 * contraction kernels gives up after a time limit, records ZP_ERR_DEVICE_TIMEOUT in the plan's
 * status word and lets all warps of the CTA return, so a lost signal can never hang the GPU.
 * This call launches one tiny product on one SM whose operand loads are deliberately never
 * issued, with the limit set to `limit_ns`: the kernel returns after about that long,
 * zp_plan_device_status then reports (and clears) ZP_ERR_DEVICE_TIMEOUT, and the library keeps
 * working.  `scratch`: at least 32 KiB of device memory, 256-byte aligned.                     */
int zp_selftest_bounded_wait(zp_plan *plan, void *scratch, size_t scratch_bytes, int64_t limit_ns,
                             void *stream);

/* Per-kernel-class device timing for benchmarks (the reference times whole steps with CUDA
 * events, bench/harness.py:88-149; there is no per-kernel counterpart).  While enabled, the
 * forward/backward drivers bracket each kernel class with CUDA events on the caller's stream.
 * zp_timing_read synchronises those events, ADDS the elapsed milliseconds and launch counts
 * since the previous read into ms[cls] / launches[cls] (arrays of ZP_N_KERNEL_CLASSES) and
 * resets.  Not thread-safe: use one thread per plan while timing is on.                     */
typedef enum zp_kernel_class {
  ZP_K_FOLD = 0,          /* weight folding / unfolding                                     */
  ZP_K_WIGNER_FWD = 1,
  ZP_K_ROTATE_IN = 2,
  ZP_K_GEMM_FWD = 3,      /* SO(2) contractions, forward                                    */
  ZP_K_GATE_FWD = 4,
  ZP_K_ROTATE_BACK = 5,   /* envelope + rotate back + segmented scatter                      */
  ZP_K_ROTATE_GRAD_OUT = 6,
  ZP_K_GEMM_DGRAD = 7,
  ZP_K_GEMM_WGRAD = 8,
  ZP_K_BIAS_GRAD = 9,
  ZP_K_GATE_BWD = 10,
  ZP_K_ROTATE_IN_BWD = 11,
  ZP_K_SRC_REDUCE = 12,
  ZP_K_WIGNER_BWD = 13,
  ZP_N_KERNEL_CLASSES = 14
} zp_kernel_class;
const char *zp_kernel_class_name(int cls);
int zp_timing_enable(zp_plan *plan, int on);
int zp_timing_read(zp_plan *plan, float *ms, int64_t *launches);

#ifdef __cplusplus
}
#endif
#endif /* ZIPPEL_B200_H */
