/*
 * sage_b200 — C ABI of the B200 (sm_100a) SAGE packed-weight matmul.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless its name
 * ends in `_host`.  `stream` is a cudaStream_t passed as void*.  Every function
 * returns SAGEB200_OK (0) or a negative SAGEB200_ERR_* code and never throws;
 * sageb200_status_string() turns a code into text.  Nothing here allocates device
 * memory except sageb200_linear_host (documented there); no call synchronises the
 * stream unless stated.
 *
 * Packed layout (tiles = ceil(N/16), groups = K/128, E = entries in {64,128,256}):
 *   codes  uint32 [tiles][groups][16][8]   two 16-bit codes per word
 *   radii  uint32 [tiles][groups][16]      sixteen 2-bit high radius fields
 *   grid   fp16   [tiles][groups][16][2]   (min, step)
 *   book   fp16   [4][E][2]                plane p = dims (2p, 2p+1) of each entry
 *   perm   int32  [K] or NULL              x_q[j] = x[perm[j]]
 * This is the layout the reference documents at csrc/sage/sage_gemv_cuda.h:7-13.
 */
#ifndef SAGE_B200_H_
#define SAGE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SAGEB200_OK 0
#define SAGEB200_ERR_INVALID_ARGUMENT (-1) /* null pointer, bad shape, bad entries      */
#define SAGEB200_ERR_ALIGNMENT (-2)        /* book not 4-byte, codes/radii/grid not 16-byte aligned */
#define SAGEB200_ERR_RANGE (-3)            /* rows > 65535 or a dimension overflows int  */
#define SAGEB200_ERR_WORKSPACE (-4)        /* workspace missing or too small             */
#define SAGEB200_ERR_CUDA (-5)             /* a CUDA call or launch failed               */
#define SAGEB200_ERR_NO_DEVICE (-6)        /* no sm_100 device is current                */
#define SAGEB200_ERR_TIMEOUT (-7)          /* a bounded device-side wait ran out         */
#define SAGEB200_ERR_STATIC_SCRATCH (-8)   /* shape too large for sageb200_linear_static */

/* Library version, major*10000 + minor*100 + patch. */
int sageb200_version(void);

/* Static text for a status code. */
const char *sageb200_status_string(int status);

/*
 * 1 if the matmul folds the input-channel permutation into its activation loads for
 * this shape, so the caller must NOT pre-gather x.  Always 1 here (any K, any rows).
 * Replaces: bool sage_gemv_fuses_permutation(int n, int k)
 *           (reference csrc/sage/sage_gemv_cuda.h:14, csrc/sage/sage_gemv_cuda.cu:114-116,
 *            which returns k <= 4096 and makes csrc/bindings.cpp:49-51 run index_select).
 */
int sageb200_gemv_fuses_permutation(int n, int k);

/*
 * Number of K slices the decode kernel will use for this shape on a device with
 * `sm_count` SMs (informational; the workspace size already accounts for it).
 * Replaces: int sage_gemm_splits(int rows, int n, int k, int sm_count)
 *           (reference csrc/sage/sage_gemv_cuda.h:21, csrc/sage/sage_gemm_cuda.cu:209-214,493-495).
 */
int sageb200_gemm_splits(int rows, int n, int k, int sm_count);

/*
 * Bytes of scratch sageb200_linear needs for this shape: partial sums of output tiles
 * that are shared between CTAs, their arrival counters and (for more than one row with a
 * permutation) the gathered activations.
 * Returns 0 when the shape needs none.  The buffer must be 256-byte aligned and
 * ZERO-FILLED ONCE when it is allocated.  Its first 64 KiB hold the arrival counters and
 * nothing else; every call leaves them zero again, so one buffer (sized for the largest
 * shape) can be reused by successive calls of any shapes on one stream.  Calls that may
 * run concurrently must not share a buffer.
 * Replaces: the workspace sizing at reference csrc/bindings.cpp:63-66.
 */
size_t sageb200_workspace_bytes(int rows, int n, int k);

/*
 * y[rows][n] (fp16) = x[rows][k] (fp16) . W^T, W given by the five packed buffers.
 * Chooses the GEMV / skinny tensor-core kernel (rows <= 16) or the prefill GEMM
 * (rows > 16) internally; the permutation is always applied inside.
 *   x     fp16 [rows][k], contiguous, any 2-byte alignment
 *   perm  NULL for identity
 *   y     fp16 [rows][n]
 *   rows may be 0 (returns OK without launching); rows <= 65535; k % 128 == 0.
 * Replaces: sage_gemv_cuda + sage_gemm_cuda and the dispatch around them
 *           (reference csrc/sage/sage_gemv_cuda.h:16-26, csrc/bindings.cpp:8-79).
 */
int sageb200_linear(const void *x, const void *codes, const void *radii, const void *grid,
                    const void *book, const int32_t *perm, void *y, void *workspace,
                    size_t workspace_bytes, int rows, int n, int k, int entries, void *stream);

/* One problem of a grouped launch: the arguments of sageb200_linear without scratch. */
typedef struct sageb200_problem {
  const void *x;
  const void *codes;
  const void *radii;
  const void *grid;
  const void *book;
  const int32_t *perm;
  void *y;
  int rows;
  int n;
  int k;
  int entries;
} sageb200_problem;

#define SAGEB200_MAX_GROUPED 16

/*
 * Several independent packed linears with rows <= 16 in ONE kernel launch (q/k/v,
 * gate/up, the experts a token routes to).  `problems_host` is a HOST array of
 * `count` <= SAGEB200_MAX_GROUPED descriptors whose pointers are device pointers.
 * The launch is planned as one resident wave: each problem gets CTAs in proportion to its
 * packed size.  Workspace: sageb200_grouped_workspace_bytes for the same descriptors (only
 * rows, n, k, entries and whether perm is NULL are read), same zero-fill rule.
 * No counterpart in the reference, which launches one kernel per linear
 * (csrc/bindings.cpp:52-61).
 */
size_t sageb200_grouped_workspace_bytes(const sageb200_problem *problems_host, int count);
int sageb200_linear_grouped(const sageb200_problem *problems_host, int count, void *workspace,
                            size_t workspace_bytes, void *stream);

/*
 * The producer of the activations, fused into a grouped decode launch: instead of reading
 * problem.x, the kernels compute the shared input row(s) of all problems themselves.
 *   kind 0  none (problem.x is read)
 *   kind 1  x = weight * fp16((a + b) * rsqrt(mean((a + b)^2) + eps)): residual add and
 *           RMSNorm as the Hugging Face Qwen3 modules round them; a + b is also written to
 *           residual_out (must not alias a); b may be NULL
 *   kind 2  x = fp16(silu(a)) * b: SwiGLU
 * a, b, residual_out are FP16 [rows][k], weight FP16 [k], all 16-byte aligned.
 */
typedef struct sageb200_activation {
  int kind;
  float eps;
  const void *a;
  const void *b;
  const void *weight;
  void *residual_out;
} sageb200_activation;

/*
 * sageb200_linear_grouped with the activations' producer fused in (all problems share rows
 * and k; problem.x is ignored).  With one row the producer runs inside the decode kernel's
 * activation staging, saving a kernel launch per norm / SwiGLU; with more rows one staging
 * launch computes the rows and writes them once per problem in that problem's channel order
 * (rows of up to 49152 channels).  Workspace: sageb200_fused_workspace_bytes.
 * No counterpart in the reference, where these are separate Hugging Face modules.
 */
size_t sageb200_fused_workspace_bytes(const sageb200_problem *problems_host, int count);
int sageb200_linear_grouped_fused(const sageb200_problem *problems_host, int count,
                                  const sageb200_activation *activation, void *workspace,
                                  size_t workspace_bytes, void *stream);

/*
 * A stack of `experts` packed linears of one shape (the experts of one MoE projection that
 * live on this GPU), every buffer with a leading expert dimension:
 *   codes [experts][tiles][groups][16][8], radii and grid likewise, book [experts][4][entries][2],
 *   perm [experts][k] or NULL.  `first_expert` is the global index of the stack's first expert.
 */
typedef struct sageb200_expert_stack {
  const void *codes;
  const void *radii;
  const void *grid;
  const void *book;
  const int32_t *perm;
  int experts;
  int first_expert;
  int n;
  int k;
  int entries;
} sageb200_expert_stack;

/*
 * Routed experts, one activation row per slot: for every slot s and stack t
 *   ys[t][s][:] = W(stack t, expert expert_ids[s]) . x[s * x_slot_stride ...]
 * `expert_ids` is a DEVICE array of `slots` global expert indices (the router's top-k, still on
 * the GPU: no host round trip); slots whose expert is outside [first_expert, first_expert +
 * experts) are skipped, so the caller zero-fills ys and, under expert parallelism, sums the
 * ranks' outputs.  x_slot_stride = 0 shares one activation row between all slots (gate/up of
 * one token), x_slot_stride = k gives each slot its own row (down).  Launches
 * SAGEB200_MAX_GROUPED problems at a time.  Workspace as for a grouped launch of the same
 * shapes (sageb200_experts_workspace_bytes).
 * No counterpart in the reference, which has no packed MoE module (its loader rejects every
 * model type but dense qwen3, weight_vq/integrations/transformers.py:88-89).
 */
size_t sageb200_experts_workspace_bytes(const sageb200_expert_stack *stacks_host, int stack_count,
                                        int slots);
int sageb200_experts(const void *x, long long x_slot_stride, const sageb200_expert_stack *stacks_host,
                     void *const *ys_host, int stack_count, const int32_t *expert_ids, int slots,
                     void *workspace, size_t workspace_bytes, void *stream);

/*
 * Routed experts, a block of up to 16 activation rows per expert visit (the compute of an
 * all-to-all expert-parallel exchange, where the rows an expert received have been sorted
 * together): for every block b and stack t
 *   ys[t][b][r][:] = W(stack t, expert block_expert_ids[b]) . x[b][r][:]      r < rows
 * x is [blocks][rows][k], ys[t] is [blocks][rows][n_t]; `block_expert_ids` is a DEVICE array of
 * `blocks` global expert indices.  A block whose id is negative or outside the stack is skipped
 * (its outputs are left untouched), so a caller sizes `blocks` for the worst case and marks the
 * unused ones with -1.  An expert that received more than `rows` rows simply owns several
 * blocks.  The packed weights of an expert are read once per block.
 * No counterpart in the reference (no packed MoE module).
 */
size_t sageb200_expert_blocks_workspace_bytes(const sageb200_expert_stack *stacks_host, int stack_count, int rows);
int sageb200_expert_blocks(const void *x, const sageb200_expert_stack *stacks_host, void *const *ys_host,
                           int stack_count, const int32_t *block_expert_ids, int blocks, int rows, void *workspace,
                           size_t workspace_bytes, void *stream);

/*
 * Dequantise to a dense fp16 matrix w[n][k]: bit-exact
 *   w = fp16_rn(float(+-dir) * fmaf(float(radius_code), step, min))
 * (reference csrc/sage/sage_gemm_cuda.cu:117-131 and tests/inference/reference.py:39-49).
 * With perm != NULL columns are scattered back to original channel order
 * (w[row][perm[j]] = w_q[row][j]); with perm == NULL they stay in quantised order.
 */
int sageb200_dequant(const void *codes, const void *radii, const void *grid, const void *book,
                     const int32_t *perm, void *w, int n, int k, int entries, void *stream);

/*
 * Export-side packing of one trained spherical linear (the step before the path): frozen
 * signs int8 [n][k] (+1 / -1), direction indices int32 [n][k/8] and radii FP32 [n][k/8]
 * (after the softplus) into the packed buffers above.  Per (row, 128-channel group) the FP16
 * grid (min, step) is fitted to the sixteen radii and each radius code is selected against
 * that rounded grid.  tiled != 0: SAGE's layout (`codes` = packed_codes, `high` = radius_codes,
 * `grid_or_scales` = radius_grid, rows padded to a multiple of 16 with zero codes and a zero
 * grid, `mins` unused); tiled == 0 (entries 64 only): SPHQuant's row-major layout (`codes` int16
 * [n][k/8], `high` int32 [n][k/128], `grid_or_scales` the FP16 scales and `mins` the FP16
 * minimums, [n][k/128] each).  The codebook and the permutation are not touched here: they are
 * small tensors the host side derives (see sage_b200/packing.py).  Bit-identical to the
 * reference's tensor program.
 * Replaces: pack_spherical (reference weight_vq/sphquant/packing.py:32-75).
 */
int sageb200_pack_spherical(const void *signs, const void *indices, const void *radius, void *codes,
                            void *high, void *grid_or_scales, void *mins, int n, int k, int entries,
                            int tiled, void *stream);

/*
 * Host-buffer form of sageb200_linear for callers whose activations live in host
 * memory: copies x_host to the device, runs the matmul and copies y back, all on
 * `stream`, then synchronises the stream.  The packed weight buffers are device
 * pointers.  `staging` is a device buffer of sageb200_host_staging_bytes(rows,n,k)
 * bytes (256-byte aligned, zero-filled once, reusable) that holds x, y and the
 * workspace.  Pinned host memory makes the copies asynchronous but is not required.
 */
size_t sageb200_host_staging_bytes(int rows, int n, int k);
int sageb200_linear_host(const void *x_host, const void *codes, const void *radii,
                         const void *grid, const void *book, const int32_t *perm, void *y_host,
                         void *staging, size_t staging_bytes, int rows, int n, int k,
                         int entries, void *stream);

/*
 * Tuning knob for sweeps (debug): warps per CTA (<= 16), K slices (<= 8) and CTAs per SM
 * of the decode kernel, and how output tiles are shared out (`mode` 1: every CTA gets an
 * even share of the (tile, group) units and shared tiles are finished through scratch;
 * 2: whole tiles per CTA; 3: never stream a CTA's share through shared-memory rings, launch
 * further waves of CTAs instead); 0 restores the built-in heuristic for a field.  Not thread
 * safe, like its counterpart.
 * Replaces: _set_sage_tuning / sage_gemv_tuning (reference csrc/bindings.cpp:81-84,
 *           csrc/sage/sage_gemv_cuda.cu:3-4).
 */
int sageb200_set_tuning(int warps, int slices, int ctas_per_sm, int mode);

/*
 * SPHQuant 64/4 packed linear, y[rows][n] = x[rows][k] . W^T: replaces the reference's
 * sph_gemv_forward_cuda (csrc/sphquant/sph_gemv_cuda.cu:403-469, declared at
 * csrc/sphquant/sph_gemv_cuda.h:5-11).  Row-major buffers: codes int16 [n][k/8] (bits 0-7
 * signs, 8-13 direction index, 14-15 low radius bits; 16-byte aligned), extra int32 [n][k/128]
 * (sixteen 2-bit high radius fields), scales / mins fp16 [n][k/128], book fp16 [64][8]
 * (16-byte aligned).  k % 128 == 0, k <= 16384 (the reference's limit); x FP16 contiguous, any
 * 2-byte alignment; rows <= 65535.  The packed weights are read once per eight activation rows;
 * sums across vectors are FP32.  No scratch.
 */
int sageb200_sph_linear(const void *x, const void *codes, const void *extra, const void *scales,
                        const void *mins, const void *book, void *y, int rows, int n, int k, void *stream);

/*
 * Dense FP16 weight w[n][k] = fp16(float(+-book[index][d]) * fmaf(code, scale, min)) of an
 * SPHQuant matrix, bit-identical to the reference's arithmetic decode
 * (tests/inference/reference.py:16-22) rounded to FP16.  The reference has no such kernel.
 */
int sageb200_sph_dequant(const void *codes, const void *extra, const void *scales, const void *mins,
                         const void *book, void *w, int n, int k, void *stream);

/*
 * Allocation-free form of sageb200_linear for the decode range (rows <= 16).
 *
 * For callers that cannot provide a workspace because they are not in a position to
 * allocate device memory: engines that fixed their whole memory plan at start-up, plugins
 * that only ever receive a stream and tensor pointers from the runtime hosting them, and
 * serving loops that cannot risk the device-wide stall (or the failure) of an allocator
 * call between two tokens.  The scratch the decode kernel needs sits in a static device
 * array inside the library instead: SAGEB200_STATIC_SCRATCH_BYTES bytes on every GPU that
 * loads the library, held until the process exits.
 *
 *   - Shapes whose sageb200_workspace_bytes(rows, n, k) exceeds that size, and rows > 16,
 *     are refused with SAGEB200_ERR_STATIC_SCRATCH; nothing is launched.
 *   - It calls no cudaMalloc, cudaFree or any other allocating routine.  The first call on
 *     each device looks up the array's device address and pins the library's static status
 *     word (a one-off set-up step that may load the library's device code): make that first
 *     call outside any stream capture.
 *   - All calls on a device share the one array.  Each call re-zeroes the arrival counters
 *     on `stream` before it launches, so calls ordered on one stream are safe; calls that
 *     can overlap on the GPU (different streams, different threads) race on the array and
 *     must be serialised by the caller or use sageb200_linear with separate workspaces.
 * Arguments and results are those of sageb200_linear.
 * No counterpart in the reference, which allocates its workspace with torch::empty on
 * every call.
 */
#define SAGEB200_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int sageb200_linear_static(const void *x, const void *codes, const void *radii, const void *grid,
                           const void *book, const int32_t *perm, void *y, int rows, int n, int k,
                           int entries, void *stream);

/*
 * Every device-side wait of the library is bounded; when one runs out, the kernel records
 * SAGEB200_ERR_TIMEOUT in a status word of the current device and every later call on that
 * device returns SAGEB200_ERR_TIMEOUT without launching, until this function clears the
 * record.  Call it once the stream that reported the time-out is idle (the outputs of the
 * call that timed out are undefined).  No counterpart in the reference (its kernels never wait).
 */
int sageb200_clear_status(void);

/* Number of kernels this library has launched in this process (all entry points). */
unsigned long long sageb200_launch_count(void);

/* Kernels launched so far by the decode glue of sage_b200_decode.h (same purpose). */
unsigned long long sageb200_glue_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* SAGE_B200_H_ */
