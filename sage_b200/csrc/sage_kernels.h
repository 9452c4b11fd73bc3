// Internal launcher declarations shared by the .cu files of libsage_b200.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sageb200 {

// Problems one launch can hold.  The public grouped entry points take SAGEB200_MAX_GROUPED (16);
// the expert entry points fill launches up to this internal limit (the kernel's parameter block
// grows with it: ~12 KB, within the 32 KB the driver accepts).
constexpr int kMaxGrouped = 64;

// One packed linear as the skinny kernel sees it.
struct SkinnyProblem {
  const __half *x;
  const uint32_t *codes;
  const uint32_t *radii;
  const uint32_t *grid;
  const uint32_t *book;
  const int32_t *perm;
  __half *y;
  float *partial;       // [tiles][slots_per_tile][16*rows] pieces of tiles shared between CTAs
  unsigned *counters;   // [tiles] arrivals, zero before and after every launch
  int rows, n, k, groups, tiles;
  int entries, dbits;
  int slices;           // K slices
  int ctas_per_slice;   // CTAs that divide one slice's units evenly
  int slots_per_tile;
  int whole_tiles;      // 1: CTAs own whole tiles (no sharing); 0: even share of units
  int share_q, share_r; // (tiles or units) / ctas_per_slice and remainder, for slices == 1
  int ring;             // 1: each warp streams its units through a ring of kRingStages x kRingUnits slots
  int cta_begin;        // first CTA of this problem in the grid
  // expert indirection (null: none): the weights are those of expert expert_ids[expert_slot]
  // inside a stack of expert_count experts starting at global expert expert_first
  const int *expert_ids;
  int expert_slot, expert_first, expert_count;
  long long codes_stride, cell_stride, book_stride;  // per-expert strides in 32-bit words
};

struct SkinnyParams {
  SkinnyProblem problem[kMaxGrouped];
  int count;
  int x_bytes;          // shared bytes reserved for staged activations
  int unit_capacity;    // most units any CTA holds (640 shared bytes each)
  int warp_segments;    // most tiles any warp touches
  int lin_bytes;        // shared bytes for activations in original order (0: none)
  unsigned warps_reciprocal;  // floor(2^32 / warps) + 1
  // producer fused into the activation staging (single row only); 0 = none
  int act_kind;
  float act_eps;
  const void *act_a, *act_b, *act_weight;
  void *act_residual_out;
  int *status;          // device-visible status word, may be null
  long long *trace;     // optional: per-CTA phase clocks (16 per CTA), null in normal use
};

// Launch plan for one problem (host side).
struct SkinnyPlan {
  int warps;
  int ctas_per_sm;
  int slices;
  int ctas_per_slice;
  int ctas;
  int unit_capacity;
  int warp_segments;
  int slots_per_tile;
  int whole_tiles;
  int ring;             // the CTA's share exceeds its shared memory: warps stream it through rings
  int column_blocks;    // 1 for rows <= 8, 2 for rows <= 16
  int tiles;
  bool needs_scratch;
  size_t x_bytes;
  size_t lin_bytes;
  size_t shared_bytes;
  size_t partial_bytes;
};

// Whether one launch can hold problems whose plans need these maxima of shared memory together.
bool skinny_shared_fits(size_t x_bytes, int unit_capacity, int warps, int warp_segments, int column_blocks,
                        size_t lin_bytes);

struct Tuning {
  int warps, slices, ctas_per_sm, mode;  // mode: 0 auto, 1 even units, 2 whole tiles
};

// cta_budget: CTAs the problem may occupy at once (0: the whole device).
// act_kind: the producer fused into a single-row launch (0 none, 1 residual add + RMSNorm,
// 2 SwiGLU); it sizes the linear staging buffer and so takes part in the plan.
SkinnyPlan plan_skinny(int rows, int n, int k, int entries, int sm_count, const Tuning &tuning,
                       int cta_budget = 0, int act_kind = 0);

// Opts every skinny-kernel variant into large dynamic shared memory on the CURRENT device.
cudaError_t configure_skinny();

// Launches the problems in `params` as one grid of `total_ctas` CTAs of `warps` warps.
cudaError_t launch_skinny(const SkinnyParams &params, int warps, int column_blocks, int total_ctas,
                          cudaStream_t stream);

cudaError_t launch_dequant(const uint32_t *codes, const uint32_t *radii, const uint32_t *grid,
                           const uint32_t *book, const int32_t *perm, __half *w, int n, int k,
                           int entries, cudaStream_t stream, int sm_count);

// Export-side packing (sage_pack.cu): `tiled` = SAGE's [tile][group][16][8] words, grid (min, step)
// in grid_or_scales and `mins` unused; otherwise SPHQuant's row-major int16 codes with separate
// scales and minimums.
cudaError_t launch_pack(const int8_t *signs, const int32_t *indices, const float *radius, uint32_t *codes,
                        uint32_t *high, __half *grid_or_scales, __half *mins, int n, int k, int dbits,
                        bool tiled, cudaStream_t stream, int sm_count);

// Per-device set-up of the library on the current device (idempotent): the device-visible
// status word the kernels write on a timed-out wait, and the SM count.  Returns a
// SAGEB200_* status (SAGEB200_ERR_TIMEOUT while an earlier time-out is recorded).
int acquire_device(int **status_word, int *sm_count);
// The buffer given to sageb200_debug_trace (null: none); read by -DSAGEB200_TRACE builds only.
long long *trace_buffer();
// Adds to the count sageb200_launch_count() reports.
void count_launches(int launches);

// Launch plan of the tcgen05 prefill GEMM (host side).
struct GemmPlan {
  int tokens_per_cta;   // MMA N: multiple of 16, at most 256
  int token_blocks;
  int row_blocks;       // blocks of 128 output rows
  int stages;
  int tmem_columns;
  int accumulators;     // token blocks per CTA (1 or 2) sharing each decoded weight stage
  int pair;             // 1: clusters of two CTAs (two row blocks) run cta_group::2 MMAs
  int k_splits;         // CTAs that share one output tile along K (1: none)
  int groups_per_split; // 128-channel groups per K split
  size_t partial_bytes; // FP32 scratch of the split tiles (0 without a split)
  size_t shared_bytes;
};

// `allow_split`: false plans without a K split (no scratch available).
GemmPlan plan_gemm_tc(int rows, int n, int k, int sm_count, bool allow_split = true);
extern int g_gemm_pairs;  // debug switch: 0 = never pair CTAs (sageb200_debug_gemm_pairs)
cudaError_t configure_gemm_tc();
// xq: activations already in quantised channel order, 16-byte aligned.  `status` is a
// device-visible word that receives SAGEB200_ERR_TIMEOUT if a bounded wait runs out.
// `sph_mins` non-null selects the SPHQuant format: `codes` = row-major 16-bit codes, `radii` = the
// per-(row, group) high radius words, `grid` = FP16 scales, `sph_mins` = FP16 minimums, `book` =
// the entry-major 64 x 8 codebook, entries = 64.
// `partial` (plan.partial_bytes) and `counters` (eight zeroed words per output tile, left zero) are
// needed when plan.k_splits > 1.
cudaError_t launch_gemm_tc(const __half *xq, const uint32_t *codes, const uint32_t *radii,
                           const uint32_t *grid, const uint32_t *book, __half *y, int *status,
                           int rows, int n, int k, int entries, const GemmPlan &plan,
                           cudaStream_t stream, float *partial = nullptr, unsigned *counters = nullptr,
                           const __half *sph_mins = nullptr);

// Causal attention over prompt rows on the tensor cores (prefill_attention.cu); rows are
// [sequence][token], row (s, t) at cache position positions[s] + t.  head_dim is 128.
cudaError_t launch_prefill_attention(const __half *q, const __half *k_cache, const __half *v_cache,
                                     const int *positions, __half *out, int sequences, int tokens, int q_heads,
                                     int kv_heads, int max_seq, cudaStream_t stream);

// x_q[m][j] = x[m][perm[j]] for the prefill path.
cudaError_t launch_gather(const __half *x, const int32_t *perm, __half *xq, int rows, int k,
                          cudaStream_t stream, int sm_count);

}  // namespace sageb200
