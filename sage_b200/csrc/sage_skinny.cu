// SAGE packed GEMV / skinny GEMM for 1..16 activation rows (decode), sm_100a.
//
// Replaces the reference's sage_gemv_kernel (csrc/sage/sage_gemv_cuda.cu:8-110), which
// launches grid.y = rows and therefore re-reads and re-decodes every weight once per
// activation row.  Here one 16-row packed tile is exactly the M dimension of a
// mma.sync.m16n8k16 instruction: the decoded weights are the A operand, the (up to 8 or
// 16) activation rows are the B operand, so weights are read and decoded once for any
// row count and the FP16 products accumulate in FP32 inside the tensor core.
//
// Work split ("stream-K"): the unit of work is (16-row tile, 128-channel group).  K may be
// cut into a few slices so that the activations of one slice fit in shared memory; inside
// a slice the units, in (tile, group) order, are divided EVENLY over the slice's CTAs, so
// every CTA gets the same amount of packed data whatever the tile count.  A CTA's range
// is contiguous in memory: each warp fetches its share with a handful of TMA bulk copies
// (cp.async.bulk, 16-byte aligned, completion on an mbarrier) issued before anything
// else, so the HBM stream is in flight while the CTA stages its codebook and activations.
// Tiles that straddle CTAs are finished without spinning: every CTA that holds a piece
// writes its partial sums to scratch and bumps the tile's arrival counter; whichever CTA
// arrives last adds the pieces in a fixed (slice, position) order, so results do not
// depend on scheduling.
//
// Per lane (g = lane / 4, t = lane % 4) and per unit: rows g and g+8 of the tile, code
// words 2t and 2t+1 of each row, i.e. vectors 4t..4t+3.  Step s (0..3) turns vector
// 4t+s of both rows into two MMAs: MMA k-slots {2t,2t+1} and {2t+8,2t+9} carry dims
// (0,1),(2,3) in the first and (4,5),(6,7) in the second.  The activation row for MMA
// column g is staged in shared memory in exactly that order, so one 16-byte shared
// load yields the B fragments of both MMAs.
//
// Arithmetic per vector: direction from a bank-conflict-free replicated shared codebook
// (replica = lane % 8), signs XORed in, radius = min + code*step evaluated in FP32 as
// fma(1 + code/16, 16*step, min - 16*step) and rounded once to FP16, weight =
// hmul2(direction, radius).  (The dense dequantisation kernel, not this one, carries the
// bit-exact weight contract; this kernel is checked against an FP32 matmul.)
#include "sage_common.cuh"
#include "sage_kernels.h"
#include "sage_skinny_core.cuh"

namespace sageb200 {
namespace {

constexpr int kBookBytes = 256 * 8 * 16;  // 256 entries x 8 replicas x 16 bytes, static
constexpr unsigned long long kWaitLimitNs = 2000000000ull;
constexpr int kMaxWarps = 16;
constexpr int kMaxCtaTiles = 64;      // tiles of one CTA when tiles are shared between CTAs
constexpr int kMaxWholeTiles = 192;   // tiles of one CTA in any mode (unit capacity 192 / 1 group)
constexpr int kMaxSlices = 8;
constexpr int kUnitBytes = 640;           // 512 codes + 64 radius words + 64 grid
constexpr int kMaxDynamicShared = 184 * 1024;  // plus ~37 KiB static stays under the 227 KiB limit
// Ring mode (a CTA's share of the matrix exceeds its shared memory): every warp streams its
// contiguous units through kRingStages stages of kRingUnits units, refilling a stage as soon
// as the warp has decoded it, so the HBM stream and the decode arithmetic overlap.
constexpr int kRingStages = 3;
constexpr int kRingUnitsMax = 4;  // units per stage: 4, 2 or 1, whatever fits beside the activations

__device__ __forceinline__ void bulk_copy(uint32_t dst, const void *src, uint32_t bytes,
                                          uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ bool barrier_done(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.u32 %0, 1, 0, p;\n}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Even split of n items over `parts` (n >= parts >= 1): with q = n / parts and
// r = n % parts, part i holds q + (i < r) items starting at i*q + min(i, r).  32-bit only.
__device__ __forceinline__ int split_begin(int i, int q, int r) { return i * q + min(i, r); }
__device__ __forceinline__ int split_owner(int u, int q, int r) {
  const int big = r * (q + 1);
  return u < big ? u / (q + 1) : r + (u - big) / q;
}

// Dynamic shared memory: [x | codes | radii | grid | warp partials | x in original order].
// kLowBits: some problem of the launch has 64 or 128 codebook entries (codes carry low
// radius bits); a launch whose codebooks all have 256 entries uses the shorter variant.
// kPath specialises the once-per-launch code for the decode graph's launches (single activation
// row, permutation present and 16-byte aligned, K not sliced, no expert indirection, the row fits
// the linear staging buffer): 1 = fused residual add + RMSNorm, 2 = fused SwiGLU, 3 = plain
// 16-byte aligned x; 5 = kind 3 for routed experts (the indirection stays); 4 = one activation
// row and nothing else assumed; 6 = several rows staged beforehand (no permutation left, aligned x,
// K not sliced, no expert stack); 7 = kind 6 with K cut into slices; 0 = every case.  The special paths are the generic code with those facts
// known at compile time, so the cold instruction stream after the wait is short and contiguous.
// kRing: the CTA's share streams through per-warp rings (see kRingStages); a separate variant so
// that the resident-share kernels keep their shorter main loop.
template <int NB, bool kLowBits, int kPath, bool kRing = false>
__global__ void __launch_bounds__(512, 1) sage_skinny_kernel(const __grid_constant__ SkinnyParams params) {
  extern __shared__ __align__(128) unsigned char shared[];
  __shared__ __align__(128) unsigned char book_shared[kBookBytes];
  __shared__ __align__(8) unsigned long long barriers[kMaxWarps][kRingStages];
  __shared__ int warp_first_tile[kMaxWarps];
  __shared__ float norm_sums[kMaxWarps];
  __shared__ int tile_parts[kMaxCtaTiles];  // CTAs contributing to the tile, all slices
  __shared__ int tile_slot[kMaxCtaTiles];   // this CTA's position among them (slice-major)
  __shared__ int tile_last[kMaxCtaTiles];   // this CTA arrived last
  __shared__ unsigned char tile_warp_lo[kMaxWholeTiles];  // first and last warp holding a
  __shared__ unsigned char tile_warp_hi[kMaxWholeTiles];  // piece of the CTA's tile

  // Phase clocks for profiling exist only in a build with -DSAGEB200_TRACE (python -m
  // sage_b200.build --trace); the default build compiles every stamp out.
#ifdef SAGEB200_TRACE
  long long *trace = params.trace ? params.trace + 16 * static_cast<size_t>(blockIdx.x) : nullptr;
#define SAGE_STAMP(i) do { if (trace && threadIdx.x == 0) trace[i] = clock64(); } while (0)
#define SAGE_STAMP_NS(i) do { if (trace && threadIdx.x == 0) trace[i] = global_nanoseconds(); } while (0)
#else
#define SAGE_STAMP(i) do { } while (0)
#define SAGE_STAMP_NS(i) do { } while (0)
#endif
  SAGE_STAMP(0);
  SAGE_STAMP_NS(13);
  pdl_launch_dependents();  // the next kernel may be scheduled as SM resources free up
  int pi = 0;
  if (params.count > 1) {
    while (pi + 1 < params.count && static_cast<int>(blockIdx.x) >= params.problem[pi + 1].cta_begin)
      ++pi;
  }
  SkinnyProblem p = params.problem[pi];
  if constexpr (kPath == 6) {
    p.slices = 1;  // several rows, staged beforehand: no permutation left, x aligned
    p.expert_ids = nullptr;
    p.perm = nullptr;
  } else if constexpr (kPath == 7) {
    p.expert_ids = nullptr;  // kind 6 with the K slices left in
    p.perm = nullptr;
  } else if constexpr (kPath == 4) {
    p.rows = 1;  // the only fact kind 4 fixes
  } else if constexpr (kPath == 5) {
    p.rows = 1;  // kind 3 with the expert indirection left in
    p.slices = 1;
  } else if constexpr (kPath != 0) {
    p.rows = 1;
    p.slices = 1;
    p.expert_ids = nullptr;
  }
  if (p.expert_ids) {
    // routed expert: pick this slot's expert out of the stack; an expert that lives on
    // another rank leaves y as the caller zeroed it.  The ids may come from the kernel just
    // before this one, so they are read only after the wait for it.
    pdl_wait();
    const int expert = __ldg(p.expert_ids + p.expert_slot) - p.expert_first;
    if (expert < 0 || expert >= p.expert_count) return;
    p.codes += expert * p.codes_stride;
    p.radii += expert * p.cell_stride;
    p.grid += expert * p.cell_stride;
    p.book += expert * p.book_stride;
    if (p.perm) p.perm += static_cast<long long>(expert) * p.k;
  }

  const int tid = threadIdx.x;
  const int threads = blockDim.x;
  const int warp = tid >> 5;
  const int warps = threads >> 5;
  const int lane = tid & 31;
  const int g = lane >> 2;
  const int t = lane & 3;

  const int local = static_cast<int>(blockIdx.x) - p.cta_begin;
  const int S = p.slices;
  const int J = p.ctas_per_slice;
  if (local >= S * J) return;  // spare CTA of a grouped launch
  int slice = 0, j = local, group_begin = 0, group_count = p.groups;
  if (S > 1) {
    slice = local % S;
    j = local / S;
    group_begin = p.groups * slice / S;
    group_count = p.groups * (slice + 1) / S - group_begin;
  }
  // Two ways to share the units out.  Whole tiles (S == 1): CTA j gets an even share of the
  // tiles, so no tile is shared and nothing needs finishing afterwards.  Even units: CTA j
  // gets an even share of the slice's units; tiles that straddle CTAs are finished in step 8.
  const bool whole = p.whole_tiles != 0;
  int unit_q = p.share_q, unit_r = p.share_r;  // host-computed for an unsliced K
  if (S > 1) {
    const int share = p.tiles * group_count;  // >= J
    unit_q = share / J;
    unit_r = share - unit_q * J;
  }
  const int scale = whole ? group_count : 1;
  const int unit_begin = split_begin(j, unit_q, unit_r) * scale;
  const int unit_end = split_begin(j + 1, unit_q, unit_r) * scale;
  const int unit_count = unit_end - unit_begin;

  __half *x_shared = reinterpret_cast<__half *>(shared);
  unsigned char *codes_shared = shared + params.x_bytes;
  unsigned char *radii_shared = codes_shared + static_cast<size_t>(params.unit_capacity) * 512;
  unsigned char *grid_shared = radii_shared + static_cast<size_t>(params.unit_capacity) * 64;
  float *partial_shared =
      reinterpret_cast<float *>(grid_shared + static_cast<size_t>(params.unit_capacity) * 64);
  __half *x_linear = reinterpret_cast<__half *>(
      reinterpret_cast<unsigned char *>(partial_shared) +
      static_cast<size_t>(warps) * params.warp_segments * NB * 512);

  // This warp's contiguous share of the CTA's units.
  // unit_count / warps by multiplication (exact: unit_count * warps < 2^32)
  const int warp_q = warps == 1 ? unit_count  // (2^32 / 1 + 1 does not fit the reciprocal)
                                : static_cast<int>(__umulhi(static_cast<unsigned>(unit_count),
                                                            params.warps_reciprocal));
  const int warp_r = unit_count - warp_q * warps;
  const int warp_begin = unit_begin + split_begin(warp, warp_q, warp_r);
  const int warp_end = unit_begin + split_begin(warp + 1, warp_q, warp_r);
  const uint32_t bar = smem_address(&barriers[warp][0]);
  // (only with an unsliced K); p.ring = units per stage, 0 for a problem of the launch that fits
  const bool ring = kRing && p.ring != 0;
  const int kRingUnits = kRing ? p.ring : 1;
  const int kRingSlots = kRingStages * kRingUnits;
  const int warp_units = warp_end - warp_begin;
  // ring: chunk c of the warp = units warp_begin + c*kRingUnits ..., into stage c % kRingStages
  auto ring_issue = [&](int chunk) {
    const int first = warp_begin + chunk * kRingUnits;
    const uint32_t count = static_cast<uint32_t>(min(kRingUnits, warp_end - first));
    const uint32_t stage = static_cast<uint32_t>(chunk % kRingStages);
    const uint32_t stage_bar = bar + 8u * stage;
    const uint32_t slot = static_cast<uint32_t>(warp * kRingSlots) + stage * kRingUnits;
    const size_t cell = static_cast<size_t>(first) * 16;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(stage_bar), "r"(count * kUnitBytes)
                 : "memory");
    bulk_copy(smem_address(codes_shared) + slot * 512u, p.codes + cell * 8, count * 512u, stage_bar);
    bulk_copy(smem_address(radii_shared) + slot * 64u, p.radii + cell, count * 64u, stage_bar);
    bulk_copy(smem_address(grid_shared) + slot * 64u, p.grid + cell, count * 64u, stage_bar);
  };

  SAGE_STAMP(11);
  // ---- 1. start the weight stream: lane 0 of each warp copies the warp's units
  if (lane == 0 && ring) {
#pragma unroll
    for (int stage = 0; stage < kRingStages; ++stage)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar + 8u * stage));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int chunk = 0; chunk < kRingStages && chunk * kRingUnits < warp_units; ++chunk) ring_issue(chunk);
  } else if (lane == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (warp_end > warp_begin) {
      const uint32_t total = static_cast<uint32_t>(warp_end - warp_begin) * kUnitBytes;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(total)
                   : "memory");
      int u = warp_begin;
      while (u < warp_end) {
        // a run of units inside one tile is contiguous in all three arrays; with a single
        // K slice the unit index is the memory order and the whole share is one run
        int run = warp_end - u;
        size_t cell = static_cast<size_t>(u) * 16;
        if (S > 1) {
          const int tile = u / group_count;
          const int gi = u - tile * group_count;
          run = min(run, group_count - gi);
          cell = (static_cast<size_t>(tile) * p.groups + group_begin + gi) * 16;
        }
        const uint32_t slot = static_cast<uint32_t>(u - unit_begin);
        bulk_copy(smem_address(codes_shared) + slot * 512u, p.codes + cell * 8, run * 512u, bar);
        bulk_copy(smem_address(radii_shared) + slot * 64u, p.radii + cell, run * 64u, bar);
        bulk_copy(smem_address(grid_shared) + slot * 64u, p.grid + cell, run * 64u, bar);
        u += run;
      }
    } else {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
    }
  }

  SAGE_STAMP(12);
  // ---- 1b. which tiles does this CTA touch, and who else touches them (static
  //          arithmetic, done while the copies fly)
  const int cta_first_tile = unit_count > 0 ? unit_begin / group_count : 0;
  const int cta_tiles = unit_count > 0 ? (unit_end - 1) / group_count - cta_first_tile + 1 : 0;
  for (int ti = tid; ti < cta_tiles; ti += threads) {
    // warps whose contiguous shares overlap this tile's units inside the CTA
    const int tile = cta_first_tile + ti;
    const int u0 = max(tile * group_count, unit_begin) - unit_begin;
    const int u1 = min((tile + 1) * group_count, unit_end) - 1 - unit_begin;
    tile_warp_lo[ti] = static_cast<unsigned char>(split_owner(u0, warp_q, warp_r));
    tile_warp_hi[ti] = static_cast<unsigned char>(split_owner(u1, warp_q, warp_r));
  }
  int shared_tile = 0;
  for (int ti = tid; !whole && ti < cta_tiles; ti += threads) {
    const int tile = cta_first_tile + ti;
    int total = 0, slot = 0;
    for (int s2 = 0; s2 < S; ++s2) {
      const int gc = p.groups * (s2 + 1) / S - p.groups * s2 / S;
      const int U2 = p.tiles * gc;
      const int q2 = U2 / J, r2 = U2 - q2 * J;
      const int u0 = tile * gc;
      const int first = split_owner(u0, q2, r2);
      const int last = split_owner(u0 + gc - 1, q2, r2);
      if (s2 == slice) slot = total + (j - first);
      total += last - first + 1;
    }
    tile_parts[ti] = total;
    tile_slot[ti] = slot;
    tile_last[ti] = 0;
    shared_tile |= total > 1;
  }

  SAGE_STAMP(1);
  // ---- 2. staging.  Every global load of this phase is issued before the first value
  //         is used, so the phase costs one trip to L2, not one per item.
  //   codebook    thread e holds entry e (16 bytes, dims interleaved) and writes its eight
  //               replicas, starting at replica (lane % 8) so a warp's stores spread over
  //               all banks
  //   activations laid out so that lane (g,t), step s finds vector 4t+s of its row at
  //               [group][s][t][8 halves]; rows are 64 bytes apart modulo 128.  Ways in:
  //     a. no permutation, 16-byte aligned x: 16-byte copies
  //     b. permutation and the rows fit the linear buffer: x is copied linearly into shared
  //        memory while the permutation indices load into registers; the gather then reads
  //        shared memory (after the barrier)
  //     c. otherwise: gather from global memory, four channels per item
  const int span = group_count * 128;
  const int row_stride = span + 32;  // halves
  const bool aligned_x = (kPath != 0 && kPath != 4) || (reinterpret_cast<uintptr_t>(p.x) & 15) == 0;  // (kind 6: checked on the host)
  const bool perm_aligned = (kPath != 0 && kPath != 4) || (reinterpret_cast<uintptr_t>(p.perm) & 15) == 0;
  const bool linear_gather =
      (kPath != 0 && kPath != 4 && kPath != 6 && kPath != 7) || (p.perm != nullptr && perm_aligned &&
                     static_cast<size_t>(p.rows) * p.k * 2 <= static_cast<size_t>(params.lin_bytes));
  // Fused producer (single activation row only): the row is computed here from the
  // producer's inputs instead of being read from p.x:
  //   1  x = weight * fp16((a + b) * rsqrt(mean((a + b)^2) + eps)),  a + b also stored as the
  //      new residual by the launch's first CTA                      (residual add + RMSNorm)
  //   2  x = fp16(silu(a)) * b                                        (SwiGLU)
  const int fused = (kPath == 0 || kPath == 4) ? params.act_kind : ((kPath == 3 || kPath >= 5) ? 0 : kPath);
  const bool gather_from_linear = linear_gather || fused != 0;
  const bool direct_copy = kPath == 6 || kPath == 7 || ((kPath == 0 || kPath == 4) && p.perm == nullptr && aligned_x && fused == 0);
  constexpr int kItemBatch = 4;  // permutation items (4 channels each) held in registers
  constexpr int kCopyBatch = 4;  // 16-byte activation pieces held in registers
  int4 held[kItemBatch];
  uint4 piece[kCopyBatch];
  const int items = span >> 2;
  const int vectors = span >> 3;
  // what the first batch of 16-byte pieces copies: the slice of every row (a) or all of x (b)
  const int pieces = fused ? 0
                     : direct_copy ? vectors * p.rows
                                   : (linear_gather && aligned_x ? (p.rows * p.k) >> 3 : 0);

  uint4 entry = make_uint4(0, 0, 0, 0);
  if (tid < p.entries) {
    entry.x = __ldg(p.book + tid);
    entry.y = __ldg(p.book + p.entries + tid);
    entry.z = __ldg(p.book + 2 * p.entries + tid);
    entry.w = __ldg(p.book + 3 * p.entries + tid);
  }
  auto load_item = [&](int q) {  // source channels of quantised channels 4q .. 4q+3
    const int channel = group_begin * 128 + 4 * q;
    if ((kPath == 0 || kPath == 4 || kPath == 6 || kPath == 7) && p.perm == nullptr) return make_int4(channel, channel + 1, channel + 2, channel + 3);
    if (perm_aligned) return __ldg(reinterpret_cast<const int4 *>(p.perm) + (channel >> 2));
    return make_int4(__ldg(p.perm + channel), __ldg(p.perm + channel + 1), __ldg(p.perm + channel + 2),
                     __ldg(p.perm + channel + 3));
  };
  if (gather_from_linear) {
#pragma unroll
    for (int it = 0; it < kItemBatch; ++it) {
      const int q = tid + it * threads;
      if (q < items) held[it] = load_item(q);
    }
  }
  // Everything above read only weights, codebook and permutation (never written by a kernel);
  // from here on the activations of the previous kernel are read and global memory is written.
  pdl_wait();
  SAGE_STAMP(14);
  float square_sum = 0.0f;
  if (fused) {
    // the whole row, in original channel order, into the linear buffer (and the norm
    // weights behind it); loads of a batch first, arithmetic and stores after
    const uint4 *a4 = reinterpret_cast<const uint4 *>(params.act_a);
    const uint4 *b4 = reinterpret_cast<const uint4 *>(params.act_b);
    const uint4 *w4 = reinterpret_cast<const uint4 *>(params.act_weight);
    uint4 *out4 = reinterpret_cast<uint4 *>(x_linear);
    uint4 *weight4 = reinterpret_cast<uint4 *>(x_linear + p.k);
    uint4 *residual4 = (fused == 1 && blockIdx.x == 0) ? reinterpret_cast<uint4 *>(params.act_residual_out) : nullptr;
    const int row_pieces = p.k >> 3;
    for (int base = 0; base < row_pieces; base += kCopyBatch * threads) {
      uint4 pa[kCopyBatch], pb[kCopyBatch], pw[kCopyBatch];
#pragma unroll
      for (int it = 0; it < kCopyBatch; ++it) {
        const int i = base + tid + it * threads;
        if (i < row_pieces) {
          pa[it] = __ldg(a4 + i);
          pb[it] = b4 ? __ldg(b4 + i) : make_uint4(0, 0, 0, 0);
          if (fused == 1) pw[it] = __ldg(w4 + i);
        }
      }
#pragma unroll
      for (int it = 0; it < kCopyBatch; ++it) {
        const int i = base + tid + it * threads;
        if (i >= row_pieces) continue;
        uint4 value;
        const __half2 *ah = reinterpret_cast<const __half2 *>(&pa[it]);
        const __half2 *bh = reinterpret_cast<const __half2 *>(&pb[it]);
        __half2 *vh = reinterpret_cast<__half2 *>(&value);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          if (fused == 1) {
            vh[c] = b4 ? __hadd2(ah[c], bh[c]) : ah[c];
            const float2 f = __half22float2(vh[c]);
            square_sum = fmaf(f.x, f.x, fmaf(f.y, f.y, square_sum));
          } else {
            const float2 g2 = __half22float2(ah[c]);
            const __half2 silu = __floats2half2_rn(silu_fast(g2.x), silu_fast(g2.y));
            vh[c] = __hmul2(silu, bh[c]);
          }
        }
        out4[i] = value;
        if (fused == 1) weight4[i] = pw[it];
        if (residual4) residual4[i] = value;
      }
    }
    if (fused == 1) {
#pragma unroll
      for (int o = 16; o; o >>= 1) square_sum += __shfl_xor_sync(0xffffffffu, square_sum, o);
      if (lane == 0) norm_sums[warp] = square_sum;
    }
  }
  auto load_piece = [&](int i) {
    if (direct_copy) {
      const int m = i / vectors;
      const int v = i - m * vectors;
      return __ldg(reinterpret_cast<const uint4 *>(p.x + static_cast<size_t>(m) * p.k +
                                                    group_begin * 128 + v * 8));
    }
    return __ldg(reinterpret_cast<const uint4 *>(p.x) + i);
  };
#pragma unroll
  for (int it = 0; it < kCopyBatch; ++it) {
    const int i = tid + it * threads;
    if (i < pieces) piece[it] = load_piece(i);
  }
  // ... and now the stores
  auto store_entry = [&](int e, const uint4 &value) {
    uint4 *line = reinterpret_cast<uint4 *>(book_shared) + e * 8;
#pragma unroll
    for (int r = 0; r < 8; ++r) line[(r + lane) & 7] = value;
  };
  if (tid < p.entries) store_entry(tid, entry);
  for (int e = tid + threads; e < p.entries; e += threads) {  // CTAs with fewer threads than entries
    uint4 value;
    value.x = __ldg(p.book + e);
    value.y = __ldg(p.book + p.entries + e);
    value.z = __ldg(p.book + 2 * p.entries + e);
    value.w = __ldg(p.book + 3 * p.entries + e);
    store_entry(e, value);
  }
  auto store_direct = [&](int i, const uint4 &value) {
    const int m = i / vectors;
    const int v = i - m * vectors;
    const int vg = v & 15;
    const int target = (v >> 4) * 128 + (vg & 3) * 32 + (vg >> 2) * 8;
    *reinterpret_cast<uint4 *>(x_shared + m * row_stride + target) = value;
  };
#pragma unroll
  for (int it = 0; it < kCopyBatch; ++it) {
    const int i = tid + it * threads;
    if (i < pieces) {
      if (direct_copy) store_direct(i, piece[it]);
      else reinterpret_cast<uint4 *>(x_linear)[i] = piece[it];
    }
  }
  for (int base = kCopyBatch * threads; base < pieces; base += kCopyBatch * threads) {
    // long rows / many rows: further batches, loads before stores again
#pragma unroll
    for (int it = 0; it < kCopyBatch; ++it) {
      const int i = base + tid + it * threads;
      if (i < pieces) piece[it] = load_piece(i);
    }
#pragma unroll
    for (int it = 0; it < kCopyBatch; ++it) {
      const int i = base + tid + it * threads;
      if (i < pieces) {
        if (direct_copy) store_direct(i, piece[it]);
        else reinterpret_cast<uint4 *>(x_linear)[i] = piece[it];
      }
    }
  }
  if (linear_gather && !aligned_x && !fused) {
    const int total = p.rows * p.k;
#pragma unroll 8
    for (int i = tid; i < total; i += threads) x_linear[i] = p.x[i];
  }
  if (!direct_copy && !gather_from_linear) {
    for (int q = tid; q < items; q += threads) {
      const int channel = group_begin * 128 + 4 * q;
      int4 source = make_int4(channel, channel + 1, channel + 2, channel + 3);
      if (p.perm) {
        source.x = __ldg(p.perm + channel);
        source.y = __ldg(p.perm + channel + 1);
        source.z = __ldg(p.perm + channel + 2);
        source.w = __ldg(p.perm + channel + 3);
      }
      const int i = 4 * q;
      const int vector = (i >> 3) & 15;
      const int target = (i & ~127) + (vector & 3) * 32 + (vector >> 2) * 8 + (i & 7);
      for (int m = 0; m < p.rows; ++m) {
        const __half *row = p.x + static_cast<size_t>(m) * p.k;
        __align__(8) __half values[4] = {row[source.x], row[source.y], row[source.z], row[source.w]};
        *reinterpret_cast<uint2 *>(x_shared + m * row_stride + target) =
            *reinterpret_cast<const uint2 *>(values);
      }
    }
  }
  SAGE_STAMP(2);
  const bool any_split = __syncthreads_or(shared_tile) != 0;
  SAGE_STAMP(3);

  if (gather_from_linear) {  // warp-uniform: the gather out of shared memory, then a second barrier
    float norm_scale = 1.0f;
    if (fused == 1) {
      float total = 0.0f;
      for (int w = 0; w < warps; ++w) total += norm_sums[w];
      norm_scale = rsqrtf(total / static_cast<float>(p.k) + params.act_eps);
    }
    const __half *weight_linear = x_linear + p.k;
    for (int base = 0; base < items; base += kItemBatch * threads) {
      if (base > 0) {
#pragma unroll
        for (int it = 0; it < kItemBatch; ++it) {
          const int q = base + tid + it * threads;
          if (q < items) held[it] = load_item(q);
        }
      }
#pragma unroll
      for (int it = 0; it < kItemBatch; ++it) {
        const int q = base + tid + it * threads;
        if (q >= items) continue;
        const int4 source = held[it];
        const int i = 4 * q;
        const int vector = (i >> 3) & 15;
        const int target = (i & ~127) + (vector & 3) * 32 + (vector >> 2) * 8 + (i & 7);
        for (int m = 0; m < p.rows; ++m) {
          const __half *row = x_linear + m * p.k;
          __align__(8) __half values[4] = {row[source.x], row[source.y], row[source.z], row[source.w]};
          if (fused == 1) {  // RMSNorm: weight * fp16(value * scale), as the unfused kernel rounds
            const int sources[4] = {source.x, source.y, source.z, source.w};
#pragma unroll
            for (int c = 0; c < 4; ++c)
              values[c] = __hmul(weight_linear[sources[c]],
                                 __float2half_rn(__half2float(values[c]) * norm_scale));
          }
          *reinterpret_cast<uint2 *>(x_shared + m * row_stride + target) =
              *reinterpret_cast<const uint2 *>(values);
        }
      }
    }
    __syncthreads();
  }

  SAGE_STAMP(4);
  // ---- 4. wait (bounded) for this warp's weights
  bool ready = ring || barrier_done(bar, 0);
  if (!ready) {
    const unsigned long long begin = global_timer();
    unsigned spins = 0;
    while (!(ready = barrier_done(bar, 0))) {
      if ((++spins & 255u) == 0 && global_timer() - begin > kWaitLimitNs) break;
    }
  }
  ready = __all_sync(0xffffffffu, ready);
  if (!ready && lane == 0 && params.status) atomicExch(params.status, -7);

  SAGE_STAMP(5);
  // ---- 5. main loop over this warp's units
  FieldConsts f;
  f.index_mask = static_cast<uint32_t>(p.entries - 1) << 7;
  f.hi_shift = 27 - p.dbits;
  f.hi_mask = 3u << f.hi_shift;
  f.lo_mask = ((1u << (8 - p.dbits)) - 1u) << 19;
  f.lo_left = 11 - p.dbits;
  f.lo_right = 5 + p.dbits;
  const uint32_t lane_offset = 16u * static_cast<uint32_t>(lane & 7);
  const unsigned char *x_row_base[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int m = min(g + 8 * nb, p.rows - 1);
    x_row_base[nb] = reinterpret_cast<const unsigned char *>(x_shared + m * row_stride) + 16 * t;
  }
  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[nb][c] = 0.0f;

  constexpr int kSegmentFloats = NB * 128;
  float *my_partial =
      partial_shared + static_cast<size_t>(warp) * params.warp_segments * kSegmentFloats;
  int first_tile = 0, tile_count = 0;
  if (ready && warp_end > warp_begin) {
    const int tile0 = warp_begin / group_count;
    int gi = warp_begin - tile0 * group_count;
    first_tile = tile0;
    int slot = ring ? warp * kRingSlots : warp_begin - unit_begin;  // shared-memory slot of unit u
    int chunk = 0, in_chunk = 0;
    for (int u = warp_begin; u < warp_end; ++u) {
      if (ring && in_chunk == 0) {
        // wait (bounded) for this chunk's bytes; the stage's phase flips every kRingStages chunks
        const uint32_t stage_bar = bar + 8u * static_cast<uint32_t>(chunk % kRingStages);
        const uint32_t parity = static_cast<uint32_t>(chunk / kRingStages) & 1u;
        bool arrived = barrier_done(stage_bar, parity);
        if (!arrived) {
          const unsigned long long begin = global_timer();
          unsigned spins = 0;
          while (!(arrived = barrier_done(stage_bar, parity))) {
            if ((++spins & 255u) == 0 && global_timer() - begin > kWaitLimitNs) break;
          }
        }
        arrived = __all_sync(0xffffffffu, arrived);
        if (!arrived) {
          if (lane == 0 && params.status) atomicExch(params.status, -7);
          break;
        }
        slot = warp * kRingSlots + (chunk % kRingStages) * kRingUnits;
      }
      const unsigned char *code_ptr = codes_shared + static_cast<size_t>(slot) * 512 + g * 32 + t * 8;
      const unsigned char *radius_ptr = radii_shared + static_cast<size_t>(slot) * 64 + g * 4;
      const unsigned char *grid_ptr = grid_shared + static_cast<size_t>(slot) * 64 + g * 4;
      uint2 code[2];
      uint32_t radius_word[2], endpoints[2];
      code[0] = *reinterpret_cast<const uint2 *>(code_ptr);
      code[1] = *reinterpret_cast<const uint2 *>(code_ptr + 256);
      radius_word[0] = *reinterpret_cast<const uint32_t *>(radius_ptr);
      radius_word[1] = *reinterpret_cast<const uint32_t *>(radius_ptr + 32);
      endpoints[0] = *reinterpret_cast<const uint32_t *>(grid_ptr);
      endpoints[1] = *reinterpret_cast<const uint32_t *>(grid_ptr + 32);
      const unsigned char *x_row[NB];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) x_row[nb] = x_row_base[nb] + 256 * gi;
      compute_unit<NB, kLowBits>(code, radius_word, endpoints, acc, f, book_shared, lane_offset, x_row, t);
      ++slot;
      ++gi;
      if (ring && (++in_chunk == kRingUnits || u + 1 == warp_end)) {
        // the whole warp is done with this stage: refill it with the chunk kRingStages ahead
        __syncwarp();
        if (lane == 0 && (chunk + kRingStages) * kRingUnits < warp_units) ring_issue(chunk + kRingStages);
        ++chunk;
        in_chunk = 0;
      }
      if (gi == group_count || u + 1 == warp_end) {
        // this warp is done with the tile: park its partial sums
        float *dst = my_partial + tile_count * kSegmentFloats;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          *reinterpret_cast<float2 *>(dst + nb * 128 + g * 8 + 2 * t) =
              make_float2(acc[nb][0], acc[nb][1]);
          *reinterpret_cast<float2 *>(dst + nb * 128 + (g + 8) * 8 + 2 * t) =
              make_float2(acc[nb][2], acc[nb][3]);
#pragma unroll
          for (int c = 0; c < 4; ++c) acc[nb][c] = 0.0f;
        }
        ++tile_count;
        gi = 0;
      }
    }
  }
  if (lane == 0) {
    warp_first_tile[warp] = first_tile;
  }

  SAGE_STAMP(6);
  __syncthreads();

  SAGE_STAMP(7);
  // ---- 7. combine the warps (warp order = K order) and write y or the partial.
  //         Item e = tile * (NB*128) + the accumulator's position [nb][row][column % 8].
  const int columns = p.rows;              // valid MMA columns
  const int tile_elements = 16 * columns;  // scratch element r = row*columns + column
  const int slots = p.slots_per_tile;
  for (int e = tid; e < cta_tiles * kSegmentFloats; e += threads) {
    const int ti = e / kSegmentFloats;
    const int position = e - ti * kSegmentFloats;
    const int row = (position >> 3) & 15;
    const int column = (position >> 7) * 8 + (position & 7);
    if (column >= columns) continue;
    const int tile = cta_first_tile + ti;
    float sum = 0.0f;
    for (int w = tile_warp_lo[ti]; w <= tile_warp_hi[ti]; ++w)
      sum += partial_shared[(static_cast<size_t>(w) * params.warp_segments + (tile - warp_first_tile[w])) *
                                kSegmentFloats + position];
    if (whole || tile_parts[ti] == 1) {
      const int out = tile * 16 + row;
      if (out < p.n) p.y[static_cast<size_t>(column) * p.n + out] = __float2half_rn(sum);
    } else {
      __stcg(p.partial + (static_cast<size_t>(tile) * slots + tile_slot[ti]) * tile_elements +
                 row * columns + column, sum);
    }
  }
  SAGE_STAMP(8);
  SAGE_STAMP_NS(15);
  if (!any_split) return;

  // ---- 8. tiles shared with other CTAs: publish, count arrivals, the last one finishes.
  //         The barrier orders the CTA's partial stores before the counting thread's
  //         fence + atomic (release); the same thread's fence after the atomic and the
  //         next barrier order the other CTAs' partials before this CTA's reads (acquire).
  __syncthreads();
  for (int ti = tid; ti < cta_tiles; ti += threads) {
    if (tile_parts[ti] <= 1) continue;
    __threadfence();
    const unsigned arrived = atomicAdd(p.counters + cta_first_tile + ti, 1u);
    __threadfence();
    tile_last[ti] = (arrived == static_cast<unsigned>(tile_parts[ti]) - 1u);
  }
  __syncthreads();
  SAGE_STAMP(9);
  for (int e = tid; e < cta_tiles * tile_elements; e += threads) {
    const int ti = e / tile_elements;
    if (!tile_last[ti]) continue;
    const int r = e - ti * tile_elements;
    const int row = r / columns;
    const int column = r - row * columns;
    const int tile = cta_first_tile + ti;
    const float *pieces = p.partial + static_cast<size_t>(tile) * slots * tile_elements + r;
    float sum = 0.0f;
    for (int k = 0; k < tile_parts[ti]; ++k)
      sum += __ldcg(pieces + static_cast<size_t>(k) * tile_elements);
    const int out = tile * 16 + row;
    if (out < p.n) p.y[static_cast<size_t>(column) * p.n + out] = __float2half_rn(sum);
  }
  __syncthreads();
  for (int ti = tid; ti < cta_tiles; ti += threads)
    if (tile_last[ti]) p.counters[cta_first_tile + ti] = 0u;
  SAGE_STAMP(10);
  SAGE_STAMP_NS(15);
#undef SAGE_STAMP
#undef SAGE_STAMP_NS
}

template <int NB, bool kLowBits, int kPath = 0>
cudaError_t configure_variant() {
  if (NB == 1) {  // ring streaming exists for up to eight activation rows
    const cudaError_t status = cudaFuncSetAttribute(sage_skinny_kernel<1, kLowBits, kPath, true>,
                                                    cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicShared);
    if (status != cudaSuccess) return status;
  }
  return cudaFuncSetAttribute(sage_skinny_kernel<NB, kLowBits, kPath>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicShared);
}

size_t x_bytes_for(int rows, int group_span) {
  return (static_cast<size_t>(rows) * (static_cast<size_t>(group_span) * 256 + 64) + 127) / 128 * 128;
}

int slice_groups(int groups, int slices, int slice) {
  return static_cast<int>(static_cast<long long>(groups) * (slice + 1) / slices) -
         static_cast<int>(static_cast<long long>(groups) * slice / slices);
}

}  // namespace

SkinnyPlan plan_skinny(int rows, int n, int k, int entries, int sm_count, const Tuning &tuning,
                       int cta_budget, int act_kind) {
  (void)entries;
  SkinnyPlan plan{};
  const int tiles = (n + 15) / 16;
  const int groups = k / 128;
  plan.tiles = tiles;
  plan.column_blocks = rows > 8 ? 2 : 1;
  plan.ctas_per_sm = tuning.ctas_per_sm > 0 ? tuning.ctas_per_sm : 1;
  plan.warps = tuning.warps > 0 ? tuning.warps : 16;
  if (plan.warps > kMaxWarps) plan.warps = kMaxWarps;
  // CTAs this problem may occupy at once: the whole device, or its share of a grouped launch
  const int resident = cta_budget > 0 ? cta_budget : sm_count * plan.ctas_per_sm;
  const int unit_cap = 192;  // 192 * 640 B = 120 KiB of packed weights per CTA

  // K slices: as few as keep one slice's activations within the shared-memory budget
  // (a single row may take more: its launch streams the weights through rings if need be)
  // Several rows: whatever one resident wave's packed share and the warps' tables leave of the
  // CTA's shared memory (at least 40 KiB) - slicing K costs a trip through scratch per tile.
  size_t x_budget = 64 * 1024;
  if (rows > 1) {
    long long share_units = (static_cast<long long>(tiles) * groups + resident - 1) / resident;
    if (share_units > unit_cap) share_units = unit_cap;
    // (the warps' partial-sum tables: a warp touches its units / groups + 2 tiles at most)
    const long long warp_units = (share_units + plan.warps - 1) / plan.warps;
    const size_t tables = static_cast<size_t>(plan.warps) * static_cast<size_t>(warp_units / groups + 2) *
                          plan.column_blocks * 512;
    const size_t taken = static_cast<size_t>(share_units) * kUnitBytes + tables + 4096;
    x_budget = taken + 40 * 1024 < static_cast<size_t>(kMaxDynamicShared) ? kMaxDynamicShared - taken : 40 * 1024;
  }
  // a single row with a permutation is gathered through a linear copy in shared memory; the
  // fused residual add + RMSNorm keeps the norm weights behind it
  const size_t lin_bytes = rows == 1 ? (static_cast<size_t>(k) * (act_kind == 1 ? 4 : 2) + 127) / 128 * 128 : 0;
  int slices = tuning.slices > 0 ? tuning.slices : 1;
  if (slices > kMaxSlices) slices = kMaxSlices;
  if (slices > groups) slices = groups;
  while (slices < kMaxSlices && slices < groups &&
         x_bytes_for(rows, (groups + slices - 1) / slices) > x_budget)
    ++slices;

  // Whole tiles per CTA or an even share of units?  Sharing a tile between CTAs costs a
  // trip through scratch memory and an arrival counter, about as long as decoding
  // kFinishUnits units; whole tiles cost imbalance when tiles are few.  Compare per SM.
  constexpr int kFinishUnits = 50;
  const long long even_cost =
      (static_cast<long long>(tiles) * groups + resident - 1) / resident + kFinishUnits;
  const long long whole_cost = static_cast<long long>((tiles + resident - 1) / resident) * groups;
  bool whole = slices == 1 && whole_cost <= even_cost;
  if (tuning.mode == 1) whole = false;
  if (tuning.mode == 2 && slices == 1) whole = true;
  if (whole) {
    long long ctas = resident < tiles ? resident : tiles;
    const long long cta_tiles = (tiles + ctas - 1) / ctas;
    const long long cta_units = cta_tiles * groups;
    // a CTA's tiles either fit its shared memory or (one resident wave kept) stream through rings
    const bool ring = cta_units > unit_cap;  // (up to eight activation rows only)
    if (ring && (cta_tiles > kMaxWholeTiles || tuning.mode == 3 || plan.column_blocks != 1)) whole = false;
    if (whole) {
      plan.whole_tiles = 1;
      plan.slices = 1;
      plan.ctas_per_slice = static_cast<int>(ctas);
      plan.ctas = plan.ctas_per_slice;
      const int warp_units = static_cast<int>((cta_units + plan.warps - 1) / plan.warps);
      plan.warp_segments = warp_units / groups + 2;
      plan.slots_per_tile = 1;
      plan.x_bytes = x_bytes_for(rows, groups);
      plan.needs_scratch = false;
      plan.partial_bytes = 0;
      const size_t fixed = plan.x_bytes + lin_bytes +
                           static_cast<size_t>(plan.warps) * plan.warp_segments * plan.column_blocks * 512;
      plan.ring = 0;
      plan.unit_capacity = static_cast<int>(cta_units);
      if (ring) {  // units per ring stage: as many as fit beside the row's buffers
        int units = kRingUnitsMax;
        while (units > 0 && fixed + static_cast<size_t>(plan.warps) * kRingStages * units * kUnitBytes >
                                static_cast<size_t>(kMaxDynamicShared))
          units >>= 1;
        plan.ring = units;
        plan.unit_capacity = plan.warps * kRingStages * units;
        if (units == 0) whole = false;
      }
      if (fixed + static_cast<size_t>(plan.unit_capacity) * kUnitBytes > static_cast<size_t>(kMaxDynamicShared))
        whole = false;
    }
  }
  if (!whole) {
    plan.whole_tiles = 0;
    plan.slices = slices;
    int min_groups = groups, max_groups = 0;
    for (int s = 0; s < slices; ++s) {
      const int count = slice_groups(groups, slices, s);
      if (count < min_groups) min_groups = count;
      if (count > max_groups) max_groups = count;
    }
    // CTAs per slice: the resident grid, but never more CTAs than units, and enough CTAs
    // that one CTA's units and tiles fit its shared-memory tables
    const long long min_units = static_cast<long long>(tiles) * min_groups;
    const long long max_units = static_cast<long long>(tiles) * max_groups;
    long long per_slice = resident / slices;
    if (per_slice < 1) per_slice = 1;
    // more units than one resident wave holds in shared memory: stream them through rings
    // (unsliced K only), else add CTAs (further waves)
    bool ring = slices == 1 && per_slice * unit_cap < max_units && tuning.mode != 3 && plan.column_blocks == 1;
    if (!ring && per_slice * unit_cap < max_units) per_slice = (max_units + unit_cap - 1) / unit_cap;
    const int tile_cap = kMaxCtaTiles - 2;
    while ((max_units + per_slice - 1) / per_slice / min_groups + 2 > tile_cap) ++per_slice;
    if (per_slice > min_units) per_slice = min_units;
    const size_t fixed = x_bytes_for(rows, max_groups) + lin_bytes;
    int ring_units = 0;
    while (true) {  // more (smaller) CTAs until one CTA's units fit shared memory
      const int cta_units = static_cast<int>((max_units + per_slice - 1) / per_slice);
      if (ring && cta_units <= unit_cap) ring = false;
      const int warp_units = (cta_units + plan.warps - 1) / plan.warps;
      plan.warp_segments = warp_units / min_groups + 2;
      const size_t tables = static_cast<size_t>(plan.warps) * plan.warp_segments * plan.column_blocks * 512;
      ring_units = 0;
      if (ring) {  // units per ring stage: as many as fit beside the row's buffers
        ring_units = kRingUnitsMax;
        while (ring_units > 0 && fixed + tables + static_cast<size_t>(plan.warps) * kRingStages * ring_units * kUnitBytes >
                                     static_cast<size_t>(kMaxDynamicShared))
          ring_units >>= 1;
      }
      plan.unit_capacity = ring ? plan.warps * kRingStages * ring_units : cta_units;
      const size_t shared = fixed + tables + static_cast<size_t>(plan.unit_capacity) * kUnitBytes;
      if ((shared <= static_cast<size_t>(kMaxDynamicShared) && (!ring || ring_units > 0)) || (!ring && per_slice >= min_units)) break;
      if (ring) {  // the rings do not fit beside this row's buffers: back to further waves
        ring = false;
        if (per_slice * unit_cap < max_units) per_slice = (max_units + unit_cap - 1) / unit_cap;
        continue;
      }
      per_slice += (per_slice + 3) / 4;
      if (per_slice > min_units) per_slice = min_units;
    }
    plan.ring = ring ? ring_units : 0;
    plan.ctas_per_slice = static_cast<int>(per_slice);
    plan.ctas = plan.ctas_per_slice * slices;
    // pieces per tile: in each slice a tile's units span at most `parts` CTAs
    const long long least = min_units / per_slice;  // units in the smallest CTA range, >= 1
    const int parts = static_cast<int>((max_groups + least - 1) / least) + 1;
    plan.slots_per_tile = slices * parts;
    plan.x_bytes = x_bytes_for(rows, max_groups);
    // every tile is whole inside one CTA only if K is unsliced and CTA ranges end on tile ends
    const bool aligned = slices == 1 && max_units % per_slice == 0 &&
                         (max_units / per_slice) % groups == 0;
    plan.needs_scratch = !aligned;
    plan.partial_bytes = plan.needs_scratch ? static_cast<size_t>(tiles) * plan.slots_per_tile *
                                                  16 * rows * sizeof(float)
                                            : 0;
  }
  // a single activation row with a permutation is gathered through a linear copy in
  // shared memory (several rows arrive pre-gathered)
  plan.lin_bytes = lin_bytes;
  plan.shared_bytes = plan.x_bytes + static_cast<size_t>(plan.unit_capacity) * kUnitBytes +
                      static_cast<size_t>(plan.warps) * plan.warp_segments * plan.column_blocks * 512 +
                      plan.lin_bytes;
  return plan;
}

bool skinny_shared_fits(size_t x_bytes, int unit_capacity, int warps, int warp_segments, int column_blocks,
                        size_t lin_bytes) {
  return x_bytes + static_cast<size_t>(unit_capacity) * kUnitBytes +
             static_cast<size_t>(warps) * warp_segments * column_blocks * 512 + lin_bytes <=
         static_cast<size_t>(kMaxDynamicShared);
}

cudaError_t configure_skinny() {
  cudaError_t status = configure_variant<1, false>();
  if (status == cudaSuccess) status = configure_variant<1, true>();
  if (status == cudaSuccess) status = configure_variant<2, false>();
  if (status == cudaSuccess) status = configure_variant<2, true>();
  if (status == cudaSuccess) status = configure_variant<1, false, 1>();
  if (status == cudaSuccess) status = configure_variant<1, true, 1>();
  if (status == cudaSuccess) status = configure_variant<1, false, 2>();
  if (status == cudaSuccess) status = configure_variant<1, true, 2>();
  if (status == cudaSuccess) status = configure_variant<1, false, 3>();
  if (status == cudaSuccess) status = configure_variant<1, true, 3>();
  if (status == cudaSuccess) status = configure_variant<1, false, 4>();
  if (status == cudaSuccess) status = configure_variant<1, true, 4>();
  if (status == cudaSuccess) status = configure_variant<1, false, 5>();
  if (status == cudaSuccess) status = configure_variant<1, true, 5>();
  if (status == cudaSuccess) status = configure_variant<1, false, 6>();
  if (status == cudaSuccess) status = configure_variant<1, true, 6>();
  if (status == cudaSuccess) status = configure_variant<2, false, 6>();
  if (status == cudaSuccess) status = configure_variant<2, true, 6>();
  if (status == cudaSuccess) status = configure_variant<1, false, 7>();
  if (status == cudaSuccess) status = configure_variant<1, true, 7>();
  if (status == cudaSuccess) status = configure_variant<2, false, 7>();
  if (status == cudaSuccess) status = configure_variant<2, true, 7>();
  return status;
}

// Only in a -DSAGEB200_TRACE build: environment SAGEB200_PATHS=0 keeps every launch on the
// generic kernel (A/B timing); the default build always takes the specialised kernels.
int skinny_path_limit() {
#ifdef SAGEB200_TRACE
  static const int limit = [] {
    const char *text = getenv("SAGEB200_PATHS");
    return text ? atoi(text) : -1;
  }();
  return limit;
#else
  return -1;
#endif
}

cudaError_t launch_skinny(const SkinnyParams &params, int warps, int column_blocks, int total_ctas,
                          cudaStream_t stream) {
  const size_t shared_bytes = params.x_bytes + static_cast<size_t>(params.unit_capacity) * kUnitBytes +
                              static_cast<size_t>(warps) * params.warp_segments * column_blocks * 512 +
                              params.lin_bytes;
  if (shared_bytes > static_cast<size_t>(kMaxDynamicShared)) return cudaErrorInvalidConfiguration;
  const int threads = warps * 32;
  bool low_bits = false;
  for (int i = 0; i < params.count; ++i) low_bits = low_bits || params.problem[i].dbits != 8;
  // the decode graph's launches take a specialised instruction stream (see the kernel's comment)
  int path = column_blocks == 1 ? (params.act_kind == 0 ? 3 : params.act_kind) : 0;
  for (int i = 0; i < params.count && path != 0; ++i) {
    const SkinnyProblem &q = params.problem[i];
    const bool fits = static_cast<size_t>(q.k) * (params.act_kind == 1 ? 4 : 2) <= static_cast<size_t>(params.lin_bytes);
    if (q.expert_ids != nullptr && path == 3) path = 5;  // routed experts: kind 3 plus the indirection
    if (q.rows != 1 || q.slices != 1 || (q.expert_ids != nullptr && path != 5) || q.perm == nullptr ||
        (reinterpret_cast<uintptr_t>(q.perm) & 15) != 0 || !fits ||
        ((path == 3 || path == 5) && (reinterpret_cast<uintptr_t>(q.x) & 15) != 0))
      path = 0;
  }
  bool single_rows = column_blocks == 1;
  for (int i = 0; i < params.count; ++i) single_rows = single_rows && params.problem[i].rows == 1;
  if (path == 0 && single_rows) path = 4;  // one activation row, everything else as it comes
  if (path == 0 && params.act_kind == 0) {  // several rows staged beforehand (kind 6; 7 with K slices)
    path = 6;
    for (int i = 0; i < params.count && path != 0; ++i) {
      const SkinnyProblem &q = params.problem[i];
      if (q.expert_ids != nullptr || q.perm != nullptr || (reinterpret_cast<uintptr_t>(q.x) & 15) != 0)
        path = 0;
      else if (q.slices != 1)
        path = 7;
    }
  }
  // debug switch: 0 = generic kernel only, 3 = kinds 1-3 only, 4 = kind 4 for every single-row launch,
  // 6 = no kind 7
  const int limit = skinny_path_limit();
  if (limit == 0) path = 0;
  if (limit == 3 && path >= 4) path = 0;
  if (limit == 6 && path == 7) path = 0;
  if (limit == 4) path = single_rows ? 4 : 0;
  bool ring = false;  // (the planner gives every problem of a launch the same answer, or none)
  for (int i = 0; i < params.count; ++i) ring = ring || params.problem[i].ring != 0;
  if (ring && column_blocks != 1) return cudaErrorInvalidConfiguration;  // (the planner never asks for it)
#define SAGE_LAUNCH(NB_, LOW_, PATH_)                                                                       \
  (ring && NB_ == 1 ? launch_dependent(sage_skinny_kernel<1, LOW_, PATH_, true>, total_ctas, threads,       \
                                       shared_bytes, stream, params)                                        \
                    : launch_dependent(sage_skinny_kernel<NB_, LOW_, PATH_>, total_ctas, threads, shared_bytes, \
                                       stream, params))
  if (column_blocks == 1) {
    switch (path) {
      case 1: return low_bits ? SAGE_LAUNCH(1, true, 1) : SAGE_LAUNCH(1, false, 1);
      case 2: return low_bits ? SAGE_LAUNCH(1, true, 2) : SAGE_LAUNCH(1, false, 2);
      case 3: return low_bits ? SAGE_LAUNCH(1, true, 3) : SAGE_LAUNCH(1, false, 3);
      case 4: return low_bits ? SAGE_LAUNCH(1, true, 4) : SAGE_LAUNCH(1, false, 4);
      case 5: return low_bits ? SAGE_LAUNCH(1, true, 5) : SAGE_LAUNCH(1, false, 5);
      case 6: return low_bits ? SAGE_LAUNCH(1, true, 6) : SAGE_LAUNCH(1, false, 6);
      case 7: return low_bits ? SAGE_LAUNCH(1, true, 7) : SAGE_LAUNCH(1, false, 7);
      default: return low_bits ? SAGE_LAUNCH(1, true, 0) : SAGE_LAUNCH(1, false, 0);
    }
  }
  if (path == 6) return low_bits ? SAGE_LAUNCH(2, true, 6) : SAGE_LAUNCH(2, false, 6);
  if (path == 7) return low_bits ? SAGE_LAUNCH(2, true, 7) : SAGE_LAUNCH(2, false, 7);
  return low_bits ? SAGE_LAUNCH(2, true, 0) : SAGE_LAUNCH(2, false, 0);
#undef SAGE_LAUNCH
  return cudaGetLastError();
}

}  // namespace sageb200
