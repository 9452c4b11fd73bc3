// One decoded token of a SAGE-packed Qwen3 (batch 1, one GPU) as ONE persistent kernel.
//
// The launch-per-linear path (sage_skinny.cu + qwen3_glue.cu) spends most of a token in fixed
// per-launch latencies: instruction fetch of once-per-launch code, partition arithmetic, the
// wait for the previous kernel, tables, staging.  Here one cooperative grid of one CTA per SM
// walks the whole token - per layer: [residual add + RMSNorm + q/k/v], attention (split over
// the context) and its combination, o_proj, [residual add + RMSNorm + gate/up + SwiGLU],
// down_proj; then the final norm, the FP16 lm_head and the greedy argmax - with a grid barrier
// between dependent phases.  The code stays resident in the instruction caches, nothing is
// planned on the device, and every warp streams its share of the NEXT phase's packed weights
// into its shared-memory ring (TMA bulk copies on mbarriers) as soon as it has finished the
// current phase, so the HBM stream runs through barriers and activation staging.
//
// Replaces, for this configuration, what the reference runs as Hugging Face modules around
// 7 x layers calls of sage_gemv_cuda (csrc/sage/sage_gemv_cuda.cu:118-188) per token
// (benchmarks/model.py:112-116).  Packed-weight arithmetic is sage_skinny_core.cuh's; glue
// numerics are qwen3_glue.cu's (norms and softmax in FP32, one rounding to FP16 where the
// Hugging Face module returns FP16, RoPE products in FP16).
//
// Work split of a packed linear with `tiles` 16-row tiles over C CTAs: every CTA owns
// floor(tiles / C) whole tiles; the remaining tiles are cut into (tile, 128-channel group)
// units and shared out evenly, each CTA leaving an FP32 partial per touched tile in a fixed
// slot; the CONSUMER of the output adds the slots (fixed order: results do not depend on
// timing) while it stages its activations, so nothing waits inside a phase.
//
// Every wait (grid barrier, mbarrier) is bounded; a wait that runs out records
// SAGEB200_ERR_TIMEOUT in the status word, raises an abort word that ends every other wait,
// and the kernel returns.
#include "../../include/sage_b200.h"
#include "../../include/sage_b200_decode.h"

#include <cstring>
#include <vector>

#include "sage_common.cuh"
#include "sage_kernels.h"
#include "sage_skinny_core.cuh"

namespace sageb200 {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = 16;
constexpr int kStages = 2;        // ring stages per warp
constexpr int kStageUnits = 4;    // units per stage (one bulk copy per array and stage)
constexpr int kRingUnits = kStages * kStageUnits;
constexpr int kUnitBytes = 640;   // 512 codes + 64 radius words + 64 grid
constexpr int kBookBytes = 256 * 8 * 16;  // one codebook, 8 replicas
constexpr int kMaxRuns = 4;
constexpr int kMaxCtaTiles = 32;
constexpr int kWarpSegments = 8;
constexpr int kMaxGroup = 8;      // query heads per kv head
constexpr int kHeldItems = 5;     // permutation items (4 channels each) a thread holds across the barrier
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

// ------------------------------------------------------------------ plan (device-visible)

struct MegaProblem {
  const uint32_t *codes, *radii, *grid, *book;
  const int32_t *perm;   // null: identity
  __half *y;             // FP16 outputs of the rows in whole tiles (null for gate/up)
  float *patch;          // [leftover tile][slot][16]: partial sums of the shared-out tiles
  int n, tiles, entries, dbits;
  int main_tiles;        // tiles owned whole by some CTA; rows below 16 * main_tiles are final in y
  int slots;             // slots per leftover tile
};

struct MegaRun {         // a contiguous range of (tile, group) units of one problem
  int problem;           // index into the phase's problems
  int unit_begin, unit_count;
  int first_slot;        // < 0: whole tiles; else the slot of this CTA's piece of the run's first tile
};

struct MegaCtaPlan { MegaRun run[kMaxRuns]; };

struct MegaLayer {
  MegaProblem qkv[3], o, gate_up[2], down;
  const __half *input_norm, *post_norm, *q_norm, *k_norm;
  __half *k_cache, *v_cache;
};

struct MegaHeader {
  int layers, hidden, heads, kv_heads, intermediate, vocab, max_seq, ctas;
  float eps, attention_scale;
  int x_stage_bytes, scratch_bytes;   // shared-memory areas (see the kernel)
  const __half *embed, *lm_head, *final_norm, *cos_table, *sin_table;
  __half *residual[2];
  __half *attn;                       // [heads * 128]
  __half *act;                        // [intermediate]
  float *attn_partial;                // [heads][chunks][130]
  float2 *block_best;                 // [ctas]
  unsigned *sync;                     // [0] barrier arrivals, [1] exits, [2] abort
  const MegaLayer *layer;             // [layers]
  const MegaCtaPlan *plan[4];         // per phase kind, [ctas]
};

enum PhaseKind { kQkv = 0, kO = 1, kGateUp = 2, kDown = 3 };

struct PhaseMeta {       // what a CTA needs of one linear phase, in shared memory
  MegaRun run[kMaxRuns];
  MegaProblem problem[3];
  int count, k, groups, kind;
};

// ------------------------------------------------------------------ small device helpers

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned load_acquire(const unsigned *p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
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

// Per-head RMSNorm + rotate-half RoPE of 128 values held two + two per lane (the arithmetic of
// norm_rope_head in qwen3_glue.cu).
__device__ __forceinline__ void norm_rope(__half2 lo, __half2 hi, const __half *weight, const __half *cos_row,
                                          const __half *sin_row, float eps, int lane, __half2 &out_lo,
                                          __half2 &out_hi) {
  const float2 lof = __half22float2(lo), hif = __half22float2(hi);
  const float square = warp_sum(lof.x * lof.x + lof.y * lof.y + hif.x * hif.x + hif.y * hif.y);
  const float scale = rsqrtf(square / 128.0f + eps);
  const __half2 wl = reinterpret_cast<const __half2 *>(weight)[lane];
  const __half2 wh = reinterpret_cast<const __half2 *>(weight + 64)[lane];
  const __half2 nl = __hmul2(wl, __floats2half2_rn(lof.x * scale, lof.y * scale));
  const __half2 nh = __hmul2(wh, __floats2half2_rn(hif.x * scale, hif.y * scale));
  const __half2 c = reinterpret_cast<const __half2 *>(cos_row)[lane];
  const __half2 s = reinterpret_cast<const __half2 *>(sin_row)[lane];
  out_lo = __hadd2(__hmul2(nl, c), __hmul2(__hneg2(nh), s));
  out_hi = __hadd2(__hmul2(nh, c), __hmul2(nl, s));
}

__device__ __forceinline__ bool better(float value, int index, float than_value, int than_index) {
  return value > than_value || (value == than_value && index < than_index);
}

// Position of a warp in its CTA's unit list: (run, offset inside the run, units left).
struct Cursor {
  int run, offset, left;
};
__device__ __forceinline__ void cursor_seek(const PhaseMeta &m, int begin, int end, Cursor &c) {
  c.run = 0;
  c.offset = begin;
  c.left = end - begin;
  while (c.run < kMaxRuns - 1 && c.offset >= m.run[c.run].unit_count) {
    c.offset -= m.run[c.run].unit_count;
    ++c.run;
  }
}
// Next chunk (up to kStageUnits units contiguous in memory) at the cursor; false at the end.
__device__ __forceinline__ bool cursor_next(const PhaseMeta &m, Cursor &c, int &run, int &unit, int &count) {
  if (c.left <= 0) return false;
  while (c.run < kMaxRuns - 1 && c.offset >= m.run[c.run].unit_count) {
    c.offset = 0;
    ++c.run;
  }
  run = c.run;
  unit = m.run[run].unit_begin + c.offset;
  count = min(kStageUnits, min(m.run[run].unit_count - c.offset, c.left));
  if (count <= 0) {  // (a plan whose totals disagree: never loop on it)
    c.left = 0;
    return false;
  }
  c.offset += count;
  c.left -= count;
  return true;
}

// ------------------------------------------------------------------ the kernel

struct SharedState {
  MegaHeader header;
  PhaseMeta meta[3];     // linear phase P lives in slot P % 3
  unsigned long long barriers[kWarps][kStages];
  float reduce[kWarps];
  int warp_first_tile[kWarps], warp_tiles[kWarps];
  float best_value[kWarps];
  int best_index[kWarps];
  float chunk_max[32], chunk_sum[32];
  int abort;
};

__device__ __forceinline__ uint2 lds64(uint32_t address) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(address));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t address) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(address));
  return v;
}

// FP32 sum of a leftover row's slots in slot order, the loads of up to 16 slots in flight together.
__device__ __noinline__ float finished_row(const float *patch, int main_tiles, int slots, int row) {
  const float *base = patch + (static_cast<size_t>((row >> 4) - main_tiles) * slots) * 16 + (row & 15);
  float v[16];
#pragma unroll
  for (int s = 0; s < 16; ++s) v[s] = s < slots ? __ldcg(base + s * 16) : 0.0f;
  float sum = 0.0f;
#pragma unroll
  for (int s = 0; s < 16; ++s) sum += v[s];
#pragma unroll 1
  for (int s = 16; s < slots; ++s) sum += __ldcg(base + s * 16);
  return sum;
}

// Sum of the warps' partial sums of one of the CTA's tiles, row `row`, in warp order (= channel
// order); every shared-memory load is issued before the first add.
__device__ __noinline__ float tile_sum(const int *warp_first_tile, const int *warp_tiles, const float *partial,
                                       int cta_tile, int row) {
  float v[kWarps];
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const int first = warp_first_tile[w];
    const bool in = first >= 0 && cta_tile >= first && cta_tile < first + warp_tiles[w];
    v[w] = in ? partial[(w * kWarpSegments + cta_tile - first) * 16 + row] : 0.0f;
  }
  float sum = 0.0f;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) sum += v[w];
  return sum;
}

// Dynamic shared memory: [SharedState | codebooks 2 x 32 KiB | rings | x_stage | scratch]
//   rings    per warp kRingUnits x (512 + 64 + 64) bytes
//   x_stage  activations of the running phase in the MMA operand order (two buffers of K halves
//            when a CTA serves two problems with different permutations, i.e. gate/up)
//   scratch  the activation row in original channel order (+ norm weights), finished leftover
//            rows; later the warps' partial sums; in the attention phase the query heads, the new
//            key/value and the warps' partial results (x_stage and scratch together)
__global__ void __launch_bounds__(kThreads, 1)
    sage_decode_mega_kernel(const MegaHeader *__restrict__ header_global, long long *tokens, int *positions,
                            long long *log, int *step, __half *logits, int log_stride, int *status,
                            long long *trace) {
  extern __shared__ __align__(1024) unsigned char shared[];
  // Phase time stamps (global nanosecond timer, thread 0 of every CTA, 2048 per CTA) exist only
  // in a -DSAGEB200_TRACE build.
#ifdef SAGEB200_TRACE
  int stamp_index = 0;
#define MEGA_STAMP() do { if (trace && threadIdx.x == 0 && stamp_index < 2048) \
    trace[static_cast<size_t>(blockIdx.x) * 2048 + stamp_index] = global_nanoseconds(); ++stamp_index; } while (0)
#else
#define MEGA_STAMP() do { } while (0)
#endif
  MEGA_STAMP();
  SharedState &S = *reinterpret_cast<SharedState *>(shared);
  constexpr int kStateBytes = (sizeof(SharedState) + 1023) / 1024 * 1024;
  unsigned char *book_shared = shared + kStateBytes;
  unsigned char *codes_ring = book_shared + 2 * kBookBytes;
  unsigned char *radii_ring = codes_ring + kWarps * kRingUnits * 512;
  unsigned char *grid_ring = radii_ring + kWarps * kRingUnits * 64;
  unsigned char *work = grid_ring + kWarps * kRingUnits * 64;  // x_stage, then scratch

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int cta = blockIdx.x;

  // ---- header, state
  for (int i = tid; i < static_cast<int>(sizeof(MegaHeader) / 4); i += kThreads)
    reinterpret_cast<uint32_t *>(&S.header)[i] = __ldg(reinterpret_cast<const uint32_t *>(header_global) + i);
  if (tid == 0) S.abort = 0;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_address(&S.barriers[warp][s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const MegaHeader &H = S.header;
  const int ctas = H.ctas;
  __half *x_stage = reinterpret_cast<__half *>(work);
  unsigned char *scratch = work + H.x_stage_bytes;
  unsigned *const sync_words = H.sync;
  const int position = positions[0];
  long long token = tokens[0];
  if (token < 0 || token >= H.vocab) token = 0;
  unsigned barrier_target = 0;
  const int phases = H.layers * 4;  // linear phases: P = 4 * layer + kind

  // Loads linear phase P's metadata (this CTA's runs and the phase's problems) into its slot.
  // Called by one warp; visible to the others after the next __syncthreads.
  auto load_meta = [&](int P) {
    PhaseMeta &m = S.meta[P % 3];
    const int kind = P & 3;
    const MegaLayer *L = H.layer + (P >> 2);
    const MegaProblem *first = kind == kQkv ? L->qkv : kind == kO ? &L->o : kind == kGateUp ? L->gate_up : &L->down;
    const int count = kind == kQkv ? 3 : kind == kGateUp ? 2 : 1;
    const uint32_t *src = reinterpret_cast<const uint32_t *>(first);
    const uint32_t *runs = reinterpret_cast<const uint32_t *>(H.plan[kind] + cta);
    // both copies in flight together: 60 + 16 words, three per lane
    constexpr int kProblemWords = static_cast<int>(sizeof(MegaProblem) / 4), kRunWords = static_cast<int>(sizeof(MegaCtaPlan) / 4);
    uint32_t v[3];
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int i = lane + 32 * j;
      v[j] = i < count * kProblemWords ? __ldg(src + i) : (i - 3 * kProblemWords >= 0 && i - 3 * kProblemWords < kRunWords ? __ldg(runs + i - 3 * kProblemWords) : 0u);
    }
#pragma unroll
    for (int j = 0; j < 3; ++j) {
      const int i = lane + 32 * j;
      if (i < count * kProblemWords) reinterpret_cast<uint32_t *>(m.problem)[i] = v[j];
      else if (i - 3 * kProblemWords >= 0 && i - 3 * kProblemWords < kRunWords) reinterpret_cast<uint32_t *>(m.run)[i - 3 * kProblemWords] = v[j];
    }
    if (lane == 0) {
      m.count = count;
      m.kind = kind;
      m.k = kind == kO ? H.heads * 128 : kind == kDown ? H.intermediate : H.hidden;
      m.groups = m.k >> 7;
    }
  };
  static_assert(sizeof(MegaProblem) == 80 && sizeof(MegaCtaPlan) == 64, "load_meta moves 60 + 16 words with 96 lanes-slots");

  // ---- per-warp weight ring.  `issued` / `consumed` count chunks over the whole kernel: chunk c
  //      lives in stage c % kStages and completes that stage's barrier phase (c / kStages) & 1.
  unsigned issued = 0, consumed = 0;
  Cursor issue_cursor{0, 0, 0};
  int issue_slot = 0;  // meta slot of the phase the issue cursor walks
  const uint32_t ring_codes = smem_address(codes_ring) + warp * kRingUnits * 512;
  const uint32_t ring_radii = smem_address(radii_ring) + warp * kRingUnits * 64;
  const uint32_t ring_grid = smem_address(grid_ring) + warp * kRingUnits * 64;
  auto issue_one = [&]() -> bool {  // warp-uniform; lane 0 issues, all lanes keep the counters in step
    const PhaseMeta &m = S.meta[issue_slot];
    int run, unit, count;
    if (!cursor_next(m, issue_cursor, run, unit, count)) return false;
    {
      // lane 0 arms the stage's barrier, then lanes 0..2 issue the chunk's three copies (codes,
      // radius words, grid) as one instruction
      const MegaProblem &p = m.problem[m.run[run].problem];
      const uint32_t stage = issued % kStages;
      const uint32_t bar = smem_address(&S.barriers[warp][stage]);
      if (lane == 0)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                     "r"(static_cast<uint32_t>(count * kUnitBytes))
                     : "memory");
      __syncwarp();
      if (lane < 3) {
        const size_t cell = static_cast<size_t>(unit) * 16;
        const uint32_t *src = lane == 0 ? p.codes + cell * 8 : lane == 1 ? p.radii + cell : p.grid + cell;
        const uint32_t dst = (lane == 0 ? ring_codes + stage * kStageUnits * 512
                                        : (lane == 1 ? ring_radii : ring_grid) + stage * kStageUnits * 64);
        bulk_copy(dst, src, static_cast<uint32_t>(count) * (lane == 0 ? 512u : 64u), bar);
      }
    }
    ++issued;
    return true;
  };
  // Points the issue cursor at this warp's share of linear phase P and fills the ring.
  auto start_stream = [&](int P) {
    issue_slot = P % 3;
    const PhaseMeta &m = S.meta[issue_slot];
    int total = 0;
#pragma unroll
    for (int r = 0; r < kMaxRuns; ++r) total += m.run[r].unit_count;
    const int begin = static_cast<int>(static_cast<long long>(total) * warp / kWarps);
    const int end = static_cast<int>(static_cast<long long>(total) * (warp + 1) / kWarps);
    cursor_seek(m, begin, end, issue_cursor);
#pragma unroll 1
    for (int i = 0; i < kStages; ++i)
      if (!issue_one()) break;
  };

  // What a linear phase needs that no kernel writes, fetched before the grid barrier that precedes
  // it: the permutation items this thread will gather with (registers) and the codebooks of this
  // CTA's problems (replicated in shared memory; the previous phase's main loops are over).
  int4 held[kHeldItems];
  auto perm_item = [&](const PhaseMeta &m, int q) {
    const int quarter = m.k >> 2;
    const int which = q >= quarter ? 1 : 0;
    const int local = q - which * quarter;
    const int32_t *perm = m.problem[m.run[0].problem + which].perm;
    if (perm == nullptr) return make_int4(4 * local, 4 * local + 1, 4 * local + 2, 4 * local + 3);
    return __ldg(reinterpret_cast<const int4 *>(perm) + local);
  };
  // (two halves so that other work can run while the loads are in flight)
  uint4 book_entry[2];
  auto prestage_load = [&](int P) {
    const PhaseMeta &m = S.meta[P % 3];
    const int problems = m.kind == kGateUp ? 2 : 1;
    const int items = (m.k >> 2) * problems;
#pragma unroll
    for (int it = 0; it < kHeldItems; ++it) {
      const int q = tid + it * kThreads;
      if (q < items) held[it] = perm_item(m, q);
    }
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      if (which >= problems) break;
      const MegaProblem &p = m.problem[m.run[0].problem + which];
      if (tid < p.entries) {
        book_entry[which].x = __ldg(p.book + tid);
        book_entry[which].y = __ldg(p.book + p.entries + tid);
        book_entry[which].z = __ldg(p.book + 2 * p.entries + tid);
        book_entry[which].w = __ldg(p.book + 3 * p.entries + tid);
      }
    }
  };
  auto prestage_store = [&](int P) {
    const PhaseMeta &m = S.meta[P % 3];
    const int problems = m.kind == kGateUp ? 2 : 1;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      if (which >= problems) break;
      const MegaProblem &p = m.problem[m.run[0].problem + which];
      uint4 *book = reinterpret_cast<uint4 *>(book_shared + which * kBookBytes);
      if (tid < p.entries) {
#pragma unroll
        for (int r = 0; r < 8; ++r) book[tid * 8 + ((r + lane) & 7)] = book_entry[which];
      }
    }
  };

  // Grid barrier: all CTAs' earlier global writes are visible to all CTAs' later reads.
  auto grid_sync = [&]() -> bool {
    __syncthreads();
    barrier_target += static_cast<unsigned>(ctas);
    if (tid == 0) {
      asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(sync_words) : "memory");
      if (load_acquire(sync_words) < barrier_target) {
        const unsigned long long begin = global_timer();
        unsigned spins = 0;
        while (load_acquire(sync_words) < barrier_target) {
          if ((++spins & 63u) == 0) {
            if (load_acquire(sync_words + 2) != 0u) { S.abort = 1; break; }
            if (global_timer() - begin > kWaitLimitNs) {
              atomicExch(sync_words + 2, 1u);
              if (status) atomicExch(status, SAGEB200_ERR_TIMEOUT);
              S.abort = 1;
              break;
            }
          }
        }
      }
    }
    __syncthreads();
    return S.abort == 0;
  };
  // Leaves the kernel after a failed wait: copies in flight get time to land first.
  auto bail_out = [&]() {
    const unsigned long long begin = global_timer();
    while (global_timer() - begin < 200000ull) __nanosleep(2000);
  };

  // the first two phases' metadata, the first phase's stream, permutation items and codebooks
  if (warp == 0) load_meta(0);
  if (warp == 1 && phases > 1) load_meta(1);
  __syncthreads();
  start_stream(0);
  prestage_load(0);
  prestage_store(0);

  int residual_slot = 0;  // H.residual[residual_slot] holds the residual stream (after the first norm)
  const int chunks_max = max(1, min(ctas / H.kv_heads, 32));
  const int group_heads = H.heads / H.kv_heads;

#pragma unroll 1
  for (int P = 0; P < phases; ++P) {
    const int layer = P >> 2, kind = P & 3;
    const MegaLayer *L = H.layer + layer;
    const PhaseMeta &M = S.meta[P % 3];
    // ================================================================ linear phase
    // (the grid barrier that precedes it has been passed; codebooks and `held` are in place)
    MEGA_STAMP();  // phase start
    const int K = M.k, groups = M.groups;
    const int my_problems = kind == kGateUp ? 2 : 1;
    const int first_problem = M.run[0].problem;  // (gate/up: 0, the second is 1)
    const bool normed = kind == kQkv || kind == kGateUp;

    // ---- staging, step 1: the activation row into scratch in original channel order; every
    //      global load of the step is issued before the first value is used
    __half *x_lin = reinterpret_cast<__half *>(scratch);
    __half *norm_lin = x_lin + K;                       // norm weights behind the row (norm phases)
    __half *left_rows = norm_lin + (normed ? K : 0);    // finished leftover rows
    const int pieces = K >> 3;
    if (normed) {
      // x = weight * fp16((h + delta) * rsqrt(mean((h + delta)^2) + eps)); CTA 0 stores h + delta
      const bool first_norm = P == 0;
      const __half *h_in = first_norm ? H.embed + static_cast<size_t>(token) * H.hidden : H.residual[residual_slot];
      const MegaProblem *delta = first_norm ? nullptr : (kind == kQkv ? &H.layer[layer - 1].down : &L->o);
      const __half *weight = kind == kQkv ? L->input_norm : L->post_norm;
      __half *h_out = H.residual[first_norm ? 0 : residual_slot ^ 1];
      const __half *delta_y = nullptr;
      const float *delta_patch = nullptr;
      int main_tiles = 0, slots = 0, main_rows = K;
      if (delta) {
        delta_y = delta->y;
        delta_patch = delta->patch;
        main_tiles = delta->main_tiles;
        slots = delta->slots;
        main_rows = min(K, main_tiles * 16);
      }
      uint4 pa = make_uint4(0, 0, 0, 0), pb = make_uint4(0, 0, 0, 0), pw = make_uint4(0, 0, 0, 0);
      if (tid < pieces) {
        pa = first_norm ? __ldg(reinterpret_cast<const uint4 *>(h_in) + tid) : __ldcg(reinterpret_cast<const uint4 *>(h_in) + tid);
        if (delta && 8 * tid < main_rows) pb = __ldcg(reinterpret_cast<const uint4 *>(delta_y) + tid);
        pw = __ldg(reinterpret_cast<const uint4 *>(weight) + tid);
      }
#pragma unroll 1
      for (int r = main_rows + tid; r < K; r += kThreads)
        left_rows[r - main_rows] = __float2half_rn(finished_row(delta_patch, main_tiles, slots, r));
      __syncthreads();  // leftover rows are in shared memory
      float square_sum = 0.0f;
#pragma unroll 1
      for (int i = tid; i < pieces; i += kThreads) {
        if (i != tid) {  // rows longer than 8 * kThreads channels
          pa = first_norm ? __ldg(reinterpret_cast<const uint4 *>(h_in) + i) : __ldcg(reinterpret_cast<const uint4 *>(h_in) + i);
          pw = __ldg(reinterpret_cast<const uint4 *>(weight) + i);
          if (delta && 8 * i < main_rows) pb = __ldcg(reinterpret_cast<const uint4 *>(delta_y) + i);
        }
        if (delta && 8 * i >= main_rows) pb = *reinterpret_cast<const uint4 *>(left_rows + (8 * i - main_rows));
        uint4 value;
        const __half2 *ah = reinterpret_cast<const __half2 *>(&pa);
        const __half2 *bh = reinterpret_cast<const __half2 *>(&pb);
        __half2 *vh = reinterpret_cast<__half2 *>(&value);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          vh[c] = delta ? __hadd2(ah[c], bh[c]) : ah[c];
          const float2 f = __half22float2(vh[c]);
          square_sum = fmaf(f.x, f.x, fmaf(f.y, f.y, square_sum));
        }
        reinterpret_cast<uint4 *>(x_lin)[i] = value;
        reinterpret_cast<uint4 *>(norm_lin)[i] = pw;
        if (cta == 0) reinterpret_cast<uint4 *>(h_out)[i] = value;
      }
      square_sum = warp_sum(square_sum);
      if (lane == 0) S.reduce[warp] = square_sum;
      if (!first_norm) residual_slot ^= 1;
    } else if (kind == kO) {
#pragma unroll 1
      for (int i = tid; i < pieces; i += kThreads)
        reinterpret_cast<uint4 *>(x_lin)[i] = __ldcg(reinterpret_cast<const uint4 *>(H.attn) + i);
    } else {  // down: act rows of whole (gate, up) tiles are in H.act; the shared-out ones are finished here
      const float *gate_patch = L->gate_up[0].patch, *up_patch = L->gate_up[1].patch;
      const int main_tiles = L->gate_up[0].main_tiles, slots = L->gate_up[0].slots;
      const int main_rows = min(K, main_tiles * 16);
      uint4 held_act[4];  // the row's main part: up to 4 x 512 x 8 channels in flight
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = tid + j * kThreads;
        if (i < pieces && 8 * i < main_rows) held_act[j] = __ldcg(reinterpret_cast<const uint4 *>(H.act) + i);
      }
#pragma unroll 1
      for (int r = main_rows + tid; r < K; r += kThreads) {
        const __half gate = __float2half_rn(finished_row(gate_patch, main_tiles, slots, r));
        const __half up = __float2half_rn(finished_row(up_patch, main_tiles, slots, r));
        left_rows[r - main_rows] = __hmul(__float2half_rn(silu_fast(__half2float(gate))), up);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = tid + j * kThreads;
        if (i < pieces && 8 * i < main_rows) reinterpret_cast<uint4 *>(x_lin)[i] = held_act[j];
      }
#pragma unroll 1
      for (int i = tid + 4 * kThreads; i < pieces; i += kThreads)
        if (8 * i < main_rows) reinterpret_cast<uint4 *>(x_lin)[i] = __ldcg(reinterpret_cast<const uint4 *>(H.act) + i);
      __syncthreads();
#pragma unroll 1
      for (int i = tid; i < pieces; i += kThreads)
        if (8 * i >= main_rows)
          reinterpret_cast<uint4 *>(x_lin)[i] = *reinterpret_cast<const uint4 *>(left_rows + (8 * i - main_rows));
    }
    __syncthreads();

    // ---- staging, step 2: gather through the permutation(s) into the MMA operand order
    {
      float norm_scale = 1.0f;
      if (normed) {
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) total += S.reduce[w];
        norm_scale = rsqrtf(total / static_cast<float>(K) + H.eps);
      }
      const int items = (K >> 2) * my_problems;
#pragma unroll 1
      for (int base = 0; base < items; base += kHeldItems * kThreads) {
#pragma unroll
        for (int it = 0; it < kHeldItems; ++it) {
          const int q = base + tid + it * kThreads;
          if (q >= items) continue;
          const int4 source = base == 0 ? held[it] : perm_item(M, q);
          const int which = q >= (K >> 2) ? 1 : 0;
          const int i = 4 * (q - which * (K >> 2));
          const int vector = (i >> 3) & 15;
          const int target = (i & ~127) + (vector & 3) * 32 + (vector >> 2) * 8 + (i & 7);
          __align__(8) __half values[4] = {x_lin[source.x], x_lin[source.y], x_lin[source.z], x_lin[source.w]};
          if (normed) {
            const int sources[4] = {source.x, source.y, source.z, source.w};
#pragma unroll
            for (int c = 0; c < 4; ++c)
              values[c] = __hmul(norm_lin[sources[c]], __float2half_rn(__half2float(values[c]) * norm_scale));
          }
          *reinterpret_cast<uint2 *>(x_stage + which * K + target) = *reinterpret_cast<const uint2 *>(values);
        }
      }
    }
    __syncthreads();
    MEGA_STAMP();  // staged

    // ---- main loop: this warp's units, run by run, streamed through its ring
    float *partial = reinterpret_cast<float *>(scratch);  // [warp][segment][16]; x_lin is dead now
    int cta_tiles = 0;
    {
      int total_units = 0;
#pragma unroll
      for (int r = 0; r < kMaxRuns; ++r) total_units += M.run[r].unit_count;
      const int begin = static_cast<int>(static_cast<long long>(total_units) * warp / kWarps);
      const int end = static_cast<int>(static_cast<long long>(total_units) * (warp + 1) / kWarps);
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      int segment = 0, first_cta_tile = -1, current_tile = -1;
      const uint32_t lane_offset = 16u * static_cast<uint32_t>(lane & 7);
      const uint32_t code_lane = smem_address(codes_ring) + warp * kRingUnits * 512 + g * 32 + t * 8;
      const uint32_t radius_lane = smem_address(radii_ring) + warp * kRingUnits * 64 + g * 4;
      const uint32_t grid_lane = smem_address(grid_ring) + warp * kRingUnits * 64 + g * 4;
      bool alive = true;
      int run_offset = 0;  // list position of the run's first unit
#pragma unroll 1
      for (int r = 0; r < kMaxRuns && alive; ++r) {
        const int run_begin = M.run[r].unit_begin, run_count = M.run[r].unit_count;
        if (run_count <= 0) continue;
        const int run_first_tile = run_begin / groups;
        const int tile_base = cta_tiles;
        cta_tiles += (run_begin + run_count - 1) / groups - run_first_tile + 1;
        const int lo = max(begin, run_offset), hi = min(end, run_offset + run_count);
        run_offset += run_count;
        if (lo >= hi) continue;
        const MegaProblem &p = M.problem[M.run[r].problem];
        const int which = M.run[r].problem - first_problem;
        const int dbits = p.dbits;
        FieldConsts f;
        f.index_mask = static_cast<uint32_t>(p.entries - 1) << 7;
        f.hi_shift = 27 - dbits;
        f.hi_mask = 3u << f.hi_shift;
        f.lo_mask = ((1u << (8 - dbits)) - 1u) << 19;
        f.lo_left = 11 - dbits;
        f.lo_right = 5 + dbits;
        const uint32_t book_lane = smem_address(book_shared + which * kBookBytes) + lane_offset;
        const uint32_t x_lane = smem_address(x_stage + which * K) + 16u * t;
        int unit = run_begin + (lo - (run_offset - run_count));
        int tile = unit / groups;
        int gi = unit - tile * groups;
        int remaining = hi - lo;
#pragma unroll 1
        while (remaining > 0) {
          const int count = min(kStageUnits, remaining);
          // wait (bounded) for the chunk's bytes
          const uint32_t stage = consumed % kStages;
          const uint32_t bar = smem_address(&S.barriers[warp][stage]);
          const uint32_t parity = (consumed / kStages) & 1u;
          bool arrived = barrier_done(bar, parity);
          if (!arrived) {
            const unsigned long long t0 = global_timer();
            unsigned spins = 0;
            while (!(arrived = barrier_done(bar, parity))) {
              if ((++spins & 255u) == 0 && global_timer() - t0 > kWaitLimitNs) break;
            }
          }
          arrived = __all_sync(0xffffffffu, arrived);
          if (!arrived) {
            if (lane == 0) {
              atomicExch(sync_words + 2, 1u);
              if (status) atomicExch(status, SAGEB200_ERR_TIMEOUT);
            }
            alive = false;
            break;
          }
#pragma unroll 1
          for (int u = 0; u < count; ++u) {
            const int cta_tile = tile_base + tile - run_first_tile;
            if (cta_tile != current_tile) {
              if (current_tile >= 0) {  // park the finished tile's sums (column 0: lanes with t == 0)
                if (t == 0) {
                  float *dst = partial + (warp * kWarpSegments + segment) * 16;
                  dst[g] = acc[0];
                  dst[g + 8] = acc[2];
                }
                ++segment;
              } else {
                first_cta_tile = cta_tile;
              }
              current_tile = cta_tile;
              acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
            }
            const uint32_t slot = stage * kStageUnits + u;
            uint2 code[2];
            uint32_t radius_word[2], endpoints[2];
            code[0] = lds64(code_lane + slot * 512);
            code[1] = lds64(code_lane + slot * 512 + 256);
            radius_word[0] = lds32(radius_lane + slot * 64);
            radius_word[1] = lds32(radius_lane + slot * 64 + 32);
            endpoints[0] = lds32(grid_lane + slot * 64);
            endpoints[1] = lds32(grid_lane + slot * 64 + 32);
            if (dbits == 8)
              compute_unit_shared<false>(code, radius_word, endpoints, acc, f, book_lane, x_lane + 256u * gi, t);
            else
              compute_unit_shared<true>(code, radius_word, endpoints, acc, f, book_lane, x_lane + 256u * gi, t);
            if (++gi == groups) {
              gi = 0;
              ++tile;
            }
          }
          ++consumed;
          remaining -= count;
          // the whole warp is done with the stage: refill it with this phase's next chunk
          __syncwarp();
          issue_one();
        }
      }
      // (runs after a failed wait were skipped: count their tiles for nobody)
      if (current_tile >= 0) {
        if (t == 0) {
          float *dst = partial + (warp * kWarpSegments + segment) * 16;
          dst[g] = acc[0];
          dst[g + 8] = acc[2];
        }
        ++segment;
      }
      if (lane == 0) {
        S.warp_first_tile[warp] = first_cta_tile;
        S.warp_tiles[warp] = segment;
      }
      if (!alive) S.abort = 1;
    }
    __syncthreads();
    MEGA_STAMP();  // main loops of all warps done
    if (S.abort) {
      bail_out();
      return;
    }

    // ---- combine the warps (warp order = channel order) and write the outputs; meanwhile the
    //      last warp fetches the metadata of the phase after the next.  The small latency-bound
    //      loads go out first, then the next linear phase's weight stream (megabytes per SM wave
    //      that would otherwise queue in front of them).
    if (warp == kWarps - 1 && P + 2 < phases) load_meta(P + 2);
    if (kind != kQkv && P + 1 < phases) prestage_load(P + 1);  // (in flight during the combination)
    if (P + 1 < phases) start_stream(P + 1);
#pragma unroll 1
    for (int e = tid; e < cta_tiles * 16; e += kThreads) {
      const int cta_tile = e >> 4, row = e & 15;
      int run = 0, run_tile_base = 0, base = 0;
#pragma unroll
      for (int r = 0; r < kMaxRuns; ++r) {
        const int count = M.run[r].unit_count;
        if (count <= 0) continue;
        const int first = M.run[r].unit_begin / groups;
        const int touched = (M.run[r].unit_begin + count - 1) / groups - first + 1;
        if (cta_tile >= base) {
          run = r;
          run_tile_base = base;
        }
        base += touched;
      }
      const MegaRun R = M.run[run];
      const MegaProblem &p = M.problem[R.problem];
      const int run_first_tile = R.unit_begin / groups;
      const int tile = run_first_tile + cta_tile - run_tile_base;
      auto sum_of = [&](int ct) { return tile_sum(S.warp_first_tile, S.warp_tiles, partial, ct, row); };
      if (R.first_slot >= 0) {  // a shared-out tile: this CTA's piece into its slot
        const int slot = tile == run_first_tile ? R.first_slot : 0;
        __stcg(p.patch + (static_cast<size_t>(tile - p.main_tiles) * p.slots + slot) * 16 + row, sum_of(cta_tile));
      } else if (kind == kGateUp) {
        // run 0 = gate's whole tiles, run 2 = up's (same tiles, the same count after run 1's):
        // SwiGLU on the finished pair, rounded as the separate kernels round (gate and up to
        // FP16, silu to FP16, FP16 product)
        if (run != 0) continue;
        int up_base = 0;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int count = M.run[r].unit_count;
          if (count > 0) up_base += (M.run[r].unit_begin + count - 1) / groups - M.run[r].unit_begin / groups + 1;
        }
        const __half gate = __float2half_rn(sum_of(cta_tile));
        const __half up = __float2half_rn(sum_of(up_base + cta_tile));
        const int out = tile * 16 + row;
        if (out < p.n) H.act[out] = __hmul(__float2half_rn(silu_fast(__half2float(gate))), up);
      } else {
        const int out = tile * 16 + row;
        if (out < p.n) p.y[out] = __float2half_rn(sum_of(cta_tile));
      }
    }
    if (kind != kQkv && P + 1 < phases) prestage_store(P + 1);
    MEGA_STAMP();  // outputs written
    if (!grid_sync()) {
      bail_out();
      return;
    }
    if (kind != kQkv) continue;

    // ================================================================ attention over the cache
    {
      MEGA_STAMP();  // attention start
      const int context = min(position + 1, H.max_seq);
      const bool in_range = position >= 0 && position < H.max_seq;  // a full cache takes no new token
      const int chunks = max(1, min(chunks_max, (context + 31) / 32));
      const int kv = cta / chunks, split = cta - kv * chunks;
      float *partial_out = H.attn_partial;
      if (cta < chunks * H.kv_heads) {
        __half *q_shared = reinterpret_cast<__half *>(work);                      // [group][128]
        __half *new_k = q_shared + kMaxGroup * 128, *new_v = new_k + 128;
        float *warp_max = reinterpret_cast<float *>(new_v + 128);                 // [warps][kMaxGroup]
        float *warp_total = warp_max + kWarps * kMaxGroup;
        float *warp_acc = warp_total + kWarps * kMaxGroup;                        // [warps][group][128]
        const int table_row = min(max(position, 0), H.max_seq - 1);
        const __half *cos_row = H.cos_table + static_cast<size_t>(table_row) * 64;
        const __half *sin_row = H.sin_table + static_cast<size_t>(table_row) * 64;
        const int chunk = (context + chunks - 1) / chunks;
        const int begin = split * chunk;
        const int end = min(context, begin + chunk);
        const bool owns_new = in_range && begin <= position && position < end;
        __half *k_base = L->k_cache + static_cast<size_t>(kv) * H.max_seq * 128;
        __half *v_base = L->v_cache + static_cast<size_t>(kv) * H.max_seq * 128;
        // items 0..group-1: the query heads; item group: the new key; item group + 1: the new value.
        // A lane holds values (2 lane, 2 lane + 1) and (64 + 2 lane, 64 + 2 lane + 1) of the item.
#pragma unroll 1
        for (int item = warp; item < group_heads + (owns_new ? 2 : 0); item += kWarps) {
          const MegaProblem &p = item < group_heads ? L->qkv[0] : item == group_heads ? L->qkv[1] : L->qkv[2];
          const int row0 = (item < group_heads ? kv * group_heads + item : kv) * 128;
          const int main_tiles = p.main_tiles, slots = p.slots;
          const __half *y = p.y;
          const float *patch = p.patch;
          __half2 pair[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int row = row0 + 64 * j + 2 * lane;  // (both rows of a pair lie in one tile)
            if (row < main_tiles * 16)
              pair[j] = __ldcg(reinterpret_cast<const __half2 *>(y + row));
            else
              pair[j] = __floats2half2_rn(finished_row(patch, main_tiles, slots, row),
                                          finished_row(patch, main_tiles, slots, row + 1));
          }
          __half2 lo = pair[0], hi = pair[1];
          if (item <= group_heads) {
            __half2 out_lo, out_hi;
            norm_rope(lo, hi, item < group_heads ? L->q_norm : L->k_norm, cos_row, sin_row, H.eps, lane, out_lo, out_hi);
            lo = out_lo;
            hi = out_hi;
          }
          __half *dst = item < group_heads ? q_shared + item * 128 : item == group_heads ? new_k : new_v;
          reinterpret_cast<__half2 *>(dst)[lane] = lo;
          reinterpret_cast<__half2 *>(dst + 64)[lane] = hi;
          if (item >= group_heads) {  // append to the cache
            __half *row = (item == group_heads ? k_base : v_base) + static_cast<size_t>(position) * 128;
            reinterpret_cast<__half2 *>(row)[lane] = lo;
            reinterpret_cast<__half2 *>(row + 64)[lane] = hi;
          }
        }
        __syncthreads();
        // A warp takes two consecutive positions at a time: lanes 16 s .. 16 s + 15 share position
        // s and hold 8 dims each; up to four query heads of the group per pass over the chunk.
        const int sub = lane >> 4, piece = lane & 15;
        auto fetch = [&](int base, uint4 &kq, uint4 &vq) {
          const int p = base + sub;
          kq = vq = make_uint4(0, 0, 0, 0);
          if (p < end) {
            if (owns_new && p == position) {
              kq = reinterpret_cast<const uint4 *>(new_k)[piece];
              vq = reinterpret_cast<const uint4 *>(new_v)[piece];
            } else {
              kq = __ldcg(reinterpret_cast<const uint4 *>(k_base + static_cast<size_t>(p) * 128) + piece);
              vq = __ldcg(reinterpret_cast<const uint4 *>(v_base + static_cast<size_t>(p) * 128) + piece);
            }
          }
        };
        auto unpack8 = [](const uint4 &a, float out[8]) {
          const __half2 *h = reinterpret_cast<const __half2 *>(&a);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
          }
        };
        constexpr int kPassHeads = 4;
#pragma unroll 1
        for (int h0 = 0; h0 < group_heads; h0 += kPassHeads) {
          float qf[kPassHeads][8];
          float running_max[kPassHeads], running_sum[kPassHeads], acc[kPassHeads][8];
#pragma unroll
          for (int j = 0; j < kPassHeads; ++j) {
            unpack8(reinterpret_cast<const uint4 *>(q_shared + min(h0 + j, group_heads - 1) * 128)[piece], qf[j]);
            running_max[j] = -INFINITY;
            running_sum[j] = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[j][i] = 0.0f;
          }
          uint4 kq, vq, next_k, next_v;
          fetch(begin + warp * 2, kq, vq);
#pragma unroll 1
          for (int base = begin + warp * 2; base < end; base += kWarps * 2) {
            fetch(base + kWarps * 2, next_k, next_v);
            const bool valid = base + sub < end;
            float kf[8], vf[8];
            unpack8(kq, kf);
            unpack8(vq, vf);
#pragma unroll
            for (int j = 0; j < kPassHeads; ++j) {
              float dot = 0.0f;
#pragma unroll
              for (int i = 0; i < 8; ++i) dot = fmaf(qf[j][i], kf[i], dot);
              dot += __shfl_xor_sync(0xffffffffu, dot, 1);
              dot += __shfl_xor_sync(0xffffffffu, dot, 2);
              dot += __shfl_xor_sync(0xffffffffu, dot, 4);
              dot += __shfl_xor_sync(0xffffffffu, dot, 8);
              if (valid) {
                dot *= H.attention_scale;
                const float new_max = fmaxf(running_max[j], dot);
                const float rescale = __expf(running_max[j] - new_max);
                const float weight = __expf(dot - new_max);
                running_sum[j] = running_sum[j] * rescale + weight;
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[j][i] = fmaf(weight, vf[i], acc[j][i] * rescale);
                running_max[j] = new_max;
              }
            }
            kq = next_k;
            vq = next_v;
          }
          // merge the warp's two position streams; the warps are merged below
#pragma unroll
          for (int j = 0; j < kPassHeads; ++j) {
            const int h = h0 + j;
            const float top = fmaxf(running_max[j], __shfl_xor_sync(0xffffffffu, running_max[j], 16));
            const float f = running_max[j] == -INFINITY ? 0.0f : __expf(running_max[j] - top);
            float total = running_sum[j] * f;
            total += __shfl_xor_sync(0xffffffffu, total, 16);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float value = acc[j][i] * f;
              value += __shfl_xor_sync(0xffffffffu, value, 16);
              acc[j][i] = value;
            }
            if (h < group_heads) {
              if (lane == 0) {
                warp_max[warp * kMaxGroup + h] = top;
                warp_total[warp * kMaxGroup + h] = total;
              }
              if (sub == 0) {
                float4 *dst = reinterpret_cast<float4 *>(warp_acc + (warp * group_heads + h) * 128 + 8 * piece);
                dst[0] = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
                dst[1] = make_float4(acc[j][4], acc[j][5], acc[j][6], acc[j][7]);
              }
            }
          }
        }
        __syncthreads();
#pragma unroll 1
        for (int item = tid; item < group_heads * 128; item += kThreads) {
          const int h = item >> 7, dim = item & 127;
          float top = -INFINITY;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) top = fmaxf(top, warp_max[w * kMaxGroup + h]);
          float total = 0.0f, value = 0.0f;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) {
            const float mx = warp_max[w * kMaxGroup + h];
            const float f = mx == -INFINITY ? 0.0f : __expf(mx - top);
            total += warp_total[w * kMaxGroup + h] * f;
            value += warp_acc[(w * group_heads + h) * 128 + dim] * f;
          }
          float *out = partial_out + (static_cast<size_t>(kv * group_heads + h) * chunks + split) * 130;
          if (dim == 0) {
            __stcg(out, top);
            __stcg(out + 1, total);
          }
          __stcg(out + 2 + dim, value);
        }
      }
      MEGA_STAMP();  // partial attention done
      if (!grid_sync()) {
        bail_out();
        return;
      }
      MEGA_STAMP();  // combination start
      prestage_load(P + 1);  // o_proj's permutation items and codebook, in flight during the combination
      // ---- combination of the chunks: one CTA per query head; thread = (dim, quarter of the chunks),
      //      every global load issued before the first use
      if (cta < H.heads) {
        const float *base = partial_out + static_cast<size_t>(cta) * chunks * 130;
        const int dim = tid & 127, quarter = tid >> 7;
        float values[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int s = quarter + 4 * j;
          values[j] = s < chunks ? __ldcg(base + s * 130 + 2 + dim) : 0.0f;
        }
        if (tid < chunks) {
          S.chunk_max[tid] = __ldcg(base + tid * 130);
          S.chunk_sum[tid] = __ldcg(base + tid * 130 + 1);
        }
        __syncthreads();
        float top = -INFINITY;
#pragma unroll 1
        for (int s = 0; s < chunks; ++s) top = fmaxf(top, S.chunk_max[s]);
        float value = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int s = quarter + 4 * j;
          if (s < chunks) {
            const float mx = S.chunk_max[s];
            value += values[j] * (mx == -INFINITY ? 0.0f : __expf(mx - top));
          }
        }
        float *quarter_sums = reinterpret_cast<float *>(work);  // [4][128]
        quarter_sums[quarter * 128 + dim] = value;
        __syncthreads();
        if (tid < 128) {
          float sum = 0.0f;
#pragma unroll 1
          for (int s = 0; s < chunks; ++s) {
            const float mx = S.chunk_max[s];
            sum += S.chunk_sum[s] * (mx == -INFINITY ? 0.0f : __expf(mx - top));
          }
          const float total = (quarter_sums[dim] + quarter_sums[128 + dim]) + (quarter_sums[256 + dim] + quarter_sums[384 + dim]);
          H.attn[cta * 128 + dim] = __float2half_rn(total / sum);
        }
      }
      prestage_store(P + 1);
      MEGA_STAMP();  // combination done
      if (!grid_sync()) {
        bail_out();
        return;
      }
    }
  }

  MEGA_STAMP();  // tail start
  // ==================================================================== tail
  // x = final_norm * fp16((h + delta) * rsqrt(mean((h + delta)^2) + eps)), then this CTA's rows
  // of the lm_head and the greedy argmax (lowest index on ties)
  {
    const int hidden = H.hidden;
    __half *x_shared = reinterpret_cast<__half *>(work);
    __half *left_rows = x_shared + hidden;
    const MegaProblem &down = H.layer[H.layers - 1].down;
    const __half *down_y = down.y;
    const float *down_patch = down.patch;
    const int down_main = down.main_tiles, down_slots = down.slots;
    const int main_rows = min(hidden, down_main * 16);
#pragma unroll 1
    for (int r = main_rows + tid; r < hidden; r += kThreads)
      left_rows[r - main_rows] = __float2half_rn(finished_row(down_patch, down_main, down_slots, r));
    __syncthreads();
    const __half *h_in = H.residual[residual_slot];
    float square = 0.0f;
#pragma unroll 1
    for (int i = tid; i < hidden; i += kThreads) {
      const __half d = i < main_rows ? __ldcg(down_y + i) : left_rows[i - main_rows];
      const __half v = __hadd(__ldcg(h_in + i), d);
      x_shared[i] = v;
      const float f = __half2float(v);
      square += f * f;
    }
    square = warp_sum(square);
    if (lane == 0) S.reduce[warp] = square;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) total += S.reduce[w];
    const float scale = rsqrtf(total / hidden + H.eps);
#pragma unroll 1
    for (int i = tid; i < hidden; i += kThreads)
      x_shared[i] = __hmul(__ldg(H.final_norm + i), __float2half_rn(__half2float(x_shared[i]) * scale));
    __syncthreads();
    const int pieces = hidden / 8;
    float top_value = -INFINITY;
    int top_index = 0x7fffffff;
#pragma unroll 1
    for (int v = cta * kWarps + warp; v < H.vocab; v += ctas * kWarps) {
      const uint4 *row = reinterpret_cast<const uint4 *>(H.lm_head + static_cast<size_t>(v) * hidden);
      float sum = 0.0f;
#pragma unroll 1
      for (int first = lane; first < pieces; first += 128) {  // four 16-byte loads in flight per lane
        uint4 w4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (first + 32 * j < pieces) w4[j] = ldg_stream_u4(row + first + 32 * j);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int i = first + 32 * j;
          if (i >= pieces) break;
          const __half2 *wh = reinterpret_cast<const __half2 *>(&w4[j]);
          const uint4 a = reinterpret_cast<const uint4 *>(x_shared)[i];
          const __half2 *ah = reinterpret_cast<const __half2 *>(&a);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float2 wf = __half22float2(wh[c]), af = __half22float2(ah[c]);
            sum = fmaf(wf.x, af.x, sum);
            sum = fmaf(wf.y, af.y, sum);
          }
        }
      }
      const __half rounded = __float2half_rn(warp_sum(sum));
      if (lane == 0) logits[v] = rounded;
      const float f = __half2float(rounded);
      if (better(f, v, top_value, top_index)) {
        top_value = f;
        top_index = v;
      }
    }
    if (lane == 0) {
      S.best_value[warp] = top_value;
      S.best_index[warp] = top_index;
    }
    __syncthreads();
    if (tid == 0) {
      float value = S.best_value[0];
      int index = S.best_index[0];
      for (int w = 1; w < kWarps; ++w)
        if (better(S.best_value[w], S.best_index[w], value, index)) {
          value = S.best_value[w];
          index = S.best_index[w];
        }
      __stcg(H.block_best + cta, make_float2(value, __int_as_float(index)));
    }
    MEGA_STAMP();  // lm_head rows done
    if (!grid_sync()) {
      bail_out();
      return;
    }
    if (cta == 0 && warp == 0) {
      float value = -INFINITY;
      int index = 0x7fffffff;
#pragma unroll 1
      for (int b = lane; b < ctas; b += 32) {
        const float2 candidate = __ldcg(H.block_best + b);
        if (better(candidate.x, __float_as_int(candidate.y), value, index)) {
          value = candidate.x;
          index = __float_as_int(candidate.y);
        }
      }
      for (int o = 16; o; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, value, o);
        const int other_index = __shfl_xor_sync(0xffffffffu, index, o);
        if (better(other, other_index, value, index)) {
          value = other;
          index = other_index;
        }
      }
      if (lane == 0) {
        if (index == 0x7fffffff) index = 0;  // a row without a single ordered value (all NaN)
        tokens[0] = index;
        if (log && step && step[0] < log_stride) log[step[0]] = index;
        positions[0] = position + 1;
        if (step) step[0] += 1;
      }
    }
  }
  MEGA_STAMP();  // end
#undef MEGA_STAMP
  // the last CTA to leave re-arms the barrier words for the next launch
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(sync_words + 1, 1u) == static_cast<unsigned>(ctas) - 1u) {
      sync_words[0] = 0u;
      sync_words[1] = 0u;
      __threadfence();
    }
  }
}

// ------------------------------------------------------------------ host: planning

size_t align256(size_t bytes) { return (bytes + 255) / 256 * 256; }

struct ProblemSplit {
  int cta_begin, cta_count, whole_per_cta, main_tiles, left_tiles, slots;
};

// Whole tiles per CTA plus the shared-out remainder (see the file comment).
ProblemSplit split_problem(int tiles, int groups, int cta_begin, int cta_count) {
  ProblemSplit s{};
  s.cta_begin = cta_begin;
  s.cta_count = cta_count;
  s.whole_per_cta = tiles / cta_count;
  s.main_tiles = s.whole_per_cta * cta_count;
  s.left_tiles = tiles - s.main_tiles;
  const long long left_units = static_cast<long long>(s.left_tiles) * groups;
  int slots = 1;
  for (int tile = 0; tile < s.left_tiles; ++tile) {
    // CTAs whose range [left*j/C, left*(j+1)/C) meets the tile's units
    const long long u0 = static_cast<long long>(tile) * groups, u1 = u0 + groups;
    int touching = 0;
    for (int j = 0; j < cta_count; ++j) {
      const long long b = left_units * j / cta_count, e = left_units * (j + 1) / cta_count;
      if (b < u1 && e > u0) ++touching;
    }
    if (touching > slots) slots = touching;
  }
  s.slots = slots;
  return s;
}

// The two runs (whole tiles, shared-out piece) of CTA `j` of a problem.
void problem_runs(const ProblemSplit &s, int groups, int j, int problem, MegaRun *runs) {
  runs[0] = MegaRun{problem, j * s.whole_per_cta * groups, s.whole_per_cta * groups, -1};
  const long long left_units = static_cast<long long>(s.left_tiles) * groups;
  const long long b = left_units * j / s.cta_count, e = left_units * (j + 1) / s.cta_count;
  int first_slot = 0;
  if (e > b) {
    const long long tile = b / groups;
    const long long u0 = tile * groups, u1 = u0 + groups;
    for (int other = 0; other < j; ++other) {
      const long long ob = left_units * other / s.cta_count, oe = left_units * (other + 1) / s.cta_count;
      if (ob < u1 && oe > u0) ++first_slot;
    }
  }
  runs[1] = MegaRun{problem, static_cast<int>(s.main_tiles * static_cast<long long>(groups) + b),
                    static_cast<int>(e - b), first_slot};
}

struct ModelPlan {
  bool ok = false;
  int ctas = 0;
  ProblemSplit qkv[3], o, gate_up, down;
  size_t x_stage_bytes = 0, scratch_bytes = 0, shared_bytes = 0;
  // workspace layout (offsets)
  size_t off_header = 0, off_layers = 0, off_plans[4] = {0, 0, 0, 0}, off_sync = 0, off_residual[2] = {0, 0};
  size_t off_q = 0, off_k = 0, off_v = 0, off_attn = 0, off_o = 0, off_act = 0, off_down = 0;
  size_t off_attn_partial = 0, off_block_best = 0;
  size_t off_patch_qkv[3] = {0, 0, 0}, off_patch_o = 0, off_patch_gate = 0, off_patch_up = 0, off_patch_down = 0;
  size_t zero_bytes = 0;  // the front of the workspace that must be zero before the first step
  size_t total_bytes = 0;
};

// The runs of CTA `c` in a phase of kind `kind`.
void build_runs(const ModelPlan &plan, const sageb200_mega_model &m, int kind, int c, MegaRun *runs) {
  const int hidden_groups = m.hidden / 128, q_out = m.heads * 128;
  for (int r = 0; r < kMaxRuns; ++r) runs[r] = MegaRun{0, 0, 0, -1};
  if (kind == kQkv) {
    int problem = 0;
    while (problem < 2 && c >= plan.qkv[problem].cta_begin + plan.qkv[problem].cta_count) ++problem;
    problem_runs(plan.qkv[problem], hidden_groups, c - plan.qkv[problem].cta_begin, problem, runs);
  } else if (kind == kO) {
    problem_runs(plan.o, q_out / 128, c, 0, runs);
  } else if (kind == kGateUp) {
    problem_runs(plan.gate_up, hidden_groups, c, 0, runs);
    problem_runs(plan.gate_up, hidden_groups, c, 1, runs + 2);
  } else {
    problem_runs(plan.down, m.intermediate / 128, c, 0, runs);
  }
}

// Every CTA's and every warp's tile count must fit the kernel's tables (exact walk).
bool check_tables(const ModelPlan &plan, const sageb200_mega_model &m) {
  for (int kind = 0; kind < 4; ++kind) {
    const int groups = (kind == kO ? m.heads * 128 : kind == kDown ? m.intermediate : m.hidden) / 128;
    for (int c = 0; c < plan.ctas; ++c) {
      MegaRun runs[kMaxRuns];
      build_runs(plan, m, kind, c, runs);
      long long total = 0;
      int cta_tiles = 0;
      for (int r = 0; r < kMaxRuns; ++r) {
        total += runs[r].unit_count;
        if (runs[r].unit_count > 0)
          cta_tiles += (runs[r].unit_begin + runs[r].unit_count - 1) / groups - runs[r].unit_begin / groups + 1;
      }
      if (cta_tiles > kMaxCtaTiles) return false;
      for (int w = 0; w < kWarps; ++w) {
        long long begin = total * w / kWarps, end = total * (w + 1) / kWarps;
        int segments = 0;
        long long offset = 0;
        for (int r = 0; r < kMaxRuns && begin < end; ++r) {
          const long long run_end = offset + runs[r].unit_count;
          if (begin < run_end) {
            const long long last = (end < run_end ? end : run_end) - 1;
            const long long u0 = runs[r].unit_begin + (begin - offset), u1 = runs[r].unit_begin + (last - offset);
            segments += static_cast<int>(u1 / groups - u0 / groups + 1);
            begin = last + 1;
          }
          offset = run_end;
        }
        if (segments > kWarpSegments) return false;
      }
    }
  }
  return true;
}

ModelPlan plan_model(const sageb200_mega_model &m, int sm_count) {
  ModelPlan plan;
  if (m.layers <= 0 || m.hidden <= 0 || m.hidden % 128 || m.heads <= 0 || m.kv_heads <= 0 || m.heads % m.kv_heads ||
      m.heads / m.kv_heads > kMaxGroup || m.head_dim != 128 || m.intermediate <= 0 || m.intermediate % 128 ||
      m.vocab <= 0 || m.max_seq <= 0 || sm_count < m.heads || sm_count < m.kv_heads)
    return plan;
  const int ctas = sm_count;
  plan.ctas = ctas;
  const int q_out = m.heads * 128, kv_out = m.kv_heads * 128;
  const int hidden_groups = m.hidden / 128;
  // q/k/v: CTAs in proportion to the packed sizes (at least one each)
  const int tiles_qkv[3] = {q_out / 16, kv_out / 16, kv_out / 16};
  const int total_tiles = tiles_qkv[0] + tiles_qkv[1] + tiles_qkv[2];
  int share[3], assigned = 0;
  for (int i = 0; i < 3; ++i) {
    share[i] = static_cast<int>(static_cast<long long>(ctas) * tiles_qkv[i] / total_tiles);
    if (share[i] < 1) share[i] = 1;
    assigned += share[i];
  }
  while (assigned < ctas) {  // hand the rest to the problem with the most tiles per CTA
    int worst = 0;
    for (int i = 1; i < 3; ++i)
      if (static_cast<long long>(tiles_qkv[i]) * share[worst] > static_cast<long long>(tiles_qkv[worst]) * share[i]) worst = i;
    ++share[worst];
    ++assigned;
  }
  while (assigned > ctas) {
    int best = 0;
    for (int i = 1; i < 3; ++i)
      if (share[i] > 1 && (share[best] <= 1 || static_cast<long long>(tiles_qkv[i]) * share[best] < static_cast<long long>(tiles_qkv[best]) * share[i])) best = i;
    if (share[best] <= 1) return plan;
    --share[best];
    --assigned;
  }
  int begin = 0;
  for (int i = 0; i < 3; ++i) {
    plan.qkv[i] = split_problem(tiles_qkv[i], hidden_groups, begin, share[i]);
    begin += share[i];
  }
  plan.o = split_problem(m.hidden / 16, q_out / 128, 0, ctas);
  plan.gate_up = split_problem(m.intermediate / 16, hidden_groups, 0, ctas);
  plan.down = split_problem(m.hidden / 16, m.intermediate / 128, 0, ctas);
  if (!check_tables(plan, m)) return plan;
  // shared memory
  const int k_max = m.intermediate > q_out ? (m.intermediate > m.hidden ? m.intermediate : m.hidden)
                                           : (q_out > m.hidden ? q_out : m.hidden);
  const int group_heads = m.heads / m.kv_heads;
  size_t x_stage = static_cast<size_t>(k_max) * 2;
  if (static_cast<size_t>(m.hidden) * 4 > x_stage) x_stage = static_cast<size_t>(m.hidden) * 4;  // gate/up: two buffers
  x_stage = (x_stage + 127) / 128 * 128;
  // scratch: the row in original order, the norm weights, finished leftover rows; or the partial sums
  size_t scratch = static_cast<size_t>(k_max) * 2 + static_cast<size_t>(m.hidden) * 2 + static_cast<size_t>(k_max) * 2;
  const size_t partial = static_cast<size_t>(kWarps) * kWarpSegments * 16 * 4;
  if (partial > scratch) scratch = partial;
  // attention: query heads, new key/value, per-warp partial results (x_stage and scratch together)
  const size_t attention = (static_cast<size_t>(kMaxGroup) * 128 + 256) * 2 +
                           static_cast<size_t>(kWarps) * kMaxGroup * 2 * 4 +
                           static_cast<size_t>(kWarps) * group_heads * 128 * 4;
  if (x_stage + scratch < attention) scratch = attention - x_stage;
  const size_t tail = static_cast<size_t>(m.hidden) * 4;
  if (x_stage + scratch < tail) scratch = tail - x_stage;
  scratch = (scratch + 127) / 128 * 128;
  plan.x_stage_bytes = x_stage;
  plan.scratch_bytes = scratch;
  const size_t state = (sizeof(SharedState) + 1023) / 1024 * 1024;
  plan.shared_bytes = state + 2 * kBookBytes + static_cast<size_t>(kWarps) * kRingUnits * kUnitBytes + x_stage + scratch;
  if (plan.shared_bytes > 227 * 1024) return plan;
  // workspace: [zeroed: sync words, patches][header][layers][plans][activations]
  size_t offset = 0;
  auto take = [&](size_t bytes) {
    const size_t at = offset;
    offset += align256(bytes);
    return at;
  };
  plan.off_sync = take(256);
  auto patch_bytes = [](const ProblemSplit &s) { return static_cast<size_t>(s.left_tiles) * s.slots * 16 * 4 + 256; };
  for (int i = 0; i < 3; ++i) plan.off_patch_qkv[i] = take(patch_bytes(plan.qkv[i]));
  plan.off_patch_o = take(patch_bytes(plan.o));
  plan.off_patch_gate = take(patch_bytes(plan.gate_up));
  plan.off_patch_up = take(patch_bytes(plan.gate_up));
  plan.off_patch_down = take(patch_bytes(plan.down));
  plan.zero_bytes = offset;
  plan.off_header = take(sizeof(MegaHeader));
  plan.off_layers = take(sizeof(MegaLayer) * m.layers);
  for (int kind = 0; kind < 4; ++kind) plan.off_plans[kind] = take(sizeof(MegaCtaPlan) * ctas);
  plan.off_residual[0] = take(static_cast<size_t>(m.hidden) * 2);
  plan.off_residual[1] = take(static_cast<size_t>(m.hidden) * 2);
  plan.off_q = take(static_cast<size_t>(q_out) * 2);
  plan.off_k = take(static_cast<size_t>(kv_out) * 2);
  plan.off_v = take(static_cast<size_t>(kv_out) * 2);
  plan.off_attn = take(static_cast<size_t>(q_out) * 2);
  plan.off_o = take(static_cast<size_t>(m.hidden) * 2);
  plan.off_act = take(static_cast<size_t>(m.intermediate) * 2);
  plan.off_down = take(static_cast<size_t>(m.hidden) * 2);
  plan.off_attn_partial = take(static_cast<size_t>(m.heads) * 32 * 130 * 4);
  plan.off_block_best = take(static_cast<size_t>(ctas) * 8);
  plan.total_bytes = offset;
  plan.ok = true;
  return plan;
}

int check_linear(const sageb200_mega_linear &l, int n, int k) {
  if (l.n != n || l.k != k || direction_bits_of(l.entries) < 0 || !l.codes || !l.radii || !l.grid || !l.book)
    return SAGEB200_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(l.codes) & 15) || (reinterpret_cast<uintptr_t>(l.radii) & 15) ||
      (reinterpret_cast<uintptr_t>(l.grid) & 15) || (reinterpret_cast<uintptr_t>(l.book) & 3) ||
      (reinterpret_cast<uintptr_t>(l.perm) & 15))
    return SAGEB200_ERR_ALIGNMENT;
  return SAGEB200_OK;
}

MegaProblem make_problem(const sageb200_mega_linear &l, const ProblemSplit &s, __half *y, float *patch) {
  MegaProblem p{};
  p.codes = static_cast<const uint32_t *>(l.codes);
  p.radii = static_cast<const uint32_t *>(l.radii);
  p.grid = static_cast<const uint32_t *>(l.grid);
  p.book = static_cast<const uint32_t *>(l.book);
  p.perm = l.perm;
  p.y = y;
  p.patch = patch;
  p.n = l.n;
  p.tiles = (l.n + 15) / 16;
  p.entries = l.entries;
  p.dbits = direction_bits_of(l.entries);
  p.main_tiles = s.main_tiles;
  p.slots = s.slots;
  return p;
}

int device_sm_count(int *sm_count) {
  int device = 0, major = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_NO_DEVICE;
  }
  return major == 10 ? SAGEB200_OK : SAGEB200_ERR_NO_DEVICE;
}

}  // namespace
}  // namespace sageb200

using namespace sageb200;

extern "C" {

size_t sageb200_mega_workspace_bytes(const sageb200_mega_model *model, int sm_count) {
  if (!model) return 0;
  if (sm_count <= 0 && device_sm_count(&sm_count) != SAGEB200_OK) sm_count = 148;
  const ModelPlan plan = plan_model(*model, sm_count);
  return plan.ok ? plan.total_bytes : 0;
}

int sageb200_mega_prepare(const sageb200_mega_model *model, const sageb200_mega_layer *layers, void *workspace,
                          size_t workspace_bytes, void *stream) {
  if (!model || !layers || !workspace) return SAGEB200_ERR_INVALID_ARGUMENT;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return SAGEB200_ERR_ALIGNMENT;
  int sm_count = 0;
  int status = acquire_device(nullptr, &sm_count);
  if (status == SAGEB200_ERR_TIMEOUT) status = SAGEB200_OK;  // re-preparing after a time-out is the way back
  if (status) return status;
  const sageb200_mega_model &m = *model;
  const ModelPlan plan = plan_model(m, sm_count);
  if (!plan.ok) return SAGEB200_ERR_RANGE;
  if (workspace_bytes < plan.total_bytes) return SAGEB200_ERR_WORKSPACE;
  if (!m.embed || !m.lm_head || !m.final_norm || !m.cos_table || !m.sin_table) return SAGEB200_ERR_INVALID_ARGUMENT;
  const int q_out = m.heads * 128, kv_out = m.kv_heads * 128;
  unsigned char *base = static_cast<unsigned char *>(workspace);
  auto at = [&](size_t offset) { return base + offset; };
  std::vector<unsigned char> image(plan.off_residual[0] - plan.off_header);  // header, layers, per-CTA runs
  auto host = [&](size_t offset) { return image.data() + (offset - plan.off_header); };
  // layers
  MegaLayer *L = reinterpret_cast<MegaLayer *>(host(plan.off_layers));
  for (int i = 0; i < m.layers; ++i) {
    const sageb200_mega_layer &in = layers[i];
    const sageb200_mega_linear *qkv[3] = {&in.q, &in.k, &in.v};
    const int outs[3] = {q_out, kv_out, kv_out};
    const size_t ys[3] = {plan.off_q, plan.off_k, plan.off_v};
    for (int j = 0; j < 3; ++j) {
      status = check_linear(*qkv[j], outs[j], m.hidden);
      if (status) return status;
      L[i].qkv[j] = make_problem(*qkv[j], plan.qkv[j], reinterpret_cast<__half *>(at(ys[j])),
                                 reinterpret_cast<float *>(at(plan.off_patch_qkv[j])));
    }
    if ((status = check_linear(in.o, m.hidden, q_out)) || (status = check_linear(in.gate, m.intermediate, m.hidden)) ||
        (status = check_linear(in.up, m.intermediate, m.hidden)) ||
        (status = check_linear(in.down, m.hidden, m.intermediate)))
      return status;
    L[i].o = make_problem(in.o, plan.o, reinterpret_cast<__half *>(at(plan.off_o)),
                          reinterpret_cast<float *>(at(plan.off_patch_o)));
    L[i].gate_up[0] = make_problem(in.gate, plan.gate_up, nullptr, reinterpret_cast<float *>(at(plan.off_patch_gate)));
    L[i].gate_up[1] = make_problem(in.up, plan.gate_up, nullptr, reinterpret_cast<float *>(at(plan.off_patch_up)));
    L[i].down = make_problem(in.down, plan.down, reinterpret_cast<__half *>(at(plan.off_down)),
                             reinterpret_cast<float *>(at(plan.off_patch_down)));
    if (!in.input_norm || !in.post_norm || !in.q_norm || !in.k_norm || !in.k_cache || !in.v_cache)
      return SAGEB200_ERR_INVALID_ARGUMENT;
    L[i].input_norm = static_cast<const __half *>(in.input_norm);
    L[i].post_norm = static_cast<const __half *>(in.post_norm);
    L[i].q_norm = static_cast<const __half *>(in.q_norm);
    L[i].k_norm = static_cast<const __half *>(in.k_norm);
    L[i].k_cache = static_cast<__half *>(in.k_cache);
    L[i].v_cache = static_cast<__half *>(in.v_cache);
  }
  // per-CTA runs
  for (int kind = 0; kind < 4; ++kind) {
    MegaCtaPlan *plans = reinterpret_cast<MegaCtaPlan *>(host(plan.off_plans[kind]));
    for (int c = 0; c < plan.ctas; ++c) {
      build_runs(plan, m, kind, c, plans[c].run);
      // a problem without whole tiles still names itself in run 0 (the kernel reads run[0].problem)
      plans[c].run[0].problem = plans[c].run[1].problem;
    }
  }
  // header
  MegaHeader &H = *reinterpret_cast<MegaHeader *>(host(plan.off_header));
  std::memset(&H, 0, sizeof(H));
  H.layers = m.layers;
  H.hidden = m.hidden;
  H.heads = m.heads;
  H.kv_heads = m.kv_heads;
  H.intermediate = m.intermediate;
  H.vocab = m.vocab;
  H.max_seq = m.max_seq;
  H.ctas = plan.ctas;
  H.eps = m.eps;
  H.attention_scale = 0.08838834764831845f;  // 1 / sqrt(128)
  H.x_stage_bytes = static_cast<int>(plan.x_stage_bytes);
  H.scratch_bytes = static_cast<int>(plan.scratch_bytes);
  H.embed = static_cast<const __half *>(m.embed);
  H.lm_head = static_cast<const __half *>(m.lm_head);
  H.final_norm = static_cast<const __half *>(m.final_norm);
  H.cos_table = static_cast<const __half *>(m.cos_table);
  H.sin_table = static_cast<const __half *>(m.sin_table);
  H.residual[0] = reinterpret_cast<__half *>(at(plan.off_residual[0]));
  H.residual[1] = reinterpret_cast<__half *>(at(plan.off_residual[1]));
  H.attn = reinterpret_cast<__half *>(at(plan.off_attn));
  H.act = reinterpret_cast<__half *>(at(plan.off_act));
  H.attn_partial = reinterpret_cast<float *>(at(plan.off_attn_partial));
  H.block_best = reinterpret_cast<float2 *>(at(plan.off_block_best));
  H.sync = reinterpret_cast<unsigned *>(at(plan.off_sync));
  H.layer = reinterpret_cast<const MegaLayer *>(at(plan.off_layers));
  for (int kind = 0; kind < 4; ++kind) H.plan[kind] = reinterpret_cast<const MegaCtaPlan *>(at(plan.off_plans[kind]));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(workspace, 0, plan.zero_bytes, s) != cudaSuccess ||
      cudaMemcpyAsync(at(plan.off_header), image.data(), image.size(), cudaMemcpyHostToDevice, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess ||  // `image` is pageable host memory of this call
      cudaFuncSetAttribute(sage_decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           static_cast<int>(plan.shared_bytes)) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  return SAGEB200_OK;
}

int sageb200_mega_step(const sageb200_mega_model *model, void *workspace, void *tokens, void *positions, void *log,
                       void *step, void *logits, int log_stride, void *stream) {
  if (!model || !workspace || !tokens || !positions || !logits) return SAGEB200_ERR_INVALID_ARGUMENT;
  int sm_count = 0;
  int *status_word = nullptr;
  int status = acquire_device(&status_word, &sm_count);
  if (status) return status;
  const ModelPlan plan = plan_model(*model, sm_count);
  if (!plan.ok) return SAGEB200_ERR_RANGE;
  const MegaHeader *header = reinterpret_cast<const MegaHeader *>(static_cast<unsigned char *>(workspace) + plan.off_header);
  long long *tokens_p = static_cast<long long *>(tokens);
  int *positions_p = static_cast<int *>(positions);
  long long *log_p = static_cast<long long *>(log);
  int *step_p = static_cast<int *>(step);
  __half *logits_p = static_cast<__half *>(logits);
  long long *trace = trace_buffer();
  void *args[] = {&header, &tokens_p, &positions_p, &log_p, &step_p, &logits_p, &log_stride, &status_word, &trace};
  // cooperative: every CTA is resident, so the grid barriers cannot starve
  if (cudaLaunchCooperativeKernel(reinterpret_cast<void *>(sage_decode_mega_kernel), dim3(plan.ctas), dim3(kThreads),
                                  args, plan.shared_bytes, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    cudaGetLastError();
    return SAGEB200_ERR_CUDA;
  }
  count_launches(1);
  return SAGEB200_OK;
}

}  // extern "C"
