// SAGE packed prefill GEMM for more than 16 activation rows: dequantise weight tiles
// into shared memory, feed tcgen05 FP16 MMAs with FP32 accumulators in tensor memory.
//
// Replaces the reference's sage_gemm_kernel_base / _m64 (csrc/sage/sage_gemm_cuda.cu:35-197,
// 272-445: 32x64 / 64x64 tiles on nvcuda::wmma, every activation tile re-decoding the
// whole weight) and its separate split-K reduce kernel (:199-206).
//
// Orientation ("swap AB"): the MMA's M dimension is 128 OUTPUT rows (eight packed 16-row
// tiles), its N dimension is up to 256 activation rows (tokens), so any token count that
// is a multiple of 16 maps onto one instruction shape without padding waste:
//     D[128 outputs][TN tokens] += Wtile[128][64] . Xq[TN][64]^T      per 64-channel stage
// Both operands are K-major in shared memory with the 128-byte swizzle:
//   A (weights)      written by 16 decode warps with 16-byte stores, bit-exact
//                    w = fp16_rn(float(+-dir) * fmaf(code, step, min))
//                    (reference csrc/sage/sage_gemm_cuda.cu:117-131)
//   B (activations)  one TMA tile load per stage from the activations in quantised
//                    channel order (no cluster multicast)
// One elected thread issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=TN, K=16, four per
// stage) and releases stages with tcgen05.commit; the decode warps then read the
// accumulator with tcgen05.ld and store FP16 outputs.
//
// Every wait is bounded: a wait that exceeds its time limit sets an abort flag in shared
// memory (all later waits return at once), records SAGEB200_ERR_TIMEOUT in the status word
// and the CTA still frees its tensor memory before returning.
#include <cuda.h>

#include "sage_common.cuh"
#include "sage_kernels.h"

namespace sageb200 {
namespace {

constexpr int kDecodeWarps = 16;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kTmaWarp = kDecodeWarps;
constexpr int kMmaWarp = kDecodeWarps + 1;
constexpr int kGemmThreads = (kDecodeWarps + 2) * 32;
constexpr int kTileRows = 128;             // output rows per CTA = MMA M
constexpr int kRowThreads = kDecodeThreads / kTileRows;  // decode threads per output row (4)
constexpr int kThreadVectors = 8 / kRowThreads;          // 8-weight vectors per thread and stage (2)
static_assert(kRowThreads == 4 && kThreadVectors == 2, "the decode loop below is written for four threads per row");
constexpr int kStageK = 64;                // channels per stage = one 128-byte swizzle row
constexpr int kAStageBytes = kTileRows * kStageK * 2;
constexpr int kMaxStages = 6;
constexpr int kBookReplicas = 8;           // codebook copies in shared memory: lane % 8 reads its own
constexpr int kBookBytes = 256 * 16 * kBookReplicas;
constexpr int kGemmSharedLimit = 226 * 1024;  // dynamic shared memory the kernel opts into (227 KiB per CTA less its static words)
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s per wait

struct GemmParams {
  const uint32_t *codes;
  const uint32_t *radii;
  const uint32_t *grid;
  const uint32_t *book;
  __half *y;
  int *status;          // device-visible status word (0 = ok)
  int rows, n, k, groups, tiles;
  int entries, dbits;
  int tokens_per_cta;   // TN: multiple of 16, 16..256 (tokens of ONE accumulator)
  int stages;
  int tmem_columns;     // power of two >= max(32, TN); 512 with two accumulators
  int accumulators;     // 1 or 2 token blocks per CTA: one decoded weight stage feeds both
  long long *trace;     // profiling build only: eight clock sums per CTA (null otherwise)
  // split K (k_splits > 1): CTA z runs the 128-channel groups [z * groups_per_split, ...), leaves
  // its FP32 tile in `partial`, and the last CTA of a tile to arrive (counter) adds the splits in
  // index order and writes the FP16 output
  int k_splits, groups_per_split;
  // packed format: 0 = SAGE (tiled words, planar codebook, (min, step) grid); 1 = SPHQuant
  // (row-major 16-bit codes in `codes`, per-(row, group) high radius word in `radii`, FP16 scales
  // in `grid` and minimums in `mins`, entry-major 64 x 8 codebook, n rows need no padding)
  int format;
  const __half *mins;
  float *partial;       // [k_splits][tiles][accumulators * TN tokens][128 rows]
  unsigned *counters;   // [tiles][8]: one word per part of a tile, zero before and after the launch
};

#ifdef SAGEB200_TRACE
#define GEMM_CLOCK() clock64()
#else
#define GEMM_CLOCK() 0ll
#endif

// ---------------------------------------------------------------- PTX wrappers

__device__ __forceinline__ void mbarrier_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbarrier_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbarrier_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbarrier_test(uint32_t bar, uint32_t parity) {
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

// Suspending form of the test: the thread sleeps in hardware until the phase completes or about
// `hint_ns` have passed, so a waiting warp does not compete for issue slots with working ones.
__device__ __forceinline__ bool mbarrier_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      " selp.u32 %0, 1, 0, p;\n}"
      : "=r"(done)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return done != 0;
}

// Bounded wait.  Returns false (and raises the CTA's abort flag) when the limit passes.
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                             int *status) {
  if (mbarrier_test(bar, parity)) return true;
  const unsigned long long begin = global_timer();
  unsigned spins = 0;
  while (true) {
    if (mbarrier_try_wait(bar, parity, 2000u)) return true;
    if (*abort_flag) return false;
    if ((++spins & 15u) == 0 && global_timer() - begin > kWaitLimitNs) {
      *abort_flag = 1;
      atomicExch(status, -7);  // SAGEB200_ERR_TIMEOUT
      return false;
    }
  }
}

__device__ __forceinline__ void fence_proxy_async_shared() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_descriptor(uint32_t address) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((address & 0x3ffffu) >> 4);  // start address
  desc |= static_cast<uint64_t>(1) << 16;                    // leading byte offset (unused here)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;            // stride byte offset
  desc |= static_cast<uint64_t>(1) << 46;                    // descriptor version (sm_100)
  desc |= static_cast<uint64_t>(2) << 61;                    // layout: 128-byte swizzle
  return desc;
}

// kind::f16 instruction descriptor: FP16 A and B (both K-major), FP32 accumulator.
__device__ __forceinline__ uint32_t instruction_descriptor(int m, int n) {
  uint32_t d = 0;
  d |= 1u << 4;                                  // D format FP32
  d |= static_cast<uint32_t>(n >> 3) << 17;      // N
  d |= static_cast<uint32_t>(m >> 4) << 24;      // M
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// ---- the same for a PAIR of CTAs (cta_group::2): one MMA covers 256 output rows (128 per CTA), each
//      CTA supplies its own weight tile and HALF of the activation tile, so an SM reads half the B
//      operand from its shared memory.  Barrier addresses with bit 24 cleared name the even CTA of
//      the pair in the cluster's shared window.
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int x, int y,
                                                 uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leader_bar & kPeerBitMask)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc, uint32_t accumulate) {
  const uint32_t zero = 0;
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}" ::"r"(tmem_d),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(zero)
      : "memory");
}
// arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const unsigned short both = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(both)
      : "memory");
}
__device__ __forceinline__ void mbarrier_arrive_leader(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & kPeerBitMask) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  return rank;
}

__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_load_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- the kernel

// Dynamic shared memory, 1024-byte aligned by hand:
//   [A stages: stages x 16 KiB][B stages: stages x TN*128][codebook 4 KiB][barriers]
// kPair: the grid is launched in clusters of two CTAs along x (two neighbouring row blocks) that
// run cta_group::2 MMAs.  Both CTAs decode their own 128 rows and load their own half of every
// activation tile; the even CTA (the leader) issues the MMAs and owns the "stage full" barriers:
// its own decode warps arrive there, its TMA thread announces both CTAs' bytes, the odd CTA's
// loads complete on it remotely, and the odd CTA's otherwise idle MMA warp forwards ONE arrival
// per stage once its own decode warps are done.  Stage-free and accumulator-ready arrivals are
// multicast to both CTAs by tcgen05.commit.
template <bool kPair>
__global__ void __launch_bounds__(kGemmThreads, 1)
    sage_gemm_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap x_map) {
  extern __shared__ unsigned char raw_shared[];
  __shared__ uint32_t tmem_base_holder;
  __shared__ int abort_flag;
  __shared__ int split_last;

  const uint32_t raw = smem_address(raw_shared);
  const uint32_t base = (raw + 1023u) & ~1023u;
  unsigned char *aligned = raw_shared + (base - raw);
  const int tn = p.tokens_per_cta;
  const int accumulators = p.accumulators;
  const int tile_tokens = kPair ? tn / 2 : tn;        // tokens of one accumulator this CTA loads
  const int b_tile_bytes = tile_tokens * kStageK * 2; // one token block's activations of a stage (this CTA's part)
  const uint32_t pair_rank = kPair ? cluster_cta_rank() : 0u;
  const bool leader = pair_rank == 0;
  const int b_stage_bytes = accumulators * b_tile_bytes;
  const uint32_t a_base = base;
  const uint32_t b_base = a_base + p.stages * kAStageBytes;
  const uint32_t book_address = b_base + p.stages * b_stage_bytes;
  uint4 *book_shared = reinterpret_cast<uint4 *>(aligned + (book_address - base));
  const uint32_t bar_base = book_address + kBookBytes;
  // barriers: full[stages], empty[stages], accumulator
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  const uint32_t accum_bar = bar_base + 8u * (2 * kMaxStages);

  // Programmatic dependent launch: the next kernel of the stream may be scheduled at once; this
  // kernel's set-up, and its decode warps' first stages (packed weights and codebook: data no
  // kernel writes), run while the previous kernel (the gather pre-pass) still works.  Only the
  // activation loads and every global write wait for the previous kernel.
  pdl_launch_dependents();
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int row_block = blockIdx.x;   // 128 output rows
  const int token_block = blockIdx.y * accumulators;  // first of this CTA's blocks of TN tokens
  const int group_begin = blockIdx.z * p.groups_per_split;
  const int group_end = min(p.groups, group_begin + p.groups_per_split);
  const int stage_first = 2 * group_begin;            // first 64-channel stage of this CTA's K range
  const int stages_k = 2 * (group_end - group_begin); // stages this CTA runs

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < p.stages; ++s) {
      // full: this CTA's decode threads; + the TMA thread's announcement (and, for a leader, the
      // odd CTA's forwarded arrival)
      mbarrier_init(full_bar(s), kDecodeThreads + (kPair ? (leader ? 2 : 0) : 1));
      mbarrier_init(empty_bar(s), 1);
    }
    mbarrier_init(accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kTmaWarp) {
    if constexpr (kPair) {  // (both CTAs, the same warp, the same holder address)
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_address(&tmem_base_holder)),
                   "r"(static_cast<uint32_t>(p.tmem_columns))
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_address(&tmem_base_holder)),
                   "r"(static_cast<uint32_t>(p.tmem_columns))
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  // codebook, interleaved: entry e = 16 bytes (dims 0..7)
  for (int e = tid; e < p.entries; e += kGemmThreads) {
    uint4 entry;
    if (p.format == 1) {
      entry = reinterpret_cast<const uint4 *>(p.book)[e];
    } else {
      entry.x = p.book[e];
      entry.y = p.book[p.entries + e];
      entry.z = p.book[2 * p.entries + e];
      entry.w = p.book[3 * p.entries + e];
    }
    // eight copies, entry-major: lane l reads copy l % 8, so the eight lanes of a quarter warp hit
    // eight different 16-byte bank groups whatever their indices (rotated fill order for the same reason)
#pragma unroll
    for (int r = 0; r < kBookReplicas; ++r) book_shared[e * kBookReplicas + ((r + tid) & (kBookReplicas - 1))] = entry;
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (kPair) cluster_sync_all();  // (no remote arrival before the other CTA's barriers exist)
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_holder;
  volatile int *abort_ptr = &abort_flag;

  if (warp < kDecodeWarps) {
    // ---------------- weight decode producers: thread = (row 0..127, quarter 0..3 of the row's
    //                  64 channels); sixteen warps keep four warps per scheduler in flight, which
    //                  is what hides the codebook-load and conversion latencies of the exact decode
    const int row = tid / kRowThreads;
    const int part = tid % kRowThreads;
    const int out_row = row_block * kTileRows + row;
    const int tile = out_row >> 4;
    // rows past the last packed tile (SAGE) / past n (SPHQuant) decode to zero
    const bool row_valid = p.format == 1 ? out_row < p.n : tile < p.tiles;
    const size_t cell_base = (static_cast<size_t>(row_valid ? tile : 0) * p.groups) * 16 + (out_row & 15);
    const size_t sph_row = static_cast<size_t>(row_valid ? out_row : 0);
    const uint32_t row_offset = static_cast<uint32_t>(row >> 3) * 1024u + static_cast<uint32_t>(row & 7) * 128u;
    const uint32_t index_mask = static_cast<uint32_t>(p.entries - 1);
    // One 128-channel group feeds two stages.  The thread's packed words of a group (two code
    // words, the radius word, the grid endpoints) are fetched TWO groups ahead into a register
    // queue: the loads come from cold HBM, and a load issued at the point of use would stall every
    // decode thread for a full memory latency every second stage.
    struct GroupWords {
      uint32_t word[2], radius, endpoints;
    };
    auto fetch_group = [&](int group) {
      GroupWords g = {{0u, 0u}, 0u, 0u};
      if (row_valid && group < group_end) {
        if (p.format == 1) {
          // sixteen 16-bit codes per group and row; this thread's two of each 64-channel half
          const uint32_t *row_codes = p.codes + (sph_row * p.groups + group) * 8;
          const size_t cell = sph_row * p.groups + group;
          g.word[0] = ldg_stream_u1(row_codes + part);
          g.word[1] = ldg_stream_u1(row_codes + 4 + part);
          g.radius = ldg_stream_u1(p.radii + cell);
          const uint32_t minimum = reinterpret_cast<const unsigned short *>(p.mins)[cell];
          const uint32_t scale = reinterpret_cast<const unsigned short *>(p.grid)[cell];
          g.endpoints = minimum | (scale << 16);  // (min, step) as in the SAGE grid
        } else {
          const size_t cell = cell_base + static_cast<size_t>(group) * 16;
          g.word[0] = ldg_stream_u1(p.codes + cell * 8 + part);
          g.word[1] = ldg_stream_u1(p.codes + cell * 8 + 4 + part);
          g.radius = ldg_stream_u1(p.radii + cell);
          g.endpoints = ldg_stream_u1(p.grid + cell);
        }
      }
      return g;
    };
    GroupWords ahead0 = fetch_group(group_begin), ahead1 = fetch_group(group_begin + 1);
    long long waited = 0, worked = 0, fenced = 0, stored = 0;  // (profiling build) clock sums of the phases
    [[maybe_unused]] const long long decode_begin = GEMM_CLOCK();
    uint32_t words[2] = {0, 0};
    uint32_t radius_word = 0;
    float minimum = 0.0f, step = 0.0f;
    bool alive = true;
    for (int ks = 0; ks < stages_k && alive; ++ks) {
      const int s = ks % p.stages;
      const uint32_t phase = static_cast<uint32_t>(ks / p.stages) & 1u;
      if ((ks & 1) == 0) {
        words[0] = ahead0.word[0];
        words[1] = ahead0.word[1];
        radius_word = ahead0.radius;
        const float2 e = __half22float2(*reinterpret_cast<const __half2 *>(&ahead0.endpoints));
        minimum = e.x;
        step = e.y;
        ahead0 = ahead1;
        ahead1 = fetch_group(group_begin + (ks >> 1) + 2);
      }
      const long long t0 = GEMM_CLOCK();
      alive = bounded_wait(empty_bar(s), phase ^ 1u, abort_ptr, p.status);
      if (!alive) break;
      const long long t1 = GEMM_CLOCK();
      const uint32_t word = words[ks & 1];
      const uint32_t stage_address = a_base + s * kAStageBytes + row_offset;
#pragma unroll
      for (int j = 0; j < kThreadVectors; ++j) {
        const uint32_t code = (word >> (16 * j)) & 0xffffu;
        const int chunk = part * kThreadVectors + j;       // 16-byte chunk within the 128-byte row
        const int vector = (ks & 1) * 8 + chunk;           // vector index within the group
        uint32_t out[4] = {0, 0, 0, 0};
        if (row_valid) {
          const uint4 dir = book_shared[((code >> 8) & index_mask) * kBookReplicas + (lane & (kBookReplicas - 1))];
          const uint32_t rc = (code >> (8 + p.dbits)) |
                              (((radius_word >> (2 * vector)) & 3u) << (8 - p.dbits));
          const float radius = fmaf(static_cast<float>(rc), step, minimum);
          const uint32_t planes[4] = {dir.x, dir.y, dir.z, dir.w};
          const uint32_t signs = code & 0xffu;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            // sign bits 2q and 2q+1 land on bits 15 and 31 of one product (one multiply and one
            // three-input logic operation per pair of weights; the other product bits are masked)
            uint32_t bits = planes[q] ^ ((signs * ((1u + (1u << 15)) << (15 - 2 * q))) & 0x80008000u);
            const float2 d = __half22float2(*reinterpret_cast<const __half2 *>(&bits));
            const __half2 v = __floats2half2_rn(d.x * radius, d.y * radius);
            out[q] = *reinterpret_cast<const uint32_t *>(&v);
          }
        }
        const uint32_t swizzled = static_cast<uint32_t>(chunk ^ (row & 7)) * 16u;
        sts_u4(stage_address + swizzled, make_uint4(out[0], out[1], out[2], out[3]));
      }
      const long long t2 = GEMM_CLOCK();
      fence_proxy_async_shared();
      const long long t3 = GEMM_CLOCK();
      mbarrier_arrive(full_bar(s));
      waited += t1 - t0;
      worked += GEMM_CLOCK() - t1;
      fenced += t3 - t2;
      stored += t2 - t1;
    }
#ifdef SAGEB200_TRACE
    if (p.trace && (tid == 0 || tid == kDecodeThreads - 1)) {
      long long *record = p.trace + (static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * 16 + (tid == 0 ? 0 : 3);
      record[0] = waited;
      record[1] = worked;
      record[2] = GEMM_CLOCK() - decode_begin;
      if (tid == 0) {
        p.trace[(static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * 16 + 10] = stored;
        p.trace[(static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * 16 + 11] = fenced;
      }
    }
    const long long epilogue_begin = GEMM_CLOCK();
#endif
    // ---------------- epilogue: TMEM -> registers -> FP16 global
    pdl_wait();  // (long since satisfied: the MMAs needed the activations; required before global writes)
    if (alive) alive = bounded_wait(accum_bar, 0, abort_ptr, p.status);
    alive = __all_sync(0xffffffffu, alive);  // tcgen05.ld is warp-collective
    tcgen05_fence_after();
#ifdef SAGEB200_TRACE
    if (p.trace && tid == 0)
      p.trace[(static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * 16 + 12] = GEMM_CLOCK() - epilogue_begin;
#endif
    {
      constexpr int kColumnParts = kDecodeWarps / 4;
      const int quarter = warp & 3;                 // TMEM lanes 32*quarter .. +31
      const int column_part = warp >> 2;            // warps 0-3: first part of the tokens, ...
      const int columns_per_part = (tn / 16 + kColumnParts - 1) / kColumnParts * 16;
      const int column_begin = column_part * columns_per_part;
      const int column_end = min(tn, column_begin + columns_per_part);
      const int out = row_block * kTileRows + quarter * 32 + lane;
      // The accumulator has output rows on lanes and tokens on columns, y is [token][row]: a lane
      // storing its own values writes 2 bytes per instruction (64 bytes per warp), and the store
      // instructions themselves then bound the epilogue.  Each warp therefore turns 16 tokens x 32
      // rows around through 1 KiB of the (now idle) weight stages and stores 16 bytes per lane:
      // eight rows of one token.  Rows beyond n, or an n / y that breaks the 16-byte alignment,
      // take the direct stores.
      const uint32_t turn = a_base + static_cast<uint32_t>(warp) * 1024u;
      const int out_base = row_block * kTileRows + quarter * 32;
      const bool wide = (p.n & 7) == 0 && out_base + 32 <= p.n && (reinterpret_cast<uintptr_t>(p.y) & 15) == 0;
      auto store_chunk = [&](const uint32_t (&r)[16], int a, int c) {
        const int token_base = (token_block + a) * tn + c;
        if (wide) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const __half h = __float2half_rn(__uint_as_float(r[i]));
            asm volatile("st.shared.u16 [%0], %1;" ::"r"(turn + i * 64u + lane * 2u),
                         "h"(*reinterpret_cast<const unsigned short *>(&h)));
          }
          __syncwarp();
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int piece = lane + 32 * q;          // token = piece / 4, eight rows = piece % 4
            const int token = token_base + (piece >> 2);
            const uint4 v = lds_u4(turn + static_cast<uint32_t>(piece) * 16u);
            if (token < p.rows)
              *reinterpret_cast<uint4 *>(p.y + static_cast<size_t>(token) * p.n + out_base + (piece & 3) * 8) = v;
          }
          __syncwarp();
        } else if (out < p.n) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int token = token_base + i;
            if (token < p.rows)
              p.y[static_cast<size_t>(token) * p.n + out] = __float2half_rn(__uint_as_float(r[i]));
          }
        }
      };
      if (p.k_splits == 1) {
        if (alive) {
          for (int a = 0; a < accumulators; ++a) {
            for (int c = column_begin; c < column_end; c += 16) {
              uint32_t r[16];
              tmem_load_16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * 256 + c, r);
              tmem_load_wait();
              store_chunk(r, a, c);
            }
          }
        }
      } else {
        // ---- split K: FP32 tile to scratch, in up to three PARTS (runs of 16-token chunks).  Split z
        //      writes the parts in the order z, z+1, ...; whoever completes a part's arrival
        //      counter adds that part's splits in index order and stores it.  CTAs that finish
        //      together are each the last writer of a different part, so the reduction spreads over
        //      the tile's CTAs without anyone waiting (a straggler simply reduces more parts).
        const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
        const size_t tile_floats = static_cast<size_t>(accumulators) * tn * kTileRows;
        const size_t split_stride = static_cast<size_t>(gridDim.x) * gridDim.y * tile_floats;
        float *tile_partial = p.partial + static_cast<size_t>(tile_id) * tile_floats;
        float *mine = tile_partial + blockIdx.z * split_stride;
        const int chunks_per_accumulator = tn / 16;
        const int chunks = accumulators * chunks_per_accumulator;
        const size_t lane_row = static_cast<size_t>(quarter) * 32 + lane;
        [[maybe_unused]] long long wrote = 0, synced = 0, reduced = 0;
        const int parts = min(p.k_splits, 3);  // (each part costs a fence and two barriers)
        for (int step = 0; step < parts; ++step) {
          const long long e0 = GEMM_CLOCK();
          const int part = (static_cast<int>(blockIdx.z) + step) % parts;
          const int chunk_begin = part * chunks / parts, chunk_end = (part + 1) * chunks / parts;
          if (alive) {
            for (int chunk = chunk_begin + column_part; chunk < chunk_end; chunk += kColumnParts) {
              const int a = chunk / chunks_per_accumulator, c = (chunk % chunks_per_accumulator) * 16;
              uint32_t r[16];
              tmem_load_16(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * 256 + c, r);
              tmem_load_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i)
                mine[static_cast<size_t>(a * tn + c + i) * kTileRows + lane_row] = __uint_as_float(r[i]);
            }
          }
          const long long e1 = GEMM_CLOCK();
          __threadfence();
          asm volatile("bar.sync 1, %0;" ::"n"(kDecodeThreads) : "memory");  // (decode warps only, all of them)
          if (tid == 0) {
            unsigned *counter = p.counters + tile_id * 8 + part;
            const bool last = atomicAdd(counter, 1u) == static_cast<unsigned>(p.k_splits - 1);
            if (last) *counter = 0u;  // (zero again for the next launch)
            split_last = last && abort_flag == 0;
          }
          asm volatile("bar.sync 1, %0;" ::"n"(kDecodeThreads) : "memory");
          const long long e2 = GEMM_CLOCK();
          wrote += e1 - e0;
          synced += e2 - e1;
          if (split_last) {
            __threadfence();
            for (int chunk = chunk_begin + column_part; chunk < chunk_end; chunk += kColumnParts) {
              const int a = chunk / chunks_per_accumulator, c = (chunk % chunks_per_accumulator) * 16;
              float sum[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) sum[i] = 0.0f;
              // (index order: the result does not depend on who came last; two splits' loads in
              //  flight at a time, the adds still in index order)
              const float *base = tile_partial + static_cast<size_t>(a * tn + c) * kTileRows + lane_row;
              int z = 0;
              for (; z + 1 < p.k_splits; z += 2) {
                float first[16], second[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) first[i] = __ldcg(base + z * split_stride + static_cast<size_t>(i) * kTileRows);
#pragma unroll
                for (int i = 0; i < 16; ++i) second[i] = __ldcg(base + (z + 1) * split_stride + static_cast<size_t>(i) * kTileRows);
#pragma unroll
                for (int i = 0; i < 16; ++i) sum[i] = (sum[i] + first[i]) + second[i];
              }
              if (z < p.k_splits) {
#pragma unroll
                for (int i = 0; i < 16; ++i) sum[i] += __ldcg(base + z * split_stride + static_cast<size_t>(i) * kTileRows);
              }
              uint32_t r[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(sum[i]);
              store_chunk(r, a, c);
            }
          }
          reduced += GEMM_CLOCK() - e2;
        }
#ifdef SAGEB200_TRACE
        if (p.trace && tid == 0) {
          long long *record = p.trace + static_cast<size_t>(tile_id) * 16;
          record[13] = wrote;
          record[14] = synced;
          record[15] = reduced;
        }
#endif
      }
    }
#ifdef SAGEB200_TRACE
    if (p.trace && tid == 0)
      p.trace[(static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * 16 + 6] = GEMM_CLOCK() - epilogue_begin;
#endif
  } else if (warp == kTmaWarp) {
    // ---------------- activation tile loads
    if (lane == 0) {
      pdl_wait();  // the activations are the previous kernel's output
      bool alive = true;
      long long waited = 0;
      for (int ks = 0; ks < stages_k && alive; ++ks) {
        const int s = ks % p.stages;
        const uint32_t phase = static_cast<uint32_t>(ks / p.stages) & 1u;
        const long long t0 = GEMM_CLOCK();
        alive = bounded_wait(empty_bar(s), phase ^ 1u, abort_ptr, p.status);
        if (!alive) break;
        waited += GEMM_CLOCK() - t0;
        if constexpr (kPair) {
          // the leader announces both CTAs' bytes; each CTA loads its half of every token block and
          // the copies complete on the leader's barrier
          if (leader) mbarrier_arrive_expect_tx(full_bar(s), static_cast<uint32_t>(2 * b_stage_bytes));
          for (int a = 0; a < accumulators; ++a)
            tma_load_2d_pair(b_base + s * b_stage_bytes + a * b_tile_bytes, &x_map, (stage_first + ks) * kStageK,
                             (token_block + a) * tn + static_cast<int>(pair_rank) * tile_tokens, full_bar(s));
        } else {
          mbarrier_arrive_expect_tx(full_bar(s), static_cast<uint32_t>(b_stage_bytes));
          for (int a = 0; a < accumulators; ++a)  // (a block past the last token reads the fill value)
            tma_load_2d(b_base + s * b_stage_bytes + a * b_tile_bytes, &x_map, (stage_first + ks) * kStageK,
                        (token_block + a) * tn, full_bar(s));
        }
      }
#ifdef SAGEB200_TRACE
      if (p.trace) p.trace[(static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * 16 + 7] = waited;
#endif
    }
  } else {
    // ---------------- MMA issue
    if (kPair && !leader) {
      // ---------------- odd CTA of a pair: forward "my decode warps have filled the stage"
      if (lane == 0) {
        bool alive = true;
        for (int ks = 0; ks < stages_k && alive; ++ks) {
          const int s = ks % p.stages;
          const uint32_t phase = static_cast<uint32_t>(ks / p.stages) & 1u;
          alive = bounded_wait(full_bar(s), phase, abort_ptr, p.status);
          if (!alive) break;
          mbarrier_arrive_leader(full_bar(s));
        }
      }
    } else if (lane == 0) {
      const uint32_t idesc = instruction_descriptor(kPair ? 2 * kTileRows : kTileRows, tn);
      bool alive = true;
      long long waited = 0;
      [[maybe_unused]] const long long mma_begin = GEMM_CLOCK();
      for (int ks = 0; ks < stages_k && alive; ++ks) {
        const int s = ks % p.stages;
        const uint32_t phase = static_cast<uint32_t>(ks / p.stages) & 1u;
        const long long t0 = GEMM_CLOCK();
        alive = bounded_wait(full_bar(s), phase, abort_ptr, p.status);
        if (!alive) break;
        waited += GEMM_CLOCK() - t0;
        tcgen05_fence_after();
        const uint64_t a_desc = smem_descriptor(a_base + s * kAStageBytes);
        for (int a = 0; a < accumulators; ++a) {
          const uint64_t b_desc = smem_descriptor(b_base + s * b_stage_bytes + a * b_tile_bytes);
#pragma unroll
          for (int j = 0; j < kStageK / 16; ++j) {
            // advancing 16 channels = 32 bytes = 2 units of the descriptor's address field
            if constexpr (kPair)
              umma_f16_pair(tmem_base + a * 256, a_desc + 2 * j, b_desc + 2 * j, idesc, (ks > 0 || j > 0) ? 1u : 0u);
            else
              umma_f16(tmem_base + a * 256, a_desc + 2 * j, b_desc + 2 * j, idesc, (ks > 0 || j > 0) ? 1u : 0u);
          }
        }
        if constexpr (kPair) umma_commit_pair(empty_bar(s));
        else umma_commit(empty_bar(s));
      }
      if (alive) {
        if constexpr (kPair) umma_commit_pair(accum_bar);
        else umma_commit(accum_bar);
      }
#ifdef SAGEB200_TRACE
      if (p.trace) {
        long long *record = p.trace + (static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * 16;
        record[8] = waited;
        record[9] = GEMM_CLOCK() - mma_begin;
      }
#endif
    }
  }

  // Let in-flight TMA copies land before the CTA's shared memory goes away: every issued
  // load targets a full barrier that the MMA thread has waited on unless we aborted; on
  // abort, wait (bounded) for each stage's barrier once more.
  tcgen05_fence_before();
  __syncthreads();
  // (a pair leaves together: the leader's MMAs read the other CTA's shared memory, and both CTAs'
  //  barriers receive remote arrivals until the last commit)
  if constexpr (kPair) cluster_sync_all();
  if (warp == kTmaWarp) {
    if (abort_flag && lane == 0) {
      const unsigned long long begin = global_timer();
      while (global_timer() - begin < 2000000ull) __nanosleep(1000);  // 2 ms grace for copies in flight
    }
    __syncwarp();
    if constexpr (kPair)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(static_cast<uint32_t>(p.tmem_columns))
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(static_cast<uint32_t>(p.tmem_columns))
                   : "memory");
  }
}

// x_q[m][j] = x[m][perm[j]]  (or a plain copy when perm is null).  One CTA per activation row at a
// time: the row is brought into shared memory with 16-byte (or, for an odd base address, 2-byte)
// loads, the permutation is read eight indices at a time, the gathered values come out of shared
// memory and leave as 16-byte stores - no 2-byte global loads, which cost a sector each.
constexpr int kGatherThreads = 256;
__global__ void __launch_bounds__(kGatherThreads) sage_gather_kernel(const __half *__restrict__ x,
                                                                     const int32_t *__restrict__ perm,
                                                                     __half *__restrict__ xq, int rows, int k) {
  extern __shared__ __align__(16) unsigned char gather_shared[];
  __half *row_shared = reinterpret_cast<__half *>(gather_shared);
  pdl_launch_dependents();  // (the GEMM behind this kernel sets up and decodes its first stages meanwhile)
  pdl_wait();               // the activations are the previous kernel's output
  const int vectors = k >> 3;
  const bool perm_wide = (reinterpret_cast<uintptr_t>(perm) & 15) == 0;
  for (int m = blockIdx.x; m < rows; m += gridDim.x) {
    const __half *source = x + static_cast<size_t>(m) * k;
    if ((reinterpret_cast<uintptr_t>(source) & 15) == 0) {
      for (int v = threadIdx.x; v < vectors; v += kGatherThreads)
        reinterpret_cast<uint4 *>(row_shared)[v] = reinterpret_cast<const uint4 *>(source)[v];
    } else {
      for (int j = threadIdx.x; j < k; j += kGatherThreads) row_shared[j] = source[j];
    }
    __syncthreads();
    uint4 *destination = reinterpret_cast<uint4 *>(xq + static_cast<size_t>(m) * k);
    for (int v = threadIdx.x; v < vectors; v += kGatherThreads) {
      if (perm == nullptr) {
        destination[v] = reinterpret_cast<const uint4 *>(row_shared)[v];
        continue;
      }
      int index[8];
      if (perm_wide) {
        *reinterpret_cast<int4 *>(index) = reinterpret_cast<const int4 *>(perm)[2 * v];
        *reinterpret_cast<int4 *>(index + 4) = reinterpret_cast<const int4 *>(perm)[2 * v + 1];
      } else {
#pragma unroll
        for (int d = 0; d < 8; ++d) index[d] = perm[v * 8 + d];
      }
      __align__(16) __half values[8];
#pragma unroll
      for (int d = 0; d < 8; ++d) values[d] = row_shared[index[d]];
      destination[v] = *reinterpret_cast<const uint4 *>(values);
    }
    __syncthreads();
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *symbol = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &query) ==
            cudaSuccess &&
        query == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(symbol);
  }
  return fn;
}

}  // namespace

cudaError_t launch_gather(const __half *x, const int32_t *perm, __half *xq, int rows, int k,
                          cudaStream_t stream, int sm_count) {
  const size_t shared = static_cast<size_t>(k) * sizeof(__half);
  if (shared > 200 * 1024) return cudaErrorInvalidValue;  // (K beyond 102400 channels)
  static bool configured[64] = {};
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return error;
  if (shared > 48 * 1024 && device >= 0 && device < 64 && !configured[device]) {
    error = cudaFuncSetAttribute(sage_gather_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (error != cudaSuccess) return error;
    configured[device] = true;
  }
  int blocks = rows;
  const int cap = (sm_count > 0 ? sm_count : 148) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return launch_dependent<1>(sage_gather_kernel, dim3(static_cast<unsigned>(blocks)), dim3(kGatherThreads), shared,
                             stream, x, perm, xq, rows, k);
}

int g_gemm_pairs = 1;  // debug switch (sageb200_debug_gemm_pairs): 0 = never pair CTAs

GemmPlan plan_gemm_tc(int rows, int n, int k, int sm_count, bool allow_split) {
  GemmPlan plan{};
  plan.row_blocks = (n + kTileRows - 1) / kTileRows;
  if (sm_count <= 0) sm_count = 148;
  const int groups = k / 128;
  // Tokens per accumulator (at most 256, 128 or 64, the rows split evenly), accumulators per CTA
  // (two token blocks sharing every decoded weight stage) and CTAs per output tile along K.
  // Cost model per 64-channel stage of one CTA, in cycles - the kernel runs at the slowest of
  //   shared-memory traffic / 128 bytes per cycle: the MMA's operand reads (A again for every
  //     accumulator), the activation tile written by TMA, the decoded weights and codebook reads
  //   the tensor pipe: 135 cycles per 128 x 256 x 16 instruction
  //   the decode warps: ~1200 cycles per stage (measured with the per-role clock sums of the
  //     profiling build)
  // times the stages per CTA and the waves the grid needs, plus, with a K split, the last CTA's
  // pass over all splits' FP32 tiles.  Large grids end up with 256 tokens x 2 (least decode work
  // per output); grids that would leave most SMs idle split K, so the decode work of one weight
  // tile is spread over several SMs.
  int tn = 0, best_accumulators = 1, best_splits = 1;
  double best_cost = 0.0;
  const int split_choices[] = {1, 2, 3, 4, 5, 6, 8};
  for (int cap = 256; cap >= 64; cap /= 2) {
    const int blocks = (rows + cap - 1) / cap;
    const int candidate = ((rows + blocks - 1) / blocks + 15) / 16 * 16;
    const int token_blocks = (rows + candidate - 1) / candidate;
    for (int accumulators = 2; accumulators >= 1; --accumulators) {
      if (accumulators == 2 && token_blocks < 2) continue;
      const double traffic = accumulators * 4.0 * (4096.0 + candidate * 32.0) + accumulators * candidate * 128.0 + 32768.0;
      const double tensor = accumulators * 4.0 * 135.0 * candidate / 256.0;
      double stage = traffic / 128.0;
      if (stage < tensor) stage = tensor;
      if (stage < 1200.0) stage = 1200.0;
      const long long tiles = static_cast<long long>(plan.row_blocks) * ((token_blocks + accumulators - 1) / accumulators);
      for (int wanted : split_choices) {
        // (a split only where the split grid still fits one wave: it exists to fill idle SMs, and
        //  its FP32 tiles would cost more HBM traffic than they save on a grid of several waves)
        if (wanted > 1 && (!allow_split || wanted * 2 > groups || tiles * wanted > sm_count || tiles > 2048)) continue;
        const int per_split = (groups + wanted - 1) / wanted;
        const int splits = (groups + per_split - 1) / per_split;  // (no empty split)
        if (splits != wanted) continue;
        const long long waves = (tiles * splits + sm_count - 1) / sm_count;
        double cost = 2.0 * per_split * stage * static_cast<double>(waves);
        if (splits > 1)  // tile written once per split, then read back by the last CTA (~64 bytes per cycle)
          cost += 2000.0 + (splits + 1.0) * accumulators * candidate * 128.0 * 4.0 / 64.0;
        if (tn == 0 || cost < best_cost * 0.97) {  // (prefer the earlier, simpler choice on near ties)
          tn = candidate;
          best_accumulators = accumulators;
          best_splits = splits;
          best_cost = cost;
        }
      }
    }
  }
  plan.tokens_per_cta = tn;
  plan.token_blocks = (rows + tn - 1) / tn;
  plan.accumulators = best_accumulators;
  // Pairs of CTAs (cta_group::2) whenever the row blocks pair up and each CTA's half of a token
  // block is a whole number of 16-token MMA columns: half the B operand per SM.
  plan.pair = g_gemm_pairs && (plan.row_blocks % 2 == 0) && (tn % 32 == 0) ? 1 : 0;
  plan.k_splits = best_splits;
  plan.groups_per_split = (groups + best_splits - 1) / best_splits;
  {
    const size_t tiles = static_cast<size_t>(plan.row_blocks) * ((plan.token_blocks + plan.accumulators - 1) / plan.accumulators);
    plan.partial_bytes = best_splits > 1 ? tiles * best_splits * plan.accumulators * tn * kTileRows * sizeof(float) : 0;
  }
  const int stage_bytes = kAStageBytes + plan.accumulators * (plan.pair ? tn / 2 : tn) * kStageK * 2;
  int stages = (kGemmSharedLimit - kBookBytes - 2 * 1024) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages < 2) stages = 2;
  plan.stages = stages;
  int columns = 32;
  while (columns < tn) columns *= 2;
  plan.tmem_columns = plan.accumulators == 2 ? 512 : columns;
  plan.shared_bytes = static_cast<size_t>(stages) * stage_bytes + kBookBytes + (2 * kMaxStages + 1) * 8 + 1024;
  return plan;
}

cudaError_t configure_gemm_tc() {
  cudaError_t error = cudaFuncSetAttribute(sage_gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kGemmSharedLimit);
  if (error != cudaSuccess) return error;
  return cudaFuncSetAttribute(sage_gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              kGemmSharedLimit);
}

// xq: activations in quantised channel order, 16-byte aligned, [rows][k].
cudaError_t launch_gemm_tc(const __half *xq, const uint32_t *codes, const uint32_t *radii,
                           const uint32_t *grid, const uint32_t *book, __half *y, int *status,
                           int rows, int n, int k, int entries, const GemmPlan &plan,
                           cudaStream_t stream, float *partial, unsigned *counters, const __half *sph_mins) {
  if (plan.k_splits > 1 && (!partial || !counters)) return cudaErrorInvalidValue;
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return cudaErrorNotSupported;
  CUtensorMap map;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k) * 2};
  const cuuint32_t box[2] = {kStageK, static_cast<cuuint32_t>(plan.pair ? plan.tokens_per_cta / 2 : plan.tokens_per_cta)};
  const cuuint32_t element_strides[2] = {1, 1};
  const CUresult encoded = encode(
      &map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half *>(xq), dims, strides, box,
      element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (encoded != CUDA_SUCCESS) return cudaErrorInvalidValue;
  GemmParams p{};
  p.codes = codes;
  p.radii = radii;
  p.grid = grid;
  p.book = book;
  p.y = y;
  p.status = status;
  p.rows = rows;
  p.n = n;
  p.k = k;
  p.groups = k / 128;
  p.tiles = (n + 15) / 16;
  p.entries = entries;
  p.dbits = direction_bits_of(entries);
  p.tokens_per_cta = plan.tokens_per_cta;
  p.stages = plan.stages;
  p.tmem_columns = plan.tmem_columns;
  p.accumulators = plan.accumulators;
  p.trace = trace_buffer();
  p.k_splits = plan.k_splits;
  p.groups_per_split = plan.groups_per_split;
  p.partial = partial;
  p.counters = counters;
  p.format = sph_mins ? 1 : 0;
  p.mins = sph_mins;
  const dim3 blocks(plan.row_blocks, (plan.token_blocks + plan.accumulators - 1) / plan.accumulators, plan.k_splits);
  cudaLaunchConfig_t config = {};
  config.gridDim = blocks;
  config.blockDim = dim3(kGemmThreads);
  config.dynamicSmemBytes = plan.shared_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  unsigned attributes = 0;
  if (g_sageb200_pdl & 1) {  // (the same switch as the decode kernels: sageb200_set_pdl)
    attribute[attributes].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[attributes].val.programmaticStreamSerializationAllowed = 1;
    ++attributes;
  }
  if (plan.pair) {
    attribute[attributes].id = cudaLaunchAttributeClusterDimension;
    attribute[attributes].val.clusterDim.x = 2;
    attribute[attributes].val.clusterDim.y = 1;
    attribute[attributes].val.clusterDim.z = 1;
    ++attributes;
  }
  config.attrs = attribute;
  config.numAttrs = attributes;
  return plan.pair ? cudaLaunchKernelEx(&config, sage_gemm_tc_kernel<true>, p, map)
                   : cudaLaunchKernelEx(&config, sage_gemm_tc_kernel<false>, p, map);
}

}  // namespace sageb200
