// SAGE packed GEMV / skinny GEMM for 1..16 activation rows (decode), sm_100a.
//
// Replaces the reference's sage_gemv_kernel (csrc/sage/sage_gemv_cuda.cu:8-110), which
// launches grid.y = rows and therefore re-reads and re-decodes every weight once per
// activation row.  Here one 16-row packed tile is exactly the M dimension of a
// mma.sync.m16n8k16 instruction: the decoded weights are the A operand, the (up to 8 or
// 16) activation rows are the B operand, so weights are read and decoded once for any
// row count and the FP16 products accumulate in FP32 inside the tensor core.
//
// Work split: CTA = (block of TB consecutive 16-row tiles) x (one of S splits of K).
// The CTA's (tile, 128-channel group) units are dealt round-robin to its warps.  Warp
// partials are combined through shared memory in a fixed order; with S > 1 the CTA's
// partial goes to global scratch and the last CTA to arrive for that tile block (an
// arrival counter, no spinning) adds the S partials in split order, so results do not
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

namespace sageb200 {
namespace {

struct UnitRegs {
  uint2 code[2];
  uint32_t radius[2];
  uint32_t grid[2];
};

__device__ __forceinline__ void load_unit(UnitRegs &r, const SkinnyProblem &p, int tile,
                                          int group, int g, int t) {
  const size_t cell = (static_cast<size_t>(tile) * p.groups + group) * 16 + g;
  r.code[0] = ldg_stream_u2(p.codes + cell * 8 + 2 * t);
  r.code[1] = ldg_stream_u2(p.codes + (cell + 8) * 8 + 2 * t);
  r.radius[0] = ldg_stream_u1(p.radii + cell);
  r.radius[1] = ldg_stream_u1(p.radii + cell + 8);
  r.grid[0] = ldg_stream_u1(p.grid + cell);
  r.grid[1] = ldg_stream_u1(p.grid + cell + 8);
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Bit-field constants that depend on the direction-bit count D, hoisted per problem.
struct FieldConsts {
  uint32_t index_mask;   // (entries-1) << L, L = 4 + replica_log2
  uint32_t shift_lo;     // 8 - L: moves the low code's index to bit L
  uint32_t shift_hi;     // 24 - L: same for the high code
  uint32_t hi_mask;      // 3 << (27 - D): the two high radius bits at mantissa position
  uint32_t hi_shift;     // 27 - D
  uint32_t lo_mask;      // ((1 << (8-D)) - 1) << 19: the low radius bits at mantissa position
  uint32_t lo_left;      // 11 - D: low code's radius bits -> bit 19
  uint32_t lo_right;     // 5 + D: high code's radius bits -> bit 19
};

template <int NB>
__device__ __forceinline__ void compute_unit(const UnitRegs &r, float (&acc)[NB][4],
                                             const FieldConsts &f, uint32_t book_base,
                                             uint32_t lane_offset,
                                             const uint32_t (&x_address)[NB], int t) {
  float step16[2], base[2];
  uint32_t high[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float2 e = __half22float2(*reinterpret_cast<const __half2 *>(&r.grid[h]));
    step16[h] = e.y * 16.0f;
    base[h] = fmaf(-16.0f, e.y, e.x);
    high[h] = (r.radius[h] >> (8 * t)) << f.hi_shift;
  }
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    uint32_t a[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t word = (s < 2) ? r.code[h].x : r.code[h].y;
      uint32_t address, signs, radius_bits;
      if (s & 1) {
        address = ((word >> f.shift_hi) & f.index_mask) | lane_offset;
        signs = (word >> 16) & 0xffu;
        radius_bits = (word >> f.lo_right) & f.lo_mask;
      } else {
        address = ((word >> f.shift_lo) & f.index_mask) | lane_offset;
        signs = word & 0xffu;
        radius_bits = (word << f.lo_left) & f.lo_mask;
      }
      // entry offset and replica offset never overlap, so OR; the base is a link-time
      // constant of the static array and folds into the load's immediate
      const uint4 dir = lds_u4(book_base + address);
      radius_bits |= ((high[h] >> (2 * s)) & f.hi_mask) | 0x3f800000u;
      const float radius = fmaf(__uint_as_float(radius_bits), step16[h], base[h]);
      const __half2 rr = __floats2half2_rn(radius, radius);
      // sign bit 2p -> bit 15 and sign bit 2p+1 -> bit 31 of half2 word p
      const uint32_t spread = signs * 0x8001u;
      const uint32_t d[4] = {dir.x ^ ((spread << 15) & 0x80008000u),
                             dir.y ^ ((spread << 13) & 0x80008000u),
                             dir.z ^ ((spread << 11) & 0x80008000u),
                             dir.w ^ ((spread << 9) & 0x80008000u)};
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const __half2 w = __hmul2(*reinterpret_cast<const __half2 *>(&d[p]), rr);
        a[h][p] = *reinterpret_cast<const uint32_t *>(&w);
      }
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const uint4 b = lds_u4(x_address[nb] + s * 64);
      mma_16816(acc[nb], a[0][0], a[1][0], a[0][1], a[1][1], b.x, b.y);
      mma_16816(acc[nb], a[0][2], a[1][2], a[0][3], a[1][3], b.z, b.w);
    }
  }
}

// The replicated codebook lives in STATIC shared memory (32 KiB: 256 entries x 8
// replicas x 16 bytes) so that its base address is a compile-time immediate.
constexpr int kBookBytes = 256 * 8 * 16;

// Shared memory map (dynamic): [staged x | warp partials].
template <int NB, int TB>
__global__ void __launch_bounds__(256) sage_skinny_kernel(const __grid_constant__ SkinnyParams params) {
  extern __shared__ __align__(16) unsigned char shared[];
  __shared__ __align__(128) unsigned char book_shared[kBookBytes];
  __shared__ int last_flag;

  int pi = 0;
  while (pi + 1 < params.count && static_cast<int>(blockIdx.x) >= params.problem[pi + 1].cta_begin)
    ++pi;
  const SkinnyProblem &p = params.problem[pi];

  const int tid = threadIdx.x;
  const int threads = blockDim.x;
  const int warp = tid >> 5;
  const int launched_warps = threads >> 5;
  const int warps = p.warps;  // warps that take units; a grouped launch may carry more
  const int lane = tid & 31;
  const int g = lane >> 2;
  const int t = lane & 3;

  const int local = static_cast<int>(blockIdx.x) - p.cta_begin;
  const int split = local % p.splits;
  const int tile_block = local / p.splits;
  const int group_begin = split * p.groups_per_split;
  const int group_count = min(p.groups_per_split, p.groups - group_begin);
  const int tile_begin = tile_block * TB;
  const int tile_count = min(TB, p.tiles - tile_begin);
  const int units = tile_count * group_count;

  // First unit of this warp: start its loads before anything else.
  int unit = warp;
  int ti = 0, gi = warp;
  while (gi >= group_count && ti < tile_count) {
    gi -= group_count;
    ++ti;
  }
  UnitRegs current;
  const bool has_work = warp < warps && unit < units;
  if (has_work) load_unit(current, p, tile_begin + ti, group_begin + gi, g, t);

  const int replica_log2 = params.replica_log2;
  const int line_log2 = 4 + replica_log2;
  __half *x_shared = reinterpret_cast<__half *>(shared);
  float *partial_shared = reinterpret_cast<float *>(shared + params.x_bytes);

  // Codebook: entry e, replica j at byte (e << line_log2) + 16*j, dims 0..7 contiguous.
  for (int e = tid; e < p.entries; e += threads) {
    uint4 entry;
    entry.x = p.book[e];
    entry.y = p.book[p.entries + e];
    entry.z = p.book[2 * p.entries + e];
    entry.w = p.book[3 * p.entries + e];
    const uint32_t base = smem_address(book_shared) + (static_cast<uint32_t>(e) << line_log2);
    for (int j = 0; j < (1 << replica_log2); ++j) sts_u4(base + 16 * j, entry);
  }

  // Activations of this K range, gathered through the permutation and laid out so that
  // lane (g,t), step s finds vector 4t+s of its row at [group][s][t][8 halves].
  const int span = group_count * 128;
  const int row_stride = span + 32;  // halves; +64 bytes staggers rows across banks
  for (int i = tid; i < span; i += threads) {
    const int j = group_begin * 128 + i;
    const int source = p.perm ? p.perm[j] : j;
    const int vector = (i >> 3) & 15;
    const int target = (i & ~127) + (vector & 3) * 32 + (vector >> 2) * 8 + (i & 7);
    for (int m = 0; m < p.rows; ++m)
      x_shared[m * row_stride + target] = p.x[static_cast<size_t>(m) * p.k + source];
  }
  const int partial_floats = launched_warps * TB * NB * 128;
  for (int i = tid; i < partial_floats; i += threads) partial_shared[i] = 0.0f;
  __syncthreads();

  FieldConsts f;
  f.index_mask = static_cast<uint32_t>(p.entries - 1) << line_log2;
  f.shift_lo = 8 - line_log2;
  f.shift_hi = 24 - line_log2;
  f.hi_shift = 27 - p.dbits;
  f.hi_mask = 3u << f.hi_shift;
  f.lo_mask = ((1u << (8 - p.dbits)) - 1u) << 19;
  f.lo_left = 11 - p.dbits;
  f.lo_right = 5 + p.dbits;
  const uint32_t book_base = smem_address(book_shared);
  const uint32_t lane_offset = 16u * static_cast<uint32_t>(lane & ((1 << replica_log2) - 1));
  uint32_t x_row_address[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int m = min(g + 8 * nb, p.rows - 1);
    x_row_address[nb] = smem_address(x_shared) + 2u * static_cast<uint32_t>(m * row_stride) + 16u * t;
  }

  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[nb][c] = 0.0f;

  auto flush = [&](int tile_index) {
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float *dst = partial_shared + ((warp * TB + tile_index) * NB + nb) * 128;
      *reinterpret_cast<float2 *>(dst + g * 8 + 2 * t) = make_float2(acc[nb][0], acc[nb][1]);
      *reinterpret_cast<float2 *>(dst + (g + 8) * 8 + 2 * t) = make_float2(acc[nb][2], acc[nb][3]);
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[nb][c] = 0.0f;
    }
  };

  if (has_work) {
    while (true) {
      // advance to the next unit of this warp and prefetch it
      int next_ti = ti, next_gi = gi + warps;
      while (next_gi >= group_count) {
        next_gi -= group_count;
        ++next_ti;
      }
      const bool more = next_ti < tile_count;
      UnitRegs next;
      if (more) load_unit(next, p, tile_begin + next_ti, group_begin + next_gi, g, t);

      uint32_t x_address[NB];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) x_address[nb] = x_row_address[nb] + 256u * gi;
      compute_unit<NB>(current, acc, f, book_base, lane_offset, x_address, t);

      if (!more || next_ti != ti) flush(ti);
      if (!more) break;
      current = next;
      ti = next_ti;
      gi = next_gi;
    }
  }
  __syncthreads();

  // Combine warps in warp order.  Element index e = ((tile*NB + nb)*16 + row)*8 + column.
  const int elements = tile_count * NB * 128;
  const bool direct = p.splits == 1;
  float *partial_global =
      direct ? nullptr
             : p.partial + (static_cast<size_t>(tile_block) * p.splits + split) * (TB * NB * 128);
  for (int e = tid; e < elements; e += threads) {
    float sum = 0.0f;
    for (int w = 0; w < warps; ++w) sum += partial_shared[w * (TB * NB * 128) + e];
    if (direct) {
      const int column = e & 7, row = (e >> 3) & 15;
      const int nb = (e >> 7) % NB, tile_index = (e >> 7) / NB;
      const int m = nb * 8 + column;
      const int out = (tile_begin + tile_index) * 16 + row;
      if (m < p.rows && out < p.n) p.y[static_cast<size_t>(m) * p.n + out] = __float2half_rn(sum);
    } else {
      __stcg(partial_global + e, sum);
    }
  }
  if (direct) return;

  // Split-K: publish, count arrivals, the last CTA reduces in split order.
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned arrived = atomicAdd(p.counters + tile_block, 1u);
    last_flag = (arrived == static_cast<unsigned>(p.splits) - 1u);
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  const float *all = p.partial + static_cast<size_t>(tile_block) * p.splits * (TB * NB * 128);
  for (int e = tid; e < elements; e += threads) {
    float sum = 0.0f;
    for (int s = 0; s < p.splits; ++s) sum += __ldcg(all + s * (TB * NB * 128) + e);
    const int column = e & 7, row = (e >> 3) & 15;
    const int nb = (e >> 7) % NB, tile_index = (e >> 7) / NB;
    const int m = nb * 8 + column;
    const int out = (tile_begin + tile_index) * 16 + row;
    if (m < p.rows && out < p.n) p.y[static_cast<size_t>(m) * p.n + out] = __float2half_rn(sum);
  }
  if (tid == 0) p.counters[tile_block] = 0u;
}

constexpr int kMaxDynamicShared = 160 * 1024;

template <int NB, int TB>
cudaError_t launch_variant(const SkinnyParams &params, int ctas, int threads, size_t shared_bytes,
                           cudaStream_t stream) {
  sage_skinny_kernel<NB, TB><<<ctas, threads, shared_bytes, stream>>>(params);
  return cudaGetLastError();
}

template <int NB, int TB>
cudaError_t configure_variant() {
  return cudaFuncSetAttribute(sage_skinny_kernel<NB, TB>,
                              cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicShared);
}

int best_warps(int units, int limit) {
  // fewest round-robin passes over the units, then the fewest warps that achieve it
  const int most = units < limit ? units : limit;
  const int passes = (units + most - 1) / most;
  return (units + passes - 1) / passes;
}

}  // namespace

SkinnyPlan plan_skinny(int rows, int n, int k, int entries, int sm_count, const Tuning &tuning) {
  SkinnyPlan plan{};
  const int tiles = (n + 15) / 16;
  const int groups = k / 128;
  plan.column_blocks = rows > 8 ? 2 : 1;
  plan.replicas = tuning.replicas > 0 ? tuning.replicas : 8;
  plan.tiles_per_cta = tuning.tiles_per_cta > 0 ? tuning.tiles_per_cta : 1;
  if (plan.tiles_per_cta > 2 && plan.column_blocks == 2) plan.tiles_per_cta = 2;
  if (plan.tiles_per_cta > 4) plan.tiles_per_cta = 4;
  if (plan.tiles_per_cta == 3) plan.tiles_per_cta = 2;
  plan.tile_blocks = (tiles + plan.tiles_per_cta - 1) / plan.tiles_per_cta;

  int splits = tuning.splits;
  if (splits <= 0) {
    // enough CTAs for ~4 per SM, at least two groups per CTA
    const int want = 4 * sm_count;
    splits = (want + plan.tile_blocks - 1) / plan.tile_blocks;
    const int most = groups >= 2 ? groups / 2 : 1;
    if (splits > most) splits = most;
    if (splits < 1) splits = 1;
  }
  if (splits > groups) splits = groups;
  // staged activations must fit: rows * (span*2 + 64) bytes <= 96 KiB
  while (static_cast<size_t>(rows) * (((groups + splits - 1) / splits) * 256 + 64) > 96 * 1024 &&
         splits < groups)
    ++splits;
  plan.groups_per_split = (groups + splits - 1) / splits;
  plan.splits = (groups + plan.groups_per_split - 1) / plan.groups_per_split;
  const int units = plan.groups_per_split * plan.tiles_per_cta;
  plan.warps = tuning.warps > 0 ? tuning.warps : best_warps(units, 8);
  if (plan.warps > 8) plan.warps = 8;
  if (plan.warps > units) plan.warps = units;
  if (plan.splits > 1) {
    plan.partial_bytes = static_cast<size_t>(plan.tile_blocks) * plan.splits * plan.tiles_per_cta *
                         plan.column_blocks * 128 * sizeof(float);
    plan.counter_bytes = static_cast<size_t>(plan.tile_blocks) * sizeof(unsigned);
  }
  return plan;
}

cudaError_t configure_skinny() {
  cudaError_t status;
  if ((status = configure_variant<1, 1>()) != cudaSuccess) return status;
  if ((status = configure_variant<1, 2>()) != cudaSuccess) return status;
  if ((status = configure_variant<1, 4>()) != cudaSuccess) return status;
  if ((status = configure_variant<2, 1>()) != cudaSuccess) return status;
  return configure_variant<2, 2>();
}

cudaError_t launch_skinny(SkinnyParams &params, const SkinnyPlan &plan, int total_ctas,
                          cudaStream_t stream) {
  int replica_log2 = 0;
  while ((1 << (replica_log2 + 1)) <= plan.replicas) ++replica_log2;
  params.replica_log2 = replica_log2;
  int max_entries = 0;
  size_t x_bytes = 0;
  for (int i = 0; i < params.count; ++i) {
    const SkinnyProblem &p = params.problem[i];
    if (p.entries > max_entries) max_entries = p.entries;
    const size_t need = static_cast<size_t>(p.rows) * (p.groups_per_split * 256 + 64);
    if (need > x_bytes) x_bytes = need;
  }
  (void)max_entries;
  params.x_bytes = static_cast<int>((x_bytes + 15) / 16 * 16);
  const size_t partial_bytes =
      static_cast<size_t>(plan.warps) * plan.tiles_per_cta * plan.column_blocks * 128 * sizeof(float);
  const size_t shared_bytes = params.x_bytes + partial_bytes;
  if (shared_bytes > static_cast<size_t>(kMaxDynamicShared)) return cudaErrorInvalidConfiguration;
  const int threads = plan.warps * 32;
#define SAGEB200_LAUNCH(NB, TB) \
  return launch_variant<NB, TB>(params, total_ctas, threads, shared_bytes, stream)
  if (plan.column_blocks == 1) {
    if (plan.tiles_per_cta == 1) SAGEB200_LAUNCH(1, 1);
    if (plan.tiles_per_cta == 2) SAGEB200_LAUNCH(1, 2);
    SAGEB200_LAUNCH(1, 4);
  }
  if (plan.tiles_per_cta == 1) SAGEB200_LAUNCH(2, 1);
  SAGEB200_LAUNCH(2, 2);
#undef SAGEB200_LAUNCH
}

}  // namespace sageb200
