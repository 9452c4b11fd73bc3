// Causal attention over a whole prompt on the tensor cores (the prompt pass of the decode glue).
//
// No counterpart in the reference's native code: there the prompt runs through Hugging Face
// modules and torch SDPA (benchmarks/model.py:43-76).  The per-row decode kernel re-reads K/V for
// every prompt row; this kernel is the usual tiled form: a CTA of four warps owns 64 query rows of
// one head, walks the key/value positions 64 at a time (double-buffered cp.async into 128-byte
// swizzled shared memory), keeps S = Q K^T and O in mma.sync.m16n8k16 accumulators (FP16 inputs,
// FP32 accumulation) with the running maximum / sum of the streaming softmax in registers, and
// feeds P to the second product straight from the first product's accumulator layout.
//
// Rows are [sequence][token]; row (s, t) sits at cache position positions[s] + t and attends to
// cache positions 0 .. its own.  q is [rows][q_heads][128] (already normalised and rotated), the
// caches are [sequence][kv_head][max_seq][128], out is [rows][q_heads][128].
#include "sage_common.cuh"
#include "sage_kernels.h"

namespace sageb200 {
namespace {

constexpr int kQueryRows = 64;    // query rows per CTA (16 per warp)
constexpr int kKeyRows = 64;      // key/value positions per tile
constexpr int kHeadDim = 128;
constexpr int kTileBytes = 64 * kHeadDim * 2;  // 16 KiB
constexpr int kAttentionThreads = 128;
constexpr int kAttentionShared = kTileBytes * 5;  // Q + two stages of (K, V)

// Byte offset of 16-byte chunk `chunk` (0..15) of row `row` in a 64 x 128 FP16 tile whose rows
// are 256 bytes: the chunk index is XORed with the row so that the eight rows an ldmatrix reads
// fall into eight different bank groups.
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return static_cast<uint32_t>(row) * 256u + static_cast<uint32_t>((chunk ^ (row & 7)) & 15) * 16u;
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src, bool valid) {
  const int bytes = valid ? 16 : 0;  // (zero-fills the 16 bytes when the source row does not exist)
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t address, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t address, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(address));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}

__global__ void __launch_bounds__(kAttentionThreads)
    prefill_attention_kernel(const __half *__restrict__ q, const __half *__restrict__ k_cache,
                             const __half *__restrict__ v_cache, const int *__restrict__ positions,
                             __half *__restrict__ out, int tokens, int q_heads, int kv_heads, int max_seq,
                             float scale_log2) {
  extern __shared__ __align__(1024) unsigned char attention_shared[];
  const uint32_t q_tile = smem_address(attention_shared);
  const uint32_t kv_tiles = q_tile + kTileBytes;  // stage s: K at kv_tiles + s * 2 * kTileBytes, V one tile later

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int query_block = gridDim.x - 1 - blockIdx.x;  // (the longest contexts start first)
  const int head = blockIdx.y, sequence = blockIdx.z;
  const int kv_head = head / (q_heads / kv_heads);
  const int first = positions[sequence];               // cache position of the sequence's token 0
  const int q0 = query_block * kQueryRows;             // first token of this CTA
  const int rows_here = min(kQueryRows, tokens - q0);
  // last cache position any row of this CTA attends to
  const int last_position = min(first + q0 + rows_here - 1, max_seq - 1);
  const int tiles = last_position / kKeyRows + 1;

  const __half *q_base = q + (static_cast<size_t>(sequence) * tokens + q0) * q_heads * kHeadDim + head * kHeadDim;
  const size_t cache_base = (static_cast<size_t>(sequence) * kv_heads + kv_head) * max_seq * kHeadDim;

  auto load_kv = [&](int tile, int stage) {
    const uint32_t k_tile = kv_tiles + static_cast<uint32_t>(stage) * 2u * kTileBytes;
    const uint32_t v_tile = k_tile + kTileBytes;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int id = tid + kAttentionThreads * i;
      const int row = id >> 4, chunk = id & 15;
      const int position = tile * kKeyRows + row;
      const bool valid = position <= last_position;
      const size_t source = cache_base + static_cast<size_t>(valid ? position : 0) * kHeadDim + chunk * 8;
      cp_async_16(k_tile + tile_offset(row, chunk), k_cache + source, valid);
      cp_async_16(v_tile + tile_offset(row, chunk), v_cache + source, valid);
    }
  };

  // Q tile and the first K/V tile
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int id = tid + kAttentionThreads * i;
    const int row = id >> 4, chunk = id & 15;
    const bool valid = row < rows_here;
    cp_async_16(q_tile + tile_offset(row, chunk),
                q_base + static_cast<size_t>(valid ? row : 0) * q_heads * kHeadDim + chunk * 8, valid);
  }
  load_kv(0, 0);
  cp_async_commit();

  float o[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
  float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
  uint32_t q_frag[8][4];
  const int query_position[2] = {first + q0 + warp * 16 + g, first + q0 + warp * 16 + g + 8};

  for (int tile = 0; tile < tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < tiles) load_kv(tile + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();  // this tile's group (and Q) have landed; the next one may be in flight
    __syncthreads();
    if (tile == 0) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        ldmatrix_x4(q_tile + tile_offset(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)), q_frag[kk]);
    }
    const uint32_t k_tile = kv_tiles + static_cast<uint32_t>(stage) * 2u * kTileBytes;
    const uint32_t v_tile = k_tile + kTileBytes;

    // ---- S = Q K^T for this warp's 16 rows x 64 positions
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
      for (int pair = 0; pair < 4; ++pair) {  // two 8-position column tiles per ldmatrix
        uint32_t b[4];
        const int matrix = lane >> 3;
        ldmatrix_x4(k_tile + tile_offset(pair * 16 + (matrix >> 1) * 8 + (lane & 7), kk * 2 + (matrix & 1)), b);
        mma_16816(s[2 * pair], q_frag[kk], b[0], b[1]);
        mma_16816(s[2 * pair + 1], q_frag[kk], b[2], b[3]);
      }
    }

    // ---- causal mask, streaming softmax (base 2)
    const int tile_start = tile * kKeyRows;
    const bool diagonal = tile_start + kKeyRows - 1 > first + q0 + warp * 16;  // (some column beyond the warp's first row)
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int column = tile_start + n * 8 + 2 * t + (e & 1);
        if (diagonal && column > query_position[e >> 1]) s[n][e] = -INFINITY;
        tile_max[e >> 1] = fmaxf(tile_max[e >> 1], s[n][e]);
      }
    }
    float correction[2], offset[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
      tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
      const float new_max = fmaxf(row_max[r], tile_max[r]);
      // (position 0 is visible to every row, so new_max is finite from the first tile on)
      correction[r] = exp2f((row_max[r] - new_max) * scale_log2);
      row_max[r] = new_max;
      offset[r] = new_max * scale_log2;
      row_sum[r] *= correction[r];
    }
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      o[n][0] *= correction[0];
      o[n][1] *= correction[0];
      o[n][2] *= correction[1];
      o[n][3] *= correction[1];
    }
    uint32_t p_frag[4][4];  // P as the A operand of the second product, 16 positions per step
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const float p0 = exp2f(s[n][0] * scale_log2 - offset[0]);
      const float p1 = exp2f(s[n][1] * scale_log2 - offset[0]);
      const float p2 = exp2f(s[n][2] * scale_log2 - offset[1]);
      const float p3 = exp2f(s[n][3] * scale_log2 - offset[1]);
      row_sum[0] += p0 + p1;
      row_sum[1] += p2 + p3;
      p_frag[n >> 1][(n & 1) * 2] = pack_half2(p0, p1);
      p_frag[n >> 1][(n & 1) * 2 + 1] = pack_half2(p2, p3);
    }

    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int pair = 0; pair < 8; ++pair) {  // two 8-wide slices of the head dimension per ldmatrix
        uint32_t b[4];
        const int matrix = lane >> 3;
        ldmatrix_x4_trans(v_tile + tile_offset(kk * 16 + (matrix & 1) * 8 + (lane & 7), pair * 2 + (matrix >> 1)), b);
        mma_16816(o[2 * pair], p_frag[kk], b[0], b[1]);
        mma_16816(o[2 * pair + 1], p_frag[kk], b[2], b[3]);
      }
    }
    __syncthreads();  // everyone is done with this stage before the next iteration refills it
  }
  cp_async_wait<0>();

  // ---- normalise and store
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
    row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = warp * 16 + g + 8 * r;
    if (row >= rows_here) continue;
    const float inverse = 1.0f / row_sum[r];
    __half *destination = out + (static_cast<size_t>(sequence) * tokens + q0 + row) * q_heads * kHeadDim + head * kHeadDim;
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      const uint32_t packed = pack_half2(o[n][2 * r] * inverse, o[n][2 * r + 1] * inverse);
      *reinterpret_cast<uint32_t *>(destination + n * 8 + 2 * t) = packed;
    }
  }
}

}  // namespace

cudaError_t launch_prefill_attention(const __half *q, const __half *k_cache, const __half *v_cache,
                                     const int *positions, __half *out, int sequences, int tokens, int q_heads,
                                     int kv_heads, int max_seq, cudaStream_t stream) {
  static bool configured[64] = {};
  int device = 0;
  cudaError_t error = cudaGetDevice(&device);
  if (error != cudaSuccess) return error;
  if (device >= 0 && device < 64 && !configured[device]) {
    error = cudaFuncSetAttribute(prefill_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kAttentionShared);
    if (error != cudaSuccess) return error;
    configured[device] = true;
  }
  const dim3 grid((tokens + kQueryRows - 1) / kQueryRows, q_heads, sequences);
  const float scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(kHeadDim));
  prefill_attention_kernel<<<grid, kAttentionThreads, kAttentionShared, stream>>>(
      q, k_cache, v_cache, positions, out, tokens, q_heads, kv_heads, max_seq, scale_log2);
  return cudaGetLastError();
}

}  // namespace sageb200
