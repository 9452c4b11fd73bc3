// Everything in a Qwen3 decode step that is not a packed linear, as small fused kernels for
// 1..16 sequences decoding one token each.  In the reference these steps are Hugging Face
// `transformers` modules driven by benchmarks/model.py:43-133 (RMSNorm eps 1e-6, per-head
// q/k RMSNorm, rotate-half RoPE, static KV cache, SDPA, SwiGLU, FP16 lm_head, argmax); here
// they exist so that a whole decode step can be captured in one CUDA graph with no host
// round trip: token ids and positions live in device memory.
//
// Numerics follow the Hugging Face modules: norms and softmax in FP32, one rounding to FP16
// where the module returns FP16, RoPE products in FP16 with FP16 cos/sin tables.
#include "../../include/sage_b200_decode.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <cooperative_groups.h>

#include "sage_common.cuh"
#include "sage_kernels.h"

namespace {

constexpr int kNormThreads = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blockDim.x <= 1024 (result in every thread).
__device__ float block_sum(float v, float *scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float total = 0.0f;
  const int warps = (blockDim.x + 31) >> 5;
  for (int w = 0; w < warps; ++w) total += scratch[w];
  return total;
}

// h[m][:] = embedding[token[m]][:]
// A token id outside [0, vocab) (a corrupted id, or the "no candidate" value of an argmax over a
// row of NaNs) reads row 0 instead of memory far beyond the table.
__global__ void embed_kernel(const __half *__restrict__ table, const long long *__restrict__ tokens,
                             __half *__restrict__ h, int hidden, int vocab) {
  // programmatic dependent launch: let the next kernel be scheduled, then wait for the
  // previous one before touching memory
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();

  const int m = blockIdx.x;
  long long token = tokens[m];
  if (token < 0 || token >= vocab) token = 0;
  const __half *row = table + static_cast<size_t>(token) * hidden;
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x)
    reinterpret_cast<uint4 *>(h + static_cast<size_t>(m) * hidden)[i] =
        reinterpret_cast<const uint4 *>(row)[i];
}

// residual[m] += delta[m] (FP16 add, skipped when delta is null);
// x[m] = weight * fp16(residual[m] * rsqrt(mean(residual[m]^2) + eps))
__global__ void __launch_bounds__(kNormThreads)
    add_rmsnorm_kernel(__half *__restrict__ residual, const __half *__restrict__ delta,
                       const __half *__restrict__ weight, __half *__restrict__ x, int hidden,
                       float eps) {
  // programmatic dependent launch: let the next kernel be scheduled, then wait for the
  // previous one before touching memory
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();

  __shared__ float scratch[32];
  extern __shared__ __half row_shared[];
  const int m = blockIdx.x;
  __half *r = residual + static_cast<size_t>(m) * hidden;
  const __half *d = delta ? delta + static_cast<size_t>(m) * hidden : nullptr;
  float square = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
    __half v = r[i];
    if (d) {
      v = __hadd(v, d[i]);
      r[i] = v;
    }
    row_shared[i] = v;
    const float f = __half2float(v);
    square += f * f;
  }
  const float total = block_sum(square, scratch);
  const float scale = rsqrtf(total / hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
    const __half normed = __float2half_rn(__half2float(row_shared[i]) * scale);
    x[static_cast<size_t>(m) * hidden + i] = __hmul(weight[i], normed);
  }
}


// add_rmsnorm_kernel with the normalised row written once per consumer, each in that consumer's
// quantised channel order (out[j][m][c] = x[m][perm[j][c]]): the packed linears behind it then
// take their activations as they lie and need no gather pre-pass.  Same arithmetic and summation
// order as add_rmsnorm_kernel; `x` (plain order) is written as well when non-null.
struct PermutedOutputs {
  const int *perm[4];
  __half *out[4];
  int count;
};
__global__ void __launch_bounds__(kNormThreads)
    add_rmsnorm_permuted_kernel(__half *__restrict__ residual, const __half *__restrict__ delta,
                                const __half *__restrict__ weight, __half *__restrict__ x,
                                const __grid_constant__ PermutedOutputs outputs, int hidden, float eps) {
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();
  __shared__ float scratch[32];
  extern __shared__ __half row_shared[];
  const int m = blockIdx.x;
  __half *r = residual + static_cast<size_t>(m) * hidden;
  const __half *d = delta ? delta + static_cast<size_t>(m) * hidden : nullptr;
  float square = 0.0f;
  for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
    __half v = r[i];
    if (d) {
      v = __hadd(v, d[i]);
      r[i] = v;
    }
    row_shared[i] = v;
    const float f = __half2float(v);
    square += f * f;
  }
  const float total = block_sum(square, scratch);
  const float scale = rsqrtf(total / hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
    const __half normed = __float2half_rn(__half2float(row_shared[i]) * scale);
    const __half value = __hmul(weight[i], normed);
    row_shared[i] = value;
    if (x) x[static_cast<size_t>(m) * hidden + i] = value;
  }
  __syncthreads();
  for (int j = 0; j < outputs.count; ++j) {
    const int4 *perm = reinterpret_cast<const int4 *>(outputs.perm[j]);
    uint4 *destination = reinterpret_cast<uint4 *>(outputs.out[j] + static_cast<size_t>(m) * hidden);
    for (int v = threadIdx.x; v < (hidden >> 3); v += kNormThreads) {
      const int4 lo = __ldg(perm + 2 * v), hi = __ldg(perm + 2 * v + 1);
      __align__(16) __half values[8] = {row_shared[lo.x], row_shared[lo.y], row_shared[lo.z], row_shared[lo.w],
                                        row_shared[hi.x], row_shared[hi.y], row_shared[hi.z], row_shared[hi.w]};
      destination[v] = *reinterpret_cast<const uint4 *>(values);
    }
  }
}

// act_q[m][c] = silu(gate[m][perm[c]]) * up[m][perm[c]]: SwiGLU written in the consumer's
// quantised channel order (one CTA per row at a time; the row is formed in shared memory with the
// rounding of swiglu_kernel, then gathered).
__global__ void __launch_bounds__(256)
    swiglu_permuted_kernel(const __half *__restrict__ gate, const __half *__restrict__ up,
                           const int *__restrict__ perm, __half *__restrict__ act, int rows, int k) {
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();
  extern __shared__ __half row_shared[];
  for (int m = blockIdx.x; m < rows; m += gridDim.x) {
    const uint4 *g4 = reinterpret_cast<const uint4 *>(gate + static_cast<size_t>(m) * k);
    const uint4 *u4 = reinterpret_cast<const uint4 *>(up + static_cast<size_t>(m) * k);
    for (int v = threadIdx.x; v < (k >> 3); v += 256) {
      const uint4 g = g4[v], u = u4[v];
      const __half2 *g2 = reinterpret_cast<const __half2 *>(&g), *u2 = reinterpret_cast<const __half2 *>(&u);
      uint4 out;
      __half2 *o2 = reinterpret_cast<__half2 *>(&out);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __half22float2(g2[q]);
        o2[q] = __hmul2(__halves2half2(__float2half_rn(sageb200::silu_fast(f.x)),
                                       __float2half_rn(sageb200::silu_fast(f.y))), u2[q]);
      }
      reinterpret_cast<uint4 *>(row_shared)[v] = out;
    }
    __syncthreads();
    uint4 *destination = reinterpret_cast<uint4 *>(act + static_cast<size_t>(m) * k);
    for (int v = threadIdx.x; v < (k >> 3); v += 256) {
      const int4 lo = __ldg(reinterpret_cast<const int4 *>(perm) + 2 * v);
      const int4 hi = __ldg(reinterpret_cast<const int4 *>(perm) + 2 * v + 1);
      __align__(16) __half values[8] = {row_shared[lo.x], row_shared[lo.y], row_shared[lo.z], row_shared[lo.w],
                                        row_shared[hi.x], row_shared[hi.y], row_shared[hi.z], row_shared[hi.w]};
      destination[v] = *reinterpret_cast<const uint4 *>(values);
    }
    __syncthreads();
  }
}

// One warp per (sequence, head): per-head RMSNorm of q or k (head_dim 128), rotate-half
// RoPE at the sequence's position, q written in place, k and v written into the cache.
// Heads 0..q_heads-1 are query heads, then kv_heads key heads, then kv_heads value heads.
__global__ void qk_norm_rope_cache_kernel(__half *__restrict__ q, const __half *__restrict__ k,
                                          const __half *__restrict__ v,
                                          const __half *__restrict__ q_weight,
                                          const __half *__restrict__ k_weight,
                                          const __half *__restrict__ cos_table,
                                          const __half *__restrict__ sin_table,
                                          const int *__restrict__ positions,
                                          __half *__restrict__ k_cache, __half *__restrict__ v_cache,
                                          int q_heads, int kv_heads, int max_seq, float eps,
                                          int rows_per_sequence) {
  // programmatic dependent launch: let the next kernel be scheduled, then wait for the
  // previous one before touching memory
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();

  const int lane = threadIdx.x & 31;
  const int head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int m = blockIdx.y;
  const int heads = q_heads + 2 * kv_heads;
  if (head >= heads) return;
  // decode: row = sequence, at positions[row]; prefill: rows_per_sequence consecutive rows are
  // the tokens of one sequence, at positions[sequence] + token
  const int sequence = m / rows_per_sequence;
  const int position = positions[sequence] + (m - sequence * rows_per_sequence);
  if (position < 0 || position >= max_seq) return;  // a full cache: write nothing out of range
  if (head >= q_heads + kv_heads) {  // value head: plain copy into the cache
    const int j = head - q_heads - kv_heads;
    const uint2 value = reinterpret_cast<const uint2 *>(v + (static_cast<size_t>(m) * kv_heads + j) * 128)[lane];
    reinterpret_cast<uint2 *>(v_cache + ((static_cast<size_t>(sequence) * kv_heads + j) * max_seq + position) * 128)[lane] = value;
    return;
  }
  const bool is_query = head < q_heads;
  const int j = is_query ? head : head - q_heads;
  const __half *source = is_query ? q + (static_cast<size_t>(m) * q_heads + j) * 128
                                  : k + (static_cast<size_t>(m) * kv_heads + j) * 128;
  const __half *weight = is_query ? q_weight : k_weight;
  // lane holds dims lane*2, lane*2+1 of the first half and the same of the second half
  const __half2 lo = reinterpret_cast<const __half2 *>(source)[lane];
  const __half2 hi = reinterpret_cast<const __half2 *>(source + 64)[lane];
  const float2 lof = __half22float2(lo), hif = __half22float2(hi);
  const float square = warp_sum(lof.x * lof.x + lof.y * lof.y + hif.x * hif.x + hif.y * hif.y);
  const float scale = rsqrtf(square / 128.0f + eps);
  const __half2 wl = reinterpret_cast<const __half2 *>(weight)[lane];
  const __half2 wh = reinterpret_cast<const __half2 *>(weight + 64)[lane];
  const __half2 nl = __hmul2(wl, __floats2half2_rn(lof.x * scale, lof.y * scale));
  const __half2 nh = __hmul2(wh, __floats2half2_rn(hif.x * scale, hif.y * scale));
  const __half2 c = reinterpret_cast<const __half2 *>(cos_table + static_cast<size_t>(position) * 64)[lane];
  const __half2 s = reinterpret_cast<const __half2 *>(sin_table + static_cast<size_t>(position) * 64)[lane];
  // out_lo = x_lo*cos - x_hi*sin ; out_hi = x_hi*cos + x_lo*sin  (FP16 products and sums)
  const __half2 out_lo = __hadd2(__hmul2(nl, c), __hmul2(__hneg2(nh), s));
  const __half2 out_hi = __hadd2(__hmul2(nh, c), __hmul2(nl, s));
  __half *target = is_query ? q + (static_cast<size_t>(m) * q_heads + j) * 128
                            : k_cache + ((static_cast<size_t>(sequence) * kv_heads + j) * max_seq + position) * 128;
  reinterpret_cast<__half2 *>(target)[lane] = out_lo;
  reinterpret_cast<__half2 *>(target + 64)[lane] = out_hi;
}

// Attention for one new token per sequence, split over the context ("flash decoding").
// CTA = (split, kv head, sequence); its `group` query heads share the K/V chunk.  Each warp
// walks positions of the chunk; partial (max, sum, weighted V) per query head go to scratch.
constexpr int kAttnWarps = 8;
constexpr int kMaxGroup = 8;

__global__ void __launch_bounds__(kAttnWarps * 32)
    attention_partial_kernel(const __half *__restrict__ q, const __half *__restrict__ k_cache,
                             const __half *__restrict__ v_cache, const int *__restrict__ positions,
                             float *__restrict__ partial, int q_heads, int kv_heads, int max_seq,
                             int splits, float scale) {
  // programmatic dependent launch: let the next kernel be scheduled, then wait for the
  // previous one before touching memory
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();

  __shared__ float shared_max[kAttnWarps][kMaxGroup];
  __shared__ float shared_sum[kAttnWarps][kMaxGroup];
  __shared__ float shared_acc[kAttnWarps][kMaxGroup][128];
  const int split = blockIdx.x, kv = blockIdx.y, m = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = q_heads / kv_heads;
  const int context = min(positions[m] + 1, max_seq);
  const int chunk = (context + splits - 1) / splits;
  const int begin = split * chunk;
  const int end = min(context, begin + chunk);
  // lane holds dims 4*lane .. 4*lane+3
  float2 qa[kMaxGroup], qb[kMaxGroup];
  for (int g = 0; g < group; ++g) {
    const __half *qh = q + (static_cast<size_t>(m) * q_heads + kv * group + g) * 128 + 4 * lane;
    qa[g] = __half22float2(reinterpret_cast<const __half2 *>(qh)[0]);
    qb[g] = __half22float2(reinterpret_cast<const __half2 *>(qh)[1]);
  }
  float running_max[kMaxGroup], running_sum[kMaxGroup], acc[kMaxGroup][4];
  for (int g = 0; g < kMaxGroup; ++g) {
    running_max[g] = -INFINITY;
    running_sum[g] = 0.0f;
    acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.0f;
  }
  const __half *k_base = k_cache + (static_cast<size_t>(m) * kv_heads + kv) * max_seq * 128;
  const __half *v_base = v_cache + (static_cast<size_t>(m) * kv_heads + kv) * max_seq * 128;
  for (int p = begin + warp; p < end; p += kAttnWarps) {
    const uint2 kw = reinterpret_cast<const uint2 *>(k_base + static_cast<size_t>(p) * 128)[lane];
    const uint2 vw = reinterpret_cast<const uint2 *>(v_base + static_cast<size_t>(p) * 128)[lane];
    const float2 ka = __half22float2(*reinterpret_cast<const __half2 *>(&kw.x));
    const float2 kb = __half22float2(*reinterpret_cast<const __half2 *>(&kw.y));
    const float2 va = __half22float2(*reinterpret_cast<const __half2 *>(&vw.x));
    const float2 vb = __half22float2(*reinterpret_cast<const __half2 *>(&vw.y));
    for (int g = 0; g < group; ++g) {
      float dot = qa[g].x * ka.x + qa[g].y * ka.y + qb[g].x * kb.x + qb[g].y * kb.y;
      dot = warp_sum(dot) * scale;
      const float new_max = fmaxf(running_max[g], dot);
      const float rescale = __expf(running_max[g] - new_max);
      const float weight = __expf(dot - new_max);
      running_sum[g] = running_sum[g] * rescale + weight;
      acc[g][0] = acc[g][0] * rescale + weight * va.x;
      acc[g][1] = acc[g][1] * rescale + weight * va.y;
      acc[g][2] = acc[g][2] * rescale + weight * vb.x;
      acc[g][3] = acc[g][3] * rescale + weight * vb.y;
      running_max[g] = new_max;
    }
  }
  for (int g = 0; g < group; ++g) {
    if (lane == 0) {
      shared_max[warp][g] = running_max[g];
      shared_sum[warp][g] = running_sum[g];
    }
    for (int c = 0; c < 4; ++c) shared_acc[warp][g][4 * lane + c] = acc[g][c];
  }
  __syncthreads();
  // combine the warps: thread = (query head of the group, dim)
  for (int item = threadIdx.x; item < group * 128; item += blockDim.x) {
    const int g = item >> 7, dim = item & 127;
    float top = -INFINITY;
    for (int w = 0; w < kAttnWarps; ++w) top = fmaxf(top, shared_max[w][g]);
    float sum = 0.0f, value = 0.0f;
    for (int w = 0; w < kAttnWarps; ++w) {
      const float f = shared_max[w][g] == -INFINITY ? 0.0f : __expf(shared_max[w][g] - top);
      sum += shared_sum[w][g] * f;
      value += shared_acc[w][g][dim] * f;
    }
    // partial layout: [sequence][query head][split][130] = (max, sum, 128 values)
    float *out = partial + ((static_cast<size_t>(m) * q_heads + kv * group + g) * splits + split) * 130;
    if (dim == 0) {
      out[0] = top;
      out[1] = sum;
    }
    out[2 + dim] = value;
  }
}

// out[m][head][:] = sum over splits, softmax-normalised; one warp-quad (128 threads) per head.
__global__ void attention_combine_kernel(const float *__restrict__ partial, __half *__restrict__ out,
                                         int q_heads, int splits) {
  // programmatic dependent launch: let the next kernel be scheduled, then wait for the
  // previous one before touching memory
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();

  const int head = blockIdx.x, m = blockIdx.y, dim = threadIdx.x;
  const float *base = partial + (static_cast<size_t>(m) * q_heads + head) * splits * 130;
  float top = -INFINITY;
  for (int s = 0; s < splits; ++s) top = fmaxf(top, base[s * 130]);
  float sum = 0.0f, value = 0.0f;
  for (int s = 0; s < splits; ++s) {
    const float mx = base[s * 130];
    const float f = mx == -INFINITY ? 0.0f : __expf(mx - top);
    sum += base[s * 130 + 1] * f;
    value += base[s * 130 + 2 + dim] * f;
  }
  out[(static_cast<size_t>(m) * q_heads + head) * 128 + dim] = __float2half_rn(value / sum);
}

// The whole attention step of one new token per sequence in ONE launch: per-head RMSNorm +
// RoPE of q and of the new k, the new k/v written into the cache, attention over the context.
// A thread-block cluster of `splits` CTAs shares one (sequence, kv head, block of up to four
// query heads): CTA r attends to the r-th chunk of the context, leaves its (max, sum, weighted
// V) in its own shared memory, and after a cluster barrier every CTA combines a slice of the
// output dims by reading all CTAs' partials through distributed shared memory - no scratch in
// global memory, no second launch.  q/k arithmetic and the cache contents are those of
// qk_norm_rope_cache_kernel, bit for bit; the attention sums run in another order than
// attention_partial_kernel's (same FP32 math).
__device__ __forceinline__ void norm_rope_head(const __half *source, const __half *weight,
                                               const __half *cos_row, const __half *sin_row,
                                               float eps, int lane, __half2 &out_lo, __half2 &out_hi) {
  const __half2 lo = reinterpret_cast<const __half2 *>(source)[lane];
  const __half2 hi = reinterpret_cast<const __half2 *>(source + 64)[lane];
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

// kStepHeads query heads (of one kv head) per CTA: 4, 2 or 1.  kExact: the group size is a
// multiple of it, so no CTA has fewer (the guards disappear).  kPrompt: prompt rows (see below).
// The variants only remove code the launch cannot reach: this kernel's cost is mostly the
// fetch of instructions that run once.

__device__ __forceinline__ void unpack16(const uint4 &a, const uint4 &b, float out[16]) {
  const __half2 *ha = reinterpret_cast<const __half2 *>(&a);
  const __half2 *hb = reinterpret_cast<const __half2 *>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = __half22float2(ha[i]), fb = __half22float2(hb[i]);
    out[2 * i] = fa.x;
    out[2 * i + 1] = fa.y;
    out[8 + 2 * i] = fb.x;
    out[8 + 2 * i + 1] = fb.y;
  }
}

// (one or two heads per CTA: at most 128 registers, so that two CTAs fit an SM and the clusters of a
//  step always find room at once - with 142 the one-sequence step was measured 8 % slower)
template <int kStepHeads, bool kExact, bool kPrompt, bool kIndexed = false>
__global__ void __launch_bounds__(kAttnWarps * 32, kStepHeads <= 2 ? 2 : 0)
    attention_step_kernel(const __half *__restrict__ q, const __half *__restrict__ k,
                          const __half *__restrict__ v, const __half *__restrict__ q_weight,
                          const __half *__restrict__ k_weight, const __half *__restrict__ cos_table,
                          const __half *__restrict__ sin_table, const int *__restrict__ positions,
                          __half *k_cache, __half *v_cache, __half *__restrict__ out, int q_heads,
                          int kv_heads, int max_seq, float eps, float scale, int rows_per_sequence,
                          const int *__restrict__ out_index) {
  sageb200::pdl_launch_dependents();
  // Prompt rows read a cache the previous kernel filled: wait at once.  A decode step waits
  // further down, after it has requested its first cache rows (written by earlier steps).
  if (kPrompt) sageb200::pdl_wait();

  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ float warp_max[kAttnWarps][kStepHeads];
  __shared__ float warp_total[kAttnWarps][kStepHeads];
  __shared__ __align__(16) float warp_acc[kAttnWarps][kStepHeads][128];
  __shared__ float cta_max[kStepHeads], cta_total[kStepHeads];
  __shared__ __align__(16) float cta_acc[kStepHeads][128];
  __shared__ __align__(16) __half q_shared[kStepHeads][128];
  __shared__ __align__(16) __half new_k[128], new_v[128];
  const int splits = gridDim.x, split = blockIdx.x, m = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = q_heads / kv_heads;
  const int parts = (group + kStepHeads - 1) / kStepHeads;
  const int kv = blockIdx.y / parts, part = blockIdx.y - kv * parts;
  const int heads = kExact ? kStepHeads : min(kStepHeads, group - part * kStepHeads);
  const int first_head = kv * group + part * kStepHeads;
  // rows_per_sequence == 0: a decode step (row = sequence; q and the new k are normalised and
  // rotated here and the new k/v appended).  > 0: prompt rows - that many consecutive rows are
  // the tokens of one sequence at positions[sequence] + token, q is already normalised and
  // rotated and the cache already holds every token's k/v.
  constexpr bool prompt = kPrompt;
  const int sequence = prompt ? m / rows_per_sequence : m;
  const int position = positions[sequence] + (prompt ? m - sequence * rows_per_sequence : 0);
  const bool in_range = !prompt && position >= 0 && position < max_seq;  // a full cache takes no new token
  const int table_row = min(max(position, 0), max_seq - 1);
  const int context = min(position + 1, max_seq);
  const int chunk = (context + splits - 1) / splits;
  const int begin = split * chunk;
  const int end = min(context, begin + chunk);
  const bool owns_new = in_range && begin <= position && position < end;
  const __half *cos_row = cos_table + static_cast<size_t>(table_row) * 64;
  const __half *sin_row = sin_table + static_cast<size_t>(table_row) * 64;
  __half *k_base = k_cache + (static_cast<size_t>(sequence) * kv_heads + kv) * max_seq * 128;
  __half *v_base = v_cache + (static_cast<size_t>(sequence) * kv_heads + kv) * max_seq * 128;

  // A warp takes four consecutive positions at a time: lanes 8s..8s+7 share position s and hold
  // 16 dims each (dims 16*piece .. 16*piece+15), so a dot product needs three shuffles.
  const int sub = lane >> 3, piece = lane & 7;
  // Decode step: the warp's first four cache rows are requested now, before the wait for the
  // kernel that produced q, k and v - earlier steps wrote them (the position being appended is
  // patched in from shared memory below) - so their trip to memory overlaps the producer's tail.
  uint4 k0, k1, v0, v1;
  k0 = k1 = v0 = v1 = make_uint4(0, 0, 0, 0);
  // (the same for the output index of this thread's first output value: a constant of the model)
  [[maybe_unused]] int first_target = 0;
  if constexpr (kIndexed) {
    const int items_all = heads * 128;
    const int item = split * ((items_all + splits - 1) / splits) + static_cast<int>(threadIdx.x);
    if (item < items_all) first_target = __ldg(out_index + (first_head + (item >> 7)) * 128 + (item & 127));
  }
  if (!kPrompt) {
    const int p = begin + warp * 4 + sub;
    if (p < end) {
      const uint4 *k_row = reinterpret_cast<const uint4 *>(k_base + static_cast<size_t>(p) * 128);
      const uint4 *v_row = reinterpret_cast<const uint4 *>(v_base + static_cast<size_t>(p) * 128);
      k0 = k_row[2 * piece];
      k1 = k_row[2 * piece + 1];
      v0 = v_row[2 * piece];
      v1 = v_row[2 * piece + 1];
    }
    sageb200::pdl_wait();
  }

  // items 0..heads-1: this CTA's query heads; item `heads`: the new token's key and value
  // (every part needs them, part 0 stores them)
  for (int item = warp; item < heads + (owns_new ? 1 : 0); item += kAttnWarps) {
    __half2 lo, hi;
    if (item < heads) {
      const __half *source = q + (static_cast<size_t>(m) * q_heads + first_head + item) * 128;
      if (prompt) {
        lo = reinterpret_cast<const __half2 *>(source)[lane];
        hi = reinterpret_cast<const __half2 *>(source + 64)[lane];
      } else {
        norm_rope_head(source, q_weight, cos_row, sin_row, eps, lane, lo, hi);
      }
      reinterpret_cast<__half2 *>(q_shared[item])[lane] = lo;
      reinterpret_cast<__half2 *>(q_shared[item] + 64)[lane] = hi;
    } else {
      norm_rope_head(k + (static_cast<size_t>(m) * kv_heads + kv) * 128, k_weight, cos_row, sin_row, eps,
                     lane, lo, hi);
      reinterpret_cast<__half2 *>(new_k)[lane] = lo;
      reinterpret_cast<__half2 *>(new_k + 64)[lane] = hi;
      const uint2 value = reinterpret_cast<const uint2 *>(v + (static_cast<size_t>(m) * kv_heads + kv) * 128)[lane];
      reinterpret_cast<uint2 *>(new_v)[lane] = value;
      if (part == 0) {
        reinterpret_cast<__half2 *>(k_base + static_cast<size_t>(position) * 128)[lane] = lo;
        reinterpret_cast<__half2 *>(k_base + static_cast<size_t>(position) * 128 + 64)[lane] = hi;
        reinterpret_cast<uint2 *>(v_base + static_cast<size_t>(position) * 128)[lane] = value;
      }
    }
  }
  __syncthreads();

  float qf[kStepHeads][16];
#pragma unroll
  for (int g = 0; g < kStepHeads; ++g) {
    const uint4 *source = reinterpret_cast<const uint4 *>(q_shared[g < heads ? g : 0] + 16 * piece);
    unpack16(source[0], source[1], qf[g]);
  }
  float running_max[kStepHeads], running_sum[kStepHeads], acc[kStepHeads][16];
#pragma unroll
  for (int g = 0; g < kStepHeads; ++g) {
    running_max[g] = -INFINITY;
    running_sum[g] = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[g][i] = 0.0f;
  }
  // the rows of the next four positions are requested before the current ones are used
  auto fetch = [&](int base, uint4 &k0, uint4 &k1, uint4 &v0, uint4 &v1) {
    const int p = base + sub;
    k0 = k1 = v0 = v1 = make_uint4(0, 0, 0, 0);
    if (p < end) {
      const bool fresh = owns_new && p == position;
      const uint4 *k_row = fresh ? reinterpret_cast<const uint4 *>(new_k)
                                 : reinterpret_cast<const uint4 *>(k_base + static_cast<size_t>(p) * 128);
      const uint4 *v_row = fresh ? reinterpret_cast<const uint4 *>(new_v)
                                 : reinterpret_cast<const uint4 *>(v_base + static_cast<size_t>(p) * 128);
      k0 = k_row[2 * piece];
      k1 = k_row[2 * piece + 1];
      v0 = v_row[2 * piece];
      v1 = v_row[2 * piece + 1];
    }
  };
  uint4 next_k0, next_k1, next_v0, next_v1;
  if (kPrompt || (owns_new && begin + warp * 4 + sub == position))
    fetch(begin + warp * 4, k0, k1, v0, v1);  // (decode: only the appended position, from shared memory)
  for (int base = begin + warp * 4; base < end; base += kAttnWarps * 4) {
    fetch(base + kAttnWarps * 4, next_k0, next_k1, next_v0, next_v1);
    const bool valid = base + sub < end;
    float kf[16], vf[16];
    unpack16(k0, k1, kf);
    unpack16(v0, v1, vf);
#pragma unroll
    for (int g = 0; g < kStepHeads; ++g) {
      if (!kExact && g >= heads) break;
      float dot = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) dot = fmaf(qf[g][i], kf[i], dot);
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      dot += __shfl_xor_sync(0xffffffffu, dot, 4);
      if (valid) {
        dot *= scale;
        const float new_max = fmaxf(running_max[g], dot);
        const float rescale = __expf(running_max[g] - new_max);
        const float weight = __expf(dot - new_max);
        running_sum[g] = running_sum[g] * rescale + weight;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[g][i] = fmaf(weight, vf[i], acc[g][i] * rescale);
        running_max[g] = new_max;
      }
    }
    k0 = next_k0;
    k1 = next_k1;
    v0 = next_v0;
    v1 = next_v1;
  }
  // merge the warp's four position streams, then the warps, then (across the cluster) the splits
#pragma unroll
  for (int g = 0; g < kStepHeads; ++g) {
    if (!kExact && g >= heads) break;
    float top = fmaxf(running_max[g], __shfl_xor_sync(0xffffffffu, running_max[g], 8));
    top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, 16));
    const float f = running_max[g] == -INFINITY ? 0.0f : __expf(running_max[g] - top);
    float total = running_sum[g] * f;
    total += __shfl_xor_sync(0xffffffffu, total, 8);
    total += __shfl_xor_sync(0xffffffffu, total, 16);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float value = acc[g][i] * f;
      value += __shfl_xor_sync(0xffffffffu, value, 8);
      value += __shfl_xor_sync(0xffffffffu, value, 16);
      acc[g][i] = value;
    }
    if (lane == 0) {
      warp_max[warp][g] = top;
      warp_total[warp][g] = total;
    }
    if (sub == 0) {
#pragma unroll
      for (int i = 0; i < 16; i += 4)
        *reinterpret_cast<float4 *>(&warp_acc[warp][g][16 * piece + i]) =
            make_float4(acc[g][i], acc[g][i + 1], acc[g][i + 2], acc[g][i + 3]);
    }
  }
  __syncthreads();
  for (int item = threadIdx.x; item < heads * 128; item += blockDim.x) {
    const int g = item >> 7, dim = item & 127;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) top = fmaxf(top, warp_max[w][g]);
    float total = 0.0f, value = 0.0f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float f = warp_max[w][g] == -INFINITY ? 0.0f : __expf(warp_max[w][g] - top);
      total += warp_total[w][g] * f;
      value += warp_acc[w][g][dim] * f;
    }
    if (dim == 0) {
      cta_max[g] = top;
      cta_total[g] = total;
    }
    cta_acc[g][dim] = value;
  }
  cluster.sync();  // every CTA's partial is in its shared memory
  const int items = heads * 128;
  const int per_cta = (items + splits - 1) / splits;
  for (int local = threadIdx.x; local < per_cta; local += blockDim.x) {
    const int item = split * per_cta + local;
    if (item >= items) break;
    const int g = item >> 7, dim = item & 127;
    float top = -INFINITY;
    for (int s = 0; s < splits; ++s) top = fmaxf(top, *cluster.map_shared_rank(&cta_max[g], s));
    float total = 0.0f, value = 0.0f;
    for (int s = 0; s < splits; ++s) {
      const float mx = *cluster.map_shared_rank(&cta_max[g], s);
      const float f = mx == -INFINITY ? 0.0f : __expf(mx - top);
      total += *cluster.map_shared_rank(&cta_total[g], s) * f;
      value += *cluster.map_shared_rank(&cta_acc[g][dim], s) * f;
    }
    // kIndexed: out_index says where each channel of a row goes - the consumer's quantised channel
    // order, so the packed linear behind this kernel needs no gather of its own (a variant of its
    // own: the plain kernel keeps its registers and instruction stream)
    if constexpr (kIndexed) {
      const int target = local == static_cast<int>(threadIdx.x) ? first_target
                                                                 : __ldg(out_index + (first_head + g) * 128 + dim);
      out[static_cast<size_t>(m) * q_heads * 128 + target] = __float2half_rn(value / total);
    } else {
      out[(static_cast<size_t>(m) * q_heads + first_head + g) * 128 + dim] = __float2half_rn(value / total);
    }
  }
  cluster.sync();  // nobody leaves while its shared memory may still be read
}

// act = silu(gate) * up, FP32 math on FP16 inputs, rounded as the FP16 modules round:
// silu(gate) to FP16, then the FP16 product.
__global__ void swiglu_kernel(const __half *__restrict__ gate, const __half *__restrict__ up,
                              __half *__restrict__ act, long long count) {
  // programmatic dependent launch: let the next kernel be scheduled, then wait for the
  // previous one before touching memory
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();

  // eight elements per thread (16-byte loads and stores) when the three arrays allow it
  const bool wide = ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) |
                      reinterpret_cast<uintptr_t>(act)) & 15) == 0;
  const long long first = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
  if (first >= count) return;
  if (wide && first + 8 <= count) {
    const uint4 g4 = *reinterpret_cast<const uint4 *>(gate + first);
    const uint4 u4 = *reinterpret_cast<const uint4 *>(up + first);
    uint4 out;
    const __half2 *g2 = reinterpret_cast<const __half2 *>(&g4);
    const __half2 *u2 = reinterpret_cast<const __half2 *>(&u4);
    __half2 *o2 = reinterpret_cast<__half2 *>(&out);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 g = __half22float2(g2[q]);
      const __half2 silu = __halves2half2(__float2half_rn(sageb200::silu_fast(g.x)),
                                          __float2half_rn(sageb200::silu_fast(g.y)));
      o2[q] = __hmul2(silu, u2[q]);
    }
    *reinterpret_cast<uint4 *>(act + first) = out;
    return;
  }
  for (long long i = first; i < count && i < first + 8; ++i) {
    const float g = __half2float(gate[i]);
    const __half silu = __float2half_rn(sageb200::silu_fast(g));
    act[i] = __hmul(silu, up[i]);
  }
}

// ---- logits of 2..16 sequences on the tensor cores.  mma.sync.m16n8k16 with 16 vocabulary rows as
// the A operand and 8 sequences as the B operand per column block.  K runs in blocks of 32 in a
// permuted order (slot 2t+e of step j <-> channel 8t+4j+e, slot 2t+8+e <-> channel 8t+4j+2+e), the
// same for both operands, so that a lane's fragments of both steps are ONE 16-byte load: 16
// contiguous bytes of a head row from global memory, and 16 bytes of a sequence's row from the
// blocked shared copy xs[k block][column block][8 sequences][32 channels] (a quarter warp reads 128
// contiguous bytes: no bank conflicts).  HBM-bound on the head matrix for any row count.
__device__ __forceinline__ int head_x_index(int m, int i, int column_blocks) {
  return (((i >> 5) * column_blocks + (m >> 3)) * 8 + (m & 7)) * 32 + (i & 31);
}
__device__ __forceinline__ void head_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// acc[nb][e]: vocabulary row v0 + g + 8 * (e >> 1), sequence nb * 8 + 2 * t + (e & 1)
template <int kColumnBlocks>
__device__ __forceinline__ void head_rows_mma(const __half *__restrict__ head, const __half *xs, int v0, int vocab,
                                              int hidden, int lane, float (&acc)[kColumnBlocks][4]) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nb = 0; nb < kColumnBlocks; ++nb) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.0f;
  const uint4 *row0 = reinterpret_cast<const uint4 *>(head + static_cast<size_t>(min(v0 + g, vocab - 1)) * hidden) + t;
  const uint4 *row1 = reinterpret_cast<const uint4 *>(head + static_cast<size_t>(min(v0 + g + 8, vocab - 1)) * hidden) + t;
  const uint4 *x_lane = reinterpret_cast<const uint4 *>(xs) + g * 4 + t;  // + (kb * blocks + nb) * 32
  const int blocks = hidden >> 5;
  for (int first = 0; first < blocks; first += 4) {  // eight 16-byte loads in flight per lane
    uint4 w0[4], w1[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (first + u < blocks) {
        w0[u] = sageb200::ldg_stream_u4(row0 + (first + u) * 4);
        w1[u] = sageb200::ldg_stream_u4(row1 + (first + u) * 4);
      }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (first + u >= blocks) break;
#pragma unroll
      for (int nb = 0; nb < kColumnBlocks; ++nb) {
        const uint4 xb = x_lane[((first + u) * kColumnBlocks + nb) * 32];
        head_mma(acc[nb], w0[u].x, w1[u].x, w0[u].y, w1[u].y, xb.x, xb.y);
        head_mma(acc[nb], w0[u].z, w1[u].z, w0[u].w, w1[u].w, xb.z, xb.w);
      }
    }
  }
}

// logits[m][v] = dot(head[v][:], x[m][:]) in FP32, rounded to FP16.  One warp per vocabulary
// row; the (up to 16) activation rows sit in shared memory.  HBM-bound on the head matrix.
constexpr int kHeadWarps = 8;

__global__ void __launch_bounds__(kHeadWarps * 32)
    lm_head_kernel(const __half *__restrict__ head, const __half *__restrict__ x,
                   __half *__restrict__ logits, int vocab, int hidden, int rows) {
  // programmatic dependent launch: let the next kernel be scheduled, then wait for the
  // previous one before touching memory
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();

  extern __shared__ __half x_shared[];
  const int lane = threadIdx.x & 31;
  if (rows > 1 && (hidden & 31) == 0) {
    // several sequences: blocked copy of the rows, then 16 vocabulary rows per warp and step
    const int column_blocks = rows > 8 ? 2 : 1;
    for (int e = threadIdx.x; e < column_blocks * 8 * hidden; e += blockDim.x) {
      const int m = e / hidden, i = e - m * hidden;
      x_shared[head_x_index(m, i, column_blocks)] = m < rows ? x[static_cast<size_t>(m) * hidden + i] : __float2half_rn(0.0f);
    }
    __syncthreads();
    const int g = lane >> 2, t = lane & 3;
    for (int v0 = (blockIdx.x * kHeadWarps + (threadIdx.x >> 5)) * 16; v0 < vocab; v0 += gridDim.x * kHeadWarps * 16) {
      float acc[2][4];
      if (column_blocks == 2) {
        head_rows_mma<2>(head, x_shared, v0, vocab, hidden, lane, acc);
      } else {
        float one[1][4];
        head_rows_mma<1>(head, x_shared, v0, vocab, hidden, lane, one);
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[0][e] = one[0][e];
      }
      for (int nb = 0; nb < column_blocks; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int v = v0 + g + 8 * (e >> 1), m = nb * 8 + 2 * t + (e & 1);
          if (v < vocab && m < rows) logits[static_cast<size_t>(m) * vocab + v] = __float2half_rn(acc[nb][e]);
        }
    }
    return;
  }
  for (int i = threadIdx.x; i < rows * hidden / 8; i += blockDim.x)
    reinterpret_cast<uint4 *>(x_shared)[i] = reinterpret_cast<const uint4 *>(x)[i];
  __syncthreads();
  const int pieces = hidden / 8;
  for (int v = blockIdx.x * kHeadWarps + (threadIdx.x >> 5); v < vocab; v += gridDim.x * kHeadWarps) {
    const uint4 *row = reinterpret_cast<const uint4 *>(head + static_cast<size_t>(v) * hidden);
    float sums[16];
    for (int m = 0; m < rows; ++m) sums[m] = 0.0f;
    for (int i = lane; i < pieces; i += 32) {
      uint4 w;
      asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                   : "l"(row + i));
      const __half2 *wh = reinterpret_cast<const __half2 *>(&w);
      for (int m = 0; m < rows; ++m) {
        const uint4 a = reinterpret_cast<const uint4 *>(x_shared + static_cast<size_t>(m) * hidden)[i];
        const __half2 *ah = reinterpret_cast<const __half2 *>(&a);
        float s = sums[m];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float2 wf = __half22float2(wh[c]), af = __half22float2(ah[c]);
          s = fmaf(wf.x, af.x, s);
          s = fmaf(wf.y, af.y, s);
        }
        sums[m] = s;
      }
    }
    for (int m = 0; m < rows; ++m) {
      const float total = warp_sum(sums[m]);
      if (lane == 0) logits[static_cast<size_t>(m) * vocab + v] = __float2half_rn(total);
    }
  }
}

// The tail of a decode step in ONE launch: final residual add + RMSNorm (recomputed by every
// CTA, same arithmetic and summation order as add_rmsnorm_kernel), the lm_head rows of this
// CTA, and the greedy argmax: every CTA leaves its best (value, index) per sequence in
// `block_best`, and the last CTA to arrive (a counter, zero before and after the launch) picks
// the overall best (lowest index on ties), appends it to the log and advances positions and
// the step counter.  The residual stream itself is left as it was.
__device__ __forceinline__ bool better(float value, int index, float than_value, int than_index) {
  return value > than_value || (value == than_value && index < than_index);
}

// kRows bounds `rows` (1, 8 or 16): one sequence runs the FP32 dot products below, several run the
// tensor-core path with one (8) or two (16) column blocks.
template <int kRows>
__global__ void __launch_bounds__(kHeadWarps * 32)
    lm_head_step_kernel(const __half *__restrict__ head, const __half *__restrict__ residual,
                        const __half *__restrict__ delta, const __half *__restrict__ norm_weight,
                        __half *__restrict__ x_out, __half *__restrict__ logits,
                        long long *__restrict__ tokens, int *__restrict__ positions,
                        long long *__restrict__ log, int *__restrict__ step, float2 *block_best,
                        unsigned *counter, int vocab, int hidden, int rows, float eps, int log_stride) {
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();

  extern __shared__ __half x_shared[];
  __shared__ float scratch[32];
  __shared__ float best_value[kHeadWarps][16];
  __shared__ int best_index[kHeadWarps][16];
  __shared__ int is_last;
  static_assert(kHeadWarps * 32 == kNormThreads, "the norm must sum in add_rmsnorm_kernel's order");
  // several sequences: the rows live in the blocked layout of head_rows_mma (same arithmetic and
  // summation order of the norm either way)
  constexpr int kColumnBlocks = kRows > 8 ? 2 : 1;
  const bool blocked = kRows > 1 && (hidden & 31) == 0;
  auto at = [&](int m, int i) { return blocked ? head_x_index(m, i, kColumnBlocks) : m * hidden + i; };
  if (blocked)
    for (int e = rows * hidden + threadIdx.x; e < kColumnBlocks * 8 * hidden; e += kNormThreads)
      x_shared[head_x_index(e / hidden, e % hidden, kColumnBlocks)] = __float2half_rn(0.0f);  // unused sequences
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool wide = ((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(delta) |
                      reinterpret_cast<uintptr_t>(norm_weight) | reinterpret_cast<uintptr_t>(x_out)) & 15) == 0;
  if (kRows > 1 && blocked && wide) {
    // Several sequences: all rows at once instead of one row after the other (every CTA does this,
    // so a serial pass per row - a trip to L2, two barriers - times the rows sat in front of the
    // whole head).  1. residual + delta of every row with 16-byte loads, none depending on another;
    // 2. each row's squares summed by thread and element exactly as the scalar loop does, out of
    // shared memory, and the block sums in block_sum's order; 3. scaling and weights, eight values
    // at a time.  Bit-identical to the loop below.
    __shared__ float row_sums[kRows][kHeadWarps];
    __shared__ float row_scale[kRows];
    const int vectors = hidden >> 3;
    const int total_vectors = rows * vectors;
    const uint4 *residual4 = reinterpret_cast<const uint4 *>(residual);
    const uint4 *delta4 = reinterpret_cast<const uint4 *>(delta);
    for (int base = 0; base < total_vectors; base += 4 * kNormThreads) {
      uint4 rv[4], dv[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = base + threadIdx.x + u * kNormThreads;
        if (e < total_vectors) {
          rv[u] = residual4[e];
          if (delta4) dv[u] = delta4[e];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int e = base + threadIdx.x + u * kNormThreads;
        if (e >= total_vectors) break;
        if (delta4) {
          __half2 *a = reinterpret_cast<__half2 *>(&rv[u]);
          const __half2 *b = reinterpret_cast<const __half2 *>(&dv[u]);
#pragma unroll
          for (int c = 0; c < 4; ++c) a[c] = __hadd2(a[c], b[c]);
        }
        const int m = e / vectors;
        *reinterpret_cast<uint4 *>(x_shared + at(m, (e - m * vectors) * 8)) = rv[u];
      }
    }
    __syncthreads();
    float square[kRows];
#pragma unroll
    for (int m = 0; m < kRows; ++m) {
      square[m] = 0.0f;
      if (m < rows) {
        for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
          const float f = __half2float(x_shared[at(m, i)]);
          square[m] += f * f;
        }
        square[m] = warp_sum(square[m]);
        if (lane == 0) row_sums[m][warp] = square[m];
      }
    }
    __syncthreads();
    if (threadIdx.x < rows) {
      float total = 0.0f;
      for (int w = 0; w < kHeadWarps; ++w) total += row_sums[threadIdx.x][w];
      row_scale[threadIdx.x] = rsqrtf(total / hidden + eps);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < total_vectors; e += kNormThreads) {
      const int m = e / vectors, i = (e - m * vectors) * 8;
      const float scale = row_scale[m];
      uint4 value = *reinterpret_cast<const uint4 *>(x_shared + at(m, i));
      const uint4 weight4 = *reinterpret_cast<const uint4 *>(norm_weight + i);
      __half *v = reinterpret_cast<__half *>(&value);
      const __half *w = reinterpret_cast<const __half *>(&weight4);
#pragma unroll
      for (int c = 0; c < 8; ++c) v[c] = __hmul(w[c], __float2half_rn(__half2float(v[c]) * scale));
      *reinterpret_cast<uint4 *>(x_shared + at(m, i)) = value;
      if (blockIdx.x == 0) *reinterpret_cast<uint4 *>(x_out + static_cast<size_t>(m) * hidden + i) = value;
    }
  } else {
    for (int m = 0; m < rows; ++m) {
      const __half *r = residual + static_cast<size_t>(m) * hidden;
      const __half *d = delta ? delta + static_cast<size_t>(m) * hidden : nullptr;
      float square = 0.0f;
      for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
        __half v = r[i];
        if (d) v = __hadd(v, d[i]);
        x_shared[at(m, i)] = v;
        const float f = __half2float(v);
        square += f * f;
      }
      const float total = block_sum(square, scratch);
      const float scale = rsqrtf(total / hidden + eps);
      for (int i = threadIdx.x; i < hidden; i += kNormThreads) {
        const __half normed = __float2half_rn(__half2float(x_shared[at(m, i)]) * scale);
        const __half value = __hmul(norm_weight[i], normed);
        x_shared[at(m, i)] = value;
        if (blockIdx.x == 0) x_out[static_cast<size_t>(m) * hidden + i] = value;
      }
    }
  }
  __syncthreads();
  if (blocked) {
    // ---- tensor-core path: 16 vocabulary rows per warp and step, best (value, index) per sequence
    const int g = lane >> 2, t = lane & 3;
    float slot_value[kColumnBlocks * 2];
    int slot_index[kColumnBlocks * 2];
#pragma unroll
    for (int q = 0; q < kColumnBlocks * 2; ++q) {
      slot_value[q] = -INFINITY;
      slot_index[q] = 0x7fffffff;
    }
    // The warps take 16-row tiles of the vocabulary in turn off a ticket counter (the word behind
    // the arrival counter; the last CTA zeroes both): the grid is one resident wave, and a static
    // split of ~2.7 tiles per warp would leave a third of the warps idle for the last pass.  The
    // next ticket is requested before the current tile is computed.  Which warp computes a tile
    // changes nothing in the logits, and the argmax does not depend on the order (lowest index on
    // ties).
    const int tiles = (vocab + 15) / 16;
    unsigned ticket = lane == 0 ? atomicAdd(counter + 1, 1u) : 0u;
    for (;;) {
      const int tile = static_cast<int>(__shfl_sync(0xffffffffu, ticket, 0));
      if (tile >= tiles) break;
      if (lane == 0) ticket = atomicAdd(counter + 1, 1u);
      const int v0 = tile * 16;
      float acc[kColumnBlocks][4];
      head_rows_mma<kColumnBlocks>(head, x_shared, v0, vocab, hidden, lane, acc);
#pragma unroll
      for (int nb = 0; nb < kColumnBlocks; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {  // (e = 0, 1: row v0 + g; e = 2, 3: row v0 + g + 8)
          const int v = v0 + g + 8 * (e >> 1), m = nb * 8 + 2 * t + (e & 1);
          if (v < vocab && m < rows) {
            const __half rounded = __float2half_rn(acc[nb][e]);
            logits[static_cast<size_t>(m) * vocab + v] = rounded;
            const float f = __half2float(rounded);
            const int q = nb * 2 + (e & 1);
            if (better(f, v, slot_value[q], slot_index[q])) {
              slot_value[q] = f;
              slot_index[q] = v;
            }
          }
        }
    }
    // the eight lanes that share t hold the same sequences: best over them, then lanes 0..3 publish
#pragma unroll
    for (int q = 0; q < kColumnBlocks * 2; ++q) {
      for (int o = 4; o < 32; o <<= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, slot_value[q], o);
        const int other_index = __shfl_xor_sync(0xffffffffu, slot_index[q], o);
        if (better(other, other_index, slot_value[q], slot_index[q])) {
          slot_value[q] = other;
          slot_index[q] = other_index;
        }
      }
      const int m = (q >> 1) * 8 + 2 * t + (q & 1);
      if (g == 0 && m < rows) {
        best_value[warp][m] = slot_value[q];
        best_index[warp][m] = slot_index[q];
      }
    }
  } else {
  const int pieces = hidden / 8;
  float top_value[kRows];
  int top_index[kRows];
#pragma unroll
  for (int m = 0; m < kRows; ++m) {
    top_value[m] = -INFINITY;
    top_index[m] = 0x7fffffff;
  }
  for (int v = blockIdx.x * kHeadWarps + warp; v < vocab; v += gridDim.x * kHeadWarps) {
    const uint4 *row = reinterpret_cast<const uint4 *>(head + static_cast<size_t>(v) * hidden);
    float sums[kRows];
#pragma unroll
    for (int m = 0; m < kRows; ++m) sums[m] = 0.0f;
    for (int first = lane; first < pieces; first += 128) {  // four 16-byte loads in flight per lane
      uint4 w4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (first + 32 * j < pieces) w4[j] = sageb200::ldg_stream_u4(row + first + 32 * j);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = first + 32 * j;
        if (i >= pieces) break;
        const __half2 *wh = reinterpret_cast<const __half2 *>(&w4[j]);
#pragma unroll
        for (int m = 0; m < kRows; ++m) {
          if (m >= rows) break;
          const uint4 a = reinterpret_cast<const uint4 *>(x_shared + static_cast<size_t>(m) * hidden)[i];
          const __half2 *ah = reinterpret_cast<const __half2 *>(&a);
          float s = sums[m];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float2 wf = __half22float2(wh[c]), af = __half22float2(ah[c]);
            s = fmaf(wf.x, af.x, s);
            s = fmaf(wf.y, af.y, s);
          }
          sums[m] = s;
        }
      }
    }
#pragma unroll
    for (int m = 0; m < kRows; ++m) {
      if (m < rows) {
        const __half rounded = __float2half_rn(warp_sum(sums[m]));
        if (lane == 0) logits[static_cast<size_t>(m) * vocab + v] = rounded;
        const float f = __half2float(rounded);
        if (better(f, v, top_value[m], top_index[m])) {
          top_value[m] = f;
          top_index[m] = v;
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < kRows; ++m)
    if (m < rows && lane == 0) {
      best_value[warp][m] = top_value[m];
      best_index[warp][m] = top_index[m];
    }
  }  // (scalar path)
  __syncthreads();
  if (threadIdx.x < rows) {
    const int m = threadIdx.x;
    float value = best_value[0][m];
    int index = best_index[0][m];
    for (int w = 1; w < kHeadWarps; ++w)
      if (better(best_value[w][m], best_index[w][m], value, index)) {
        value = best_value[w][m];
        index = best_index[w][m];
      }
    block_best[static_cast<size_t>(blockIdx.x) * rows + m] = make_float2(value, __int_as_float(index));
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(counter, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int m = 0; m < rows; ++m) {
    float value = -INFINITY;
    int index = 0x7fffffff;
    for (int b = threadIdx.x; b < static_cast<int>(gridDim.x); b += blockDim.x) {
      const float2 candidate = __ldcg(block_best + static_cast<size_t>(b) * rows + m);
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
    __syncthreads();
    if (lane == 0) {
      best_value[warp][0] = value;
      best_index[warp][0] = index;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < kHeadWarps; ++w)
        if (better(best_value[w][0], best_index[w][0], value, index)) {
          value = best_value[w][0];
          index = best_index[w][0];
        }
      if (index == 0x7fffffff) index = 0;  // a row without a single ordered value (all NaN)
      tokens[m] = index;
      if (log && step && step[0] < log_stride) log[static_cast<size_t>(m) * log_stride + step[0]] = index;
      positions[m] += 1;
    }
  }
  if (threadIdx.x == 0) {
    if (step) step[0] += 1;
    counter[0] = 0u;  // zero again for the next launch: arrivals and tile tickets
    counter[1] = 0u;
  }
}

// Mixture-of-experts routing for one token per CTA, in one launch: residual add + RMSNorm (the
// arithmetic and summation order of add_rmsnorm_kernel, run by the CTA's first 256 threads),
// the FP16 router (logit = fp16(FP32 dot), one warp per four experts at a time), softmax over
// all experts, top-k (lowest index on ties) and renormalised weights - Qwen3-MoE's routing.
constexpr int kRouteThreads = 1024;
constexpr int kMaxExperts = 256;

__global__ void __launch_bounds__(kRouteThreads)
    moe_route_kernel(__half *__restrict__ residual, const __half *__restrict__ delta,
                     const __half *__restrict__ norm_weight, const __half *__restrict__ router,
                     __half *__restrict__ x, int *__restrict__ ids, float *__restrict__ weights, int hidden,
                     int experts, int top_k, float eps) {
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();

  extern __shared__ __half row_shared[];
  __shared__ float scratch[32];
  __shared__ float logits[kMaxExperts];
  const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __half *r = residual + static_cast<size_t>(m) * hidden;
  const __half *d = delta ? delta + static_cast<size_t>(m) * hidden : nullptr;
  float square = 0.0f;
  if (tid < kNormThreads) {
    for (int i = tid; i < hidden; i += kNormThreads) {
      __half v = r[i];
      if (d) {
        v = __hadd(v, d[i]);
        r[i] = v;
      }
      row_shared[i] = v;
      const float f = __half2float(v);
      square += f * f;
    }
    square = warp_sum(square);
    if (lane == 0) scratch[warp] = square;
  }
  __syncthreads();
  float total = 0.0f;
  for (int w = 0; w < kNormThreads / 32; ++w) total += scratch[w];
  const float scale = rsqrtf(total / hidden + eps);
  __syncthreads();
  for (int i = tid; i < hidden; i += kRouteThreads) {
    const __half normed = __float2half_rn(__half2float(row_shared[i]) * scale);
    const __half value = __hmul(norm_weight[i], normed);
    row_shared[i] = value;
    x[static_cast<size_t>(m) * hidden + i] = value;
  }
  __syncthreads();
  const int pieces = hidden / 8;
  for (int e = warp; e < experts; e += kRouteThreads / 32) {
    const uint4 *row = reinterpret_cast<const uint4 *>(router + static_cast<size_t>(e) * hidden);
    float sum = 0.0f;
    for (int i = lane; i < pieces; i += 32) {
      const uint4 w = __ldg(row + i);
      const uint4 a = reinterpret_cast<const uint4 *>(row_shared)[i];
      const __half2 *wh = reinterpret_cast<const __half2 *>(&w);
      const __half2 *ah = reinterpret_cast<const __half2 *>(&a);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float2 wf = __half22float2(wh[c]), af = __half22float2(ah[c]);
        sum = fmaf(wf.x, af.x, sum);
        sum = fmaf(wf.y, af.y, sum);
      }
    }
    sum = warp_sum(sum);
    if (lane == 0) logits[e] = __half2float(__float2half_rn(sum));
  }
  __syncthreads();
  if (warp != 0) return;
  // warp 0: lane holds experts lane, lane + 32, ...
  constexpr int kPerLane = kMaxExperts / 32;
  float mine[kPerLane];
  float top = -INFINITY;
#pragma unroll
  for (int j = 0; j < kPerLane; ++j) {
    const int e = lane + 32 * j;
    mine[j] = e < experts ? logits[e] : -INFINITY;
    top = fmaxf(top, mine[j]);
  }
  top = warp_max(top);
  float chosen_sum = 0.0f;
  float chosen_weight = 0.0f;  // lane s keeps the s-th choice
  int chosen_id = 0;
  for (int s = 0; s < top_k; ++s) {
    float best = -INFINITY;
    int best_id = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < kPerLane; ++j) {
      const int e = lane + 32 * j;
      if (mine[j] > best || (mine[j] == best && e < best_id && mine[j] != -INFINITY)) {
        best = mine[j];
        best_id = e;
      }
    }
    for (int o = 16; o; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_id = __shfl_xor_sync(0xffffffffu, best_id, o);
      if (other > best || (other == best && other_id < best_id)) {
        best = other;
        best_id = other_id;
      }
    }
    const float weight = __expf(best - top);
    chosen_sum += weight;
    if (lane == (s & 31)) {
      chosen_weight = weight;
      chosen_id = best_id;
    }
#pragma unroll
    for (int j = 0; j < kPerLane; ++j)
      if (lane + 32 * j == best_id) mine[j] = -INFINITY;
  }
  if (lane < top_k) {
    ids[m * top_k + lane] = chosen_id;
    weights[m * top_k + lane] = chosen_weight / chosen_sum;
  }
}

// out[m][:] = fp16(sum over the token's slots of weight * expert output), FP32 sum in slot order.
__global__ void moe_mix_kernel(const __half *__restrict__ slot_outputs, const float *__restrict__ weights,
                               __half *__restrict__ out, int hidden, int top_k) {
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();
  const int m = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= hidden) return;
  float sum = 0.0f;
  for (int s = 0; s < top_k; ++s)
    sum += weights[m * top_k + s] * __half2float(slot_outputs[(static_cast<size_t>(m) * top_k + s) * hidden + i]);
  out[static_cast<size_t>(m) * hidden + i] = __float2half_rn(sum);
}


// ---- sorted expert compute: where each received (token, expert) slot goes.
// One CTA.  Slot j (received order) of local expert e takes position p = number of earlier slots of
// e (a stable counting sort: warp votes, per-warp counts, a scan over the warps per expert);
// expert e owns ceil(count_e / rows_per_block) consecutive blocks starting at the running sum;
// target[j] = row of the block buffer, block_experts[b] = the global expert id of block b (-1 for a
// block nobody uses).  Slots without a local expert go to the row `dump` = blocks * rows_per_block.
constexpr int kPlanThreads = 1024;
constexpr int kPlanMaxExperts = 256;
constexpr int kPlanMaxChunks = 4;  // received <= 4096

__global__ void __launch_bounds__(kPlanThreads)
    dispatch_plan_kernel(const int *__restrict__ ids, int *__restrict__ target, int *__restrict__ block_experts,
                         int received, int first_expert, int local_experts, int rows_per_block, int blocks) {
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();
  __shared__ int running[kPlanMaxExperts];          // slots of the expert seen so far, then its first block
  __shared__ unsigned short warp_counts[32][kPlanMaxExperts];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int e = tid; e < kPlanMaxExperts; e += kPlanThreads) running[e] = 0;
  for (int b = tid; b < blocks; b += kPlanThreads) block_experts[b] = -1;
  int expert[kPlanMaxChunks], position[kPlanMaxChunks];
#pragma unroll
  for (int c = 0; c < kPlanMaxChunks; ++c) {
    const int j = c * kPlanThreads + tid;
    int e = -1;
    if (j < received) {
      const int id = ids[j];
      if (id >= first_expert && id < first_expert + local_experts) e = id - first_expert;
    }
    expert[c] = e;
    position[c] = 0;
    if (c * kPlanThreads >= received) continue;  // (uniform: the whole chunk is past the end)
    for (int i = tid; i < 32 * kPlanMaxExperts; i += kPlanThreads) (&warp_counts[0][0])[i] = 0;
    __syncthreads();
    const unsigned same = __match_any_sync(0xffffffffu, e >= 0 ? e : -1 - lane);
    const int rank = __popc(same & ((1u << lane) - 1u));
    if (e >= 0 && rank == 0) warp_counts[warp][e] = static_cast<unsigned short>(__popc(same));
    __syncthreads();
    if (tid < local_experts) {  // exclusive scan over the warps, continuing the expert's running count
      int sum = running[tid];
      for (int w = 0; w < 32; ++w) {
        const int count = warp_counts[w][tid];
        warp_counts[w][tid] = static_cast<unsigned short>(sum);
        sum += count;
      }
      running[tid] = sum;
    }
    __syncthreads();
    if (e >= 0) position[c] = warp_counts[warp][e] + rank;
    __syncthreads();
  }
  // counts -> first block of each expert (one thread: at most 256 experts)
  if (tid == 0) {
    int next = 0;
    for (int e = 0; e < local_experts; ++e) {
      const int count = running[e];
      running[e] = next;
      next += (count + rows_per_block - 1) / rows_per_block;
    }
  }
  __syncthreads();
  const int dump = blocks * rows_per_block;
#pragma unroll
  for (int c = 0; c < kPlanMaxChunks; ++c) {
    const int j = c * kPlanThreads + tid;
    if (j >= received) continue;
    const int e = expert[c];
    if (e < 0) {
      target[j] = dump;
      continue;
    }
    const int block = running[e] + position[c] / rows_per_block;
    const int within = position[c] % rows_per_block;
    target[j] = block < blocks ? block * rows_per_block + within : dump;
    if (within == 0 && block < blocks) block_experts[block] = e + first_expert;
  }
}

// rows[target[j]][:] = x[j / source_div][:] for every slot that has a row (16-byte copies)
__global__ void __launch_bounds__(128)
    dispatch_rows_kernel(const __half *__restrict__ x, const int *__restrict__ target, __half *__restrict__ rows,
                         int hidden, int dump, int source_div) {
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();
  const int j = blockIdx.x;
  const int row = target[j];
  if (row >= dump) return;
  const uint4 *source = reinterpret_cast<const uint4 *>(x + static_cast<size_t>(j / source_div) * hidden);
  uint4 *destination = reinterpret_cast<uint4 *>(rows + static_cast<size_t>(row) * hidden);
  for (int v = threadIdx.x; v < (hidden >> 3); v += 128) destination[v] = source[v];
}

// back[j][:] = outputs[target[j]][:], zeros for a slot without a row
__global__ void __launch_bounds__(128)
    combine_rows_kernel(const __half *__restrict__ outputs, const int *__restrict__ target, __half *__restrict__ back,
                        int hidden, int dump) {
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();
  const int j = blockIdx.x;
  const int row = target[j];
  uint4 *destination = reinterpret_cast<uint4 *>(back + static_cast<size_t>(j) * hidden);
  if (row >= dump) {
    for (int v = threadIdx.x; v < (hidden >> 3); v += 128) destination[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4 *source = reinterpret_cast<const uint4 *>(outputs + static_cast<size_t>(row) * hidden);
  for (int v = threadIdx.x; v < (hidden >> 3); v += 128) destination[v] = source[v];
}

// next[m] = argmax(logits[m]), lowest index on ties; also appends the token to the output
// log at column step[0] and advances the sequence's position.
__global__ void __launch_bounds__(1024)
    argmax_advance_kernel(const __half *__restrict__ logits, long long *__restrict__ tokens,
                          int *__restrict__ positions, long long *__restrict__ log,
                          int *__restrict__ step, int vocab, int log_stride) {
  // programmatic dependent launch: let the next kernel be scheduled, then wait for the
  // previous one before touching memory
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();

  __shared__ float best_value[32];
  __shared__ int best_index[32];
  const int m = blockIdx.x;
  const __half *row = logits + static_cast<size_t>(m) * vocab;
  float value = -INFINITY;
  int index = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float f = __half2float(row[i]);
    if (f > value || (f == value && i < index)) {
      value = f;
      index = i;
    }
  }
  for (int o = 16; o; o >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, value, o);
    const int other_index = __shfl_xor_sync(0xffffffffu, index, o);
    if (other > value || (other == value && other_index < index)) {
      value = other;
      index = other_index;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    best_value[warp] = value;
    best_index[warp] = index;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w)
      if (best_value[w] > value || (best_value[w] == value && best_index[w] < index)) {
        value = best_value[w];
        index = best_index[w];
      }
    if (index == 0x7fffffff) index = 0;  // a row without a single ordered value (all NaN)
    tokens[m] = index;
    if (log && step[0] < log_stride) log[static_cast<size_t>(m) * log_stride + step[0]] = index;
    positions[m] += 1;
  }
}

// The step counter advances once per decode step, after every row's argmax has used it.
__global__ void advance_step_kernel(int *step) {
  sageb200::pdl_launch_dependents();
  sageb200::pdl_wait();
  step[0] += 1;
}

int launch_status() { return cudaGetLastError() == cudaSuccess ? 0 : -5; }

}  // namespace

extern "C" {

int sageb200_glue_embed(const void *table, const void *tokens, void *h, int rows, int hidden,
                        int vocab, void *stream) {
  if (hidden % 8 || vocab <= 0) return -1;
  sageb200::launch_dependent<2>(embed_kernel, rows, 128, 0, static_cast<cudaStream_t>(stream),
      static_cast<const __half *>(table), static_cast<const long long *>(tokens),
      static_cast<__half *>(h), hidden, vocab);
  return launch_status();
}

int sageb200_glue_add_rmsnorm(void *residual, const void *delta, const void *weight, void *x,
                              int rows, int hidden, float eps, void *stream) {
  if (hidden > 24576) return -1;
  sageb200::launch_dependent<2>(add_rmsnorm_kernel, rows, kNormThreads, hidden * sizeof(__half), static_cast<cudaStream_t>(stream),
      static_cast<__half *>(residual), static_cast<const __half *>(delta),
      static_cast<const __half *>(weight), static_cast<__half *>(x), hidden, eps);
  return launch_status();
}

int sageb200_glue_qk_norm_rope_cache(void *q, const void *k, const void *v, const void *q_weight,
                                     const void *k_weight, const void *cos_table,
                                     const void *sin_table, const void *positions, void *k_cache,
                                     void *v_cache, int rows, int q_heads, int kv_heads, int head_dim,
                                     int max_seq, float eps, void *stream) {
  if (head_dim != 128) return -1;
  const int heads = q_heads + 2 * kv_heads;
  const dim3 grid((heads + 3) / 4, rows);
  sageb200::launch_dependent<2>(qk_norm_rope_cache_kernel, grid, 128, 0, static_cast<cudaStream_t>(stream),
      static_cast<__half *>(q), static_cast<const __half *>(k), static_cast<const __half *>(v),
      static_cast<const __half *>(q_weight), static_cast<const __half *>(k_weight),
      static_cast<const __half *>(cos_table), static_cast<const __half *>(sin_table),
      static_cast<const int *>(positions), static_cast<__half *>(k_cache),
      static_cast<__half *>(v_cache), q_heads, kv_heads, max_seq, eps, 1);
  return launch_status();
}

int sageb200_glue_prefill_qk_norm_rope_cache(void *q, const void *k, const void *v, const void *q_weight,
                                             const void *k_weight, const void *cos_table,
                                             const void *sin_table, const void *positions, void *k_cache,
                                             void *v_cache, int sequences, int tokens, int q_heads,
                                             int kv_heads, int head_dim, int max_seq, float eps, void *stream) {
  if (head_dim != 128 || sequences < 1 || tokens < 1 || static_cast<long long>(sequences) * tokens > 65535)
    return -1;
  const int heads = q_heads + 2 * kv_heads;
  const dim3 grid((heads + 3) / 4, sequences * tokens);
  sageb200::launch_dependent<2>(qk_norm_rope_cache_kernel, grid, 128, 0, static_cast<cudaStream_t>(stream),
      static_cast<__half *>(q), static_cast<const __half *>(k), static_cast<const __half *>(v),
      static_cast<const __half *>(q_weight), static_cast<const __half *>(k_weight),
      static_cast<const __half *>(cos_table), static_cast<const __half *>(sin_table),
      static_cast<const int *>(positions), static_cast<__half *>(k_cache),
      static_cast<__half *>(v_cache), q_heads, kv_heads, max_seq, eps, tokens);
  return launch_status();
}

size_t sageb200_glue_attention_scratch_bytes(int rows, int q_heads, int splits) {
  return static_cast<size_t>(rows) * q_heads * splits * 130 * sizeof(float);
}

int sageb200_glue_attention_decode(const void *q, const void *k_cache, const void *v_cache,
                                   const void *positions, void *out, void *scratch, int rows,
                                   int q_heads, int kv_heads, int head_dim, int max_seq, int splits,
                                   void *stream) {
  if (head_dim != 128 || q_heads % kv_heads || q_heads / kv_heads > kMaxGroup || splits < 1) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(splits, kv_heads, rows);
  sageb200::launch_dependent<2>(attention_partial_kernel, grid, kAttnWarps * 32, 0, s,
      static_cast<const __half *>(q), static_cast<const __half *>(k_cache),
      static_cast<const __half *>(v_cache), static_cast<const int *>(positions),
      static_cast<float *>(scratch), q_heads, kv_heads, max_seq, splits, rsqrtf(128.0f));
  sageb200::launch_dependent<2>(attention_combine_kernel, dim3(q_heads, rows), 128, 0, s, static_cast<const float *>(scratch),
                                                              static_cast<__half *>(out), q_heads,
                                                              splits);
  return launch_status();
}

}  // extern "C"

namespace {

using AttentionKernel = void (*)(const __half *, const __half *, const __half *, const __half *, const __half *,
                                 const __half *, const __half *, const int *, __half *, __half *, __half *, int, int,
                                 int, float, float, int, const int *);

// debug: environment SAGEB200_ATTN_HEADS = 1, 2 or 4 forces the query heads per CTA
int attention_heads_override() {
  static const int value = [] {
    const char *text = getenv("SAGEB200_ATTN_HEADS");
    return text ? atoi(text) : 0;
  }();
  return value;
}

// Query heads per CTA: four when the group allows (K/V rows are read once per four heads),
// fewer when that leaves most SMs without a CTA.
int attention_heads_per_cta(int group, int units_at_four, int sm_count) {
  const int forced = attention_heads_override();
  if (forced == 1 || forced == 2 || forced == 4) return forced;
  if (group % 4 == 0 && units_at_four * 2 > sm_count) return 4;
  if (group % 2 == 0) return group % 4 == 0 && units_at_four * 4 <= sm_count ? 1 : 2;
  return group >= 3 ? 4 : 1;
}

template <bool kPrompt, bool kIndexed = false>
AttentionKernel attention_variant(int heads_per_cta, bool exact) {
  if (heads_per_cta == 4)
    return exact ? attention_step_kernel<4, true, kPrompt, kIndexed> : attention_step_kernel<4, false, kPrompt, kIndexed>;
  if (heads_per_cta == 2)
    return exact ? attention_step_kernel<2, true, kPrompt, kIndexed> : attention_step_kernel<2, false, kPrompt, kIndexed>;
  return attention_step_kernel<1, true, kPrompt, kIndexed>;
}

int launch_attention(bool prompt_rows, const void *q, const void *k, const void *v, const void *q_weight,
                     const void *k_weight, const void *cos_table, const void *sin_table, const void *positions,
                     void *k_cache, void *v_cache, void *out, int grid_rows, int q_heads, int kv_heads, int max_seq,
                     int splits, float eps, int rows_per_sequence, bool dependent, void *stream,
                     const void *out_index = nullptr) {
  const int group = q_heads / kv_heads;
  static int sm_count = 0;
  if (sm_count == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sm_count <= 0)
      sm_count = 148;
  }
  const int per_cta = attention_heads_per_cta(group, splits * kv_heads * ((group + 3) / 4) * grid_rows, sm_count);
  const int parts = (group + per_cta - 1) / per_cta;
  const bool exact = group % per_cta == 0;
  AttentionKernel kernel = prompt_rows  ? attention_variant<true>(per_cta, exact)
                           : out_index ? attention_variant<false, true>(per_cta, exact)
                                       : attention_variant<false>(per_cta, exact);
  if (splits == 16) {  // beyond the portable cluster size: opt in, and check that one fits at all
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(splits, kv_heads * parts, grid_rows);
  config.blockDim = dim3(kAttnWarps * 32);
  config.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attributes[2];
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = splits;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = dependent ? 2 : 1;
  if (splits == 16) {
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &config) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      return -1;
    }
  }
  __atomic_fetch_add(&sageb200::g_sageb200_glue_launches, 1ull, __ATOMIC_RELAXED);
  const cudaError_t error = cudaLaunchKernelEx(
      &config, kernel, static_cast<const __half *>(q), static_cast<const __half *>(k),
      static_cast<const __half *>(v), static_cast<const __half *>(q_weight), static_cast<const __half *>(k_weight),
      static_cast<const __half *>(cos_table), static_cast<const __half *>(sin_table),
      static_cast<const int *>(positions), static_cast<__half *>(k_cache), static_cast<__half *>(v_cache),
      static_cast<__half *>(out), q_heads, kv_heads, max_seq, eps, rsqrtf(128.0f), rows_per_sequence,
      static_cast<const int *>(out_index));
  return error == cudaSuccess ? launch_status() : -5;
}

}  // namespace

extern "C" {

int sageb200_glue_attention_step(const void *q, const void *k, const void *v, const void *q_weight,
                                 const void *k_weight, const void *cos_table, const void *sin_table,
                                 const void *positions, void *k_cache, void *v_cache, void *out, int rows,
                                 int q_heads, int kv_heads, int head_dim, int max_seq, int splits, float eps,
                                 void *stream) {
  if (head_dim != 128 || kv_heads < 1 || q_heads % kv_heads || max_seq < 1 || rows < 1) return -1;
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8 && splits != 16) return -1;
  return launch_attention(false, q, k, v, q_weight, k_weight, cos_table, sin_table, positions, k_cache, v_cache, out,
                          rows, q_heads, kv_heads, max_seq, splits, eps, 0, (sageb200::g_sageb200_pdl & 6) != 0, stream);
}

int sageb200_glue_attention_step_permuted(const void *q, const void *k, const void *v, const void *q_weight,
                                          const void *k_weight, const void *cos_table, const void *sin_table,
                                          const void *positions, void *k_cache, void *v_cache, void *out,
                                          const void *out_index, int rows, int q_heads, int kv_heads, int head_dim,
                                          int max_seq, int splits, float eps, void *stream) {
  if (head_dim != 128 || kv_heads < 1 || q_heads % kv_heads || max_seq < 1 || rows < 1) return -1;
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8 && splits != 16) return -1;
  if (reinterpret_cast<uintptr_t>(out_index) & 3) return -1;
  return launch_attention(false, q, k, v, q_weight, k_weight, cos_table, sin_table, positions, k_cache, v_cache, out,
                          rows, q_heads, kv_heads, max_seq, splits, eps, 0, (sageb200::g_sageb200_pdl & 6) != 0, stream,
                          out_index);
}

int sageb200_glue_prefill_attention(const void *q, const void *k_cache, const void *v_cache,
                                    const void *positions, void *out, int sequences, int tokens, int q_heads,
                                    int kv_heads, int head_dim, int max_seq, void *stream) {
  if (head_dim != 128 || kv_heads < 1 || q_heads % kv_heads || max_seq < 1 || sequences < 1 || tokens < 1 ||
      static_cast<long long>(sequences) * tokens > 65535)
    return -1;
  if (tokens >= 32 && sequences <= 65535 && q_heads <= 65535) {
    // the tiled tensor-core kernel; a handful of rows stay on the per-row decode kernel
    __atomic_fetch_add(&sageb200::g_sageb200_glue_launches, 1ull, __ATOMIC_RELAXED);
    const cudaError_t error = sageb200::launch_prefill_attention(
        static_cast<const __half *>(q), static_cast<const __half *>(k_cache), static_cast<const __half *>(v_cache),
        static_cast<const int *>(positions), static_cast<__half *>(out), sequences, tokens, q_heads, kv_heads,
        max_seq, static_cast<cudaStream_t>(stream));
    return error == cudaSuccess ? 0 : -5;
  }
  return launch_attention(true, q, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, positions,
                          const_cast<void *>(k_cache), const_cast<void *>(v_cache), out, sequences * tokens, q_heads,
                          kv_heads, max_seq, 1, 0.0f, tokens, false, stream);
}

int sageb200_glue_add_rmsnorm_permuted(void *residual, const void *delta, const void *weight, void *x,
                                       const void *const *perms, void *const *outs, int count, int rows,
                                       int hidden, float eps, void *stream) {
  if (hidden > 24576 || hidden % 8 || count < 1 || count > 4 || !perms || !outs || rows < 1) return -1;
  PermutedOutputs outputs = {};
  outputs.count = count;
  for (int j = 0; j < count; ++j) {
    if (!perms[j] || !outs[j] || ((reinterpret_cast<uintptr_t>(perms[j]) | reinterpret_cast<uintptr_t>(outs[j])) & 15))
      return -1;
    outputs.perm[j] = static_cast<const int *>(perms[j]);
    outputs.out[j] = static_cast<__half *>(outs[j]);
  }
  const size_t shared = hidden * sizeof(__half);
  static bool configured = false;
  if (shared > 40 * 1024 && !configured) {
    if (cudaFuncSetAttribute(add_rmsnorm_permuted_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024) !=
        cudaSuccess)
      return -5;
    configured = true;
  }
  sageb200::launch_dependent<2>(add_rmsnorm_permuted_kernel, rows, kNormThreads, shared,
                                static_cast<cudaStream_t>(stream), static_cast<__half *>(residual),
                                static_cast<const __half *>(delta), static_cast<const __half *>(weight),
                                static_cast<__half *>(x), outputs, hidden, eps);
  return launch_status();
}

int sageb200_glue_swiglu_permuted(const void *gate, const void *up, const void *perm, void *act, int rows, int k,
                                  int sm_count, void *stream) {
  if (rows < 1 || k < 8 || k % 8 || k > 100 * 1024 || !gate || !up || !perm || !act ||
      ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(perm) |
        reinterpret_cast<uintptr_t>(act)) & 15))
    return -1;
  const size_t shared = static_cast<size_t>(k) * sizeof(__half);
  static bool configured = false;
  if (shared > 40 * 1024 && !configured) {
    if (cudaFuncSetAttribute(swiglu_permuted_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
        cudaSuccess)
      return -5;
    configured = true;
  }
  int blocks = rows;
  const int cap = (sm_count > 0 ? sm_count : 148) * 4;
  if (blocks > cap) blocks = cap;
  sageb200::launch_dependent<2>(swiglu_permuted_kernel, blocks, 256, shared, static_cast<cudaStream_t>(stream),
                                static_cast<const __half *>(gate), static_cast<const __half *>(up),
                                static_cast<const int *>(perm), static_cast<__half *>(act), rows, k);
  return launch_status();
}

int sageb200_glue_swiglu(const void *gate, const void *up, void *act, long long count, void *stream) {
  const unsigned blocks = static_cast<unsigned>((count + 2047) / 2048);  // eight elements per thread
  sageb200::launch_dependent<2>(swiglu_kernel, blocks, 256, 0, static_cast<cudaStream_t>(stream),
      static_cast<const __half *>(gate), static_cast<const __half *>(up), static_cast<__half *>(act),
      count);
  return launch_status();
}

int sageb200_glue_lm_head(const void *head, const void *x, void *logits, int rows, int vocab,
                          int hidden, int sm_count, void *stream) {
  if (rows > 16 || hidden % 8) return -1;
  const int staged_rows = rows > 1 && hidden % 32 == 0 ? (rows > 8 ? 16 : 8) : rows;  // (blocked copy: whole column blocks)
  const size_t shared = static_cast<size_t>(staged_rows) * hidden * sizeof(__half);
  static bool configured = false;
  if (shared > 48 * 1024 && !configured) {
    if (cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=
        cudaSuccess)
      return -5;
    configured = true;
  }
  const int blocks = (sm_count > 0 ? sm_count : 148) * 4;
  sageb200::launch_dependent<2>(lm_head_kernel, blocks, kHeadWarps * 32, shared, static_cast<cudaStream_t>(stream),
      static_cast<const __half *>(head), static_cast<const __half *>(x), static_cast<__half *>(logits),
      vocab, hidden, rows);
  return launch_status();
}

size_t sageb200_glue_lm_head_step_scratch_bytes(int rows, int sm_count) {
  const int blocks = (sm_count > 0 ? sm_count : 148) * 4;
  return 256 + static_cast<size_t>(blocks) * rows * sizeof(float2);
}

int sageb200_glue_lm_head_step(const void *head, const void *residual, const void *delta,
                               const void *norm_weight, void *x, void *logits, void *tokens,
                               void *positions, void *log, void *step, void *scratch, int rows, int vocab,
                               int hidden, float eps, int log_stride, int sm_count, void *stream) {
  if (rows < 1 || rows > 16 || hidden % 8 || vocab < 1) return -1;
  const int staged_rows = rows > 1 && hidden % 32 == 0 ? (rows > 8 ? 16 : 8) : rows;  // (blocked copy: whole column blocks)
  const size_t shared = static_cast<size_t>(staged_rows) * hidden * sizeof(__half);
  if (shared > 200 * 1024) return -1;
  auto kernel = rows == 1 ? lm_head_step_kernel<1> : rows <= 8 ? lm_head_step_kernel<8> : lm_head_step_kernel<16>;
  if (shared > 40 * 1024 &&
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
    return -5;
  int blocks = (sm_count > 0 ? sm_count : 148) * 4;
  if (rows > 1 && hidden % 32 == 0) {
    // several sequences (tiles handed out by ticket): exactly the CTAs that are resident at once
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kHeadWarps * 32, shared) != cudaSuccess) {
      cudaGetLastError();
      per_sm = 0;
    }
    if (per_sm >= 1 && per_sm < 4) blocks = (sm_count > 0 ? sm_count : 148) * per_sm;
  }
  sageb200::launch_dependent<2>(
      kernel, blocks, kHeadWarps * 32, shared, static_cast<cudaStream_t>(stream),
      static_cast<const __half *>(head), static_cast<const __half *>(residual),
      static_cast<const __half *>(delta), static_cast<const __half *>(norm_weight), static_cast<__half *>(x),
      static_cast<__half *>(logits), static_cast<long long *>(tokens), static_cast<int *>(positions),
      static_cast<long long *>(log), static_cast<int *>(step),
      reinterpret_cast<float2 *>(static_cast<char *>(scratch) + 256), static_cast<unsigned *>(scratch), vocab,
      hidden, rows, eps, log_stride);
  return launch_status();
}

int sageb200_glue_moe_route(void *residual, const void *delta, const void *norm_weight, const void *router,
                            void *x, void *ids, void *weights, int rows, int hidden, int experts, int top_k,
                            float eps, void *stream) {
  if (rows < 1 || hidden % 8 || hidden > 24576 || experts < 1 || experts > kMaxExperts || top_k < 1 ||
      top_k > 32 || top_k > experts)
    return -1;
  const size_t shared = static_cast<size_t>(hidden) * sizeof(__half);
  sageb200::launch_dependent<2>(
      moe_route_kernel, dim3(rows), dim3(kRouteThreads), shared, static_cast<cudaStream_t>(stream),
      static_cast<__half *>(residual), static_cast<const __half *>(delta), static_cast<const __half *>(norm_weight),
      static_cast<const __half *>(router), static_cast<__half *>(x), static_cast<int *>(ids),
      static_cast<float *>(weights), hidden, experts, top_k, eps);
  return launch_status();
}

int sageb200_glue_moe_mix(const void *slot_outputs, const void *weights, void *out, int rows, int hidden,
                          int top_k, void *stream) {
  if (rows < 1 || hidden < 1 || top_k < 1) return -1;
  sageb200::launch_dependent<2>(moe_mix_kernel, dim3((hidden + 255) / 256, rows), dim3(256), 0,
                                static_cast<cudaStream_t>(stream), static_cast<const __half *>(slot_outputs),
                                static_cast<const float *>(weights), static_cast<__half *>(out), hidden, top_k);
  return launch_status();
}

int sageb200_glue_dispatch_plan(const void *ids, void *target, void *block_experts, int received,
                                int first_expert, int local_experts, int rows_per_block, int blocks, void *stream) {
  if (!ids || !target || !block_experts || received < 1 || received > kPlanThreads * kPlanMaxChunks ||
      local_experts < 1 || local_experts > kPlanMaxExperts || rows_per_block < 1 || blocks < 1)
    return -1;
  sageb200::launch_dependent<2>(dispatch_plan_kernel, 1, kPlanThreads, 0, static_cast<cudaStream_t>(stream),
                                static_cast<const int *>(ids), static_cast<int *>(target),
                                static_cast<int *>(block_experts), received, first_expert, local_experts,
                                rows_per_block, blocks);
  return launch_status();
}

int sageb200_glue_dispatch_rows(const void *x, const void *target, void *rows, int received, int hidden, int dump,
                                int source_div, void *stream) {
  if (!x || !target || !rows || received < 1 || hidden < 8 || hidden % 8 || source_div < 1 ||
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(rows)) & 15))
    return -1;
  sageb200::launch_dependent<2>(dispatch_rows_kernel, received, 128, 0, static_cast<cudaStream_t>(stream),
                                static_cast<const __half *>(x), static_cast<const int *>(target),
                                static_cast<__half *>(rows), hidden, dump, source_div);
  return launch_status();
}

int sageb200_glue_combine_rows(const void *outputs, const void *target, void *back, int received, int hidden,
                               int dump, void *stream) {
  if (!outputs || !target || !back || received < 1 || hidden < 8 || hidden % 8 ||
      ((reinterpret_cast<uintptr_t>(outputs) | reinterpret_cast<uintptr_t>(back)) & 15))
    return -1;
  sageb200::launch_dependent<2>(combine_rows_kernel, received, 128, 0, static_cast<cudaStream_t>(stream),
                                static_cast<const __half *>(outputs), static_cast<const int *>(target),
                                static_cast<__half *>(back), hidden, dump);
  return launch_status();
}

int sageb200_glue_argmax_advance(const void *logits, void *tokens, void *positions, void *log,
                                 void *step, int rows, int vocab, int log_stride, void *stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  sageb200::launch_dependent<2>(argmax_advance_kernel, rows, 1024, 0, s, static_cast<const __half *>(logits),
                                               static_cast<long long *>(tokens),
                                               static_cast<int *>(positions),
                                               static_cast<long long *>(log), static_cast<int *>(step),
                                               vocab, log_stride);
  if (step) sageb200::launch_dependent<2>(advance_step_kernel, 1, 1, 0, s, static_cast<int *>(step));
  return launch_status();
}

}  // extern "C"
