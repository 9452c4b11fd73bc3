// Export-side packing: frozen signs / direction indices and trained radii of a spherical
// (SAGE or SPHQuant) linear into the packed buffers the inference kernels read.
//
// Replaces the tensor program of the reference's exporter
// (weight_vq/sphquant/packing.py:32-75): per (row, 128-channel group)
//     minimum = min of the 16 radii, step = fp16((max - min) / levels), minimum = fp16(minimum)
//     code_v  = clamp(round_half_even((radius_v - minimum) / step), 0, levels)    (0 where step == 0)
//     word_v  = sign bits | index << 8 | low (8 - D) bits of code_v << (8 + D)
//     high    = the two high bits of the sixteen codes, two bits per vector
// and the words laid out either in SAGE's tiled form (two codes per 32-bit word,
// [tile][group][16 rows][8 words], rows padded to a multiple of 16 with zero codes and a zero
// grid) or in SPHQuant's row-major int16 form.  Integer work plus a handful of FP32 operations
// that round exactly as the tensor program's do (IEEE division, round-half-even, one rounding
// to FP16), so the packed buffers are identical bit for bit.
//
// One thread per (row, group): 16 radii (64 bytes), 16 indices, 128 signs in; 32 + 4 + 4 bytes
// out.  HBM-bound on the signs (1 byte per weight in, 0.31 byte per weight out).
#include "sage_common.cuh"
#include "sage_kernels.h"

namespace sageb200 {
namespace {

constexpr int kPackThreads = 128;

template <bool kTiled>
__global__ void __launch_bounds__(kPackThreads) sage_pack_kernel(
    const int8_t *__restrict__ signs, const int32_t *__restrict__ indices,
    const float *__restrict__ radius, uint32_t *__restrict__ codes, uint32_t *__restrict__ high_out,
    __half *__restrict__ grid_or_scales, __half *__restrict__ mins, int n, int n_padded, int k,
    int dbits) {
  const int groups = k >> 7;
  const long long total = static_cast<long long>(n_padded) * groups;
  const int levels = (1 << (10 - dbits)) - 1;
  const int low_bits = 8 - dbits;
  for (long long item = static_cast<long long>(blockIdx.x) * kPackThreads + threadIdx.x; item < total;
       item += static_cast<long long>(gridDim.x) * kPackThreads) {
    const int row = static_cast<int>(item / groups);
    const int group = static_cast<int>(item - static_cast<long long>(row) * groups);
    uint32_t words[16];
    uint32_t high = 0;
    __half minimum_h = __float2half_rn(0.0f), step_h = __float2half_rn(0.0f);
    if (row < n) {
      const float *r = radius + static_cast<size_t>(row) * (k >> 3) + group * 16;
      float values[16];
#pragma unroll
      for (int q = 0; q < 4; ++q)
        *reinterpret_cast<float4 *>(values + 4 * q) = reinterpret_cast<const float4 *>(r)[q];
      float lowest = values[0], highest = values[0];
#pragma unroll
      for (int v = 1; v < 16; ++v) {
        lowest = fminf(lowest, values[v]);
        highest = fmaxf(highest, values[v]);
      }
      // the step is rounded to FP16 from the FP32 minimum, then the minimum itself is rounded
      step_h = __float2half_rn(__fdiv_rn(__fsub_rn(highest, lowest), static_cast<float>(levels)));
      minimum_h = __float2half_rn(lowest);
      const float step = __half2float(step_h), minimum = __half2float(minimum_h);
      const bool live = step > 0.0f;
      const float safe_step = live ? step : 1.0f;
      const int32_t *index = indices + static_cast<size_t>(row) * (k >> 3) + group * 16;
      const int8_t *sign = signs + static_cast<size_t>(row) * k + group * 128;
#pragma unroll
      for (int v = 0; v < 16; ++v) {
        int code = 0;
        if (live) {
          const float scaled = rintf(__fdiv_rn(__fsub_rn(values[v], minimum), safe_step));
          code = static_cast<int>(fminf(fmaxf(scaled, 0.0f), static_cast<float>(levels)));
        }
        const uint2 packed_signs = *reinterpret_cast<const uint2 *>(sign + v * 8);
        uint32_t bits = 0;
#pragma unroll
        for (int d = 0; d < 8; ++d) {
          const uint32_t byte = ((d < 4 ? packed_signs.x : packed_signs.y) >> (8 * (d & 3))) & 0xffu;
          bits |= (byte >> 7) << d;  // a negative int8 has bit 7 set
        }
        words[v] = bits | (static_cast<uint32_t>(index[v]) << 8) |
                   (static_cast<uint32_t>(code & ((1 << low_bits) - 1)) << (8 + dbits));
        high |= static_cast<uint32_t>(code >> low_bits) << (2 * v);
      }
    } else {
#pragma unroll
      for (int v = 0; v < 16; ++v) words[v] = 0;
    }
    if constexpr (kTiled) {
      const size_t cell = (static_cast<size_t>(row >> 4) * groups + group) * 16 + (row & 15);
      uint4 *out = reinterpret_cast<uint4 *>(codes + cell * 8);
      out[0] = make_uint4(words[0] | (words[1] << 16), words[2] | (words[3] << 16),
                          words[4] | (words[5] << 16), words[6] | (words[7] << 16));
      out[1] = make_uint4(words[8] | (words[9] << 16), words[10] | (words[11] << 16),
                          words[12] | (words[13] << 16), words[14] | (words[15] << 16));
      high_out[cell] = high;
      reinterpret_cast<__half2 *>(grid_or_scales)[cell] = __halves2half2(minimum_h, step_h);
    } else {
      // row-major int16 codes [n][k/8], per-(row, group) high word, scale and minimum
      const size_t cell = static_cast<size_t>(row) * groups + group;
      uint4 *out = reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(codes) + cell * 16);
      out[0] = make_uint4(words[0] | (words[1] << 16), words[2] | (words[3] << 16),
                          words[4] | (words[5] << 16), words[6] | (words[7] << 16));
      out[1] = make_uint4(words[8] | (words[9] << 16), words[10] | (words[11] << 16),
                          words[12] | (words[13] << 16), words[14] | (words[15] << 16));
      high_out[cell] = high;
      grid_or_scales[cell] = step_h;
      mins[cell] = minimum_h;
    }
  }
}

}  // namespace

cudaError_t launch_pack(const int8_t *signs, const int32_t *indices, const float *radius, uint32_t *codes,
                        uint32_t *high, __half *grid_or_scales, __half *mins, int n, int k, int dbits,
                        bool tiled, cudaStream_t stream, int sm_count) {
  const int n_padded = tiled ? (n + 15) / 16 * 16 : n;
  const long long total = static_cast<long long>(n_padded) * (k >> 7);
  long long blocks = (total + kPackThreads - 1) / kPackThreads;
  const long long cap = static_cast<long long>(sm_count) * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (tiled)
    sage_pack_kernel<true><<<static_cast<unsigned>(blocks), kPackThreads, 0, stream>>>(
        signs, indices, radius, codes, high, grid_or_scales, mins, n, n_padded, k, dbits);
  else
    sage_pack_kernel<false><<<static_cast<unsigned>(blocks), kPackThreads, 0, stream>>>(
        signs, indices, radius, codes, high, grid_or_scales, mins, n, n_padded, k, dbits);
  return cudaGetLastError();
}

}  // namespace sageb200
