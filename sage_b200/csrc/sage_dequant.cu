// Dense FP16 dequantisation of a SAGE-packed matrix: w[n][k].
//
// Bit-exact with the reference's own dequantisation
// (csrc/sage/sage_gemm_cuda.cu:117-131: radius = fmaf(code, step, min) in FP32,
// w = fp16_rn(float(+-dir) * radius)) and with its Python decoder followed by .half()
// (tests/inference/reference.py:39-49, tests/inference/test_sage.py:113-115).
//
// HBM-bound: reads 2.5 bit/weight, writes 16 bit/weight.  One thread decodes one
// 8-wide vector and stores 16 bytes (or eight scattered halves when the inverse
// channel permutation is applied).
#include "sage_common.cuh"
#include "sage_kernels.h"

namespace sageb200 {
namespace {

constexpr int kDequantThreads = 256;

template <bool kScatter>
__global__ void __launch_bounds__(kDequantThreads) sage_dequant_kernel(
    const uint32_t *__restrict__ codes, const uint32_t *__restrict__ radii,
    const uint32_t *__restrict__ grid, const uint32_t *__restrict__ book,
    const int32_t *__restrict__ perm, __half *__restrict__ w, int n, int k, int entries,
    int dbits) {
  __shared__ uint32_t shared_book[4 * 256];
  for (int i = threadIdx.x; i < 4 * entries; i += kDequantThreads) shared_book[i] = book[i];
  __syncthreads();
  const int vectors_per_row = k >> 3;
  const int groups = k >> 7;
  const long long total = static_cast<long long>(n) * vectors_per_row;
  for (long long item = static_cast<long long>(blockIdx.x) * kDequantThreads + threadIdx.x;
       item < total; item += static_cast<long long>(gridDim.x) * kDequantThreads) {
    const int row = static_cast<int>(item / vectors_per_row);
    const int vi = static_cast<int>(item - static_cast<long long>(row) * vectors_per_row);
    const int group = vi >> 4;
    const int v = vi & 15;
    const size_t cell = (static_cast<size_t>(row >> 4) * groups + group) * 16 + (row & 15);
    const uint32_t word = codes[cell * 8 + (v >> 1)];
    const uint32_t code = (word >> (16 * (v & 1))) & 0xffffu;
    const uint32_t endpoints = grid[cell];
    const float2 e = __half22float2(*reinterpret_cast<const __half2 *>(&endpoints));
    uint32_t out[4];
    dequant_vector_exact(code, radii[cell], v, e.x, e.y, shared_book, entries, dbits, out);
    if constexpr (!kScatter) {
      *reinterpret_cast<uint4 *>(w + static_cast<size_t>(row) * k + static_cast<size_t>(vi) * 8) =
          make_uint4(out[0], out[1], out[2], out[3]);
    } else {
      const __half *values = reinterpret_cast<const __half *>(out);
      const int32_t *p = perm + vi * 8;
#pragma unroll
      for (int d = 0; d < 8; ++d) w[static_cast<size_t>(row) * k + p[d]] = values[d];
    }
  }
}

}  // namespace

cudaError_t launch_dequant(const uint32_t *codes, const uint32_t *radii, const uint32_t *grid,
                           const uint32_t *book, const int32_t *perm, __half *w, int n, int k,
                           int entries, cudaStream_t stream, int sm_count) {
  const long long total = static_cast<long long>(n) * (k >> 3);
  long long blocks = (total + kDequantThreads - 1) / kDequantThreads;
  const long long cap = static_cast<long long>(sm_count) * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const int dbits = direction_bits_of(entries);
  if (perm) {
    sage_dequant_kernel<true><<<static_cast<unsigned>(blocks), kDequantThreads, 0, stream>>>(
        codes, radii, grid, book, perm, w, n, k, entries, dbits);
  } else {
    sage_dequant_kernel<false><<<static_cast<unsigned>(blocks), kDequantThreads, 0, stream>>>(
        codes, radii, grid, book, perm, w, n, k, entries, dbits);
  }
  return cudaGetLastError();
}

}  // namespace sageb200
