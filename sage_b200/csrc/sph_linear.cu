// SPHQuant 64/4 packed-weight matmul and dequantisation for sm_100a.
//
// Replaces the reference's csrc/sphquant/sph_gemv_cuda.cu (kernel :251-399, host entry
// :403-469) behind the same operator (weight_vq/inference/ops.py:21-39).  Format (row-major,
// no tiles, no permutation):
//   packed_codes  int16 [N][K/8]   bits 0-7 signs (1 = negative), 8-13 direction index,
//                                  14-15 low radius bits
//   radius_extra  int32 [N][K/128] sixteen 2-bit high radius fields; code = low | high << 2
//   radius_scales / radius_mins fp16 [N][K/128]   radius = fmaf(code, scale, min) in FP32
//   codebook      fp16 [64][8]     entry-major
//   W[n][8v + d] = (+-codebook[index][d]) * radius
//
// Differences from the reference kernel, by design: the packed weights are read ONCE for up to
// eight activation rows (the reference launches grid.y = rows and re-reads them per row), and
// sums across vectors are FP32 (the reference accumulates in FP16).
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sage_b200.h"
#include "sage_common.cuh"
#include "sage_kernels.h"

namespace sageb200 {
namespace {

constexpr int kSphWarps = 16;
constexpr int kSphThreads = kSphWarps * 32;
constexpr int kSphBookBytes = 64 * 8 * 16;  // 64 entries x 8 replicas x 16 bytes
constexpr int kSphChunkHalves = 72;         // a 64-channel chunk of x plus 16 bytes of padding

struct SphChunk {  // what one lane needs for 64 consecutive weights of one output row
  uint4 codes;
  uint32_t extra;
  float scale, minimum;
};

__device__ __forceinline__ SphChunk load_chunk(const uint16_t *codes, const uint32_t *extra,
                                               const __half *scales, const __half *mins, long long row,
                                               int chunk, int chunks, int groups, bool valid) {
  SphChunk c;
  c.codes = make_uint4(0, 0, 0, 0);
  c.extra = 0;
  c.scale = c.minimum = 0.0f;
  if (valid) {
    const long long cell = row * groups + (chunk >> 1);
    c.codes = ldg_stream_u4(reinterpret_cast<const uint4 *>(codes) + row * chunks + chunk);
    c.extra = __ldg(extra + cell);
    c.scale = __half2float(__ldg(scales + cell));
    c.minimum = __half2float(__ldg(mins + cell));
  }
  return c;
}

// One warp = 32 / L output rows at a time (L = 8, 16 or 32 lanes each: fewer rows per warp when
// the matrix has few rows, so that every SM still gets work); a lane walks every L-th 64-weight
// chunk of its row.  Per code: direction from the replicated codebook (one LDS.128, replica =
// lane % 8, conflict-free), signs XORed in, FP16 dot with the eight activations per row of x,
// FP32 multiply by the radius and FP32 accumulation.
template <int M, int L>
__global__ void __launch_bounds__(kSphThreads)
    sph_skinny_kernel(const __half *__restrict__ x, const uint16_t *__restrict__ codes,
                      const uint32_t *__restrict__ extra, const __half *__restrict__ scales,
                      const __half *__restrict__ mins, const uint4 *__restrict__ book,
                      __half *__restrict__ y, int rows, int n, int k) {
  extern __shared__ __align__(16) unsigned char shared[];
  uint4 *book_shared = reinterpret_cast<uint4 *>(shared);
  __half *x_shared = reinterpret_cast<__half *>(shared + kSphBookBytes);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  pdl_launch_dependents();
  if (tid < 64) {  // codebook: static data, fetched before the wait for the previous kernel
    const uint4 entry = __ldg(book + tid);
#pragma unroll
    for (int r = 0; r < 8; ++r) book_shared[tid * 8 + ((r + lane) & 7)] = entry;
  }
  pdl_wait();
  // activations: M rows (zero beyond `rows`), each 64-channel chunk padded to 72 halves so that
  // the eight lanes of a row, which read chunks 128 bytes apart, hit different banks
  const int chunks = k >> 6, groups = k >> 7;
  const int row_halves = chunks * kSphChunkHalves;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const int row_pieces = k >> 3;
  for (int i = tid; i < M * row_pieces; i += kSphThreads) {
    const int m = i / row_pieces, piece = i - m * row_pieces;
    uint4 value = make_uint4(0, 0, 0, 0);
    if (m < rows) {
      const __half *source = x + static_cast<size_t>(m) * k + piece * 8;
      if (aligned) {
        value = __ldg(reinterpret_cast<const uint4 *>(source));
      } else {
        __half *parts = reinterpret_cast<__half *>(&value);
#pragma unroll
        for (int h = 0; h < 8; ++h) parts[h] = source[h];
      }
    }
    *reinterpret_cast<uint4 *>(x_shared + m * row_halves + (piece >> 3) * kSphChunkHalves + (piece & 7) * 8) = value;
  }
  __syncthreads();

  constexpr int kRowsPerWarp = 32 / L;
  const int sub = lane / L, l = lane % L;
  const uint32_t book_base = smem_address(book_shared) + static_cast<uint32_t>(lane & 7) * 16u;
  const int quads = (n + kRowsPerWarp - 1) / kRowsPerWarp;
  for (int quad = blockIdx.x * kSphWarps + warp; quad < quads; quad += gridDim.x * kSphWarps) {
    const int row = quad * kRowsPerWarp + sub;
    const bool row_valid = row < n;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
    SphChunk current = load_chunk(codes, extra, scales, mins, row, l, chunks, groups, row_valid && l < chunks);
    for (int chunk = l; chunk < chunks; chunk += L) {
      const SphChunk next = load_chunk(codes, extra, scales, mins, row, chunk + L, chunks, groups,
                                       row_valid && chunk + L < chunks);
      const uint32_t words[4] = {current.codes.x, current.codes.y, current.codes.z, current.codes.w};
      const uint32_t high = current.extra >> ((chunk & 1) * 16);  // this half group's eight fields
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t code = (words[j >> 1] >> ((j & 1) * 16)) & 0xffffu;
        const uint32_t signs = code & 0xffu;
        const uint32_t index = (code >> 8) & 63u;
        const uint32_t radius_code = (code >> 14) | (((high >> (2 * j)) & 3u) << 2);
        const float radius = fmaf(static_cast<float>(radius_code), current.scale, current.minimum);
        uint4 direction = lds_u4(book_base + index * 128u);
        // sign of dim 2p in bit 15, of dim 2p+1 in bit 31 of pair p
        direction.x ^= ((signs & 1u) << 15) | ((signs & 2u) << 30);
        direction.y ^= ((signs & 4u) << 13) | ((signs & 8u) << 28);
        direction.z ^= ((signs & 16u) << 11) | ((signs & 32u) << 26);
        direction.w ^= ((signs & 64u) << 9) | ((signs & 128u) << 24);
        const __half2 *d = reinterpret_cast<const __half2 *>(&direction);
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const uint4 xv = *reinterpret_cast<const uint4 *>(x_shared + m * row_halves + chunk * kSphChunkHalves + j * 8);
          const __half2 *xh = reinterpret_cast<const __half2 *>(&xv);
          __half2 dot = __hmul2(d[0], xh[0]);
          dot = __hfma2(d[1], xh[1], dot);
          dot = __hfma2(d[2], xh[2], dot);
          dot = __hfma2(d[3], xh[3], dot);
          const float2 f = __half22float2(dot);
          acc[m] = fmaf(radius, f.x + f.y, acc[m]);
        }
      }
      current = next;
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float total = acc[m];
#pragma unroll
      for (int o = 1; o < L; o <<= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
      if (l == 0 && row_valid && m < rows) y[static_cast<size_t>(m) * n + row] = __float2half_rn(total);
    }
  }
}

// Dense FP16 weight, one thread per 8-weight vector: fp16_rn(float(+-dir) * radius).
__global__ void sph_dequant_kernel(const uint16_t *__restrict__ codes, const uint32_t *__restrict__ extra,
                                   const __half *__restrict__ scales, const __half *__restrict__ mins,
                                   const __half *__restrict__ book, __half *__restrict__ w, long long vectors,
                                   int vectors_per_row) {
  __shared__ __align__(16) __half book_shared[64 * 8];
  for (int i = threadIdx.x; i < 64; i += blockDim.x)
    reinterpret_cast<uint4 *>(book_shared)[i] = __ldg(reinterpret_cast<const uint4 *>(book) + i);
  __syncthreads();
  const long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (v >= vectors) return;
  const long long row = v / vectors_per_row;
  const int vector = static_cast<int>(v - row * vectors_per_row);
  const long long cell = row * (vectors_per_row >> 4) + (vector >> 4);
  const uint32_t code = codes[v];
  const uint32_t radius_code = (code >> 14) | (((__ldg(extra + cell) >> (2 * (vector & 15))) & 3u) << 2);
  const float radius = fmaf(static_cast<float>(radius_code), __half2float(__ldg(scales + cell)),
                            __half2float(__ldg(mins + cell)));
  const __half *direction = book_shared + ((code >> 8) & 63u) * 8;
  __align__(16) __half out[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) {
    const float value = __half2float(direction[d]) * radius;
    out[d] = __float2half_rn((code >> d) & 1u ? -value : value);
  }
  reinterpret_cast<uint4 *>(w)[v] = *reinterpret_cast<const uint4 *>(out);
}

template <int M, int L>
cudaError_t launch_sph_lanes(const __half *x, const uint16_t *codes, const uint32_t *extra, const __half *scales,
                             const __half *mins, const uint4 *book, __half *y, int rows, int n, int k, int sm_count,
                             cudaStream_t stream) {
  const size_t shared = kSphBookBytes + static_cast<size_t>(M) * (k / 64) * kSphChunkHalves * sizeof(__half);
  static bool configured = false;  // per instantiation
  if (!configured) {
    const cudaError_t error = cudaFuncSetAttribute(sph_skinny_kernel<M, L>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (error != cudaSuccess) return error;
    configured = true;
  }
  const int per_sm = shared <= 100 * 1024 ? 2 : 1;
  const int quads = (n + 32 / L - 1) / (32 / L);
  int ctas = (quads + kSphWarps - 1) / kSphWarps;
  if (ctas > sm_count * per_sm) ctas = sm_count * per_sm;
  return launch_dependent(sph_skinny_kernel<M, L>, dim3(ctas), dim3(kSphThreads), shared, stream, x, codes, extra,
                          scales, mins, book, y, rows, n, k);
}

// Lanes per output row: as few as keep every SM's warps busy (more rows per warp share the
// activation reads), never more than the row has chunks.
template <int M>
cudaError_t launch_sph(const __half *x, const uint16_t *codes, const uint32_t *extra, const __half *scales,
                       const __half *mins, const uint4 *book, __half *y, int rows, int n, int k, int sm_count,
                       cudaStream_t stream) {
  const long long warps = static_cast<long long>(sm_count) * kSphWarps;
  const int chunks = k / 64;
  if (chunks >= 32 && static_cast<long long>(n) < warps * 2)
    return launch_sph_lanes<M, 32>(x, codes, extra, scales, mins, book, y, rows, n, k, sm_count, stream);
  if (chunks >= 16 && static_cast<long long>(n) < warps * 4)
    return launch_sph_lanes<M, 16>(x, codes, extra, scales, mins, book, y, rows, n, k, sm_count, stream);
  return launch_sph_lanes<M, 8>(x, codes, extra, scales, mins, book, y, rows, n, k, sm_count, stream);
}

int sph_sm_count() {
  static int count = 0;
  if (count == 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      count = 148;
  }
  return count;
}

}  // namespace
}  // namespace sageb200

extern "C" {

int sageb200_sph_linear(const void *x, const void *codes, const void *extra, const void *scales,
                        const void *mins, const void *book, void *y, int rows, int n, int k, void *stream) {
  using namespace sageb200;
  if (rows < 0 || n <= 0 || k <= 0 || k % 128 || k / 128 > 128) return SAGEB200_ERR_INVALID_ARGUMENT;
  if (rows > 65535) return SAGEB200_ERR_RANGE;
  if (rows == 0) return SAGEB200_OK;
  if (!x || !codes || !extra || !scales || !mins || !book || !y) return SAGEB200_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(book) & 15) ||
      (reinterpret_cast<uintptr_t>(extra) & 3) || (reinterpret_cast<uintptr_t>(x) & 1))
    return SAGEB200_ERR_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int sm_count = sph_sm_count();
  if (rows >= 33 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(y) & 1) == 0) {
    // Prompt-sized calls: the tcgen05 GEMM with this format's decode (no permutation, so the
    // activations are used where they lie; no scratch in this interface, so K is not split).
    int *status_word = nullptr;
    int device_sms = 0;
    const int state = acquire_device(&status_word, &device_sms);
    if (state != SAGEB200_OK) return state;
    const GemmPlan plan = plan_gemm_tc(rows, n, k, device_sms, false);
    if (launch_gemm_tc(static_cast<const __half *>(x), static_cast<const uint32_t *>(codes),
                       static_cast<const uint32_t *>(extra), static_cast<const uint32_t *>(scales),
                       static_cast<const uint32_t *>(book), static_cast<__half *>(y), status_word, rows, n, k, 64,
                       plan, s, nullptr, nullptr, static_cast<const __half *>(mins)) != cudaSuccess) {
      cudaGetLastError();
      return SAGEB200_ERR_CUDA;
    }
    count_launches(1);
    return SAGEB200_OK;
  }
  // activation rows per pass: as many as fit shared memory, at most eight
  int per_pass = 8;
  while (per_pass > 1 && kSphBookBytes + static_cast<size_t>(per_pass) * (k / 64) * kSphChunkHalves * 2 > 192 * 1024)
    per_pass >>= 1;
  for (int first = 0; first < rows; first += per_pass) {
    const int count = rows - first < per_pass ? rows - first : per_pass;
    const __half *xp = static_cast<const __half *>(x) + static_cast<size_t>(first) * k;
    __half *yp = static_cast<__half *>(y) + static_cast<size_t>(first) * n;
    const auto *c = static_cast<const uint16_t *>(codes);
    const auto *e = static_cast<const uint32_t *>(extra);
    const auto *sc = static_cast<const __half *>(scales);
    const auto *mn = static_cast<const __half *>(mins);
    const auto *bk = static_cast<const uint4 *>(book);
    cudaError_t error;
    if (count == 1) error = launch_sph<1>(xp, c, e, sc, mn, bk, yp, count, n, k, sm_count, s);
    else if (count == 2) error = launch_sph<2>(xp, c, e, sc, mn, bk, yp, count, n, k, sm_count, s);
    else if (count <= 4) error = launch_sph<4>(xp, c, e, sc, mn, bk, yp, count, n, k, sm_count, s);
    else error = launch_sph<8>(xp, c, e, sc, mn, bk, yp, count, n, k, sm_count, s);
    if (error != cudaSuccess) return SAGEB200_ERR_CUDA;
  }
  return cudaGetLastError() == cudaSuccess ? SAGEB200_OK : SAGEB200_ERR_CUDA;
}

int sageb200_sph_dequant(const void *codes, const void *extra, const void *scales, const void *mins,
                         const void *book, void *w, int n, int k, void *stream) {
  using namespace sageb200;
  if (n <= 0 || k <= 0 || k % 128) return SAGEB200_ERR_INVALID_ARGUMENT;
  if (!codes || !extra || !scales || !mins || !book || !w) return SAGEB200_ERR_INVALID_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(book) & 15)) return SAGEB200_ERR_ALIGNMENT;
  const long long vectors = static_cast<long long>(n) * (k / 8);
  const unsigned blocks = static_cast<unsigned>((vectors + 255) / 256);
  sph_dequant_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t *>(codes), static_cast<const uint32_t *>(extra),
      static_cast<const __half *>(scales), static_cast<const __half *>(mins), static_cast<const __half *>(book),
      static_cast<__half *>(w), vectors, k / 8);
  return cudaGetLastError() == cudaSuccess ? SAGEB200_OK : SAGEB200_ERR_CUDA;
}

}  // extern "C"
