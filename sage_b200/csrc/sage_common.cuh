// Shared device helpers for the SAGE packed-weight kernels (sm_100a).
//
// Bit layout of one 16-bit code (reference weight_vq/sphquant/packing.py:43-50):
//   bits 0-7        sign of dims 0-7 (1 = negative)
//   bits 8..8+D-1   direction-codebook index, D = log2(entries) in {6,7,8}
//   bits 8+D..15    low 8-D bits of the radius code
// The two high radius bits of vector v sit in bits 2v, 2v+1 of the row's radius word
// (packing.py:51).  radius = fmaf(code, step, min) in FP32 and
// weight = fp16_rn(float(+-dir) * radius) (reference csrc/sage/sage_gemm_cuda.cu:117-131).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sageb200 {

__host__ __device__ inline int direction_bits_of(int entries) {
  return entries == 64 ? 6 : entries == 128 ? 7 : entries == 256 ? 8 : -1;
}

// Streaming 64-/32-/128-bit loads of packed weights: read once, keep out of L1.
__device__ __forceinline__ uint2 ldg_stream_u2(const void *p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
               : "=r"(v.x), "=r"(v.y)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u1(const void *p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_stream_u4(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint4 lds_u4(uint32_t shared_address) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(shared_address));
  return v;
}
__device__ __forceinline__ void sts_u4(uint32_t shared_address, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(shared_address), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w));
}

// Programmatic dependent launch.  A kernel calls pdl_launch_dependents() as early as it
// likes (the next kernel in the stream may then be scheduled while this one still runs) and
// pdl_wait() before its first read of anything an earlier kernel wrote and before its first
// global write; pdl_wait() returns once all earlier kernels have completed and flushed.
// Both are no-ops for kernels launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Host side: launch `kernel` allowing it to start before the previous kernel of `stream`
// has finished (the kernel must follow the protocol above).
// `kBit` names the kernel family: 1 = packed-linear kernels, 2 = decode glue.
extern int g_sageb200_pdl;  // bit mask of families launched this way; 0: plain launches
extern unsigned long long g_sageb200_glue_launches;  // decode-glue kernels launched (bench bookkeeping)
template <int kBit = 1, typename... KernelArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t shared,
                                    cudaStream_t stream, Args &&...args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = (g_sageb200_pdl & kBit) ? 1 : 0;
  if (kBit == 2) __atomic_fetch_add(&g_sageb200_glue_launches, 1ull, __ATOMIC_RELAXED);
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// silu(g) = g / (1 + e^-g) with the fast exponential and the fast division, the same in every
// kernel that computes it (the fused and the stand-alone SwiGLU must round alike).
__device__ __forceinline__ float silu_fast(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

__device__ __forceinline__ long long global_nanoseconds() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_address(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Exact dequantisation of one code into eight FP16 values (as four half2 words).
// `book` points at the planar [4][entries] half2 codebook (global or shared).
__device__ __forceinline__ void dequant_vector_exact(uint32_t code, uint32_t radius_word,
                                                     int vector, float minimum, float step,
                                                     const uint32_t *book, int entries,
                                                     int dbits, uint32_t out[4]) {
  const uint32_t index = (code >> 8) & static_cast<uint32_t>(entries - 1);
  const uint32_t rc =
      (code >> (8 + dbits)) | (((radius_word >> (2 * vector)) & 3u) << (8 - dbits));
  const float radius = fmaf(static_cast<float>(rc), step, minimum);
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    uint32_t bits = book[p * entries + index];
    bits ^= (((code >> (2 * p)) & 1u) << 15) | (((code >> (2 * p + 1)) & 1u) << 31);
    const float2 d = __half22float2(*reinterpret_cast<const __half2 *>(&bits));
    const __half2 w = __floats2half2_rn(d.x * radius, d.y * radius);
    out[p] = *reinterpret_cast<const uint32_t *>(&w);
  }
}

}  // namespace sageb200
