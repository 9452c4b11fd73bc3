// C entry points over the reference project's own SAGE launchers, so that the
// UNMODIFIED reference kernels (csrc/sage/sage_gemv_cuda.cu, sage_gemm_cuda.cu,
// compiled from the reference checkout by oracle/Makefile) can be run beside this
// repo's kernels as a same-GPU comparator.  TEST/BENCH INFRASTRUCTURE ONLY.
//
// The dispatch below follows csrc/bindings.cpp:49-76 of the reference: rows < 16
// goes to sage_gemv_cuda (gather fused only when sage_gemv_fuses_permutation says
// so; otherwise the caller must pass pre-gathered input), larger inputs go to
// sage_gemm_cuda with a caller-supplied FP32 split-K workspace.
#include "sage_gemv_cuda.h"

extern "C" int sage_ref_fuses_permutation(int n, int k) {
  return sage_gemv_fuses_permutation(n, k) ? 1 : 0;
}

extern "C" int sage_ref_gemm_splits(int rows, int n, int k, int sm_count) {
  return sage_gemm_splits(rows, n, k, sm_count);
}

// input must already be in quantised channel order when perm == nullptr.
extern "C" int sage_ref_gemv(const void *input, const void *codes, const void *radii,
                             const void *grid, const void *book, void *output,
                             const int32_t *perm, int rows, int n, int k, int entries,
                             void *stream) {
  sage_gemv_cuda(static_cast<const half *>(input), static_cast<const uint32_t *>(codes),
                 static_cast<const uint32_t *>(radii), static_cast<const half2 *>(grid),
                 static_cast<const uint32_t *>(book), static_cast<half *>(output), perm, rows, n,
                 k, entries, static_cast<cudaStream_t>(stream));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sage_ref_gemm(const void *input, const void *codes, const void *radii,
                             const void *grid, const void *book, void *output, float *workspace,
                             int parts, int rows, int n, int k, int entries, void *stream) {
  sage_gemm_cuda(static_cast<const half *>(input), static_cast<const uint32_t *>(codes),
                 static_cast<const uint32_t *>(radii), static_cast<const half2 *>(grid),
                 static_cast<const uint32_t *>(book), static_cast<half *>(output), workspace,
                 parts, rows, n, k, entries, static_cast<cudaStream_t>(stream));
  return static_cast<int>(cudaGetLastError());
}
