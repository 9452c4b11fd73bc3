/*
 * CPU oracle for the SAGE packed-weight matmul, plain C.  TEST INFRASTRUCTURE ONLY.
 *
 * A restatement of the arithmetic the reference project defines for its packed
 * SAGE linear; used to check the CUDA kernels and as the timed CPU baseline.
 * Nothing in the sage_b200 package links or calls this file.
 *
 * Parity status: PINNED (tests/test_oracle.py compares every function here with
 * the numpy oracle and with golden vectors generated from the reference's own
 * Python decoder).
 *
 * Reference sources followed, by path inside the reference project:
 *   tests/inference/reference.py:25-49    field unpack and decode
 *   csrc/sage/sage_gemm_cuda.cu:117-131   radius = fma(code, step, min) in FP32,
 *                                         weight = fp16_rn(float(+-dir) * radius)
 *   csrc/sage/sage_gemv_cuda.h:7-13       buffer shapes
 *   tests/inference/test_sage.py:113-122  FP32 matmul on FP16-rounded weights
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static float half_bits_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exponent = (h >> 10) & 0x1fu;
  uint32_t mantissa = h & 0x3ffu;
  uint32_t bits;
  if (exponent == 0) {
    if (mantissa == 0) {
      bits = sign;
    } else { /* subnormal: normalise */
      int shift = 0;
      while (!(mantissa & 0x400u)) {
        mantissa <<= 1;
        ++shift;
      }
      mantissa &= 0x3ffu;
      bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (mantissa << 13);
    }
  } else if (exponent == 31) {
    bits = sign | 0x7f800000u | (mantissa << 13);
  } else {
    bits = sign | ((exponent + 127 - 15) << 23) | (mantissa << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* float -> half, round to nearest even (same rounding as __float2half_rn / .half()). */
static uint16_t float_to_half_bits(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7fffffffu;
  if (absx >= 0x7f800000u) /* inf / nan */
    return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x200u : 0));
  if (absx >= 0x477ff000u) /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7c00u);
  if (absx < 0x33000001u) /* below half of the smallest subnormal -> 0 */
    return (uint16_t)sign;
  int32_t exponent = (int32_t)(absx >> 23) - 127;
  uint32_t mantissa = (absx & 0x7fffffu) | 0x800000u;
  uint32_t shift;
  uint32_t result_exp;
  if (exponent < -14) { /* subnormal half */
    shift = (uint32_t)(13 + (-14 - exponent));
    result_exp = 0;
  } else {
    shift = 13;
    result_exp = (uint32_t)(exponent + 15);
  }
  uint32_t kept = mantissa >> shift;
  uint32_t rest = mantissa & ((1u << shift) - 1u);
  uint32_t halfway = 1u << (shift - 1);
  if (rest > halfway || (rest == halfway && (kept & 1u))) ++kept;
  /* kept carries the implicit bit for normals; adding handles mantissa overflow */
  uint32_t out = (result_exp == 0) ? kept : ((result_exp - 1) << 10) + kept;
  return (uint16_t)(sign | out);
}

static int direction_bits(int entries) {
  return entries == 64 ? 6 : entries == 128 ? 7 : entries == 256 ? 8 : -1;
}

/* Decode one output row into FP16 bits, columns in QUANTISED order. */
static void decode_row(const uint32_t *codes, const uint32_t *radii, const uint16_t *grid,
                       const uint16_t *book, int row, int groups, int entries, int dbits,
                       uint16_t *out) {
  const int tile = row >> 4, r = row & 15;
  for (int g = 0; g < groups; ++g) {
    const size_t cell = ((size_t)tile * groups + g) * 16 + r;
    const uint32_t *words = codes + cell * 8;
    const uint32_t extra = radii[cell];
    const float minimum = half_bits_to_float(grid[cell * 2]);
    const float step = half_bits_to_float(grid[cell * 2 + 1]);
    for (int v = 0; v < 16; ++v) {
      const uint32_t code = (words[v >> 1] >> (16 * (v & 1))) & 0xffffu;
      const uint32_t index = (code >> 8) & (uint32_t)(entries - 1);
      const uint32_t rc = (code >> (8 + dbits)) | (((extra >> (2 * v)) & 3u) << (8 - dbits));
      /* product of a <=4-bit integer and an 11-bit significand is exact in FP32,
         so mul+add rounds once, exactly like fmaf in the reference kernels */
      const float radius = minimum + (float)rc * step;
      for (int d = 0; d < 8; ++d) {
        float dir = half_bits_to_float(book[((size_t)(d >> 1) * entries + index) * 2 + (d & 1)]);
        if ((code >> d) & 1u) dir = -dir;
        out[(size_t)g * 128 + v * 8 + d] = float_to_half_bits(dir * radius);
      }
    }
  }
}

/*
 * out[n][k] = FP16 bits of the dequantised weight.  perm == NULL leaves the
 * columns in quantised order; otherwise out[row][perm[j]] = w_q[row][j].
 * Returns 0, or -1 on an invalid argument.
 */
int sage_oracle_decode_fp16(const uint32_t *codes, const uint32_t *radii, const uint16_t *grid,
                            const uint16_t *book, const int32_t *perm, int n, int k, int entries,
                            uint16_t *out) {
  const int dbits = direction_bits(entries);
  if (dbits < 0 || n <= 0 || k <= 0 || (k % 128)) return -1;
  const int groups = k / 128;
  int failed = 0;
#pragma omp parallel
  {
    uint16_t *scratch = (uint16_t *)malloc((size_t)k * sizeof(uint16_t));
    if (!scratch) {
#pragma omp atomic write
      failed = 1;
    }
#pragma omp for schedule(static)
    for (int row = 0; row < n; ++row) {
      if (!scratch) continue;
      if (!perm) {
        decode_row(codes, radii, grid, book, row, groups, entries, dbits, out + (size_t)row * k);
      } else {
        decode_row(codes, radii, grid, book, row, groups, entries, dbits, scratch);
        for (int j = 0; j < k; ++j) out[(size_t)row * k + perm[j]] = scratch[j];
      }
    }
    free(scratch);
  }
  return failed ? -2 : 0;
}

/*
 * The reference CPU path: y[rows][n] (FP32) = x.float() @ W16.float().T with W16 the
 * FP16-rounded dequantised weight in original channel order.
 * x is FP16 bits [rows][k].  threads <= 0 keeps the OpenMP default.
 */
int sage_oracle_linear(const uint16_t *x, const uint32_t *codes, const uint32_t *radii,
                       const uint16_t *grid, const uint16_t *book, const int32_t *perm, float *y,
                       int rows, int n, int k, int entries, int threads) {
  const int dbits = direction_bits(entries);
  if (dbits < 0 || n <= 0 || k <= 0 || (k % 128) || rows < 0) return -1;
  const int groups = k / 128;
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
#else
  (void)threads;
#endif
  float *xf = (float *)malloc((size_t)(rows > 0 ? rows : 1) * k * sizeof(float));
  if (!xf) return -2;
  for (size_t i = 0; i < (size_t)rows * k; ++i) xf[i] = half_bits_to_float(x[i]);
  int failed = 0;
#pragma omp parallel
  {
    uint16_t *wq = (uint16_t *)malloc((size_t)k * sizeof(uint16_t));
    float *w = (float *)malloc((size_t)k * sizeof(float));
    if (!wq || !w) {
#pragma omp atomic write
      failed = 1;
    }
#pragma omp for schedule(static)
    for (int row = 0; row < n; ++row) {
      if (!wq || !w) continue;
      decode_row(codes, radii, grid, book, row, groups, entries, dbits, wq);
      if (perm) {
        for (int j = 0; j < k; ++j) w[perm[j]] = half_bits_to_float(wq[j]);
      } else {
        for (int j = 0; j < k; ++j) w[j] = half_bits_to_float(wq[j]);
      }
      for (int m = 0; m < rows; ++m) {
        const float *xr = xf + (size_t)m * k;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int j = 0; j < k; j += 8)
          for (int c = 0; c < 8; ++c) acc[c] += xr[j + c] * w[j + c];
        y[(size_t)m * n + row] =
            ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
      }
    }
    free(wq);
    free(w);
  }
  free(xf);
  return failed ? -2 : 0;
}

int sage_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
