// Per-unit arithmetic of the SAGE decode kernel: one (16-row tile, 128-channel group)
// unit from registers/shared memory into mma.sync accumulators.  Kept in a header so the
// kernel and its micro-benchmarks share one definition.
#pragma once

#include "sage_common.cuh"

namespace sageb200 {

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
      "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// a ^ (b & c): one LOP3 (truth table 0x78)
__device__ __forceinline__ uint32_t xor_and(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x78;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// (a & b) | c: one LOP3 (truth table 0xEA)
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// byte kIndex of a, zero extended: one PRMT
template <int kIndex>
__device__ __forceinline__ uint32_t byte_of(uint32_t a) {
  uint32_t d;
  asm("prmt.b32 %0, %1, 0, %2;" : "=r"(d) : "r"(a), "n"(0x4440 | kIndex));
  return d;
}

// Bit-field constants that depend on the direction-bit count D, hoisted per problem.
struct FieldConsts {
  uint32_t index_mask;   // (entries-1) << 7: entry stride is 128 bytes (8 replicas)
  uint32_t hi_mask;      // 3 << (27 - D): the two high radius bits at mantissa position
  uint32_t hi_shift;     // 27 - D
  uint32_t lo_mask;      // ((1 << (8-D)) - 1) << 19: the low radius bits at mantissa position
  uint32_t lo_left;      // 11 - D: low code's radius bits -> bit 19
  uint32_t lo_right;     // 5 + D: high code's radius bits -> bit 19
};

// One unit (16 rows x 128 channels) into the accumulators.
//   code/radius_word/endpoints: this lane's words for rows g and g+8
//   x_row[nb]: this lane's activation row at this group in shared memory (16t bytes in)
//   kLowBits: the code carries low radius bits (64 or 128 codebook entries); with 256
//             entries the two high bits are the whole radius code
template <int NB, bool kLowBits>
__device__ __forceinline__ void compute_unit(const uint2 (&code)[2], const uint32_t (&radius_word)[2],
                                             const uint32_t (&endpoints)[2], float (&acc)[NB][4],
                                             const FieldConsts &f, const unsigned char *book,
                                             uint32_t lane_offset,
                                             const unsigned char *const (&x_row)[NB], int t) {
  float step16[2], base[2];
  uint32_t high[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float2 e = __half22float2(*reinterpret_cast<const __half2 *>(&endpoints[h]));
    step16[h] = e.y * 16.0f;
    base[h] = fmaf(-16.0f, e.y, e.x);
    high[h] = (radius_word[h] >> (8 * t)) << f.hi_shift;
  }
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    uint32_t a[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t word = (s < 2) ? code[h].x : code[h].y;
      uint32_t offset, signs, low = 0x3f800000u;
      if (s & 1) {
        offset = and_or(word >> 17, f.index_mask, lane_offset);
        signs = byte_of<2>(word);
        if constexpr (kLowBits) low = and_or(word >> f.lo_right, f.lo_mask, 0x3f800000u);
      } else {
        offset = and_or(word >> 1, f.index_mask, lane_offset);
        signs = byte_of<0>(word);
        if constexpr (kLowBits) low = and_or(word << f.lo_left, f.lo_mask, 0x3f800000u);
      }
      // entry offset and replica offset never overlap (OR); the static array's base is a
      // link-time constant and folds into the load's immediate
      const uint4 dir = *reinterpret_cast<const uint4 *>(book + offset);
      // 1 + code/16 as FP32 bits: high radius bits and low radius bits at mantissa positions
      const uint32_t radius_bits = and_or(s ? high[h] >> (2 * s) : high[h], f.hi_mask, low);
      const float radius = fmaf(__uint_as_float(radius_bits), step16[h], base[h]);
      const __half2 rr = __floats2half2_rn(radius, radius);
      // sign bit 2p -> bit 15 and sign bit 2p+1 -> bit 31 of half2 word p: one multiply by
      // (1 + 2^15) << (15 - 2p) each (integer multiplies run beside the logic pipe)
      const uint32_t d[4] = {xor_and(dir.x, signs * 0x40008000u, 0x80008000u),
                             xor_and(dir.y, signs * 0x10002000u, 0x80008000u),
                             xor_and(dir.z, signs * 0x04000800u, 0x80008000u),
                             xor_and(dir.w, signs * 0x01000200u, 0x80008000u)};
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const __half2 w = __hmul2(*reinterpret_cast<const __half2 *>(&d[p]), rr);
        a[h][p] = *reinterpret_cast<const uint32_t *>(&w);
      }
    }
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const uint4 b = *reinterpret_cast<const uint4 *>(x_row[nb] + s * 64);
      mma_16816(acc[nb], a[0][0], a[1][0], a[0][1], a[1][1], b.x, b.y);
      mma_16816(acc[nb], a[0][2], a[1][2], a[0][3], a[1][3], b.z, b.w);
    }
  }
}

// 16-byte shared-memory load by 32-bit address that the compiler may schedule early: not
// `volatile` (so it can move across arithmetic and the MMAs), "memory" clobber (so it stays on
// its side of barriers and mbarrier waits).
__device__ __forceinline__ uint4 lds_u4_early(uint32_t shared_address) {
  uint4 v;
  asm("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "r"(shared_address)
      : "memory");
  return v;
}

// The same unit for ONE activation row with every operand named by its 32-bit shared-memory
// address (ld.shared explicitly: no generic addressing, no 64-bit pointer arithmetic):
//   book_lane  address of the replicated codebook + this lane's replica offset
//   x_lane     address of the staged activation row at this group + 16 * t
template <bool kLowBits>
__device__ __forceinline__ void compute_unit_shared(const uint2 (&code)[2], const uint32_t (&radius_word)[2],
                                                    const uint32_t (&endpoints)[2], float (&acc)[4],
                                                    const FieldConsts &f, uint32_t book_lane, uint32_t x_lane,
                                                    int t) {
  float step16[2], base[2];
  uint32_t high[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float2 e = __half22float2(*reinterpret_cast<const __half2 *>(&endpoints[h]));
    step16[h] = e.y * 16.0f;
    base[h] = fmaf(-16.0f, e.y, e.x);
    high[h] = (radius_word[h] >> (8 * t)) << f.hi_shift;
  }
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    uint32_t a[2][4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t word = (s < 2) ? code[h].x : code[h].y;
      uint32_t offset, signs, low = 0x3f800000u;
      if (s & 1) {
        offset = (word >> 17) & f.index_mask;
        signs = byte_of<2>(word);
        if constexpr (kLowBits) low = and_or(word >> f.lo_right, f.lo_mask, 0x3f800000u);
      } else {
        offset = (word >> 1) & f.index_mask;
        signs = byte_of<0>(word);
        if constexpr (kLowBits) low = and_or(word << f.lo_left, f.lo_mask, 0x3f800000u);
      }
      const uint4 dir = lds_u4_early(book_lane + offset);
      const uint32_t radius_bits = and_or(s ? high[h] >> (2 * s) : high[h], f.hi_mask, low);
      const float radius = fmaf(__uint_as_float(radius_bits), step16[h], base[h]);
      const __half2 rr = __floats2half2_rn(radius, radius);
      const uint32_t d[4] = {xor_and(dir.x, signs * 0x40008000u, 0x80008000u),
                             xor_and(dir.y, signs * 0x10002000u, 0x80008000u),
                             xor_and(dir.z, signs * 0x04000800u, 0x80008000u),
                             xor_and(dir.w, signs * 0x01000200u, 0x80008000u)};
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const __half2 w = __hmul2(*reinterpret_cast<const __half2 *>(&d[p]), rr);
        a[h][p] = *reinterpret_cast<const uint32_t *>(&w);
      }
    }
    const uint4 b = lds_u4_early(x_lane + s * 64);
    mma_16816(acc, a[0][0], a[1][0], a[0][1], a[1][1], b.x, b.y);
    mma_16816(acc, a[0][2], a[1][2], a[0][3], a[1][3], b.z, b.w);
  }
}

}  // namespace sageb200
