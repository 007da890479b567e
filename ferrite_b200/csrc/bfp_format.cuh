// Packed block-float layout (see include/ferrite_b200.h) and the in-register unpack to bf16 pairs.
//
// The unpack never converts integers to floats one at a time.  A magnitude is OR-ed into the mantissa
// of the bf16 constant 128.0 (0x4300), which makes the number 128 + mag exactly; one packed bf16x2 FMA
// then computes (128 + mag) * scale - 128 * scale = mag * scale for two values at once.  The scale is a
// power of two, so every step is exact and the result is the block float's value bit for bit
// (models/gpt2.py:31-32 of the reference: +-mag * 2^(top-133)).
#pragma once
#include "common.cuh"

namespace fb {

// A packed matrix is a grid of units: 64 rows of K (KSTEP) x 64 columns (a group of 4 runs).  A unit holds its
// 4 x 64 runs' mantissas, run-major ([run][row][16 or 8 bytes]), then their 4 x 64 shared exponents ([run][row]);
// the units of one column group follow each other along K, so any stretch of K of a 64-column group is one
// contiguous piece of memory: one bulk copy per pipeline stage, and 128-bit loads for a lane walking down K.
constexpr int KSTEP = 64, GROUP_RUNS = 4;
__host__ __device__ constexpr int run_bytes(int fmt) { return fmt == FB_BFP8 ? 16 : 8; }
__host__ __device__ constexpr int unit_mant_bytes(int fmt) { return GROUP_RUNS * KSTEP * run_bytes(fmt); }
__host__ __device__ constexpr int unit_bytes(int fmt) { return unit_mant_bytes(fmt) + GROUP_RUNS * KSTEP; }
__host__ __device__ inline int64_t ksteps_of(int64_t K) { return (K + KSTEP - 1) / KSTEP; }
__host__ __device__ inline int64_t groups_of(int64_t N) { return (N + 16 * GROUP_RUNS - 1) / (16 * GROUP_RUNS); }
__host__ __device__ inline int64_t packed_bytes(int fmt, int64_t K, int64_t N) { return groups_of(N) * ksteps_of(K) * unit_bytes(fmt); }
// byte offsets of run b (= column / 16), row k inside a packed matrix
__host__ __device__ inline int64_t unit_offset(int fmt, int64_t K, int64_t b, int64_t k) {
  return ((b / GROUP_RUNS) * ksteps_of(K) + k / KSTEP) * unit_bytes(fmt);
}
__host__ __device__ inline int64_t mant_offset(int fmt, int64_t K, int64_t b, int64_t k) {
  return unit_offset(fmt, K, b, k) + ((b % GROUP_RUNS) * KSTEP + k % KSTEP) * run_bytes(fmt);
}
__host__ __device__ inline int64_t exp_offset(int fmt, int64_t K, int64_t b, int64_t k) {
  return unit_offset(fmt, K, b, k) + unit_mant_bytes(fmt) + (b % GROUP_RUNS) * KSTEP + k % KSTEP;
}

// Where a bfp4 value sits inside the 8 bytes of its (row, column block): column j of 16 is nibble
// p of word h with j = 8h + 2*(p%4) + p/4, so that masking a word with 0x000F000F yields two neighbouring
// columns in the two halves of a register.
__host__ __device__ inline int bfp4_nibble_of_column(int j) {  // j in 0..7 -> p
  return (j >> 1) + ((j & 1) << 2);
}

// bf16 bit patterns of 2^(top-133) and of -(128 * 2^(top-133)), each in both halves of a register.
struct Scale8 {
  uint32_t s2, c2;
};
__device__ __forceinline__ Scale8 scale8(uint32_t top) {
  uint32_t s = top >= 7 ? (top - 6) << 7 : 1u << top;  // below 2^-126 the scale is a bf16 denormal
  uint32_t c = 0x8000u | ((top + 1) << 7);             // -(2^(top-126))
  return {s * 0x10001u, c * 0x10001u};
}
// bfp4: value = (code - 8) * 2^(top-129): scale 2^(top-129) and -(136 * scale)
__device__ __forceinline__ Scale8 scale4(uint32_t top) {
  uint32_t s = top >= 3 ? (top - 2) << 7 : 1u << (top + 4);
  uint32_t c = 0x8000u | ((top + 5) << 7) | 0x08u;  // -(2^(top-122) * 1.0625)
  return {s * 0x10001u, c * 0x10001u};
}

__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// Four bfp8 bytes (columns j..j+3 of a run) -> two registers of bf16 pairs (j, j+1) and (j+2, j+3).
__device__ __forceinline__ void unpack8_word(uint32_t w, Scale8 sc, uint32_t& lo, uint32_t& hi) {
  uint32_t r0, r1, m, a;
  asm("prmt.b32 %0, %1, %1, 0x9180;" : "=r"(r0) : "r"(w));  // [sign-fill(b1) b1 sign-fill(b0) b0]
  asm("prmt.b32 %0, %1, %1, 0xB3A2;" : "=r"(r1) : "r"(w));  // [sign-fill(b3) b3 sign-fill(b2) b2]
  asm("lop3.b32 %0, %1, 0x807F807F, 0x43004300, 0xEA;" : "=r"(m) : "r"(r0));  // +-(128 + mag)
  asm("lop3.b32 %0, %1, 0x80008000, %2, 0x6A;" : "=r"(a) : "r"(r0), "r"(sc.c2));  // -+128*scale
  lo = fma_bf16x2(m, sc.s2, a);
  asm("lop3.b32 %0, %1, 0x807F807F, 0x43004300, 0xEA;" : "=r"(m) : "r"(r1));
  asm("lop3.b32 %0, %1, 0x80008000, %2, 0x6A;" : "=r"(a) : "r"(r1), "r"(sc.c2));
  hi = fma_bf16x2(m, sc.s2, a);
}

// One bfp4 word (8 columns) -> four registers of bf16 pairs (0,1) (2,3) (4,5) (6,7).
__device__ __forceinline__ void unpack4_word(uint32_t w, Scale8 sc, uint32_t out[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t m;
    asm("lop3.b32 %0, %1, 0x000F000F, 0x43004300, 0xEA;" : "=r"(m) : "r"(w >> (4 * i)));  // 128 + code
    out[i] = fma_bf16x2(m, sc.s2, sc.c2);
  }
}

// A whole run of 16 columns as eight bf16-pair registers (columns 2i, 2i+1 in register i).
__device__ __forceinline__ void unpack_run8(uint4 raw, uint32_t top, uint32_t v[8]) {
  Scale8 sc = scale8(top);
  unpack8_word(raw.x, sc, v[0], v[1]);
  unpack8_word(raw.y, sc, v[2], v[3]);
  unpack8_word(raw.z, sc, v[4], v[5]);
  unpack8_word(raw.w, sc, v[6], v[7]);
}
__device__ __forceinline__ void unpack_run4(uint2 raw, uint32_t top, uint32_t v[8]) {
  Scale8 sc = scale4(top);
  unpack4_word(raw.x, sc, v);
  unpack4_word(raw.y, sc, v + 4);
}

}  // namespace fb
