// Packed block-float layout (see include/ferrite_b200.h) and the in-register unpack to bf16 pairs.
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

// Where a value sits in its run's bytes.  A magnitude and ITS OWN sign do not share a byte (or nibble): the sign is
// parked one byte (three nibbles) further up, cyclically, so that masking a word - or the word rotated - leaves two
// values in the two halves of a register with each sign already on bit 15 / 31 and each magnitude on the low bits:
//   bfp8, word h of a run = columns 4h..4h+3:  byte0 = mag(c0) | sign(c3)<<7,  byte1 = mag(c2) | sign(c0)<<7,
//                                              byte2 = mag(c1) | sign(c2)<<7,  byte3 = mag(c3) | sign(c1)<<7
//   bfp4, word h of a run = columns 8h..8h+7:  nibble p = mag3(v_p) | sign(v_(p-3 mod 8))<<3, v_p = column 2*(p%4) + p/4
__host__ __device__ inline int bfp4_nibble_of_column(int j) {  // j in 0..7 -> p
  return (j >> 1) + ((j & 1) << 2);
}
__host__ __device__ inline int bfp8_byte_of_column(int j) {  // j in 0..3 -> the byte that holds its magnitude
  return j == 0 ? 0 : j == 1 ? 2 : j == 2 ? 1 : 3;
}

// Round a run of 16 bf16 values (their bits) to the block float and store it as run b of row k of the packed matrix at
// `base` (K rows).  Integer arithmetic only; bit-exact with the reference's numpy model (models/gpt2.py:21-32): the
// largest biased exponent is shared, magnitudes are the mantissas (hidden one included) shifted down to it and
// rounded half up into 7 bits (bfp8) or to the nearest 3 bits, ties up (bfp4); a zero carries no sign.
template <int FMT>
__device__ __forceinline__ void store_run(const uint32_t bits[16], uint8_t* base, int64_t K, int64_t b, int64_t k) {
  uint32_t top = 0;
#pragma unroll
  for (int j = 0; j < 16; ++j) top = max(top, (bits[j] >> 7) & 255u);
  base[exp_offset(FMT, K, b, k)] = (uint8_t)top;
  if (FMT == FB_BFP8) {
    uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      uint32_t e = (bits[j] >> 7) & 255u, m = (bits[j] & 127u) | (e ? 128u : 0u);
      uint32_t shift = min(top - e, 8u);
      uint32_t q = min((m + (1u << shift)) >> (shift + 1), 127u);
      uint32_t sign = q ? bits[j] >> 15 : 0u;
      const int at = bfp8_byte_of_column(j & 3);  // the magnitude's byte; the sign goes on top of the next byte up
      out[j >> 2] |= (q << (8 * at)) | (sign << (8 * ((at + 1) & 3) + 7));
    }
    *reinterpret_cast<uint4*>(base + mant_offset(FMT, K, b, k)) = make_uint4(out[0], out[1], out[2], out[3]);
  } else {
    uint32_t out[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      uint32_t e = (bits[j] >> 7) & 255u, m = (bits[j] & 127u) | (e ? 128u : 0u);
      uint32_t shift = min(top - e, 8u);
      uint32_t q = shift < 4 ? min((m + (16u << shift)) >> (shift + 5), 7u) : 0u;
      uint32_t sign = q ? bits[j] >> 15 : 0u;
      const int at = bfp4_nibble_of_column(j & 7);  // the magnitude's nibble; the sign tops the nibble three up
      out[j >> 3] |= (q << (4 * at)) | (sign << (4 * ((at + 3) & 7) + 3));
    }
    *reinterpret_cast<uint2*>(base + mant_offset(FMT, K, b, k)) = make_uint2(out[0], out[1]);
  }
}

// The unpack never converts integers to floats and never touches the sign.  A magnitude sitting in the mantissa
// field of a bf16 whose exponent field is zero IS a number: the subnormal mag * 2^-133.  The block float's value is
// +-mag * 2^(top-133) (models/gpt2.py:31-32), i.e. that subnormal times 2^top: two exact packed multiplications by
// powers of two (2^126, then 2^(top-126); one would overflow bf16's exponent), two values per instruction, the sign bit
// riding along.  Per four bfp8 values: two masks and one rotate on the integer pipe, four multiplies on the FMA pipe.
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
constexpr uint32_t TWO_126_X2 = 0x7E807E80u;
// bf16 pair 2^(top-126) (bfp8) / 2^(top-122) (bfp4: its 3-bit magnitude stands 4 bits higher)
__device__ __forceinline__ uint32_t scale8(uint32_t top) { return ((top + 1) << 7) * 0x10001u; }
__device__ __forceinline__ uint32_t scale4(uint32_t top) { return ((top + 5) << 7) * 0x10001u; }

// Four bfp8 bytes (columns j..j+3 of a run) -> two registers of bf16 pairs (j, j+1) and (j+2, j+3).
__device__ __forceinline__ void unpack8_word(uint32_t w, uint32_t s2, uint32_t& lo, uint32_t& hi) {
  uint32_t a, r, b;
  asm("lop3.b32 %0, %1, 0x807F807F, 0, 0xC0;" : "=r"(a) : "r"(w));
  asm("shf.r.wrap.b32 %0, %1, %1, 8;" : "=r"(r) : "r"(w));
  asm("lop3.b32 %0, %1, 0x807F807F, 0, 0xC0;" : "=r"(b) : "r"(r));
  lo = mul_bf16x2(mul_bf16x2(a, TWO_126_X2), s2);
  hi = mul_bf16x2(mul_bf16x2(b, TWO_126_X2), s2);
}

// One bfp4 word (8 columns) -> four registers of bf16 pairs (0,1) (2,3) (4,5) (6,7).
__device__ __forceinline__ void unpack4_word(uint32_t w, uint32_t s2, uint32_t out[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t r = w, m;
    if (i) asm("shf.r.wrap.b32 %0, %1, %1, %2;" : "=r"(r) : "r"(w), "r"(4 * i));
    asm("lop3.b32 %0, %1, 0x80078007, 0, 0xC0;" : "=r"(m) : "r"(r));
    out[i] = mul_bf16x2(mul_bf16x2(m, TWO_126_X2), s2);
  }
}

// The masked words alone (no multiplies): each half of a register is a column's sign and magnitude standing where a
// bf16 subnormal's are, i.e. half << 16 read as an fp32 is the (fp32-denormal) number +-mag * 2^-133 (bfp4: its 3-bit
// magnitude m, for a value of +-16m * 2^(top-133)).  A consumer that multiplies by an fp32 anyway folds 2^top into that
// factor and needs no unpack arithmetic at all.  Eight registers per run: columns 2i, 2i+1 in register i.
template <int FMT>
__device__ __forceinline__ void mask_run(const uint32_t* words, uint32_t m[8]) {
  if (FMT == FB_BFP8) {
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      uint32_t r;
      asm("lop3.b32 %0, %1, 0x807F807F, 0, 0xC0;" : "=r"(m[2 * h]) : "r"(words[h]));
      asm("shf.r.wrap.b32 %0, %1, %1, 8;" : "=r"(r) : "r"(words[h]));
      asm("lop3.b32 %0, %1, 0x807F807F, 0, 0xC0;" : "=r"(m[2 * h + 1]) : "r"(r));
    }
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        uint32_t r = words[h];
        if (i) asm("shf.r.wrap.b32 %0, %1, %1, %2;" : "=r"(r) : "r"(words[h]), "r"(4 * i));
        asm("lop3.b32 %0, %1, 0x80078007, 0, 0xC0;" : "=r"(m[4 * h + i]) : "r"(r));
      }
  }
}

// A whole run of 16 columns as eight bf16-pair registers (columns 2i, 2i+1 in register i).
__device__ __forceinline__ void unpack_run8(uint4 raw, uint32_t top, uint32_t v[8]) {
  const uint32_t s2 = scale8(top);
  unpack8_word(raw.x, s2, v[0], v[1]);
  unpack8_word(raw.y, s2, v[2], v[3]);
  unpack8_word(raw.z, s2, v[4], v[5]);
  unpack8_word(raw.w, s2, v[6], v[7]);
}
__device__ __forceinline__ void unpack_run4(uint2 raw, uint32_t top, uint32_t v[8]) {
  const uint32_t s2 = scale4(top);
  unpack4_word(raw.x, s2, v);
  unpack4_word(raw.y, s2, v + 4);
}

}  // namespace fb
