/* Block-float (bfp8 / bfp4) quantisation in plain C: a restatement of the reference's numpy model
 * models/gpt2.py:16-32 (bf16_bits with round-to-nearest-even, then per run of 16 the largest biased exponent,
 * magnitudes shifted down to it and rounded half up into 7 bits, or to the nearest 3 bits with ties up).
 * TEST INFRASTRUCTURE ONLY: it exists so that whole weight matrices can be checked and the CPU baseline's weights
 * prepared in seconds where numpy takes minutes.  Pinned against the reference by tests/test_oracle.py (it must
 * equal oracle/bfp.py, which tests/golden/make_golden.py checked against the reference itself).
 * Build: gcc -O3 -fopenmp -shared -fPIC oracle/bfp_oracle.c -o oracle/_build/libbfp_oracle.so  (oracle/build.py) */
#include <stdint.h>
#include <string.h>

static inline uint32_t bf16_bits(float f) { /* models/gpt2.py:16-18, packer=False */
  uint32_t u;
  memcpy(&u, &f, 4);
  return (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
}

/* src: rows x cols floats (cols a multiple of 16); dst: the values the block float holds, as floats.
 * fmt: 8 or 4.  Each value is +-q * 2^(top-133), exactly representable in a float unless it is below 2^-149. */
void bfp_values(const float* src, float* dst, int64_t rows, int64_t cols, int fmt) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t c0 = 0; c0 < cols; c0 += 16) {
      uint32_t bits[16], top = 0;
      for (int j = 0; j < 16; ++j) {
        bits[j] = bf16_bits(src[r * cols + c0 + j]);
        uint32_t e = (bits[j] >> 7) & 255u;
        if (e > top) top = e;
      }
      for (int j = 0; j < 16; ++j) {
        uint32_t e = (bits[j] >> 7) & 255u, m = (bits[j] & 127u) | (e ? 128u : 0u);
        uint32_t shift = top - e < 8 ? top - e : 8;
        uint32_t q;
        if (fmt == 8) {
          q = (m + (1u << shift)) >> (shift + 1);
          if (q > 127) q = 127;
        } else {
          q = shift < 4 ? (m + (16u << shift)) >> (shift + 5) : 0;
          if (q > 7) q = 7;
          q <<= 4;
        }
        /* q * 2^(top-133) built as a double scale, then narrowed: exact (q has at most 7 bits) */
        double v = (double)q;
        int ex = (int)top - 133;
        while (ex > 0) { v *= 2.0; --ex; }
        while (ex < 0) { v *= 0.5; ++ex; }
        dst[r * cols + c0 + j] = (float)((bits[j] >> 15) ? -v : v);
      }
    }
  }
}
