// Block-float GEMV on CUDA cores: one token (fb_linear sends more to the tensor-core kernel; up to 4 a pass otherwise).
//
// Work split: one column block (16 output columns, one shared-exponent run per row k) per group of warps;
// the group's lanes split K, each lane streaming 4 consecutive rows per step as 64 (bfp8) or 32 (bfp4)
// contiguous bytes plus one 32-bit word of exponents.  Lanes keep 16 fp32 sums per token and the K
// reduction is a butterfly of warp shuffles (16 shuffles per token) followed by one pass through shared
// memory across the group's warps.  The weights are read exactly once, 128 bits at a time.
#pragma once
#include "bfp_format.cuh"

namespace fb {

constexpr float GEMV_ACC_SCALE = 18446744073709551616.f;  // 2^64: gemv_accumulate's sums are kept scaled by 2^-64

template <int FMT>
struct RunBytes { static constexpr int value = FMT == FB_BFP8 ? 16 : 8; };

// raw bytes of 4 consecutive rows of one column block
template <int FMT>
struct Raw4 {
  uint4 q[FMT == FB_BFP8 ? 4 : 2];
  uint32_t tops;
};

// `col` points at the first unit of the run's column group, `run` is the run's place in the group (0..3)
template <int FMT>
__device__ __forceinline__ void load_raw4(Raw4<FMT>& r, const uint8_t* col, int run, int64_t k0) {
  const uint8_t* unit = col + (k0 / KSTEP) * unit_bytes(FMT);
  const int at = run * KSTEP + (int)(k0 % KSTEP);
  const uint4* p = reinterpret_cast<const uint4*>(unit + at * RunBytes<FMT>::value);
#pragma unroll
  for (int i = 0; i < (FMT == FB_BFP8 ? 4 : 2); ++i) r.q[i] = __ldg(p + i);
  r.tops = __ldg(reinterpret_cast<const uint32_t*>(unit + unit_mant_bytes(FMT) + at));
}

template <int FMT>
__device__ __forceinline__ void unpack_row(const Raw4<FMT>& r, int kk, uint32_t v[8]) {
  uint32_t top = (r.tops >> (8 * kk)) & 255u;
  if (FMT == FB_BFP8) {
    unpack_run8(r.q[kk], top, v);
  } else {
    uint4 q = r.q[kk >> 1];
    unpack_run4((kk & 1) ? make_uint2(q.z, q.w) : make_uint2(q.x, q.y), top, v);
  }
}

// Sum over K-slice [k_begin, k_end) stepping `stride` rows between this warp's chunks of 128 rows.
// x rows are bf16 with M rows `ldx` apart; `g` (may be null) multiplies x along K (an RMSNorm's weight).
// acc[t][j] += sum_k x[t][k] * g[k] * W[k][16b + j];  ss[t] += sum_k x[t][k]^2 over the rows this lane reads.
template <int FMT, int M, bool NORM>
__device__ __forceinline__ void gemv_accumulate(const uint8_t* __restrict__ col, int run,
                                                const uint16_t* x, int64_t ldx, const uint16_t* __restrict__ g,
                                                int64_t K, int64_t k_first, int64_t k_step, float acc[M][16], float ss[M]) {
  const int lane = threadIdx.x & 31;
  int64_t k0 = k_first + 4 * lane;
  Raw4<FMT> cur, nxt;
  if (k0 < K) load_raw4<FMT>(cur, col, run, k0);
  griddep_wait();  // the weights above are nobody's output; the activations below are the kernel before's
  for (; k0 < K; k0 += k_step) {
    int64_t kn = k0 + k_step;
    if (kn < K) load_raw4<FMT>(nxt, col, run, kn);
    float xv[M][4];
    float gv[4] = {1.f, 1.f, 1.f, 1.f};
    if (NORM) {
      uint2 gb = __ldg(reinterpret_cast<const uint2*>(g + k0));
      gv[0] = bf16_bits_to_float(gb.x & 0xFFFFu), gv[1] = bf16_bits_to_float(gb.x >> 16);
      gv[2] = bf16_bits_to_float(gb.y & 0xFFFFu), gv[3] = bf16_bits_to_float(gb.y >> 16);
    }
#pragma unroll
    for (int t = 0; t < M; ++t) {
      // (a plain load: an invariant one - __ldg - may be scheduled above griddep_wait(), whose asm it does not alias)
      uint2 xb = *reinterpret_cast<const uint2*>(x + t * ldx + k0);
      xv[t][0] = bf16_bits_to_float(xb.x & 0xFFFFu), xv[t][1] = bf16_bits_to_float(xb.x >> 16);
      xv[t][2] = bf16_bits_to_float(xb.y & 0xFFFFu), xv[t][3] = bf16_bits_to_float(xb.y >> 16);
      if (NORM) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          ss[t] = fmaf(xv[t][kk], xv[t][kk], ss[t]);
          xv[t][kk] *= gv[kk];
        }
      }
    }
    // The sums are kept scaled by 2^-64 (GEMV_ACC_SCALE undoes it): the weight enters the FMA as the fp32 denormal
    // +-mag * 2^-133 its masked bits already are, and 2^(top-64) goes into the activation - one multiply per run and
    // token instead of unpack arithmetic per value.  The products are exact inside the FMA either way, so the sums
    // round as those of the unpacked values do.  (Shared exponents above 186 - values beyond 2^53 - would overflow
    // that factor: such a run takes the unpacked route, its activations scaled by 2^-64.)
    constexpr uint32_t LIFT = FMT == FB_BFP8 ? 63 : 67;  // bfp4's 3-bit magnitude stands for 16 times itself
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const uint32_t top = (cur.tops >> (8 * kk)) & 255u;
      uint32_t v[8];
      float xs[M];
      if (top <= 186) {
        const uint32_t* words = reinterpret_cast<const uint32_t*>(cur.q) + kk * (FMT == FB_BFP8 ? 4 : 2);
        mask_run<FMT>(words, v);
        const float lift = __uint_as_float((top + LIFT) << 23);
#pragma unroll
        for (int t = 0; t < M; ++t) xs[t] = xv[t][kk] * lift;
      } else {
        unpack_row<FMT>(cur, kk, v);
#pragma unroll
        for (int t = 0; t < M; ++t) xs[t] = xv[t][kk] * 5.421010862427522e-20f;  // 2^-64
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 w2 = make_float2(__uint_as_float(v[i] << 16), __uint_as_float(v[i] & 0xFFFF0000u));
#pragma unroll
        for (int t = 0; t < M; ++t) {  // two columns per instruction (packed fp32 FMA)
          const float2 r = __ffma2_rn(w2, make_float2(xs[t], xs[t]), make_float2(acc[t][2 * i], acc[t][2 * i + 1]));
          acc[t][2 * i] = r.x, acc[t][2 * i + 1] = r.y;
        }
      }
    }
    cur = nxt;
  }
}

// Butterfly over the warp: 16 per-lane partial sums -> lane l (even) ends with the full sum of column
// column_of_lane(l); 8 + 4 + 2 + 1 + 1 shuffles.
__device__ __forceinline__ float butterfly16(float v[16]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int s = 16, n = 8; s >= 2; s >>= 1, n >>= 1) {
    const bool upper = lane & s;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (i < n) {
        float send = upper ? v[i] : v[i + n];
        float keep = upper ? v[i + n] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
      }
    }
  }
  return v[0] + __shfl_xor_sync(0xffffffffu, v[0], 1);
}
__device__ __forceinline__ int column_of_lane(int lane) {  // which of the 16 columns lane's butterfly result is
  return ((lane >> 4) & 1) << 3 | ((lane >> 3) & 1) << 2 | ((lane >> 2) & 1) << 1 | ((lane >> 1) & 1);
}

}  // namespace fb
