// bf16 <-> packed block float.  Integer arithmetic only; bit-exact with the reference's numpy model
// (models/gpt2.py:21-32): per run of 16 columns the largest biased exponent is shared, magnitudes are the
// mantissas (hidden one included) shifted down to it and rounded half up into 7 bits (bfp8) or to the
// nearest 3 bits, ties up (bfp4).  These run once per weight (upload), not in the decode loop.
#include "bfp_format.cuh"

namespace fb {

__device__ __forceinline__ void load_run_bits(const uint16_t* src, uint32_t bits[16]) {
  const uint4* p = reinterpret_cast<const uint4*>(src);
  uint4 a = p[0], b = p[1];
  uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    bits[2 * i] = w[i] & 0xFFFFu;
    bits[2 * i + 1] = w[i] >> 16;
  }
}

// One thread per (matrix, row k, column block b); neighbouring threads take neighbouring blocks of a
// row, so the bf16 reads are contiguous.
template <int FMT>
__global__ void quantize_kernel(const uint16_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t batch, int64_t K, int64_t N) {
  const int64_t NB = N / 16;
  int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= batch * K * NB) return;
  int64_t b = idx % NB, k = (idx / NB) % K, mat = idx / (NB * K);
  uint32_t bits[16];
  load_run_bits(src + (mat * K + k) * N + 16 * b, bits);
  store_run<FMT>(bits, dst + mat * packed_bytes(FMT, K, N), K, b, k);
}

// (top, sign, mag) of column j of a run, from the packed bytes
template <int FMT>
__device__ __forceinline__ void read_field(const uint8_t* base, int64_t K, int64_t b, int64_t k, int j, uint32_t& sign, uint32_t& mag) {
  if (FMT == FB_BFP8) {
    const uint32_t w = reinterpret_cast<const uint32_t*>(base + mant_offset(FMT, K, b, k))[j >> 2];
    const int at = bfp8_byte_of_column(j & 3);
    mag = (w >> (8 * at)) & 127u, sign = (w >> (8 * ((at + 1) & 3) + 7)) & 1u;
  } else {
    const uint32_t w = reinterpret_cast<const uint32_t*>(base + mant_offset(FMT, K, b, k))[j >> 3];
    const int at = bfp4_nibble_of_column(j & 7);
    mag = (w >> (4 * at)) & 7u, sign = (w >> (4 * ((at + 3) & 7) + 3)) & 1u;
  }
}

// bf16 bits of +-q * 2^(top-133), built from integers (normalised, or a bf16 denormal when it is that small)
__device__ __forceinline__ uint32_t bf16_of(uint32_t sign, uint32_t q, uint32_t top) {
  if (q == 0) return 0;
  int p = 31 - __clz(q);       // position of the leading one
  int e = (int)top + p - 6;    // biased exponent of q * 2^(top-133)
  if (e >= 1) return (sign << 15) | ((uint32_t)e << 7) | ((q << (7 - p)) & 127u);
  return (sign << 15) | (q << top);  // denormal: units of 2^-133
}

template <int FMT>
__global__ void dequantize_kernel(const uint8_t* __restrict__ src, uint16_t* __restrict__ dst, int64_t batch, int64_t K, int64_t N) {
  const int64_t NB = N / 16;
  int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= batch * K * NB) return;
  int64_t b = idx % NB, k = (idx / NB) % K, mat = idx / (NB * K);
  const uint8_t* base = src + mat * packed_bytes(FMT, K, N);
  uint32_t top = base[exp_offset(FMT, K, b, k)];
  uint32_t w[8];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    uint32_t sign, mag;
    read_field<FMT>(base, K, b, k, j, sign, mag);
    uint32_t bits = bf16_of(sign, FMT == FB_BFP4 ? mag << 4 : mag, top);
    if (j & 1) w[j >> 1] |= bits << 16; else w[j >> 1] = bits;
  }
  uint4* out = reinterpret_cast<uint4*>(dst + (mat * K + k) * N + 16 * b);
  out[0] = make_uint4(w[0], w[1], w[2], w[3]);
  out[1] = make_uint4(w[4], w[5], w[6], w[7]);
}

template <int FMT>
__global__ void fields_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ top_out, uint8_t* __restrict__ sign_out,
                              uint8_t* __restrict__ mag_out, int64_t batch, int64_t K, int64_t N) {
  const int64_t NB = N / 16;
  int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (idx >= batch * K * NB) return;
  int64_t b = idx % NB, k = (idx / NB) % K, mat = idx / (NB * K);
  const uint8_t* base = src + mat * packed_bytes(FMT, K, N);
  top_out[(mat * K + k) * NB + b] = base[exp_offset(FMT, K, b, k)];
  for (int j = 0; j < 16; ++j) {
    uint32_t sign, mag;
    read_field<FMT>(base, K, b, k, j, sign, mag);
    sign_out[(mat * K + k) * N + 16 * b + j] = (uint8_t)sign;
    mag_out[(mat * K + k) * N + 16 * b + j] = (uint8_t)mag;
  }
}

static int check_shape(int fmt, int64_t batch, int64_t K, int64_t N) {
  FB_REQUIRE(fmt == FB_BFP8 || fmt == FB_BFP4, "a block float is bfp8 or bfp4, not dtype %d", fmt);
  FB_REQUIRE(batch >= 1 && K >= 1 && N >= 16 && N % 16 == 0, "a block float's rows are runs of 16: got %lld x %lld x %lld",
             (long long)batch, (long long)K, (long long)N);
  return FB_OK;
}

}  // namespace fb

extern "C" size_t fb_packed_bytes(int fmt, int64_t K, int64_t N) {
  if ((fmt != FB_BFP8 && fmt != FB_BFP4) || K < 1 || N < 16 || N % 16) return 0;
  return (size_t)fb::packed_bytes(fmt, K, N);
}

extern "C" int fb_quantize(int fmt, const void* src, int64_t batch, int64_t K, int64_t N, void* dst, void* stream) {
  if (int rc = fb::check_shape(fmt, batch, K, N)) return rc;
  FB_REQUIRE(src && dst && (uintptr_t)src % 16 == 0 && (uintptr_t)dst % 16 == 0, "quantize: 16-byte aligned device pointers");
  int64_t total = batch * K * (N / 16);
  dim3 grid((unsigned)fb::ceil_div(total, 256)), block(256);
  auto s = (cudaStream_t)stream;
  if (K % fb::KSTEP || N % (16 * fb::GROUP_RUNS)) {  // the padding of the last units holds zeros
    if (cudaMemsetAsync(dst, 0, (size_t)batch * fb::packed_bytes(fmt, K, N), s) != cudaSuccess)
      return fb::launch_status("fb_quantize (padding)");
  }
  if (fmt == FB_BFP8) fb::quantize_kernel<FB_BFP8><<<grid, block, 0, s>>>((const uint16_t*)src, (uint8_t*)dst, batch, K, N);
  else fb::quantize_kernel<FB_BFP4><<<grid, block, 0, s>>>((const uint16_t*)src, (uint8_t*)dst, batch, K, N);
  return fb::launch_status("fb_quantize");
}

extern "C" int fb_dequantize(int fmt, const void* packed, int64_t batch, int64_t K, int64_t N, void* dst, void* stream) {
  if (int rc = fb::check_shape(fmt, batch, K, N)) return rc;
  FB_REQUIRE(packed && dst && (uintptr_t)packed % 16 == 0 && (uintptr_t)dst % 16 == 0, "dequantize: 16-byte aligned device pointers");
  int64_t total = batch * K * (N / 16);
  dim3 grid((unsigned)fb::ceil_div(total, 256)), block(256);
  auto s = (cudaStream_t)stream;
  if (fmt == FB_BFP8) fb::dequantize_kernel<FB_BFP8><<<grid, block, 0, s>>>((const uint8_t*)packed, (uint16_t*)dst, batch, K, N);
  else fb::dequantize_kernel<FB_BFP4><<<grid, block, 0, s>>>((const uint8_t*)packed, (uint16_t*)dst, batch, K, N);
  return fb::launch_status("fb_dequantize");
}

extern "C" int fb_unpack_fields(int fmt, const void* packed, int64_t batch, int64_t K, int64_t N, uint8_t* top, uint8_t* sign,
                                uint8_t* mag, void* stream) {
  if (int rc = fb::check_shape(fmt, batch, K, N)) return rc;
  FB_REQUIRE(packed && top && sign && mag, "unpack_fields: null pointer");
  int64_t total = batch * K * (N / 16);
  dim3 grid((unsigned)fb::ceil_div(total, 256)), block(256);
  auto s = (cudaStream_t)stream;
  if (fmt == FB_BFP8) fb::fields_kernel<FB_BFP8><<<grid, block, 0, s>>>((const uint8_t*)packed, top, sign, mag, batch, K, N);
  else fb::fields_kernel<FB_BFP4><<<grid, block, 0, s>>>((const uint8_t*)packed, top, sign, mag, batch, K, N);
  return fb::launch_status("fb_unpack_fields");
}
