// The small kernels of a decode step around the matmuls and attention: embedding gather, RoPE + KV-cache write,
// RMSNorm on its own, greedy argmax.  All are bandwidth-trivial; they exist so a whole step stays on the device
// (one CUDA graph) with places and ids as data, as ferrite's replayed step has them (ferrite/tensor.py:788-810).
#include "bfp_format.cuh"

namespace fb {

// out[t, :] = table[ids[t], :]  (Tensor.gather, ferrite/tensor.py:116-126; ferrite/compiler.py:1574-1580)
__global__ void gather_rows_kernel(const uint4* __restrict__ table, const int32_t* __restrict__ ids, uint4* __restrict__ out,
                                   int64_t row_vecs, int64_t table_rows) {
  griddep_launch_dependents();
  const int64_t t = blockIdx.x;
  int64_t id = ids[t];
  id = id < 0 ? 0 : id >= table_rows ? table_rows - 1 : id;  // nothing checks an id's bounds on ferrite; here it is clamped
  for (int64_t v = threadIdx.x; v < row_vecs; v += blockDim.x) out[t * row_vecs + v] = __ldg(table + id * row_vecs + v);
}

// the same for rows that are not whole 16-byte pieces (or not 16-byte aligned): two bytes at a time
__global__ void gather_rows_small_kernel(const uint16_t* __restrict__ table, const int32_t* __restrict__ ids, uint16_t* __restrict__ out,
                                         int64_t row_halves, int64_t table_rows) {
  griddep_launch_dependents();
  const int64_t t = blockIdx.x;
  int64_t id = ids[t];
  id = id < 0 ? 0 : id >= table_rows ? table_rows - 1 : id;
  for (int64_t v = threadIdx.x; v < row_halves; v += blockDim.x) out[t * row_halves + v] = table[id * row_halves + v];
}

// One block per (token, head): optional per-head RMSNorm (Qwen3's q/k norm, models/llama.py:121-123), the
// half-rotation RoPE x*cos + rotate_half(x)*sin with bf16 tables (models/llama.py:92-93, 351-368), then q heads go to
// q_out and k/v heads into the cache rows (Tensor.put, ferrite/tensor.py:128-140): cache[head][row[t]][:].
// Tables: [places, table_cols] with table_cols = hd (one head's table; v heads then do not turn) or the full
// (H + 2 KV) * hd width ferrite keeps (v's columns hold cos 1, sin 0).
struct RopeArgs {
  const uint16_t* qkv;  // [T, (H + 2KV) * hd]
  int64_t ld_qkv;
  const uint16_t *cos, *sin;
  int64_t table_cols, table_rows;
  const int32_t* places;  // [T] table row of each token (clamped into the table)
  const int32_t* rows;    // [T] cache row of each token (a row outside the cache is not written)
  const uint16_t* qk_norm;  // [(H + KV) * hd] or null
  float eps;
  uint16_t* q_out;  // [T, H * hd]
  int64_t ld_q;
  uint16_t* cache;  // [2 KV, cache_rows, hd], heads head_stride elements apart
  int64_t head_stride;
  int H, KV, hd;
  // a block-float cache (Tensor.put into a bfp8 / bfp4 tensor, ferrite/compiler.py:1648-1662): 2 KV packed matrices
  // [cache_rows, hd] one after another; each run of 16 of a row rounded as the cast rounds it
  int cache_fmt;  // 0: bf16
  int64_t cache_rows;
};

__global__ void rope_kv_kernel(RopeArgs a) {
  griddep_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y, half = a.hd / 2, d = threadIdx.x;  // blockDim.x == hd / 2
  const uint16_t* x = a.qkv + t * a.ld_qkv + (int64_t)h * a.hd;
  float x1 = bf16_bits_to_float(x[d]), x2 = bf16_bits_to_float(x[d + half]);
  const bool is_v = h >= a.H + a.KV;
  if (a.qk_norm && !is_v) {
    __shared__ float red[8];  // (hd / 2 is a whole number of warps when a norm is given: the launch checks it)
    float ss = warp_sum(x1 * x1 + x2 * x2);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) total += red[w];
    const float r = rsqrtf(total / (float)a.hd + a.eps);
    x1 *= r * bf16_bits_to_float(a.qk_norm[h * a.hd + d]);
    x2 *= r * bf16_bits_to_float(a.qk_norm[h * a.hd + d + half]);
  }
  float y1 = x1, y2 = x2;
  const bool wide = a.table_cols != a.hd;
  if (wide || !is_v) {
    const int64_t place = min(max((int64_t)a.places[t], (int64_t)0), a.table_rows - 1);
    const int64_t at = place * a.table_cols + (wide ? (int64_t)h * a.hd : 0);
    const float c1 = bf16_bits_to_float(a.cos[at + d]), c2 = bf16_bits_to_float(a.cos[at + d + half]);
    const float s1 = bf16_bits_to_float(a.sin[at + d]), s2 = bf16_bits_to_float(a.sin[at + d + half]);
    y1 = x1 * c1 - x2 * s1;
    y2 = x2 * c2 + x1 * s2;
  }
  const int64_t cache_row = a.rows[t];
  if (h >= a.H && (cache_row < 0 || cache_row >= a.cache_rows)) return;  // a row outside the cache: nothing is written
  if (h >= a.H && a.cache_fmt) {  // a key or value row into the block-float cache: a thread per run of 16 rounds and stores it
    __shared__ uint16_t row[512];
    row[d] = (uint16_t)float_to_bf16_bits(y1);
    row[d + half] = (uint16_t)float_to_bf16_bits(y2);
    __syncthreads();
    if (d < a.hd / 16) {
      uint32_t bits[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) bits[j] = row[16 * d + j];
      uint8_t* base = reinterpret_cast<uint8_t*>(a.cache) + (int64_t)(h - a.H) * packed_bytes(a.cache_fmt, a.cache_rows, a.hd);
      if (a.cache_fmt == FB_BFP8) store_run<FB_BFP8>(bits, base, a.cache_rows, d, cache_row);
      else store_run<FB_BFP4>(bits, base, a.cache_rows, d, cache_row);
    }
    return;
  }
  uint16_t* out;
  if (h < a.H) out = a.q_out + t * a.ld_q + (int64_t)h * a.hd;
  else out = a.cache + (int64_t)(h - a.H) * a.head_stride + cache_row * a.hd;  // k heads, then v heads (models/llama.py:506-514)
  out[d] = (uint16_t)float_to_bf16_bits(y1);
  out[d + half] = (uint16_t)float_to_bf16_bits(y2);
}

// out = x * rsqrt(mean(x^2) + eps) * w  (models/llama.py:82-85), one block per row
__global__ void __launch_bounds__(256) rmsnorm_kernel(const uint16_t* __restrict__ x, int64_t ldx, const uint16_t* __restrict__ w,
                                                      uint16_t* __restrict__ out, int64_t ldo, int64_t cols, float eps) {
  griddep_launch_dependents();
  const int64_t t = blockIdx.x;
  float ss = 0.f;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = bf16_bits_to_float(x[t * ldx + c]);
    ss = fmaf(v, v, ss);
  }
  __shared__ float red[8];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
  for (int i = 0; i < 8; ++i) total += red[i];
  const float r = rsqrtf(total / (float)cols + eps);
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
    out[t * ldo + c] = (uint16_t)float_to_bf16_bits(bf16_bits_to_float(x[t * ldx + c]) * r * bf16_bits_to_float(w[c]));
}

// Greedy pick: the column of each row's largest logit, the lowest column among equals (numpy's argmax).
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int64_t ld, int64_t cols, int32_t* __restrict__ out,
                                                      float* __restrict__ out_value) {
  const int64_t t = blockIdx.x;
  float best = -INFINITY;
  int64_t at = cols;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = logits[t * ld + c];
    if (v > best || (v == best && c < at)) best = v, at = c;
  }
  __shared__ float sv[32];
  __shared__ int64_t si[32];
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, at, o);
    if (ov > best || (ov == best && oi < at)) best = ov, at = oi;
  }
  if ((threadIdx.x & 31) == 0) sv[threadIdx.x >> 5] = best, si[threadIdx.x >> 5] = at;
  __syncthreads();
  if (threadIdx.x < 32) {
    best = threadIdx.x < blockDim.x / 32 ? sv[threadIdx.x] : -INFINITY;
    at = threadIdx.x < blockDim.x / 32 ? si[threadIdx.x] : cols;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, at, o);
      if (ov > best || (ov == best && oi < at)) best = ov, at = oi;
    }
    if (threadIdx.x == 0) {
      out[t] = (int32_t)(at < cols ? at : 0);
      if (out_value) out_value[t] = best;
    }
  }
}

// dst[b, ids[i], :] = src[b, i, :]; of rows with the same place the later one stays (Tensor.put, ferrite/tensor.py:128-140)
template <typename T>
__global__ void put_rows_kernel(T* dst, int64_t ds0, int64_t ds1, int64_t ds2, const T* src, int64_t ss0, int64_t ss1, int64_t ss2,
                                const int32_t* ids, int64_t n, int64_t cols, int64_t dst_rows) {
  const int64_t i = blockIdx.x, b = blockIdx.y;
  const int32_t place = ids[i];
  if (place < 0 || place >= dst_rows) return;
  for (int64_t j = i + 1; j < n; ++j)
    if (ids[j] == place) return;
  for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) dst[b * ds0 + place * ds1 + c * ds2] = src[b * ss0 + i * ss1 + c * ss2];
}

}  // namespace fb

extern "C" int fb_put_rows(void* dst, int64_t ds0, int64_t ds1, int64_t ds2, const void* src, int64_t ss0, int64_t ss1, int64_t ss2,
                           const int32_t* ids, int64_t batch, int64_t n, int64_t cols, int64_t dst_rows, int elem_bytes, void* stream) {
  FB_REQUIRE(dst && src && ids && batch >= 1 && n >= 1 && cols >= 1 && batch <= 65535, "fb_put_rows: null pointer or empty");
  FB_REQUIRE(elem_bytes == 2 || elem_bytes == 4, "fb_put_rows: 2- or 4-byte values");
  dim3 grid((unsigned)n, (unsigned)batch);
  auto s = (cudaStream_t)stream;
  if (elem_bytes == 2) fb::put_rows_kernel<uint16_t><<<grid, 128, 0, s>>>((uint16_t*)dst, ds0, ds1, ds2, (const uint16_t*)src, ss0, ss1, ss2, ids, n, cols, dst_rows);
  else fb::put_rows_kernel<uint32_t><<<grid, 128, 0, s>>>((uint32_t*)dst, ds0, ds1, ds2, (const uint32_t*)src, ss0, ss1, ss2, ids, n, cols, dst_rows);
  return fb::launch_status("fb_put_rows");
}

extern "C" int fb_gather_rows(const void* table, int64_t table_rows, int64_t row_bytes, const int32_t* ids, int64_t n, void* out,
                              void* stream) {
  FB_REQUIRE(table && ids && out && n >= 1 && table_rows >= 1, "fb_gather_rows: null pointer or empty");
  FB_REQUIRE(row_bytes >= 2 && row_bytes % 2 == 0 && (uintptr_t)table % 2 == 0 && (uintptr_t)out % 2 == 0, "fb_gather_rows: rows of whole 2-byte values");
  if (row_bytes % 16 == 0 && (uintptr_t)table % 16 == 0 && (uintptr_t)out % 16 == 0)
    fb::gather_rows_kernel<<<(unsigned)n, 128, 0, (cudaStream_t)stream>>>((const uint4*)table, ids, (uint4*)out, row_bytes / 16, table_rows);
  else
    fb::gather_rows_small_kernel<<<(unsigned)n, 128, 0, (cudaStream_t)stream>>>((const uint16_t*)table, ids, (uint16_t*)out, row_bytes / 2, table_rows);
  return fb::launch_status("fb_gather_rows");
}

extern "C" int fb_rope_kv_write(const void* qkv, int64_t T, int64_t ld_qkv, int H, int KV, int hd, const void* cos, const void* sin,
                                int64_t table_cols, int64_t table_rows, const int32_t* places, const int32_t* rows, const void* qk_norm, float eps,
                                void* q_out, int64_t ld_q, void* cache, int64_t cache_rows, int64_t cache_head_stride, void* stream) {
  FB_REQUIRE(qkv && cos && sin && places && rows && q_out && cache, "fb_rope_kv_write: null pointer");
  FB_REQUIRE(T >= 1 && H >= 1 && KV >= 1 && hd >= 2 && hd % 2 == 0 && hd <= 512, "fb_rope_kv_write: heads of an even width up to 512");
  FB_REQUIRE(!qk_norm || hd % 64 == 0, "fb_rope_kv_write: a q/k norm takes heads of a multiple of 64 columns (got %d)", hd);
  FB_REQUIRE(table_rows >= 1 && cache_rows >= 1, "fb_rope_kv_write: empty tables or cache");
  FB_REQUIRE(cache_head_stride >= cache_rows * hd, "fb_rope_kv_write: heads at least cache_rows rows apart");
  FB_REQUIRE(table_cols == hd || table_cols == (int64_t)(H + 2 * KV) * hd, "fb_rope_kv_write: tables one head wide, or as wide as q, k and v");
  fb::RopeArgs a{(const uint16_t*)qkv, ld_qkv, (const uint16_t*)cos, (const uint16_t*)sin, table_cols, table_rows, places, rows,
                 (const uint16_t*)qk_norm, eps, (uint16_t*)q_out, ld_q, (uint16_t*)cache, cache_head_stride, H, KV, hd, 0, cache_rows};
  fb::rope_kv_kernel<<<dim3((unsigned)T, (unsigned)(H + 2 * KV)), hd / 2, 0, (cudaStream_t)stream>>>(a);
  return fb::launch_status("fb_rope_kv_write");
}

extern "C" int fb_rope_kv_write_packed(int cache_fmt, const void* qkv, int64_t T, int64_t ld_qkv, int H, int KV, int hd, const void* cos,
                                       const void* sin, int64_t table_cols, int64_t table_rows, const int32_t* places, const int32_t* rows, const void* qk_norm,
                                       float eps, void* q_out, int64_t ld_q, void* cache_packed, int64_t cache_rows, void* stream) {
  FB_REQUIRE(cache_fmt == FB_BFP8 || cache_fmt == FB_BFP4, "fb_rope_kv_write_packed: a bfp8 or bfp4 cache (dtype %d given)", cache_fmt);
  FB_REQUIRE(qkv && cos && sin && places && rows && q_out && cache_packed, "fb_rope_kv_write_packed: null pointer");
  FB_REQUIRE(T >= 1 && H >= 1 && KV >= 1 && hd >= 16 && hd % 16 == 0 && hd <= 512 && cache_rows >= 1, "fb_rope_kv_write_packed: heads of whole runs of 16, up to 512 wide");
  FB_REQUIRE(table_cols == hd || table_cols == (int64_t)(H + 2 * KV) * hd, "fb_rope_kv_write_packed: tables one head wide, or as wide as q, k and v");
  FB_REQUIRE((uintptr_t)cache_packed % 16 == 0, "fb_rope_kv_write_packed: misaligned cache");
  FB_REQUIRE(!qk_norm || hd % 64 == 0, "fb_rope_kv_write_packed: a q/k norm takes heads of a multiple of 64 columns (got %d)", hd);
  FB_REQUIRE(table_rows >= 1, "fb_rope_kv_write_packed: empty tables");
  fb::RopeArgs a{(const uint16_t*)qkv, ld_qkv, (const uint16_t*)cos, (const uint16_t*)sin, table_cols, table_rows, places, rows,
                 (const uint16_t*)qk_norm, eps, (uint16_t*)q_out, ld_q, (uint16_t*)cache_packed, 0, H, KV, hd, cache_fmt, cache_rows};
  fb::rope_kv_kernel<<<dim3((unsigned)T, (unsigned)(H + 2 * KV)), hd / 2, 0, (cudaStream_t)stream>>>(a);
  return fb::launch_status("fb_rope_kv_write_packed");
}

extern "C" int fb_rmsnorm(const void* x, int64_t rows, int64_t cols, int64_t ldx, const void* w, float eps, void* out, int64_t ldo,
                          void* stream) {
  FB_REQUIRE(x && w && out && rows >= 1 && cols >= 1 && ldx >= cols && ldo >= cols, "fb_rmsnorm: bad arguments");
  fb::rmsnorm_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)x, ldx, (const uint16_t*)w, (uint16_t*)out, ldo, cols, eps);
  return fb::launch_status("fb_rmsnorm");
}

extern "C" int fb_argmax(const void* logits_f32, int64_t rows, int64_t cols, int64_t ld, int32_t* out, float* out_value, void* stream) {
  FB_REQUIRE(logits_f32 && out && rows >= 1 && cols >= 1 && ld >= cols, "fb_argmax: bad arguments");
  fb::argmax_kernel<<<(unsigned)rows, 1024, 0, (cudaStream_t)stream>>>((const float*)logits_f32, ld, cols, out, out_value);
  return fb::launch_status("fb_argmax");
}
