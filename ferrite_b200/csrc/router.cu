// The mixture-of-experts router's integer kernels: top-k with numpy's stable order, and the list of touched experts.
// Both compare values exactly as stored, so their indices match the numpy reference bit for bit on the same logits
// (models/llama.py:27; ferrite/tensor.py:373-416; ferrite/compiler.py:1716-1731, 1898-1905).
#include "common.cuh"

namespace fb {

// One block per row.  Pick j is the smallest element, in the order (value descending, column ascending), that
// comes after pick j-1: no "taken" marks, ties resolve to the lower column, -0 equals 0 (float compare).
template <typename T>
__device__ __forceinline__ float as_float(T v);
template <>
__device__ __forceinline__ float as_float<uint16_t>(uint16_t v) { return bf16_bits_to_float(v); }
template <>
__device__ __forceinline__ float as_float<float>(float v) { return v; }

template <typename T>
__global__ void __launch_bounds__(256) topk_kernel(const T* __restrict__ x, int64_t ldx, int64_t cols, int k, const int32_t* __restrict__ labels,
                                                   T* __restrict__ values, int32_t* __restrict__ ids, uint16_t* __restrict__ weights, int64_t ldo) {
  griddep_launch_dependents();
  const int64_t row = blockIdx.x;
  const T* xr = x + row * ldx;
  __shared__ float sv[8];
  __shared__ int64_t si[8];
  __shared__ float picked_v[64];
  float prev_v = INFINITY;
  int64_t prev_i = -1;
  for (int j = 0; j < k; ++j) {
    float best = -INFINITY;
    int64_t at = cols;  // "none"
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
      const float v = as_float<T>(xr[c]);
      const bool after = j == 0 || v < prev_v || (v == prev_v && c > prev_i);
      if (after && (at == cols || v > best || (v == best && c < at))) best = v, at = c;
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, at, o);
      if (oi < cols && (at == cols || ov > best || (ov == best && oi < at))) best = ov, at = oi;
    }
    if ((threadIdx.x & 31) == 0) sv[threadIdx.x >> 5] = best, si[threadIdx.x >> 5] = at;
    __syncthreads();
    best = sv[0], at = si[0];
    for (int w = 1; w < 8; ++w)
      if (si[w] < cols && (at == cols || sv[w] > best || (sv[w] == best && si[w] < at))) best = sv[w], at = si[w];
    __syncthreads();
    prev_v = best, prev_i = at;
    if (threadIdx.x == 0) {
      const int64_t c = at < cols ? at : 0;
      values[row * ldo + j] = xr[c];  // the stored bits, untouched
      ids[row * ldo + j] = labels ? labels[row * ldx + c] : (int32_t)c;
      picked_v[j] = best;
    }
  }
  if (weights) {  // softmax of the picked values (models/llama.py:288: the weights of Qwen3's and Mixtral's experts)
    __syncthreads();
    if (threadIdx.x == 0) {
      float sum = 0.f;
      for (int j = 0; j < k; ++j) sum += expf(picked_v[j] - picked_v[0]);
      for (int j = 0; j < k; ++j) weights[row * ldo + j] = (uint16_t)float_to_bf16_bits(expf(picked_v[j] - picked_v[0]) / sum);
    }
  }
}

// One block: experts some row picks with a weight that is not zero, ascending, then n; and each entry's weight per row.
// Experts are counted from `first`: a rank that holds experts first .. first + n - 1 lists those, numbered from 0.
__global__ void __launch_bounds__(256) touched_kernel(const int32_t* __restrict__ ids, const uint16_t* __restrict__ w, int64_t rows, int k, int n,
                                                      int first, int slots, int32_t* __restrict__ experts, uint16_t* __restrict__ out) {
  griddep_launch_dependents();
  extern __shared__ int32_t flag[];  // [n] then the compacted list [slots]
  int32_t* listed = flag + n;
  for (int e = threadIdx.x; e < n; e += blockDim.x) flag[e] = 0;
  __syncthreads();
  for (int64_t i = threadIdx.x; i < rows * k; i += blockDim.x) {
    const int32_t e = ids[i] - first;
    if (e >= 0 && e < n && (w[i] & 0x7FFFu) != 0) flag[e] = 1;  // (+0 and -0 are both zero)
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int count = 0;
    for (int e = 0; e < n && count < slots; ++e)
      if (flag[e]) listed[count++] = e;
    for (; count < slots; ++count) listed[count] = n;
  }
  __syncthreads();
  for (int s = threadIdx.x; s < slots; s += blockDim.x) experts[s] = listed[s];
  for (int64_t i = threadIdx.x; i < (int64_t)slots * rows; i += blockDim.x) {
    const int s = (int)(i / rows);
    const int64_t r = i % rows;
    const int32_t e = listed[s];
    float acc = 0.f;
    bool any = false;
    for (int j = 0; j < k; ++j)
      if (e < n && ids[r * k + j] - first == e) acc += bf16_bits_to_float(w[r * k + j]), any = true;
    out[i] = any ? (uint16_t)float_to_bf16_bits(acc) : 0;
  }
}

// One block of n threads (rounded up to whole warps), a thread per value (expert): Tensor.group's counting sort.  Thread
// e counts its choices, the runs' first slots are a scan over the counts rounded up to whole tiles of 32, and thread e
// hands its choices their slots in the choices' own order (row by row, choice by choice), as the reference's one-worker
// kernel does (ferrite/compiler.py:1844-1896) - so the result is that kernel's, slot for slot.
__global__ void __launch_bounds__(1024) group_kernel(const int32_t* __restrict__ ids, int rows, int k, int n, int t, int rp,
                                                     int32_t* __restrict__ order, int32_t* __restrict__ tiles, int32_t* __restrict__ places) {
  griddep_launch_dependents();
  extern __shared__ int32_t first_slot[];  // [n + 1]
  const int e = threadIdx.x, total = rows * k;
  for (int s = threadIdx.x; s < 32 * t; s += blockDim.x) order[s] = 0;
  for (int i = threadIdx.x; i < t; i += blockDim.x) tiles[i] = n;  // none: a matmul picking by them skips the tiles past those used
  for (int s = threadIdx.x; s < k * rp; s += blockDim.x) places[s] = 0;
  int count = 0;
  if (e < n)
    for (int i = 0; i < total; ++i) count += ids[i] == e;  // (every thread reads the same word: a broadcast)
  if (e <= n) first_slot[e] = e < n ? (count + 31) / 32 * 32 : 0;
  __syncthreads();  // (also: the fills above are done before any slot is written)
  if (threadIdx.x == 0) {  // the runs one after another, each a whole number of tiles
    int s = 0;
    for (int v = 0; v <= n; ++v) {
      const int room = first_slot[v];
      first_slot[v] = s;
      s += room;
    }
  }
  __syncthreads();
  if (e >= n) return;
  int s = first_slot[e];
  for (int tile = s / 32; tile < first_slot[e + 1] / 32; ++tile) tiles[tile] = e;
  for (int i = 0; i < total && count; ++i)
    if (ids[i] == e) {
      const int r = i / k, j = i - r * k;
      order[s] = r;
      places[j * rp + r] = s;
      ++s, --count;
    }
}

}  // namespace fb

extern "C" int fb_group(const int32_t* ids, int64_t rows, int k, int n, int32_t* order, int32_t* tiles, int32_t* places, void* stream) {
  FB_REQUIRE(ids && order && tiles && places && rows >= 1 && k >= 1 && k <= 32 && n >= 1 && n <= 1023, "fb_group: up to 32 choices a row of up to 1023 values");
  FB_REQUIRE(rows * k <= (1 << 22), "fb_group: up to 4 M choices");
  const int64_t t = (rows * k + 31) / 32 + (n < rows * k ? n : rows * k), rp = (rows + 31) / 32 * 32;
  const int threads = (n + 1 + 31) / 32 * 32;
  fb::group_kernel<<<1, threads, (size_t)(n + 1) * sizeof(int32_t), (cudaStream_t)stream>>>(ids, (int)rows, k, n, (int)t, (int)rp, order, tiles, places);
  return fb::launch_status("fb_group");
}

extern "C" int fb_topk(int dtype, const void* x, int64_t rows, int64_t cols, int64_t ldx, int k, const int32_t* labels, void* values,
                       int32_t* ids, void* softmax_weights_bf16, int64_t ldo, void* stream) {
  FB_REQUIRE(dtype == FB_BF16 || dtype == FB_FP32, "fb_topk: bf16 or fp32 (ferrite/tensor.py:381)");
  FB_REQUIRE(x && values && ids && rows >= 1 && k >= 1 && k <= 64 && k <= cols && ldo >= k, "fb_topk: k of at most 64 and at most the columns");
  auto s = (cudaStream_t)stream;
  if (dtype == FB_BF16)
    fb::topk_kernel<uint16_t><<<(unsigned)rows, 256, 0, s>>>((const uint16_t*)x, ldx, cols, k, labels, (uint16_t*)values, ids, (uint16_t*)softmax_weights_bf16, ldo);
  else
    fb::topk_kernel<float><<<(unsigned)rows, 256, 0, s>>>((const float*)x, ldx, cols, k, labels, (float*)values, ids, (uint16_t*)softmax_weights_bf16, ldo);
  return fb::launch_status("fb_topk");
}

extern "C" int fb_touched(const int32_t* ids, const void* weights_bf16, int64_t rows, int k, int n, int first, int32_t* experts, void* out_bf16,
                          void* stream) {
  FB_REQUIRE(ids && weights_bf16 && experts && out_bf16 && rows >= 1 && k >= 1 && k <= 32 && n >= 1 && n <= 4096, "fb_touched: up to 32 choices of up to 4096 experts");
  const int slots = (int)(rows * k < n ? rows * k : n);
  fb::touched_kernel<<<1, 256, (size_t)(n + slots) * sizeof(int32_t), (cudaStream_t)stream>>>(ids, (const uint16_t*)weights_bf16, rows, k, n, first, slots, experts,
                                                                                           (uint16_t*)out_bf16);
  return fb::launch_status("fb_touched");
}
