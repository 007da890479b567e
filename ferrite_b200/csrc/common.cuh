// Shared helpers for the sm_100a kernels: error reporting for the C ABI, bf16 bit tricks.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/ferrite_b200.h"

namespace fb {

// Last error text of the calling thread; every extern "C" entry point returns 0 or a negative
// fb_status and leaves the reason here (fb_last_error()).
void set_error(const char* fmt, ...);
int launch_status(const char* what);  // cudaGetLastError() -> FB_OK / FB_ERR_LAUNCH with the message kept
// the status words of the kernels that wait (each reads and clears its own): 0, or the code of the wait that gave up
int status_word_tcgen05();
int status_word_peer();
int status_word_gemv_stream();

#define FB_REQUIRE(cond, ...)            \
  do {                                   \
    if (!(cond)) {                       \
      fb::set_error(__VA_ARGS__);        \
      return FB_ERR_ARG;                 \
    }                                    \
  } while (0)

// True the first time it is called on the current device for this mask: what is set up per device (a kernel's
// shared-memory opt-in, a symbol's address) keeps one mask.  Two threads racing both see true at worst, which only
// repeats the set-up.
inline bool first_on_device(std::atomic<uint64_t>& seen) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return true;
  const uint64_t bit = 1ull << dev;
  return !(seen.fetch_or(bit) & bit);
}

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// float -> bf16 bits, round to nearest even (what an upload of Python floats does: ferrite/tensor.py:56)
__device__ __forceinline__ uint32_t float_to_bf16_bits(float f) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialisation attribute may start while
// the kernel before it in the stream still runs; it must call griddep_wait() before it reads anything that kernel
// wrote (the call returns once that kernel has finished and its writes are visible).  Every kernel of the decode
// step calls griddep_launch_dependents() first thing: it tells the scheduler that the next kernel in the stream may
// be started as soon as room frees up (a no-op when that kernel was launched the ordinary way).
#if defined(__CUDACC__)
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

}  // namespace fb
