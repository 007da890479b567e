// Arguments of fb_linear as the kernels see them, and the implementations it dispatches to.
#pragma once
#include "common.cuh"

namespace fb {

struct LinearArgs {
  int fmt;               // FB_BFP8 | FB_BFP4 | FB_BF16
  const void* x;         // [M, K] bf16, rows ldx apart
  int64_t M, K, ldx;
  const void* W;         // packed [K, N]
  int64_t N;
  void* out;             // [M, N] or [M, N/2] (SwiGLU), rows ldo apart
  int out_dtype;         // FB_BF16 | FB_FP32
  int64_t ldo;
  const void* norm_w;    // [K] bf16 or null: RMSNorm prologue
  float eps;
  int epilogue;          // fb_epilogue
  const void* residual;  // [M, N] bf16, rows ldr apart (FB_EPI_RESIDUAL)
  int64_t ldr;
  void* workspace;
  size_t workspace_bytes;
  bool persistent = false;  // the tcgen05 path's persistent kernel (tiles' steps shared out over the SMs) instead of a CTA per tile
  // An RMSNorm handed from the matmul that makes its input to the matmul that consumes it (fb_linear_chained), so that no
  // kernel stands between them.  As producer (with the residual epilogue, out bf16): besides out[t, n], xn_out[t, n] =
  // bf16(out[t, n] * next_norm_w[n]) and sumsq_out[part * M + t] = the sum of out[t, n]^2 over the part's columns, a part
  // per CTA.  As consumer: x is such an xn, and the row scale is rsqrt(sum over sumsq_in's parts / K + eps).
  const void* next_norm_w = nullptr;
  void* xn_out = nullptr;
  int64_t ld_xn = 0;
  float* sumsq_out = nullptr;
  const float* sumsq_in = nullptr;
  int sumsq_parts = 0;
};

// Tensor.matmul(index=) (ferrite/tensor.py:450-460): W a batch of packed matrices, index[slot] picks one per slot
struct IndexedArgs {
  int mode;  // 1: one result per slot; 2: the slots' matmuls summed (K runs through the slots)
  const int32_t* index;
  int n_experts, n_slots;
  int64_t x_slot_rows;      // mode 1: rows of x from one slot's to the next's (0: every slot multiplies the same x)
  int64_t out_slot_stride;  // mode 1: elements of out from one slot's result to the next's
  const void* row_scale;    // mode 1: bf16 [slot * M + t] multiplying the epilogue's result, or null
};

// fb_linear's workspace, shared by its kernels (calls on one stream run in order):
//   [0, 1024)     arrival words of the persistent tcgen05 kernel's CTAs: zero before the first call, and every call
//                 leaves them zero - nothing else may ever be written here;
//   [1024, 2048)  the row scales of an RMSNorm prologue;
//   [2048, 18432) arrival counters of the streaming GEMV's output tiles (one per 64 output columns): zero before the first
//                 call and left zero by every call, like the arrival words;
//   [18432, ...)  each kernel's own: partial tiles and sums, the normalised activations.
constexpr size_t WS_ARRIVED_AT = 0, WS_RSTD_AT = 1024, WS_COUNTERS_AT = 2048, WS_COUNTERS = 4096, WS_BODY_AT = WS_COUNTERS_AT + 4 * WS_COUNTERS;

int linear_gemv(const LinearArgs& a, cudaStream_t s);     // gemv.cu: one token (up to 4 a pass), CUDA cores
int linear_gemv_stream(const LinearArgs& a, cudaStream_t s);  // gemv_stream.cu: one token, persistent CTAs fed by bulk copies
bool linear_gemv_stream_supports(const LinearArgs& a);
size_t linear_gemv_stream_workspace(int64_t K, int64_t N);
int linear_tcgen05(const LinearArgs& a, cudaStream_t s);  // gemm_tcgen05.cu: tensor cores (tcgen05, tiles through shared memory)
int linear_mma(const LinearArgs& a, cudaStream_t s);      // gemm_mma.cu: up to 32 tokens, tensor cores fed from registers
bool linear_mma_supports(const LinearArgs& a);
int linear_tcgen05_indexed(const LinearArgs& a, const IndexedArgs& ix, cudaStream_t s);
bool linear_tcgen05_supports(const LinearArgs& a);
bool linear_persistent_wins(const LinearArgs& a);
int linear_tcgen05_parts(int fmt, int64_t M, int64_t K, int64_t N, int epilogue);  // CTAs (parts of sumsq_out) of the per-tile kernel's launch; 0: no chaining  // whether fb_linear, left to choose, runs the persistent kernel for this shape
size_t linear_tcgen05_workspace(int64_t M, int64_t K, int64_t N);

}  // namespace fb
