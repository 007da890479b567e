// fb_linear: argument checks (what ferrite's Tensor.matmul asserts, ferrite/tensor.py:443-485) and the
// choice between the GEMV and the tensor-core kernels.
#include "linear.cuh"

static int g_linear_kernel = FB_LINEAR_AUTO;

// The head of fb_linear's workspace (arrival words, counters: linear.cuh) has to be zero before the first kernel that
// counts in it.  A buffer this process has not been given before is zeroed here, in stream order, so that a caller's
// fresh allocation needs no memset of its own; what the library cannot see - a buffer written by someone else between
// calls, or freed and handed back at the same address with other contents - stays the caller's to zero.
#include <mutex>
static void zero_new_workspace(void* workspace, size_t bytes, cudaStream_t s) {
  static std::mutex lock;
  static const void* seen[64];
  static int n_seen = 0;
  if (!workspace || bytes < fb::WS_BODY_AT) return;
  std::lock_guard<std::mutex> hold(lock);
  for (int i = 0; i < n_seen; ++i)
    if (seen[i] == workspace) return;
  seen[n_seen < 64 ? n_seen++ : 63] = workspace;
  cudaMemsetAsync(workspace, 0, fb::WS_BODY_AT, s);
}

extern "C" int fb_linear_prefer(int kernel) {
  FB_REQUIRE(kernel >= FB_LINEAR_AUTO && kernel <= FB_LINEAR_GEMV_STREAM, "fb_linear_prefer: unknown kernel %d", kernel);
  g_linear_kernel = kernel;
  return FB_OK;
}

extern "C" size_t fb_linear_workspace_bytes(int64_t M, int64_t K, int64_t N) {
  const size_t a = fb::linear_tcgen05_workspace(M, K, N), b = M == 1 ? fb::linear_gemv_stream_workspace(K, N) : 0;
  return a > b ? a : b;
}

extern "C" int fb_linear(int fmt, const void* x, int64_t M, int64_t K, int64_t ldx, const void* W, int64_t N, void* out,
                         int out_dtype, int64_t ldo, const void* norm_w, float eps, int epilogue, const void* residual,
                         int64_t ldr, void* workspace, size_t workspace_bytes, void* stream) {
  FB_REQUIRE(fmt == FB_BFP8 || fmt == FB_BFP4, "fb_linear: W is bfp8 or bfp4 (dtype %d given)", fmt);
  FB_REQUIRE(x && W && out, "fb_linear: null pointer");
  FB_REQUIRE(M >= 1 && K >= 4 && K % 4 == 0 && N >= 16 && N % 16 == 0, "fb_linear: [%lld, %lld] @ [%lld, %lld]: K a multiple of 4, N of 16",
             (long long)M, (long long)K, (long long)K, (long long)N);
  FB_REQUIRE(out_dtype == FB_BF16 || out_dtype == FB_FP32, "fb_linear: out is bf16 or fp32");
  FB_REQUIRE(epilogue >= FB_EPI_NONE && epilogue <= FB_EPI_RESIDUAL, "fb_linear: unknown epilogue %d", epilogue);
  FB_REQUIRE(epilogue != FB_EPI_SWIGLU || N % 32 == 0, "fb_linear: SwiGLU pairs column j with j + N/2: N a multiple of 32");
  FB_REQUIRE(epilogue != FB_EPI_RESIDUAL || residual, "fb_linear: the residual epilogue needs a residual");
  const int64_t out_cols = epilogue == FB_EPI_SWIGLU ? N / 2 : N;
  FB_REQUIRE(ldx >= K && ldx % 4 == 0 && ldo >= out_cols && (epilogue != FB_EPI_RESIDUAL || ldr >= N), "fb_linear: row strides too small or unaligned");
  FB_REQUIRE((uintptr_t)x % 8 == 0 && (uintptr_t)W % 16 == 0 && (uintptr_t)out % 4 == 0 && (!norm_w || (uintptr_t)norm_w % 8 == 0),
             "fb_linear: misaligned pointer");
  fb::LinearArgs a{fmt, x, M, K, ldx, W, N, out, out_dtype, ldo, norm_w, eps, epilogue, residual, ldr, workspace, workspace_bytes};
  auto s = (cudaStream_t)stream;
  zero_new_workspace(workspace, workspace_bytes, s);
  // one token: the CUDA-core GEMV (a CTA per 16 columns; the streaming kernel - persistent CTAs fed by bulk copies -
  // is measured slower on every shape of the benchmark and runs only when asked for by FB_LINEAR_GEMV_STREAM); a few: tensor-core MMAs whose weight fragments are unpacked in registers (no bf16
  // tile in shared memory); more: the tcgen05 kernel, whose cost hardly grows with the tokens
  const int prefer = g_linear_kernel;
  if (prefer == FB_LINEAR_MMA && fb::linear_mma_supports(a)) return fb::linear_mma(a, s);
  if (prefer == FB_LINEAR_GEMV && M <= 4) return fb::linear_gemv(a, s);
  if (prefer == FB_LINEAR_GEMV_STREAM) {
    FB_REQUIRE(fb::linear_gemv_stream_supports(a), "fb_linear: [%lld, %lld] @ [%lld, %lld] is not for the streaming GEMV (one row, N a multiple of 64, the workspace given)",
               (long long)M, (long long)K, (long long)K, (long long)N);
    return fb::linear_gemv_stream(a, s);
  }
  // (measured: the register-fed kernel wins for up to 8 rows on bfp4 weights and on bfp8 matrices of up to 32 M values;
  // its legacy MMAs cost about 27 cycles each per SM quarter, so beyond 8 rows the tcgen05 kernel is faster)
  const bool few_rows_win = M > 1 && M <= 8 && K <= 8192 && (fmt == FB_BFP4 || K * N <= (int64_t)32 << 20);
  if (prefer == FB_LINEAR_AUTO && few_rows_win && fb::linear_mma_supports(a)) return fb::linear_mma(a, s);
  a.persistent = prefer == FB_LINEAR_PERSISTENT || (prefer == FB_LINEAR_AUTO && fb::linear_persistent_wins(a));
  if ((M > 1 || prefer == FB_LINEAR_PERSISTENT) && fb::linear_tcgen05_supports(a)) return fb::linear_tcgen05(a, s);
  return fb::linear_gemv(a, s);
}

extern "C" int fb_linear_chain_parts(int fmt, int64_t M, int64_t K, int64_t N, int epilogue) {
  if ((fmt != FB_BFP8 && fmt != FB_BFP4) || K % 8 || N % 16) return 0;
  return fb::linear_tcgen05_parts(fmt, M, K, N, epilogue);
}

extern "C" int fb_linear_chained(int fmt, const void* x, int64_t M, int64_t K, int64_t ldx, const void* W, int64_t N, void* out, int out_dtype,
                                 int64_t ldo, float eps, int epilogue, const void* residual, int64_t ldr, const float* sumsq_in, int sumsq_parts,
                                 const void* next_norm_w, void* xn_out, int64_t ld_xn, float* sumsq_out, void* workspace, size_t workspace_bytes,
                                 void* stream) {
  FB_REQUIRE(fmt == FB_BFP8 || fmt == FB_BFP4, "fb_linear_chained: W is bfp8 or bfp4 (dtype %d given)", fmt);
  FB_REQUIRE(x && W && out, "fb_linear_chained: null pointer");
  FB_REQUIRE(M >= 2 && M <= 128 && K >= 8 && K % 8 == 0 && N >= 16 && N % 16 == 0, "fb_linear_chained: 2 to 128 rows, K a multiple of 8, N of 16");
  FB_REQUIRE(out_dtype == FB_BF16 || out_dtype == FB_FP32, "fb_linear_chained: out is bf16 or fp32");
  FB_REQUIRE(epilogue >= FB_EPI_NONE && epilogue <= FB_EPI_RESIDUAL && (epilogue != FB_EPI_SWIGLU || N % 128 == 0), "fb_linear_chained: epilogue %d (SwiGLU: N a multiple of 128)", epilogue);
  FB_REQUIRE(epilogue != FB_EPI_RESIDUAL || residual, "fb_linear_chained: the residual epilogue needs a residual");
  FB_REQUIRE(sumsq_in || next_norm_w, "fb_linear_chained: neither takes a norm over nor hands one on (fb_linear does the rest)");
  FB_REQUIRE(!sumsq_in || sumsq_parts >= 1, "fb_linear_chained: the sums of squares come in at least one part");
  FB_REQUIRE(!next_norm_w || (xn_out && sumsq_out && ld_xn >= N && out_dtype == FB_BF16 && epilogue != FB_EPI_SWIGLU),
             "fb_linear_chained: handing a norm on takes xn_out and sumsq_out, a bf16 result and no SwiGLU");
  FB_REQUIRE(ldx >= K && ldx % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)W % 16 == 0, "fb_linear_chained: misaligned x or W");
  fb::LinearArgs a{fmt, x, M, K, ldx, W, N, out, out_dtype, ldo, nullptr, eps, epilogue, residual, ldr, workspace, workspace_bytes};
  a.sumsq_in = sumsq_in, a.sumsq_parts = sumsq_parts;
  a.next_norm_w = next_norm_w, a.xn_out = xn_out, a.ld_xn = ld_xn, a.sumsq_out = sumsq_out;
  FB_REQUIRE(fb::linear_tcgen05_supports(a), "fb_linear_chained: a shape the tensor-core kernel does not take");
  return fb::linear_tcgen05(a, (cudaStream_t)stream);
}

extern "C" int fb_linear_indexed(int fmt, const void* x, int64_t M, int64_t K, int64_t ldx, int64_t x_slot_rows, const void* W, int64_t N,
                                 int n_experts, const int32_t* index, int n_slots, int sum_slots, void* out, int out_dtype, int64_t ldo,
                                 int64_t out_slot_stride, const void* norm_w, float eps, int epilogue, const void* residual, int64_t ldr,
                                 const void* row_scale_bf16, void* workspace, size_t workspace_bytes, void* stream) {
  FB_REQUIRE(fmt == FB_BFP8 || fmt == FB_BFP4, "fb_linear_indexed: W is bfp8 or bfp4 (dtype %d given)", fmt);
  FB_REQUIRE(x && W && out && index && n_experts >= 1 && n_slots >= 1, "fb_linear_indexed: null pointer or no experts");
  FB_REQUIRE(M >= 1 && M <= 128 && K >= 8 && K % 8 == 0 && N >= 16 && N % 16 == 0, "fb_linear_indexed: up to 128 rows, K a multiple of 8, N of 16");
  FB_REQUIRE(out_dtype == FB_BF16 || out_dtype == FB_FP32, "fb_linear_indexed: out is bf16 or fp32");
  FB_REQUIRE(epilogue >= FB_EPI_NONE && epilogue <= FB_EPI_RESIDUAL && (epilogue != FB_EPI_SWIGLU || N % 128 == 0), "fb_linear_indexed: epilogue %d (SwiGLU: N a multiple of 128)", epilogue);
  FB_REQUIRE(!sum_slots || (epilogue != FB_EPI_SWIGLU && !row_scale_bf16 && K % 64 == 0), "fb_linear_indexed: summed slots take whole 64-row units of K, no SwiGLU, no row scale");
  FB_REQUIRE(epilogue != FB_EPI_RESIDUAL || residual, "fb_linear_indexed: the residual epilogue needs a residual");
  FB_REQUIRE(ldx % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)W % 16 == 0, "fb_linear_indexed: misaligned x or W");
  fb::LinearArgs a{fmt, x, M, K, ldx, W, N, out, out_dtype, ldo, norm_w, eps, epilogue, residual, ldr, workspace, workspace_bytes};
  fb::IndexedArgs ix{sum_slots ? 2 : 1, index, n_experts, n_slots, x_slot_rows, out_slot_stride, row_scale_bf16};
  return fb::linear_tcgen05_indexed(a, ix, (cudaStream_t)stream);
}
