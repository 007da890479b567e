// fb_linear for a few tokens: the block-float GEMV with RMSNorm prologue and SwiGLU / residual epilogue.
#include "gemv.cuh"
#include "linear.cuh"
#include "sm100.cuh"

namespace fb {

// One CTA of 8 warps per column block (per gate/up pair of blocks with the SwiGLU epilogue: warps 0-3
// take the gate's block, 4-7 the up's).  See gemv.cuh for the per-lane work.
template <int FMT, int M, bool NORM>
__global__ void __launch_bounds__(256) linear_gemv_kernel(LinearArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool swiglu = a.epilogue == FB_EPI_SWIGLU;
  const int G = swiglu ? 4 : 8;
  const int grp = swiglu ? warp >> 2 : 0, wg = swiglu ? warp & 3 : warp;
  const int64_t NB = a.N / 16, K = a.K;
  const int64_t b = blockIdx.x + (grp ? NB / 2 : 0);
  const uint8_t* col = static_cast<const uint8_t*>(a.W) + (b / GROUP_RUNS) * ksteps_of(K) * unit_bytes(FMT);
  // The CTAs of a column group's four runs read interleaved 1 KB pieces of one contiguous strip; the CTA of run 0 asks
  // for the whole strip to be brought into L2 up front (the bulk path keeps far more bytes in flight than a CTA's
  // loads can), so the loads below mostly find their bytes there.
  if (b % GROUP_RUNS == 0 && wg == 0 && lane == 0) {
    const int64_t bytes = ksteps_of(K) * unit_bytes(FMT);
    for (int64_t at = 0; at < bytes; at += 32768) bulk_prefetch_l2(col + at, (uint32_t)(bytes - at < 32768 ? bytes - at : 32768));
  }

  float acc[M][16], ss[M];
#pragma unroll
  for (int t = 0; t < M; ++t) {
    ss[t] = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[t][j] = 0.f;
  }
  gemv_accumulate<FMT, M, NORM>(col, (int)(b % GROUP_RUNS), static_cast<const uint16_t*>(a.x), a.ldx, static_cast<const uint16_t*>(a.norm_w), K,
                                wg * 128, G * 128, acc, ss);
  // Only now may the next kernel's CTAs move in beside this one's (four of these fit an SM): were they let in at the
  // start, the L2 prefetches of several kernels ahead would compete with this kernel's loads and evict one another.
  griddep_launch_dependents();

  __shared__ float red[8][M][16];
  __shared__ float ssred[8][M];
#pragma unroll
  for (int t = 0; t < M; ++t) {
    float r = butterfly16(acc[t]);
    if (!(lane & 1)) red[warp][t][column_of_lane(lane)] = r;
    if (NORM) {
      float s = warp_sum(ss[t]);
      if (lane == 0) ssred[warp][t] = s;
    }
  }
  __syncthreads();
  if (threadIdx.x >= M * 16) return;
  const int t = threadIdx.x >> 4, j = threadIdx.x & 15;
  float v = 0.f, u = 0.f, s2 = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    if (w < G) v += red[w][t][j]; else u += red[w][t][j];
    if (NORM && w < G) s2 += ssred[w][t];  // a group's lanes read every row once
  }
  v *= GEMV_ACC_SCALE, u *= GEMV_ACC_SCALE;
  if (NORM) {
    float rstd = rsqrtf(s2 / (float)K + a.eps);
    v *= rstd, u *= rstd;
  }
  const int64_t n = 16 * (int64_t)blockIdx.x + j;
  float y = v;
  if (swiglu) y = v / (1.f + __expf(-v)) * u;
  else if (a.epilogue == FB_EPI_RESIDUAL) y += bf16_bits_to_float(static_cast<const uint16_t*>(a.residual)[t * a.ldr + n]);
  if (a.out_dtype == FB_FP32) static_cast<float*>(a.out)[t * a.ldo + n] = y;
  else static_cast<uint16_t*>(a.out)[t * a.ldo + n] = (uint16_t)float_to_bf16_bits(y);
}

template <int FMT, int M>
static void launch_gemv(const LinearArgs& a, cudaStream_t s) {
  unsigned blocks = (unsigned)(a.N / 16 / (a.epilogue == FB_EPI_SWIGLU ? 2 : 1));
  // a programmatic dependent of the kernel before it: the L2 prefetch and the first weight loads do not wait for it
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(blocks), cfg.blockDim = dim3(256), cfg.dynamicSmemBytes = 0, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  if (a.norm_w) cudaLaunchKernelEx(&cfg, linear_gemv_kernel<FMT, M, true>, a);
  else cudaLaunchKernelEx(&cfg, linear_gemv_kernel<FMT, M, false>, a);
}

template <int FMT>
static void launch_gemv_m(const LinearArgs& a, cudaStream_t s) {
  switch (a.M) {
    case 1: launch_gemv<FMT, 1>(a, s); break;
    case 2: launch_gemv<FMT, 2>(a, s); break;
    case 3: launch_gemv<FMT, 3>(a, s); break;
    default: launch_gemv<FMT, 4>(a, s); break;
  }
}

// Rows in chunks of at most 4; each chunk is one pass over the weights.
int linear_gemv(const LinearArgs& args, cudaStream_t s) {
  const int64_t out_cols_elem = args.out_dtype == FB_FP32 ? 4 : 2;
  for (int64_t m0 = 0; m0 < args.M; m0 += 4) {
    LinearArgs a = args;
    a.M = args.M - m0 < 4 ? args.M - m0 : 4;
    a.x = static_cast<const uint16_t*>(args.x) + m0 * args.ldx;
    a.out = static_cast<char*>(args.out) + m0 * args.ldo * out_cols_elem;
    if (args.residual) a.residual = static_cast<const uint16_t*>(args.residual) + m0 * args.ldr;
    if (args.fmt == FB_BFP8) launch_gemv_m<FB_BFP8>(a, s); else launch_gemv_m<FB_BFP4>(a, s);
  }
  return launch_status("fb_linear (gemv)");
}

}  // namespace fb
