// fb_linear for ONE token as a streaming kernel: persistent CTAs (two an SM), the packed weights arriving in shared memory
// by bulk copies (cp.async.bulk, one 64 x 64 unit of 4352 / 2304 bytes a copy, no multicast) into a ring of mbarrier-guarded
// stages that keeps ~50 KB in flight per CTA, eight consumer warps unpacking from shared memory.
//
// Work: the packed matrix is one run of units, a column group's units one after another (bfp_format.cuh), and CTA c takes
// the c-th of equal contiguous stretches of that run - so every CTA streams one contiguous piece of memory of the same
// length whatever the shape.  A stretch crosses column groups; the part of one group it holds is a SEGMENT.  Inside a
// unit a thread owns one row k of one run of 16 columns: one 16-byte read of shared memory, the masked bits entering packed
// fp32 FMAs as denormals (gemv.cuh), 16 sums kept over the segment; at its end the 64 rows' sums meet by a butterfly of
// shuffles and a pass through shared memory, and the segment's 64 column sums go to the workspace.  Each output tile
// (64 columns: a group, or with SwiGLU a gate group and its up group) counts the units that have arrived; the CTA that
// completes the count adds the tile's segments in their own order - the result is the same every run -, applies the
// RMSNorm's scale, SwiGLU or the residual, stores, and leaves the counter at zero for the next call.  Every wait on an
// mbarrier is bounded (sm100.cuh).
#include "gemv.cuh"
#include "linear.cuh"
#include "sm100.cuh"
#include <algorithm>
#include <atomic>

namespace fb {

namespace {

constexpr int GS_CONSUMERS = 256, GS_THREADS = GS_CONSUMERS + 32, GS_MAX_STAGES = 24, GS_SMEM = 112 * 1024;
enum { WAIT_GS_FULL = 301, WAIT_GS_EMPTY };

struct GemvStreamParams {
  LinearArgs a;
  int units, ksteps, groups, tiles, stages, max_segments;
  float* partials;      // [groups][max_segments][64]
  uint32_t* counters;   // [tiles], zero between calls
};

struct Slot {
  int at = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void next(int n) {
    if (++at == n) at = 0, phase ^= 1;
  }
};

__host__ __device__ inline int stretch_begin(int cta, int units, int ctas) { return (int)((int64_t)cta * units / ctas); }
// the CTA whose stretch holds unit u
__host__ __device__ inline int cta_of_unit(int u, int units, int ctas) {
  int c = (int)((int64_t)u * ctas / units);
  while (c + 1 < ctas && stretch_begin(c + 1, units, ctas) <= u) ++c;
  while (c > 0 && stretch_begin(c, units, ctas) > u) --c;
  return c;
}

__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(GS_CONSUMERS) : "memory"); }

template <int FMT>
__global__ void __launch_bounds__(GS_THREADS) linear_gemv_stream_kernel(const GemvStreamParams p) {
  constexpr int UNIT = unit_bytes(FMT), UNIT_MANT = unit_mant_bytes(FMT), RUN = run_bytes(FMT);
  extern __shared__ __align__(128) uint8_t smem[];
  const LinearArgs& a = p.a;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int KS = p.ksteps, ctas = gridDim.x;
  const bool swiglu = a.epilogue == FB_EPI_SWIGLU;
  uint8_t* ring = smem;                                                  // [stages][UNIT]
  float* xg = reinterpret_cast<float*>(ring + p.stages * UNIT);          // [KS * 64]: x (times the norm's weight), zeros past K
  float* red = xg + KS * KSTEP;                                          // [2][8 warps][16]: segments alternate between the two
  float* ssred = red + 2 * 8 * 16;                                       // [8]
  uint64_t* full = reinterpret_cast<uint64_t*>(ssred + 8);
  uint64_t* empty = full + GS_MAX_STAGES;
  uint32_t* flags = reinterpret_cast<uint32_t*>(empty + GS_MAX_STAGES);  // [0] a wait gave up, [1] this CTA completes the tile
  const uint32_t abort_flag = smem_u32(flags);

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) mbar_init(smem_u32(full + s), 1), mbar_init(smem_u32(empty + s), GS_CONSUMERS / 32);
    flags[0] = flags[1] = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const int u_begin = stretch_begin(blockIdx.x, p.units, ctas), u_end = stretch_begin(blockIdx.x + 1, p.units, ctas);

  if (warp == GS_CONSUMERS / 32) {
    // ---- the producer: one thread feeds the ring with the stretch's units in order (the weights are nobody's output, so
    // this does not wait for the kernel before)
    if (lane == 0) {
      const uint8_t* W = static_cast<const uint8_t*>(a.W);
      Slot r;
      for (int u = u_begin; u < u_end; ++u, r.next(p.stages)) {
        if (!mbar_wait(smem_u32(empty + r.at), r.phase ^ 1, abort_flag, WAIT_GS_EMPTY)) break;
        mbar_expect_tx(smem_u32(full + r.at), UNIT);
        bulk_copy_g2s(smem_u32(ring + r.at * UNIT), W + (int64_t)u * UNIT, UNIT, smem_u32(full + r.at));
      }
    }
    return;
  }

  // ---- the consumers.  The token first: xg[k] = x[k] (* g[k]) as fp32, and the sum of its squares for the norm
  griddep_wait();
  float ss = 0.f;
  {
    const uint16_t* x = static_cast<const uint16_t*>(a.x);
    const uint16_t* g = static_cast<const uint16_t*>(a.norm_w);
    for (int k = 4 * tid; k < KS * KSTEP; k += 4 * GS_CONSUMERS) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k < a.K) {  // (K is a multiple of 4)
        const uint2 xb = *reinterpret_cast<const uint2*>(x + k);
        v = make_float4(bf16_bits_to_float(xb.x & 0xFFFFu), bf16_bits_to_float(xb.x >> 16), bf16_bits_to_float(xb.y & 0xFFFFu), bf16_bits_to_float(xb.y >> 16));
        if (g) {
          ss = fmaf(v.x, v.x, ss), ss = fmaf(v.y, v.y, ss), ss = fmaf(v.z, v.z, ss), ss = fmaf(v.w, v.w, ss);
          const uint2 gb = __ldg(reinterpret_cast<const uint2*>(g + k));
          v.x *= bf16_bits_to_float(gb.x & 0xFFFFu), v.y *= bf16_bits_to_float(gb.x >> 16);
          v.z *= bf16_bits_to_float(gb.y & 0xFFFFu), v.w *= bf16_bits_to_float(gb.y >> 16);
        }
      }
      *reinterpret_cast<float4*>(xg + k) = v;
    }
    ss = warp_sum(ss);
    if (lane == 0) ssred[warp] = ss;
  }
  consumers_sync();
  griddep_launch_dependents();
  float rstd = 1.f;
  if (a.norm_w) {
    float s2 = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s2 += ssred[w];
    rstd = rsqrtf(s2 / (float)a.K + a.eps);
  }

  const int run = tid >> 6, krow = tid & 63;  // a warp: 32 rows of one run
  const uint32_t my_q = (uint32_t)(run * KSTEP + krow) * RUN, my_top = UNIT_MANT + run * KSTEP + krow;
  constexpr uint32_t LIFT = FMT == FB_BFP8 ? 63 : 67;
  Slot r;
  int segment_parity = 0;
  for (int u = u_begin; u < u_end;) {
    const int group = u / KS, k0 = u - group * KS, n = min(KS - k0, u_end - u);
    float acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0.f;
    bool alive = true;
    for (int i = 0; i < n; ++i, r.next(p.stages)) {
      if (!mbar_wait(smem_u32(full + r.at), r.phase, abort_flag, WAIT_GS_FULL)) { alive = false; break; }
      const uint8_t* unit = ring + r.at * UNIT;
      uint32_t words[4];
      if (FMT == FB_BFP8) {
        const uint4 q = *reinterpret_cast<const uint4*>(unit + my_q);
        words[0] = q.x, words[1] = q.y, words[2] = q.z, words[3] = q.w;
      } else {
        const uint2 q = *reinterpret_cast<const uint2*>(unit + my_q);
        words[0] = q.x, words[1] = q.y;
      }
      const uint32_t top = unit[my_top];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(empty + r.at));
      const float xk = xg[(k0 + i) * KSTEP + krow];
      uint32_t v[8];
      float xs;
      if (top <= 186) {  // (gemv.cuh: the masked bits as fp32 denormals, 2^(top-64) in the activation's factor)
        mask_run<FMT>(words, v);
        xs = xk * __uint_as_float((top + LIFT) << 23);
      } else {
        if (FMT == FB_BFP8) unpack_run8(make_uint4(words[0], words[1], words[2], words[3]), top, v);
        else unpack_run4(make_uint2(words[0], words[1]), top, v);
        xs = xk * 5.421010862427522e-20f;  // 2^-64
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 w2 = make_float2(__uint_as_float(v[j] << 16), __uint_as_float(v[j] & 0xFFFF0000u));
        const float2 s = __ffma2_rn(w2, make_float2(xs, xs), make_float2(acc[2 * j], acc[2 * j + 1]));
        acc[2 * j] = s.x, acc[2 * j + 1] = s.y;
      }
    }
    if (!alive) return;  // (the status word says which wait; the other consumers see the abort flag in their own waits)
    // ---- the segment's end: the rows' sums meet (warps 2r and 2r+1 hold run r's two halves of the rows)
    const float mine = butterfly16(acc);
    float* rd = red + segment_parity * 8 * 16;
    segment_parity ^= 1;
    if (!(lane & 1)) rd[warp * 16 + column_of_lane(lane)] = mine;
    consumers_sync();
    if (ld_shared_volatile(abort_flag)) return;  // (all consumers together: nobody is left waiting at a barrier)
    u += n;
    if (warp >= 2) continue;  // the other warps go on with the next segment while these two publish this one
    const int col = tid, tile = swiglu && group >= p.groups / 2 ? group - p.groups / 2 : group;
    {
      const float sum = rd[(2 * (col >> 4)) * 16 + (col & 15)] + rd[(2 * (col >> 4) + 1) * 16 + (col & 15)];
      const int segment = (int)blockIdx.x - cta_of_unit(group * KS, p.units, ctas);
      __stcg(p.partials + ((int64_t)group * p.max_segments + segment) * 64 + col, sum);
      __threadfence();
    }
    asm volatile("bar.sync 2, 64;" ::: "memory");
    if (tid == 0) {
      const uint32_t whole = (uint32_t)(swiglu ? 2 * KS : KS);
      flags[1] = atomicAdd(p.counters + tile, (uint32_t)n) + (uint32_t)n == whole;
    }
    asm volatile("bar.sync 2, 64;" ::: "memory");
    if (!flags[1]) continue;
    // ---- this CTA brought the tile's last units: add the segments in their order, finish the 64 columns
    __threadfence();
    auto column_sum = [&](int g) {
      const int c0 = cta_of_unit(g * KS, p.units, ctas), c1 = cta_of_unit(g * KS + KS - 1, p.units, ctas);
      const float* at = p.partials + (int64_t)g * p.max_segments * 64 + col;
      float s = 0.f;
      for (int c = c0; c <= c1; ++c, at += 64) s += __ldcg(at);
      return s * GEMV_ACC_SCALE * rstd;
    };
    float y = column_sum(tile);
    const int64_t ncol = (int64_t)tile * 64 + col;
    if (swiglu) y = y / (1.f + __expf(-y)) * column_sum(tile + p.groups / 2);
    else if (a.epilogue == FB_EPI_RESIDUAL) y += bf16_bits_to_float(static_cast<const uint16_t*>(a.residual)[ncol]);
    if (a.out_dtype == FB_FP32) static_cast<float*>(a.out)[ncol] = y;
    else static_cast<uint16_t*>(a.out)[ncol] = (uint16_t)float_to_bf16_bits(y);
    if (tid == 0) p.counters[tile] = 0;
  }
}

int sms_of_device() {
  static int sms[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
  return sms[dev] > 0 ? sms[dev] : 148;
}

struct Plan {
  int ksteps, groups, units, ctas, max_segments;
};
Plan plan_of(int64_t K, int64_t N) {
  Plan pl;
  pl.ksteps = (int)ksteps_of(K), pl.groups = (int)(N / 64);
  pl.units = pl.ksteps * pl.groups;
  pl.ctas = std::max(1, std::min(2 * sms_of_device(), pl.units / 4));
  pl.max_segments = pl.ksteps / (pl.units / pl.ctas) + 2;
  return pl;
}

int stages_of(int fmt, int64_t K, int units_per_cta) {
  const int64_t fixed = ksteps_of(K) * KSTEP * 4 + 2048;
  const int64_t fit = (GS_SMEM - fixed) / unit_bytes(fmt);
  return (int)std::min<int64_t>(std::min<int64_t>(GS_MAX_STAGES, fit), units_per_cta + 1);
}

template <int FMT>
int launch(const GemvStreamParams& p, int ctas, size_t smem, cudaStream_t s) {
  static std::atomic<uint64_t> opted{0};  // the shared-memory opt-in, once per device
  if (first_on_device(opted)) cudaFuncSetAttribute(linear_gemv_stream_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, GS_SMEM);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(ctas), cfg.blockDim = dim3(GS_THREADS), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, linear_gemv_stream_kernel<FMT>, p);
  return launch_status("fb_linear (streaming gemv)");
}

}  // namespace

size_t linear_gemv_stream_workspace(int64_t K, int64_t N) {
  if (N % 64 || N / 64 * ksteps_of(K) >= (int64_t)1 << 30) return 0;
  const Plan pl = plan_of(K, N);
  return WS_BODY_AT + (size_t)pl.groups * pl.max_segments * 64 * sizeof(float);
}

bool linear_gemv_stream_supports(const LinearArgs& a) {
  if (a.M != 1 || (a.fmt != FB_BFP8 && a.fmt != FB_BFP4) || a.N % 64 || a.next_norm_w || a.sumsq_in) return false;
  if (a.epilogue == FB_EPI_SWIGLU && a.N % 128) return false;
  const size_t need = linear_gemv_stream_workspace(a.K, a.N);
  if (!need || !a.workspace || a.workspace_bytes < need || (uintptr_t)a.workspace % 16) return false;
  const Plan pl = plan_of(a.K, a.N);
  if ((a.epilogue == FB_EPI_SWIGLU ? pl.groups / 2 : pl.groups) > (int)WS_COUNTERS) return false;
  return stages_of(a.fmt, a.K, (pl.units + pl.ctas - 1) / pl.ctas) >= std::min(4, (pl.units + pl.ctas - 1) / pl.ctas + 1);
}

int linear_gemv_stream(const LinearArgs& a, cudaStream_t s) {
  const Plan pl = plan_of(a.K, a.N);
  GemvStreamParams p;
  p.a = a;
  p.units = pl.units, p.ksteps = pl.ksteps, p.groups = pl.groups, p.max_segments = pl.max_segments;
  p.tiles = a.epilogue == FB_EPI_SWIGLU ? pl.groups / 2 : pl.groups;
  p.stages = stages_of(a.fmt, a.K, (pl.units + pl.ctas - 1) / pl.ctas);
  p.partials = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + WS_BODY_AT);
  p.counters = reinterpret_cast<uint32_t*>(static_cast<char*>(a.workspace) + WS_COUNTERS_AT);
  const size_t smem = (size_t)p.stages * unit_bytes(a.fmt) + (size_t)pl.ksteps * KSTEP * 4 + 2048;
  return a.fmt == FB_BFP8 ? launch<FB_BFP8>(p, pl.ctas, smem, s) : launch<FB_BFP4>(p, pl.ctas, smem, s);
}

int status_word_gemv_stream() { return read_and_clear_status_word(); }

}  // namespace fb
