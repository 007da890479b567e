// fb_linear on the 5th-generation tensor cores: block-float weights x a batch of tokens (5 <= M <= 128 per pass).
//
// The weight matrix is the MMA's A operand (128 output columns per CTA = the 128 accumulator lanes in TMEM) and the
// tokens are its N dimension, so a decode batch of 32 tokens costs one 128x32x16 tcgen05.mma per 16 rows of K and
// the kernel stays bound by the HBM stream of packed weights, which it reads exactly once:
//
//   raw producer (1 thread)  cp.async.bulk: 8 column blocks x 64 rows of packed mantissas + exponents -> smem ring
//   x producer   (1 thread)  TMA tile [tokens x 64] of the (normalised) activations, 128B-swizzled   -> smem ring
//   8 worker warps           raw bytes -> bf16 pairs in registers (bfp_format.cuh) -> MN-major 128B-swizzled A tile
//   MMA issuer   (1 thread)  4 x tcgen05.mma (K = 16 each) per stage, accumulating in TMEM; tcgen05.commit frees stages
//   epilogue (worker warps)  tcgen05.ld -> RMSNorm row scale, SwiGLU / residual, bf16 / fp32 store
//
// Few column tiles (N = 4096 gives 32) cannot fill 148 SMs, so K is split across CTAs; partial tiles go through an
// fp32 workspace and the last CTA of a tile to finish sums them in split order (deterministic) and runs the epilogue.
// Every mbarrier wait is bounded (sm100.cuh).
#include <cuda.h>

#include "bfp_format.cuh"
#include "linear.cuh"
#include "sm100.cuh"

namespace fb {

namespace {

constexpr int TILE_N = 128;  // output columns per CTA (MMA M)
constexpr int KC = 64;       // rows of K per pipeline stage
constexpr int WORKERS = 256;
constexpr int WARP_RAW = 8, WARP_MMA = 9, WARP_X = 10;
constexpr int THREADS = 11 * 32;
constexpr int A_STAGES = 2, A_STAGE_BYTES = TILE_N * KC * 2;
constexpr int MAX_STAGES = 8;
constexpr int WS_COUNTERS = 4096, WS_RSTD = 1024;  // workspace: tile counters, row scales, then x', then partials

template <int FMT>
struct RawStage {
  static constexpr int RUN = FMT == FB_BFP8 ? 16 : 8;
  static constexpr int BLOCK = KC * RUN;            // one column block's mantissas
  static constexpr int BYTES = 8 * (BLOCK + KC);    // + its exponents
};

struct GemmParams {
  LinearArgs a;
  int nt;  // MMA N: tokens rounded up to a multiple of 16
  int tmem_cols;
  int splits, chunks_per_split, chunks_total;
  int raw_stages, x_stages;
  const float* rstd;  // [M] row scales of the RMSNorm prologue, or null
  float* partials;
  int* counters;
};

enum WaitCode { WAIT_RAW_EMPTY = 101, WAIT_RAW_FULL, WAIT_X_EMPTY, WAIT_X_FULL, WAIT_A_EMPTY, WAIT_A_FULL, WAIT_ACC };

template <int FMT>
__global__ void __launch_bounds__(THREADS) linear_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  using RS = RawStage<FMT>;
  extern __shared__ uint8_t smem_unaligned[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int nt = p.nt, R = p.raw_stages, SX = p.x_stages;
  const LinearArgs& a = p.a;
  const bool swiglu = a.epilogue == FB_EPI_SWIGLU;
  const int64_t K = a.K, NB = a.N / 16;

  uint8_t* sA = smem;
  uint8_t* sX = sA + A_STAGES * A_STAGE_BYTES;
  uint8_t* sRaw = sX + SX * nt * 128;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sRaw + R * RS::BYTES);
  uint64_t* raw_full = bars, *raw_empty = bars + MAX_STAGES, *x_full = bars + 2 * MAX_STAGES, *x_empty = bars + 3 * MAX_STAGES;
  uint64_t* a_full = bars + 4 * MAX_STAGES, *a_empty = a_full + A_STAGES, *acc_full = a_empty + A_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* is_last = const_cast<int*>(abort_flag) + 1;

  if (tid == 0) {
    for (int s = 0; s < R; ++s) mbar_init(smem_u32(raw_full + s), 1), mbar_init(smem_u32(raw_empty + s), WORKERS / 32);
    for (int s = 0; s < SX; ++s) mbar_init(smem_u32(x_full + s), 1), mbar_init(smem_u32(x_empty + s), 1);
    for (int s = 0; s < A_STAGES; ++s) mbar_init(smem_u32(a_full + s), WORKERS / 32), mbar_init(smem_u32(a_empty + s), 1);
    mbar_init(smem_u32(acc_full), 1);
    *abort_flag = 0;
    *is_last = 1;
    fence_barrier_init();
  }
  if (warp == WARP_MMA) tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  const int c0 = split * p.chunks_per_split;
  const int n_chunks = min(p.chunks_total - c0, p.chunks_per_split);

  // which column block each of the tile's 8 raw slots holds: 8 neighbours, or 4 gate blocks then their 4 up blocks
  auto block_of = [&](int bl) -> int64_t {
    if (!swiglu) { int64_t b = 8 * (int64_t)tile + bl; return b < NB ? b : -1; }
    int64_t g = 4 * (int64_t)tile + (bl & 3);
    return g < NB / 2 ? g + (bl >> 2) * (NB / 2) : -1;
  };

  if (warp == WARP_RAW && lane == 0) {
    const uint8_t* W = static_cast<const uint8_t*>(a.W);
    const uint8_t* Wexp = W + mant_bytes(FMT, K, a.N);
    int valid = 0;
    for (int bl = 0; bl < 8; ++bl) valid += block_of(bl) >= 0;
    for (int i = 0; i < n_chunks; ++i) {
      const int r = i % R;
      mbar_wait(smem_u32(raw_empty + r), ((i / R) & 1) ^ 1, abort_flag, WAIT_RAW_EMPTY);
      const int64_t k0 = (int64_t)(c0 + i) * KC;
      const uint32_t bar = smem_u32(raw_full + r), dst = smem_u32(sRaw + r * RS::BYTES);
      mbar_expect_tx(bar, valid * (RS::BLOCK + KC));
      for (int bl = 0; bl < 8; ++bl) {
        const int64_t b = block_of(bl);
        if (b < 0) continue;
        bulk_copy_g2s(dst + bl * RS::BLOCK, W + (b * K + k0) * RS::RUN, RS::BLOCK, bar);
        bulk_copy_g2s(dst + 8 * RS::BLOCK + bl * KC, Wexp + b * K + k0, KC, bar);
      }
    }
  } else if (warp == WARP_X && lane == 0) {
    for (int i = 0; i < n_chunks; ++i) {
      const int s = i % SX;
      mbar_wait(smem_u32(x_empty + s), ((i / SX) & 1) ^ 1, abort_flag, WAIT_X_EMPTY);
      mbar_expect_tx(smem_u32(x_full + s), nt * 128);
      tma_load_2d(smem_u32(sX + s * nt * 128), &tmap_x, (c0 + i) * KC, 0, smem_u32(x_full + s));
    }
  } else if (warp == WARP_MMA && lane == 0) {
    const uint32_t idesc = umma_idesc_bf16(nt, true, false);
    for (int i = 0; i < n_chunks; ++i) {
      const int sa = i % A_STAGES, sx = i % SX;
      mbar_wait(smem_u32(a_full + sa), (i / A_STAGES) & 1, abort_flag, WAIT_A_FULL);
      mbar_wait(smem_u32(x_full + sx), (i / SX) & 1, abort_flag, WAIT_X_FULL);
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < KC / 16; ++kk) {
        // A: MN-major, 64-column swizzle atoms 1024 B apart, groups of 8 rows of K 2048 B apart; 16 rows of K per MMA
        const uint64_t da = umma_smem_desc(smem_u32(sA + sa * A_STAGE_BYTES + kk * 4096), 1024, 2048);
        // X: K-major, one 128-byte swizzled row per token, groups of 8 tokens 1024 B apart; 32 bytes of K per MMA
        const uint64_t dx = umma_smem_desc(smem_u32(sX + sx * nt * 128 + kk * 32), 16, 1024);
        umma_bf16(tmem, da, dx, idesc, (i | kk) != 0);
      }
      umma_commit(smem_u32(a_empty + sa));
      umma_commit(smem_u32(x_empty + sx));
    }
    umma_commit(smem_u32(acc_full));
  } else if (warp < WORKERS / 32) {
    for (int i = 0; i < n_chunks; ++i) {
      const int r = i % R, sa = i % A_STAGES;
      mbar_wait(smem_u32(raw_full + r), (i / R) & 1, abort_flag, WAIT_RAW_FULL);
      mbar_wait(smem_u32(a_empty + sa), ((i / A_STAGES) & 1) ^ 1, abort_flag, WAIT_A_EMPTY);
      const uint8_t* raw = sRaw + r * RS::BYTES;
#pragma unroll
      for (int j = 0; j < 8 * KC / WORKERS; ++j) {
        const int u = tid + WORKERS * j, bl = u >> 6, k = u & 63;
        const uint32_t top = raw[8 * RS::BLOCK + bl * KC + k];
        uint32_t v[8];
        if (FMT == FB_BFP8) unpack_run8(*reinterpret_cast<const uint4*>(raw + bl * RS::BLOCK + k * 16), top, v);
        else unpack_run4(*reinterpret_cast<const uint2*>(raw + bl * RS::BLOCK + k * 8), top, v);
        const int slot = swiglu ? ((bl & 3) << 1 | bl >> 2) : bl;  // gate and up blocks alternate: rows r and r+16 pair up
        uint8_t* row = sA + sa * A_STAGE_BYTES + ((k >> 3) * 2 + (slot >> 2)) * 1024 + (k & 7) * 128;
        const int c = (slot & 3) * 2;
        *reinterpret_cast<uint4*>(row + ((c ^ (k & 7)) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<uint4*>(row + (((c + 1) ^ (k & 7)) << 4)) = make_uint4(v[4], v[5], v[6], v[7]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(raw_empty + r));
        mbar_arrive(smem_u32(a_full + sa));
      }
    }
  }

  // ---- epilogue: worker warp w reads TMEM lanes 32*(w%4).. (its quarter) and half of the token columns
  const int q = warp & 3, ncol = nt / 2, col0 = (warp >> 2) * ncol, row = 32 * q + lane;
  const bool worker = warp < WORKERS / 32;
  const int64_t M = a.M;

  auto finish = [&](int t, float val) {  // t is the same for the whole warp
    if (t >= M) return;
    if (p.rstd) val *= p.rstd[t];
    int64_t n;
    bool store;
    if (swiglu) {
      const float up = __shfl_xor_sync(0xffffffffu, val, 16);
      val = val / (1.f + __expf(-val)) * up;
      n = 64 * (int64_t)tile + 16 * q + lane;
      store = lane < 16 && n < a.N / 2;
    } else {
      n = TILE_N * (int64_t)tile + row;
      store = n < a.N;
      if (store && a.epilogue == FB_EPI_RESIDUAL) val += bf16_bits_to_float(static_cast<const uint16_t*>(a.residual)[t * a.ldr + n]);
    }
    if (!store) return;
    if (a.out_dtype == FB_FP32) static_cast<float*>(a.out)[t * a.ldo + n] = val;
    else static_cast<uint16_t*>(a.out)[t * a.ldo + n] = (uint16_t)float_to_bf16_bits(val);
  };

  if (worker) {
    mbar_wait(smem_u32(acc_full), 0, abort_flag, WAIT_ACC);
    tc_fence_after();
    float* mine = p.partials + ((size_t)(tile * p.splits + split) * nt) * TILE_N;
    for (int cb = 0; cb < ncol; cb += 8) {
      float v[8];
      tmem_ld8(tmem + ((uint32_t)(32 * q) << 16) + col0 + cb, v);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        if (p.splits == 1) finish(col0 + cb + e, v[e]);
        else mine[(size_t)(col0 + cb + e) * TILE_N + row] = v[e];
      }
    }
  }
  if (p.splits > 1) {
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int done = atomicAdd(p.counters + tile, 1);
      *is_last = done == p.splits - 1;
      if (*is_last) p.counters[tile] = 0;  // ready for the next launch (a replayed graph)
    }
    __syncthreads();
    if (*is_last && worker) {
      __threadfence();
      const float* all = p.partials + ((size_t)tile * p.splits * nt) * TILE_N;
      for (int t = col0; t < col0 + ncol && t < M; ++t) {
        float val = 0.f;
        for (int s = 0; s < p.splits; ++s) val += __ldcg(all + ((size_t)s * nt + t) * TILE_N + row);
        finish(t, val);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem, p.tmem_cols);
  }
}

// x' = bf16(x * g) and rstd[t] = rsqrt(mean(x^2) + eps): the RMSNorm prologue's two factors, once per call.
// The row scale commutes with the matmul, so the GEMM applies it to the accumulators.
__global__ void __launch_bounds__(256) rms_prepare_kernel(const uint16_t* __restrict__ x, int64_t ldx, const uint16_t* __restrict__ g,
                                                          int64_t K, float eps, uint16_t* __restrict__ xn, float* __restrict__ rstd) {
  const int t = blockIdx.x;
  float ss = 0.f;
  for (int64_t k = 2 * threadIdx.x; k < K; k += 2 * blockDim.x) {
    const uint32_t xb = *reinterpret_cast<const uint32_t*>(x + t * ldx + k), gb = *reinterpret_cast<const uint32_t*>(g + k);
    const float x0 = bf16_bits_to_float(xb & 0xFFFFu), x1 = bf16_bits_to_float(xb >> 16);
    ss = fmaf(x0, x0, fmaf(x1, x1, ss));
    *reinterpret_cast<uint32_t*>(xn + t * K + k) = pack_bf16x2(x0 * bf16_bits_to_float(gb & 0xFFFFu), x1 * bf16_bits_to_float(gb >> 16));
  }
  __shared__ float red[8];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += red[w];
    rstd[t] = rsqrtf(s / (float)K + eps);
  }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
  static EncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess && res == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiled>(p);
  }
  return fn;
}

struct Plan {
  int nt, tmem_cols, tiles, splits, cps, chunks, raw_stages, x_stages;
  size_t smem;
};

Plan make_plan(int fmt, int64_t M, int64_t K, int64_t N, int epilogue) {
  Plan pl;
  pl.nt = (int)((M + 15) / 16 * 16);
  pl.tmem_cols = pl.nt <= 32 ? 32 : pl.nt <= 64 ? 64 : 128;
  pl.tiles = (int)(epilogue == FB_EPI_SWIGLU ? ceil_div(N / 2, 64) : ceil_div(N, TILE_N));
  pl.chunks = (int)(K / KC);
  int want = 296 / pl.tiles;  // two CTAs per SM
  want = want < 1 ? 1 : want;
  int most = pl.chunks / 4 < 1 ? 1 : pl.chunks / 4;  // at least 4 stages of work per CTA
  int splits = want < most ? want : most;
  pl.cps = (int)ceil_div(pl.chunks, splits);
  pl.splits = (int)ceil_div(pl.chunks, pl.cps);
  const int raw = fmt == FB_BFP8 ? RawStage<FB_BFP8>::BYTES : RawStage<FB_BFP4>::BYTES;
  pl.x_stages = pl.nt <= 64 ? 4 : 3;
  const size_t fixed = 1024 + A_STAGES * A_STAGE_BYTES + (size_t)pl.x_stages * pl.nt * 128 + 5 * MAX_STAGES * 8 + 64;
  const size_t budget = pl.nt <= 64 ? 112 * 1024 : 200 * 1024;  // small batches: two CTAs share an SM
  int stages = (int)((budget - fixed) / raw);
  pl.raw_stages = stages > MAX_STAGES ? MAX_STAGES : stages;
  pl.smem = fixed + (size_t)pl.raw_stages * raw;
  return pl;
}

}  // namespace

bool linear_tcgen05_supports(const LinearArgs& a) {
  return a.K % KC == 0 && a.M >= 1 && a.ldx % 8 == 0 && (uintptr_t)a.x % 16 == 0 && encode_tiled() != nullptr &&
         (a.epilogue != FB_EPI_SWIGLU || a.N % 32 == 0);
}

size_t linear_tcgen05_workspace(int64_t M, int64_t K, int64_t N) {
  if (M <= 4 || K % KC) return 0;
  const int64_t rows = M < 128 ? M : 128;
  const int nt = (int)((rows + 15) / 16 * 16);
  // partial tiles: never more than ~296 CTAs' worth, each nt x 128 floats
  return WS_COUNTERS + WS_RSTD + (size_t)rows * K * 2 + (size_t)(296 + 148) * nt * TILE_N * 4;
}

static int run_pass(const LinearArgs& a, cudaStream_t s) {
  Plan pl = make_plan(a.fmt, a.M, a.K, a.N, a.epilogue);
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  const size_t xn_bytes = a.norm_w ? (size_t)a.M * a.K * 2 : 0;
  const size_t need = WS_COUNTERS + WS_RSTD + xn_bytes + (pl.splits > 1 ? (size_t)pl.tiles * pl.splits * pl.nt * TILE_N * 4 : 0);
  if (need > WS_COUNTERS + WS_RSTD && (!ws || a.workspace_bytes < need)) {
    set_error("fb_linear: workspace of %zu bytes needed, %zu given (fb_linear_workspace_bytes)", need, a.workspace_bytes);
    return FB_ERR_MEMORY;
  }
  GemmParams p{};
  p.a = a;
  p.nt = pl.nt, p.tmem_cols = pl.tmem_cols, p.splits = pl.splits, p.chunks_per_split = pl.cps, p.chunks_total = pl.chunks;
  p.raw_stages = pl.raw_stages, p.x_stages = pl.x_stages;
  p.counters = reinterpret_cast<int*>(ws);
  const void* x = a.x;
  int64_t ldx = a.ldx;
  if (a.norm_w) {
    float* rstd = reinterpret_cast<float*>(ws + WS_COUNTERS);
    uint16_t* xn = reinterpret_cast<uint16_t*>(ws + WS_COUNTERS + WS_RSTD);
    rms_prepare_kernel<<<(unsigned)a.M, 256, 0, s>>>(static_cast<const uint16_t*>(a.x), a.ldx, static_cast<const uint16_t*>(a.norm_w), a.K,
                                                     a.eps, xn, rstd);
    p.rstd = rstd, x = xn, ldx = a.K;
  }
  p.partials = reinterpret_cast<float*>(ws + WS_COUNTERS + WS_RSTD + xn_bytes);

  CUtensorMap tmap;
  const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
  const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
  const cuuint32_t box[2] = {KC, (cuuint32_t)pl.nt}, estr[2] = {1, 1};
  CUresult rc = encode_tiled()(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    set_error("fb_linear: cuTensorMapEncodeTiled failed (%d) for x [%lld, %lld] stride %lld", (int)rc, (long long)a.M, (long long)a.K, (long long)ldx);
    return FB_ERR_LAUNCH;
  }
  dim3 grid(pl.tiles, pl.splits);
  auto kernel = a.fmt == FB_BFP8 ? linear_tcgen05_kernel<FB_BFP8> : linear_tcgen05_kernel<FB_BFP4>;
  static bool attr_set[2] = {false, false};
  if (!attr_set[a.fmt == FB_BFP8]) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    attr_set[a.fmt == FB_BFP8] = true;
  }
  kernel<<<grid, THREADS, pl.smem, s>>>(tmap, p);
  return launch_status("fb_linear (tcgen05)");
}

int linear_tcgen05(const LinearArgs& args, cudaStream_t s) {
  const int64_t esz = args.out_dtype == FB_FP32 ? 4 : 2;
  for (int64_t m0 = 0; m0 < args.M; m0 += 128) {
    LinearArgs a = args;
    a.M = args.M - m0 < 128 ? args.M - m0 : 128;
    a.x = static_cast<const uint16_t*>(args.x) + m0 * args.ldx;
    a.out = static_cast<char*>(args.out) + m0 * args.ldo * esz;
    if (args.residual) a.residual = static_cast<const uint16_t*>(args.residual) + m0 * args.ldr;
    if (int rc = run_pass(a, s)) return rc;
  }
  return FB_OK;
}

}  // namespace fb

extern "C" int fb_status_word(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, fb::g_status_word, sizeof v) != cudaSuccess) return FB_ERR_LAUNCH;
  if (v) cudaMemcpyToSymbol(fb::g_status_word, &zero, sizeof zero);
  return v;
}
