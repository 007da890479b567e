// fb_linear on the 5th-generation tensor cores: block-float weights x a batch of tokens (up to 128 per pass).
//
// The weight matrix is the MMA's A operand (128 output columns per CTA = the 128 accumulator lanes in TMEM) and the
// tokens are its N dimension, so a decode batch of 32 tokens costs one 128x32x16 tcgen05.mma per 16 rows of K and
// the kernel stays bound by the HBM stream of packed weights, which it reads exactly once:
//
//   x producer   (1 thread)  TMA tiles [tokens x 64] of the (normalised) activations, 128B-swizzled     -> smem ring
//                            (the packed weights are NOT prefetched into L2: the workers' own loads stream at the full
//                            HBM rate, and a bulk L2 prefetch running ten steps ahead was measured to cost 5 %)
//   16 worker warps          in 4 teams, each taking every fourth step: packed bytes by 128-bit global loads into
//                            registers that are refilled for the team's next step as soon as they are unpacked (no
//                            staging in shared memory, whose bandwidth the bf16 operand tiles need) -> bf16 pairs
//                            (bfp_format.cuh) -> MN-major 128B-swizzled A tiles
//   2 MMA issuers (1 thread each) 8 x tcgen05.mma (K = 16 each) per 128 rows; one takes the even steps, the other the
//                            odd ones, each into its own TMEM accumulator, so that one thread's barrier waits and
//                            descriptor arithmetic hide behind the other's MMAs; tcgen05.commit frees the slots
//   epilogue (worker warps)  tcgen05.ld -> shared memory -> RMSNorm row scale, SwiGLU / residual, bf16 / fp32 store
//
// Few column tiles (N = 4096 gives 32) cannot fill 148 SMs, so K is split across the CTAs of a thread-block cluster
// (up to 8); each CTA owns a slice of the tile's rows, the others send it their partial sums through distributed
// shared memory, and it adds them in rank order (deterministic) before the epilogue.  No global scratch is needed for
// the reduction.  Every mbarrier wait is bounded (sm100.cuh).
#include <cuda.h>

#include <type_traits>

#include "bfp_format.cuh"
#include "linear.cuh"
#include "sm100.cuh"

namespace fb {

namespace {

constexpr int TILE_N = 128;     // output columns per CTA (MMA M): two 64-column groups
constexpr int STEP_UNITS = 2;   // 64-row units of K per pipeline step: 128 rows
constexpr int STEP_ROWS = STEP_UNITS * KSTEP;
constexpr int WORKERS = 512;    // one CTA per SM (a kernel that allocates tensor memory gets the SM to itself)
constexpr int WARP_MMA = 16, WARP_X = 18;  // warps 16 and 17 issue MMAs
constexpr int THREADS = 19 * 32;
constexpr int TEAMS = 4;        // teams of worker warps, each unpacking every fourth step on its own
constexpr int A_SLOT_BYTES = TILE_N * STEP_ROWS * 2;
constexpr int MAX_STAGES = 8;
// workspace (linear.cuh): arrival words of the persistent kernel's CTAs | row scales | partial tiles | normalised activations
constexpr int MAX_GRID = (int)(WS_RSTD_AT - WS_ARRIVED_AT) / 4;

struct GemmParams {
  LinearArgs a;
  int nt;  // MMA N: tokens rounded up to a multiple of 16
  int tmem_cols;
  int splits, steps_per_split, steps_total;  // K in steps of 128 rows
  int x_slots, a_slots;
  const float* rstd;  // [M] row scales of the RMSNorm prologue, or null
  const float* sumsq_in;  // or: [sumsq_parts, M] partial sums of squares of the rows x was normalised from (LinearArgs)
  int sumsq_parts;
  // a mixture of experts' matmul (Tensor.matmul(index=), ferrite/tensor.py:450-460): W is a batch of n_experts packed
  // matrices expert_bytes apart and index[slot] picks one per slot (n_experts or more: none, zeros).
  //   mode 1: one result per slot (grid z): out + slot * out_slot_stride, x rows from slot * x_slot_rows on
  //   mode 2: the slots' matmuls summed: K runs through slot 0's rows, then slot 1's, ... (x columns slot * K + k)
  int mode;
  const int32_t* index;
  int n_experts, n_slots, steps_per_slot;
  int64_t expert_bytes, x_slot_rows, out_slot_stride;
  const uint16_t* row_scale;  // mode 1: bf16 [slot * M + t] multiplying the epilogue's result, or null
  // the persistent kernel (a plain matmul): CTA c takes steps [c * work / grid, (c + 1) * work / grid) of the
  // tiles x steps_total steps laid end to end; a tile shared by several CTAs meets in `partials` (fp32 [grid][nt][128],
  // a CTA's own slot) with one arrival word per CTA in `arrived` (0 between launches)
  int tiles, work;
  float* partials;
  uint32_t* arrived;
};

enum WaitCode { WAIT_X_EMPTY = 103, WAIT_X_FULL, WAIT_A_EMPTY, WAIT_A_FULL, WAIT_ACC, WAIT_ACC_EMPTY, WAIT_SHARED_TILE };

// a ring position: slot index and the parity of the phase its barriers are in (no division in the loops)
struct Ring {
  int slot = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void next(int n) {
    if (++slot == n) slot = 0, phase ^= 1;
  }
};
__device__ __forceinline__ void cluster_sync() {  // every thread of every CTA of the cluster
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared window, of CTA `rank`'s copy of a shared-memory location of this CTA
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ void store_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

template <int FMT>
__global__ void __launch_bounds__(THREADS) linear_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  constexpr int UNIT = unit_bytes(FMT), UNIT_MANT = unit_mant_bytes(FMT), RUN = run_bytes(FMT);
  extern __shared__ uint8_t smem_unaligned[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int nt = p.nt, SX = p.x_slots, SA = p.a_slots;
  const LinearArgs& a = p.a;
  const bool swiglu = a.epilogue == FB_EPI_SWIGLU;
  const int64_t K = a.K, KS = ksteps_of(K), G = groups_of(a.N);

  uint8_t* sA = smem;  // A slots; reused as the split-K exchange buffer once the MMAs are done
  const int x_slot_bytes = STEP_UNITS * nt * 128;  // a [tokens x 64] tile per 64 rows of K
  uint8_t* sX = sA + SA * A_SLOT_BYTES;
  uint32_t* lut = reinterpret_cast<uint32_t*>(sX + SX * x_slot_bytes);  // exponent byte -> its power of two as a bf16 pair
  float* tok_rstd = reinterpret_cast<float*>(lut + 256);  // per token (nt of them): the RMSNorm row scale, the mixture's weight (or ones)
  float* tok_scale = tok_rstd + nt;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tok_scale + nt);
  uint64_t* x_full = bars, *x_empty = bars + MAX_STAGES, *a_full = bars + 2 * MAX_STAGES, *a_empty = bars + 3 * MAX_STAGES;
  uint64_t* acc_full = bars + 4 * MAX_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  const uint32_t abort_flag = smem_u32(tmem_slot + 1);

  // The kernel is launched as a programmatic dependent of the kernel before it: everything up to a griddep_wait()
  // (barriers, tensor memory, the first weight loads - weights are never written by a kernel of
  // the stream) overlaps that kernel's last CTAs; the activations, row scales, residual and expert index are read after.
  griddep_launch_dependents();
  if (p.mode != 0) griddep_wait();  // the expert index decides what is read at all
  // an indexed matmul's slot that picks no expert is zeros, with nothing read (ferrite/tensor.py:458-460)
  const int zslot = p.mode == 1 ? (int)blockIdx.z : 0;
  int expert = 0;
  if (p.mode == 1) {
    expert = p.index[zslot];
    if (expert < 0 || expert >= p.n_experts) {
      if (split == 0) {
        const int64_t cols = swiglu ? 64 : TILE_N, n0 = cols * tile, n_end = swiglu ? a.N / 2 : a.N;
        for (int64_t i = tid; i < a.M * cols; i += THREADS) {
          const int64_t t = i / cols, n = n0 + i % cols;
          if (n >= n_end) continue;
          const int64_t at = zslot * p.out_slot_stride + t * a.ldo + n;
          if (a.out_dtype == FB_FP32) static_cast<float*>(a.out)[at] = 0.f;
          else static_cast<uint16_t*>(a.out)[at] = 0;
        }
      }
      return;  // (every CTA of a cluster shares the slot: they all leave here, before any cluster barrier)
    }
  }
  if (tid == 0) {
    for (int s = 0; s < SX; ++s) mbar_init(smem_u32(x_full + s), 1), mbar_init(smem_u32(x_empty + s), 1);
    for (int s = 0; s < SA; ++s) mbar_init(smem_u32(a_full + s), WORKERS / 32 / TEAMS), mbar_init(smem_u32(a_empty + s), 1);
    mbar_init(smem_u32(acc_full), 2);
    tmem_slot[1] = 0;
    fence_barrier_init();
  }
  if (tid < 256) {
    lut[tid] = FMT == FB_BFP8 ? scale8(tid) : scale4(tid);
  }
  if (warp == WARP_MMA) tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  const int s0 = split * p.steps_per_split;
  const int n_steps = min(p.steps_total - s0, p.steps_per_split);
  const int units_total = (int)KS;  // the last step of K may hold one unit only

  // the tile's two 64-column groups: neighbours, or a group of gate columns and the group of their up columns
  const int64_t g0 = swiglu ? tile : 2 * (int64_t)tile, g1 = swiglu ? tile + G / 2 : 2 * (int64_t)tile + 1;
  const bool has_g1 = g1 < G;

  // steps are numbered through the slots in mode 2: step gs is rows (gs % S) * 128.. of slot gs / S
  const int S = p.mode == 2 ? p.steps_per_slot : p.steps_total;
  if (warp == WARP_X && lane >= 16) {  // the epilogue's per-token factors, fetched while the matmul runs
    griddep_wait();
    for (int t = lane - 16; t < nt; t += 16) {
      float rs = p.rstd && t < a.M ? p.rstd[t] : 1.f;
      if (p.sumsq_in && t < a.M) {  // the matmul before this one left the rows' sums of squares, a part per CTA: added in part order
        float ss = 0.f;
        for (int q = 0; q < p.sumsq_parts; ++q) ss += p.sumsq_in[(int64_t)q * a.M + t];
        rs = rsqrtf(ss / (float)K + a.eps);
      }
      tok_rstd[t] = rs;
      tok_scale[t] = p.row_scale && t < a.M ? bf16_bits_to_float(p.row_scale[(int64_t)zslot * a.M + t]) : 1.f;
    }
  } else if (warp == WARP_X && lane == 0) {
    Ring rx;
    int ks = s0 % S, slot = s0 / S;
    const int y = p.mode == 1 ? (int)(zslot * p.x_slot_rows) : 0;
    prefetch_tensormap(&tmap_x);
    griddep_wait();  // the activations come from the kernel before
    for (int i = 0; i < n_steps; ++i, rx.next(SX)) {
      const int s = rx.slot;
      mbar_wait(smem_u32(x_empty + s), rx.phase ^ 1, abort_flag, WAIT_X_EMPTY);
      mbar_expect_tx(smem_u32(x_full + s), x_slot_bytes);
      const int x0 = (p.mode == 2 ? slot * (int)K : 0) + ks * STEP_ROWS;
#pragma unroll
      for (int u = 0; u < STEP_UNITS; ++u)  // rows of K past the end read as zeros (or meet zeros in A)
        tma_load_2d(smem_u32(sX + s * x_slot_bytes + u * nt * 128), &tmap_x, x0 + u * KSTEP, y, smem_u32(x_full + s));
      if (++ks == S) ks = 0, ++slot;
    }
  } else if ((warp == WARP_MMA || warp == WARP_MMA + 1) && lane == 0) {
    const int me = warp - WARP_MMA;  // steps me, me + 2, ... into accumulator `me`
    const uint32_t idesc = umma_idesc_bf16(nt, true, false);
    // A: MN-major, 64-column swizzle atoms 1024 B apart, groups of 8 rows of K 2048 B apart; 16 rows of K per MMA
    // X: K-major, one 128-byte swizzled row per token, groups of 8 tokens 1024 B apart; 32 bytes of K per MMA
    // The address field is the low 14 bits (units of 16 B): slots and K offsets are added to it directly.
    const uint64_t da0 = umma_smem_desc(smem_u32(sA), 1024, 2048), dx0 = umma_smem_desc(smem_u32(sX), 16, 1024);
    const uint32_t x_slot16 = (uint32_t)x_slot_bytes >> 4, x_unit16 = (uint32_t)(nt * 128) >> 4;
    Ring ra, rx;
    if (me) ra.next(SA), rx.next(SX);
    const uint32_t acc = tmem + me * nt;
    for (int i = me; i < n_steps; i += 2, ra.next(SA), ra.next(SA), rx.next(SX), rx.next(SX)) {
      mbar_wait(smem_u32(a_full + ra.slot), ra.phase, abort_flag, WAIT_A_FULL);
      mbar_wait(smem_u32(x_full + rx.slot), rx.phase, abort_flag, WAIT_X_FULL);
      tc_fence_after();
      const uint64_t da = da0 + (uint32_t)ra.slot * (A_SLOT_BYTES >> 4), dx = dx0 + (uint32_t)rx.slot * x_slot16;
#pragma unroll
      for (int kk = 0; kk < STEP_ROWS / 16; ++kk)
        umma_bf16(acc, da + kk * (4096 >> 4), dx + (kk >> 2) * x_unit16 + (kk & 3) * (32 >> 4), idesc, (i - me) | kk);
      umma_commit(smem_u32(a_empty + ra.slot));
      umma_commit(smem_u32(x_empty + rx.slot));
    }
    umma_commit(smem_u32(acc_full));
  } else if (warp < WORKERS / 32) {
    // The worker warps form TEAMS teams; team t unpacks steps t, t + TEAMS, ... on its own, so a warp synchronises
    // (slot wait, proxy fence, arrive) once per 8 runs of 16 values instead of once per 2, and while one team waits
    // for its loads the others unpack.  A thread owns one row k of the step and walks the tile's 8 runs.
    constexpr int TEAM_THREADS = WORKERS / TEAMS;
    const int team = tid / TEAM_THREADS, k = tid % TEAM_THREADS;  // TEAM_THREADS == STEP_ROWS
    const uint8_t* W = static_cast<const uint8_t*>(a.W) + (p.mode == 1 ? expert * p.expert_bytes : 0);
    const int unit = k >> 6, ku = k & 63;
    using RawT = typename std::conditional<FMT == FB_BFP8, uint4, uint2>::type;
    const uint32_t sA32 = smem_u32(sA), lut32 = smem_u32(lut);
    const uint32_t row_base = (uint32_t)((k >> 3) * 2 * 1024 + (k & 7) * 128);
    Ring ra;
    for (int t = 0; t < team; ++t) ra.next(SA);
    RawT q[8];
    uint32_t top[8];
    // where step i's bytes lie: its expert's matrix (mode 2), its 128 rows of K; null past the end or with no expert
    auto rows_of = [&](int i) -> const uint8_t* {
      if (i >= n_steps) return nullptr;
      const int gs = s0 + i, slot_i = gs / S, ks = gs - slot_i * S;
      const uint8_t* w = W;
      if (p.mode == 2) {
        const int e = p.index[slot_i];
        if (e < 0 || e >= p.n_experts) return nullptr;
        w = static_cast<const uint8_t*>(a.W) + e * p.expert_bytes;
      }
      if (ks * STEP_UNITS + unit >= units_total) return nullptr;
      return w + ((int64_t)ks * STEP_UNITS + unit) * UNIT;
    };
    // this thread's bytes of a step's two column groups, from the step's first unit on: mantissas, exponents (the runs
    // of a group lie at fixed distances behind them, so a load is a pointer and an immediate)
    const int64_t my_q0 = g0 * KS * UNIT + ku * RUN, my_q1 = g1 * KS * UNIT + ku * RUN;
    const int64_t my_e0 = g0 * KS * UNIT + UNIT_MANT + ku, my_e1 = g1 * KS * UNIT + UNIT_MANT + ku;
    auto load = [&](const uint8_t* rows, int j) {  // run j of the tile: group j / 4, run j % 4 of it
      const int grp = j >> 2, run = j & 3;
      if (rows != nullptr && (grp == 0 || has_g1)) {
        q[j] = __ldg(reinterpret_cast<const RawT*>(rows + (grp ? my_q1 : my_q0) + run * KSTEP * RUN));
        top[j] = __ldg(rows + (grp ? my_e1 : my_e0) + run * KSTEP);
      } else {  // past the end of K, a column group past N, or no expert: zeros
        q[j] = RawT{};
        top[j] = 0;
      }
    };
    {
      const uint8_t* rows = rows_of(team);
#pragma unroll
      for (int j = 0; j < 8; ++j) load(rows, j);
    }
    const uint32_t k7 = (uint32_t)(k & 7);  // 16-byte chunk c of this thread's row goes to chunk c ^ k7 of its swizzled line
    for (int i = team; i < n_steps; i += TEAMS) {
      const uint8_t* next = rows_of(i + TEAMS);
      const int sa = ra.slot;
      mbar_wait(smem_u32(a_empty + sa), ra.phase ^ 1, abort_flag, WAIT_A_EMPTY);
      const uint32_t slot = sA32 + sa * A_SLOT_BYTES + row_base, slot7 = slot | (k7 << 4);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t sc = ld_shared_u32(lut32 + top[j] * 4);
        uint32_t v[8];
        if constexpr (FMT == FB_BFP8) {
          unpack8_word(q[j].x, sc, v[0], v[1]);
          unpack8_word(q[j].y, sc, v[2], v[3]);
          unpack8_word(q[j].z, sc, v[4], v[5]);
          unpack8_word(q[j].w, sc, v[6], v[7]);
        } else {
          unpack4_word(q[j].x, sc, v);
          unpack4_word(q[j].y, sc, v + 4);
        }
        load(next, j);  // this register's next bytes are on their way while the rest of the step is unpacked
        const int sl = swiglu ? ((j & 3) << 1 | j >> 2) : j;  // gate and up runs alternate: rows r and r + 16 pair up
        // chunk c of the row goes to chunk c ^ k7 of its 128-byte line: the line's address has its low seven bits clear,
        // so (line | k7 << 4) ^ (c << 4) is that chunk's address - one operation per store
        const uint32_t c0 = (uint32_t)(sl & 3) * 2;
        st_shared_v4((slot7 ^ (c0 << 4)) + (sl >> 2) * 1024, v[0], v[1], v[2], v[3]);
        st_shared_v4((slot7 ^ ((c0 + 1) << 4)) + (sl >> 2) * 1024, v[4], v[5], v[6], v[7]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(a_full + sa));
      for (int t = 0; t < TEAMS; ++t) ra.next(SA);
    }
  }

  // ---- accumulators -> the owning CTA's shared memory.  CTA `rank` of the cluster (= its K split) owns rows
  // [rank * rows_per, (rank + 1) * rows_per) of the tile; exchange[src][t][row] is what CTA src summed for them.
  const bool worker = warp < WORKERS / 32;
  const int splits = p.splits, rows_per = (TILE_N + splits - 1) / splits;  // (the last rank may own fewer rows)
  float* exchange = reinterpret_cast<float*>(sA);
  if (worker) {
    mbar_wait(smem_u32(acc_full), 0, abort_flag, WAIT_ACC);
    tc_fence_after();
  }
  if (splits > 1) cluster_sync();  // every CTA of the cluster is past its MMAs: the A slots are free to receive
  else __syncthreads();
  // worker warps sharing one quarter of the TMEM lanes split the token columns, in runs of whole 8-column loads
  const int col_groups = nt % 32 == 0 ? 4 : nt % 16 == 0 ? 2 : 1;
  if (splits == 1 && worker && (warp >> 2) < col_groups) {
    // ---- no K split: the epilogue runs straight from tensor memory.  Lane = tile row = output column, so a warp's
    // store of one token is 32 consecutive columns; SwiGLU's gate (lanes 0-15) meets its up (lanes 16-31) by a shuffle.
    griddep_wait();  // (long since true: the MMAs consumed that kernel's activations) - the residual is its output too
    const int q = warp & 3, ncol = nt / col_groups, col0 = (warp >> 2) * ncol, row = 32 * q + lane;
    const int64_t n = swiglu ? 64 * (int64_t)tile + 16 * q + (lane & 15) : TILE_N * (int64_t)tile + row;
    const bool live = swiglu ? lane < 16 && n < a.N / 2 : n < a.N;
    for (int cb = 0; cb < ncol && col0 + cb < a.M; cb += 8) {
      float v[8], res[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {  // the residual reads of the eight tokens are in flight together
        const int t = col0 + cb + e;
        res[e] = live && t < a.M && a.epilogue == FB_EPI_RESIDUAL
                     ? bf16_bits_to_float(static_cast<const uint16_t*>(a.residual)[t * a.ldr + n]) : 0.f;
      }
      tmem_ld8(tmem + ((uint32_t)(32 * q) << 16) + col0 + cb, v);
      if (n_steps > 1) {  // the odd steps' accumulator
        float w[8];
        tmem_ld8(tmem + ((uint32_t)(32 * q) << 16) + nt + col0 + cb, w);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += w[e];
      }
      // (the eight tokens side by side, step by step: eight independent chains instead of one eight times as long)
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] *= tok_rstd[col0 + cb + e];
      if (swiglu) {
        float up[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) up[e] = __shfl_down_sync(0xffffffffu, v[e], 16);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = v[e] / (1.f + __expf(-v[e])) * up[e] * tok_scale[col0 + cb + e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = v[e] * tok_scale[col0 + cb + e] + res[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int t = col0 + cb + e;
        if (t < a.M && live) {
          const int64_t at = zslot * p.out_slot_stride + t * a.ldo + n;
          if (a.out_dtype == FB_FP32) static_cast<float*>(a.out)[at] = v[e];
          else static_cast<uint16_t*>(a.out)[at] = (uint16_t)float_to_bf16_bits(v[e]);
        }
      }
    }
  } else if (worker && (warp >> 2) < col_groups) {
    const int q = warp & 3, ncol = nt / col_groups, col0 = (warp >> 2) * ncol, row = 32 * q + lane;
    const uint32_t owner = row / rows_per;
    uint32_t at = smem_u32(exchange) + (uint32_t)(((split * nt + col0) * rows_per + row % rows_per) * 4);
    if (splits > 1) at = map_to_rank(at, owner);  // (a CTA's window is contiguous: offsets carry over)
    for (int cb = 0; cb < ncol; cb += 8) {
      float v[8];
      tmem_ld8(tmem + ((uint32_t)(32 * q) << 16) + col0 + cb, v);
      if (n_steps > 1) {  // the odd steps' accumulator
        float w[8];
        tmem_ld8(tmem + ((uint32_t)(32 * q) << 16) + nt + col0 + cb, w);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += w[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t addr = at + (uint32_t)((cb + e) * rows_per * 4);
        if (splits > 1) store_cluster_f32(addr, v[e]);
        else asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v[e]) : "memory");
      }
    }
  }
  tc_fence_before();
  if (splits > 1) cluster_sync();

  // ---- epilogue over this CTA's rows: sum the splits in rank order, scale, SwiGLU / residual, store
  if (worker && splits > 1) {
    griddep_wait();  // (long since true: the MMAs consumed that kernel's activations) - the residual is its output too
    const int64_t M = a.M;
    const int own = min(rows_per, TILE_N - split * rows_per);   // rows of the tile this CTA owns
    const int out_rows = swiglu ? own / 2 : own;  // SwiGLU: rows 32q..32q+15 are gates, the next 16 their ups
    const int total = out_rows * (int)min((int64_t)nt, M);
    const uint32_t inv_rows = 0xFFFFFFFFu / (uint32_t)max(out_rows, 1) + 1;  // idx / out_rows == umulhi(idx, inv_rows) for idx < 2^14
    for (int base = tid; base < total; base += 4 * WORKERS) {
      float res[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {  // the residual reads of four outputs are in flight together
        const int idx = base + e * WORKERS;
        res[e] = 0.f;
        if (idx < total && a.epilogue == FB_EPI_RESIDUAL) {
          const int t = (int)__umulhi((uint32_t)idx, inv_rows), n = TILE_N * tile + split * rows_per + (idx - t * out_rows);
          if (n < a.N) res[e] = bf16_bits_to_float(static_cast<const uint16_t*>(a.residual)[t * a.ldr + n]);
        }
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int idx = base + e * WORKERS;
        if (idx >= total) break;
        const int t = (int)__umulhi((uint32_t)idx, inv_rows), o = idx - t * out_rows;
        const int lr = swiglu ? (o / 16) * 32 + o % 16 : o;  // row inside this CTA's slice
        float val = 0.f, up = 0.f;
        for (int s = 0; s < splits; ++s) {
          const float* src = exchange + ((size_t)s * nt + t) * rows_per;
          val += src[lr];
          if (swiglu) up += src[lr + 16];
        }
        val *= tok_rstd[t], up *= tok_rstd[t];
        const float scale = tok_scale[t];
        const int tr = split * rows_per + lr;  // row inside the tile
        int64_t n;
        if (swiglu) {
          val = val / (1.f + __expf(-val)) * up * scale;
          n = 64 * (int64_t)tile + (tr / 32) * 16 + tr % 16;
          if (n >= a.N / 2) continue;
        } else {
          n = TILE_N * (int64_t)tile + tr;
          if (n >= a.N) continue;
          val = val * scale + res[e];
        }
        const int64_t at = zslot * p.out_slot_stride + t * a.ldo + n;
        if (a.out_dtype == FB_FP32) static_cast<float*>(a.out)[at] = val;
        else static_cast<uint16_t*>(a.out)[at] = (uint16_t)float_to_bf16_bits(val);
      }
    }
  }
  __syncthreads();
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem, p.tmem_cols);
  }
  // ---- the next matmul's RMSNorm, handed on (LinearArgs::next_norm_w): over the columns this CTA has just written - a
  // slice of the tile's with a K split - xn = bf16(out * g) and each token's sum of out^2, one part per CTA.  The values
  // are read back as stored (bf16), so xn and the sums are those a separate pass over `out` would compute; the sum over
  // a part's columns is a warp's butterfly, the same every run.
  if (a.xn_out != nullptr && worker) {
    const int n0 = TILE_N * tile + (splits > 1 ? split * rows_per : 0);
    const int own = min(splits > 1 ? min(rows_per, TILE_N - split * rows_per) : TILE_N, (int)a.N - n0);
    const uint16_t* out = static_cast<const uint16_t*>(a.out);
    const uint16_t* g = static_cast<const uint16_t*>(a.next_norm_w);
    uint16_t* xn = static_cast<uint16_t*>(a.xn_out);
    const int64_t part = (int64_t)tile * splits + split;
    for (int t = warp; t < a.M; t += WORKERS / 32) {
      float ss = 0.f;
      for (int r = lane; r < own; r += 32) {
        const float x0 = bf16_bits_to_float(out[t * a.ldo + n0 + r]);
        ss = fmaf(x0, x0, ss);
        xn[t * a.ld_xn + n0 + r] = (uint16_t)float_to_bf16_bits(x0 * bf16_bits_to_float(g[n0 + r]));
      }
      ss = warp_sum(ss);
      if (lane == 0) a.sumsq_out[part * a.M + t] = ss;
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// The plain matmul (no expert index) as a PERSISTENT kernel: one CTA per SM, and the tiles' steps of K laid end to end
// (tile 0's steps, then tile 1's, ...) are cut into equal runs, one per CTA, so every SM streams the same number of
// weight bytes whatever the tile count (224 tiles on 148 SMs would otherwise cost two rounds).  A CTA's run is a tail
// of one tile, whole tiles, and a head of another: its SEGMENTS.  Weight loads, unpacking and MMAs run on across the
// segment boundaries without a pause: the accumulators are double-buffered in tensor memory, and four warps of their
// own (one per quarter of the TMEM lanes) empty a finished segment's while the next segment's MMAs fill the other pair:
//   a whole tile:  epilogue straight from tensor memory;
//   a tail (the run begins inside a tile):  the partial sums go to this CTA's slot of `partials` and its arrival word
//                  is set - this is the FIRST segment of the CTA, so it is long done when it is needed;
//   a head (the run ends inside a tile):  the LAST segment of the CTA; it owns the tile: waits (bounded) for the CTAs
//                  after it that hold the rest of the tile, adds their partial sums to its own in CTA order - a fixed
//                  order, so the result does not change from run to run - and runs the epilogue.
// The wait is for CTAs with HIGHER numbers that did their part first, so it is short when the whole grid is resident
// (grid <= SMs, one CTA each); were some CTA never to run, the wait gives up after its bound and reports.
// Arrival words are cleared by the owner; the next launch touches them only after its griddep_wait(), i.e. after this
// grid has finished.
//
// Warps: 0-15 unpack (4 teams; together they also run the epilogue of the run's last segment), 16 and 17 issue MMAs, 18 feeds
// activations, 19 idles, 20-23 run the epilogues.  The unpacking warps need ~96 registers, the others few: the kernel is compiled for 768 threads (80 each)
// and setmaxnreg moves registers from warps 16-19 to the unpacking warps.
constexpr int P_THREADS = 24 * 32, WARP_EPI = 20;

struct Segment {
  int tile, k_first, k_steps;  // steps [k_first, k_first + k_steps) of the tile's p.steps_total
  int i_first;                 // its first step, counted from the start of the CTA's run
};

template <int FMT>
__global__ void __launch_bounds__(P_THREADS) linear_persistent_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
  constexpr int UNIT = unit_bytes(FMT), UNIT_MANT = unit_mant_bytes(FMT), RUN = run_bytes(FMT);
  extern __shared__ uint8_t smem_unaligned[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_unaligned) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int nt = p.nt, SX = p.x_slots, SA = p.a_slots;
  const LinearArgs& a = p.a;
  const bool swiglu = a.epilogue == FB_EPI_SWIGLU;
  const int KS = (int)ksteps_of(a.K), G = (int)groups_of(a.N);
  const int S = p.steps_total;

  uint8_t* sA = smem;
  const int x_slot_bytes = STEP_UNITS * nt * 128;
  uint8_t* sX = sA + SA * A_SLOT_BYTES;
  uint32_t* lut = reinterpret_cast<uint32_t*>(sX + SX * x_slot_bytes);
  float* tok_rstd = reinterpret_cast<float*>(lut + 256);  // per token (nt of them): the RMSNorm row scale (or 1), read by the epilogue warps only
  uint64_t* bars = reinterpret_cast<uint64_t*>(tok_rstd + nt);
  uint64_t* x_full = bars, *x_empty = bars + MAX_STAGES, *a_full = bars + 2 * MAX_STAGES, *a_empty = bars + 3 * MAX_STAGES;
  uint64_t* acc_full = bars + 4 * MAX_STAGES, *acc_empty = acc_full + 2;  // one of each per accumulator pair
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  const uint32_t abort_flag = smem_u32(tmem_slot + 1);

  griddep_launch_dependents();
  if (tid == 0) {
    for (int s = 0; s < SX; ++s) mbar_init(smem_u32(x_full + s), 1), mbar_init(smem_u32(x_empty + s), 1);
    for (int s = 0; s < SA; ++s) mbar_init(smem_u32(a_full + s), WORKERS / 32 / TEAMS), mbar_init(smem_u32(a_empty + s), 1);
    for (int b = 0; b < 2; ++b) mbar_init(smem_u32(acc_full + b), 2), mbar_init(smem_u32(acc_empty + b), 4);
    tmem_slot[1] = 0;
    fence_barrier_init();
  }
  if (tid < 256) lut[tid] = FMT == FB_BFP8 ? scale8(tid) : scale4(tid);
  if (warp == WARP_MMA) tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // this CTA's run of the work, and the work index -> (tile, step of K)
  const int lo = (int)((int64_t)blockIdx.x * p.work / gridDim.x), hi = (int)((int64_t)(blockIdx.x + 1) * p.work / gridDim.x);
  const int n_steps = hi - lo;
  const int tile_lo = lo / S, k_lo = lo - tile_lo * S;
  // (tile, step of K) of the run's step i, moved on by `by` steps at a time: no division in the loops
  struct At {
    int tile, ks;
    __device__ __forceinline__ void advance(int by, int S) {
      ks += by;
      while (ks >= S) ks -= S, ++tile;
    }
  };
  // segment number s of the run (0, 1, ...): the tile it lies in and its steps
  auto segment = [&](int s) -> Segment {
    Segment g;
    g.tile = tile_lo + s;
    g.k_first = s == 0 ? k_lo : 0;
    g.i_first = s == 0 ? 0 : s * S - k_lo;
    g.k_steps = min(S - g.k_first, n_steps - g.i_first);
    return g;
  };
  const int n_segments = n_steps > 0 ? (k_lo + n_steps + S - 1) / S : 0;
  // the two 64-column groups of a tile: neighbours, or a group of gate columns and the group of their up columns
  auto groups = [&](int tile, int& g0, int& g1) { g0 = swiglu ? tile : 2 * tile, g1 = swiglu ? tile + G / 2 : 2 * tile + 1; };
  const uint8_t* W = static_cast<const uint8_t*>(a.W);

  // ---- a segment's epilogue for quarter qd of the TMEM lanes (tile rows 32 qd .. 32 qd + 31, a row per lane): passes
  // of 16 tokens first_pass, first_pass + pass_stride, ...  The row scales come from shared memory (the epilogue warps'
  // copy) or, with rs == nullptr, from where the norm's kernel left them.
  struct SegmentEnd {
    bool tail;   // the segment does not start its tile: its sums went to the tile's owner
    int others;  // CTAs after this one whose sums of an owned tile were added
  };
  auto epilogue = [&](auto pass_width, int s, int qd, int first_pass, int pass_stride, const float* rs) -> SegmentEnd {
    constexpr int PW = decltype(pass_width)::value;  // tokens a pass: 16, or 8 where more warps share a segment
    const int row = 32 * qd + lane;
    const Segment g = segment(s);
    const int pair = s & 1;
    const bool whole_end = g.k_first + g.k_steps == S;  // the segment reaches the tile's last step
    const bool tail = g.k_first > 0;
    const int64_t n = swiglu ? 64 * (int64_t)g.tile + 16 * qd + (lane & 15) : TILE_N * (int64_t)g.tile + row;
    const bool live = swiglu ? lane < 16 && n < a.N / 2 : n < a.N;
    // the CTAs after this one that hold the rest of an owned tile: c + 1 .. while their runs begin inside the tile
    int others = 0;
    if (!tail && !whole_end) {
      const int64_t tile_end = (int64_t)(g.tile + 1) * S;
      while ((int)blockIdx.x + others + 1 < (int)gridDim.x && (int64_t)(blockIdx.x + others + 1) * p.work / gridDim.x < tile_end) ++others;
    }
    mbar_wait(smem_u32(acc_full + pair), (uint32_t)(s >> 1) & 1, abort_flag, WAIT_ACC);
    tc_fence_after();
    for (int o = lane; o < others; o += 32) {  // a lane per CTA waited for (every warp waits for itself)
      const uint32_t* flag = p.arrived + blockIdx.x + 1 + o;
      const long long start = clock64();
      for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v || ld_shared_volatile(abort_flag)) break;
        if (clock64() - start > WAIT_CLOCKS) {
          asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(abort_flag), "r"(1u) : "memory");
          atomicCAS(&g_status_word, 0, (int)WAIT_SHARED_TILE);
          break;
        }
        __nanosleep(32);
      }
    }
    __syncwarp();
    const bool even = g.k_steps > 1 || !(g.i_first & 1), odd = g.k_steps > 1 || (g.i_first & 1);  // which accumulators hold steps
    const uint32_t acc = tmem + ((uint32_t)(32 * qd) << 16) + 2 * pair * nt;
    float* mine = p.partials + (size_t)blockIdx.x * nt * TILE_N;
    // PW tokens at a time (nt is a multiple of 16), one kind of load after another, every load of a kind in flight
    // before the first is used: a pass is ONE trip to tensor memory, one per CTA whose sums are added, one to the
    // residual - not one per token, and the arithmetic is PW independent chains
    for (int c0 = PW * first_pass; c0 < nt && c0 < a.M; c0 += PW * pass_stride) {
      float v[PW], w[PW];
      if constexpr (PW == 16) {
        if (even) tmem_ld16_nowait(acc + c0, v);
        if (odd) tmem_ld16_nowait(acc + nt + c0, w);
      } else {
        if (even) tmem_ld8_nowait(acc + c0, v);
        if (odd) tmem_ld8_nowait(acc + nt + c0, w);
      }
      tmem_ld_wait();
      if (odd) {
#pragma unroll
        for (int e = 0; e < PW; ++e) v[e] = even ? v[e] + w[e] : w[e];
      }
      if (tail) {
#pragma unroll
        for (int e = 0; e < PW; ++e) mine[(c0 + e) * TILE_N + row] = v[e];
        continue;
      }
      for (int o = 0; o < others; ++o) {  // the rest of the tile, added in CTA order
        const float* theirs = p.partials + (size_t)(blockIdx.x + 1 + o) * nt * TILE_N + (size_t)c0 * TILE_N + row;
#pragma unroll
        for (int e = 0; e < PW; ++e) w[e] = c0 + e < a.M ? __ldcg(theirs + e * TILE_N) : 0.f;
#pragma unroll
        for (int e = 0; e < PW; ++e) v[e] += w[e];
      }
#pragma unroll
      for (int e = 0; e < PW; ++e) v[e] *= rs ? rs[c0 + e] : p.rstd && c0 + e < a.M ? p.rstd[c0 + e] : 1.f;
      if (swiglu) {
#pragma unroll
        for (int e = 0; e < PW; ++e) w[e] = __shfl_down_sync(0xffffffffu, v[e], 16);
#pragma unroll
        for (int e = 0; e < PW; ++e) v[e] = v[e] / (1.f + __expf(-v[e])) * w[e];
      } else if (a.epilogue == FB_EPI_RESIDUAL) {
#pragma unroll
        for (int e = 0; e < PW; ++e)
          w[e] = live && c0 + e < a.M ? bf16_bits_to_float(static_cast<const uint16_t*>(a.residual)[(c0 + e) * a.ldr + n]) : 0.f;
#pragma unroll
        for (int e = 0; e < PW; ++e) v[e] += w[e];
      }
#pragma unroll
      for (int e = 0; e < PW; ++e) {
        const int t = c0 + e;
        if (t < a.M && live) {
          const int64_t at = t * a.ldo + n;
          if (a.out_dtype == FB_FP32) static_cast<float*>(a.out)[at] = v[e];
          else static_cast<uint16_t*>(a.out)[at] = (uint16_t)float_to_bf16_bits(v[e]);
        }
      }
    }
    return SegmentEnd{tail, others};
  };

  if (warp < WORKERS / 32) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 96;");
    // ---- the unpacking warps: team t turns steps t, t + 4, ... of the run into bf16 A tiles, whatever tile they are of
    constexpr int TEAM_THREADS = WORKERS / TEAMS;
    const int team = tid / TEAM_THREADS, k = tid % TEAM_THREADS;
    const int unit = k >> 6, ku = k & 63;
    using RawT = typename std::conditional<FMT == FB_BFP8, uint4, uint2>::type;
    const uint32_t sA32 = smem_u32(sA), lut32 = smem_u32(lut);
    const uint32_t row_base = (uint32_t)((k >> 3) * 2 * 1024 + (k & 7) * 128);
    Ring ra;
    for (int t = 0; t < team; ++t) ra.next(SA);
    RawT q[8];
    uint32_t top[8];
    // where step i's bytes lie for this thread's row of K: the number of its unit of each of the tile's two column
    // groups, counted through the whole packed matrix (below 2^31: a matrix of under 4 TB); -1: zeros
    auto locate = [&](int i, At at, int& u0, int& u1) {
      u0 = u1 = -1;
      if (i >= n_steps || at.ks * STEP_UNITS + unit >= KS) return;
      int g0, g1;
      groups(at.tile, g0, g1);
      u0 = g0 * KS + at.ks * STEP_UNITS + unit;
      if (g1 < G) u1 = g1 * KS + at.ks * STEP_UNITS + unit;
    };
    // (a step's two pointers - this thread's row in each group's unit, nullptr: zeros - are made once; a run's bytes
    // lie at fixed distances behind them, so a load is a pointer and an immediate)
    const uint8_t* const my_row = W + ku * RUN;
    auto rows_at = [&](int u) -> const uint8_t* { return u >= 0 ? my_row + (int64_t)u * UNIT : nullptr; };
    auto load = [&](const uint8_t* r0, const uint8_t* r1, int j) {  // run j of the tile: group j / 4, run j % 4 of it
      const uint8_t* r = (j >> 2) ? r1 : r0;
      const int run = j & 3;
      if (r != nullptr) {
        q[j] = __ldg(reinterpret_cast<const RawT*>(r + run * KSTEP * RUN));
        top[j] = __ldg(r + (UNIT_MANT + run * KSTEP) - ku * (RUN - 1));
      } else {
        q[j] = RawT{};
        top[j] = 0;
      }
    };
    At next{tile_lo, k_lo};  // where the step after this team's current one lies
    next.advance(team, S);
    {
      int u0, u1;
      locate(team, next, u0, u1);
      const uint8_t* r0 = rows_at(u0), *r1 = rows_at(u1);
#pragma unroll
      for (int j = 0; j < 8; ++j) load(r0, r1, j);
    }
    const uint32_t k7 = (uint32_t)(k & 7);
    for (int i = team; i < n_steps; i += TEAMS) {
      int n0, n1;
      next.advance(TEAMS, S);
      locate(i + TEAMS, next, n0, n1);
      const uint8_t* r0 = rows_at(n0), *r1 = rows_at(n1);
      const int sa = ra.slot;
      mbar_wait(smem_u32(a_empty + sa), ra.phase ^ 1, abort_flag, WAIT_A_EMPTY);
      const uint32_t slot = sA32 + sa * A_SLOT_BYTES + row_base, slot7 = slot | (k7 << 4);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t sc = ld_shared_u32(lut32 + top[j] * 4);
        uint32_t v[8];
        if constexpr (FMT == FB_BFP8) {
          unpack8_word(q[j].x, sc, v[0], v[1]);
          unpack8_word(q[j].y, sc, v[2], v[3]);
          unpack8_word(q[j].z, sc, v[4], v[5]);
          unpack8_word(q[j].w, sc, v[6], v[7]);
        } else {
          unpack4_word(q[j].x, sc, v);
          unpack4_word(q[j].y, sc, v + 4);
        }
        load(r0, r1, j);  // this register's next bytes are on their way while the rest of the step is unpacked
        const int sl = swiglu ? ((j & 3) << 1 | j >> 2) : j;  // gate and up runs alternate: rows r and r + 16 pair up
        // chunk c of the row goes to chunk c ^ k7 of its 128-byte line: the line's address has its low seven bits clear,
        // so (line | k7 << 4) ^ (c << 4) is that chunk's address - one operation per store
        const uint32_t c0 = (uint32_t)(sl & 3) * 2;
        st_shared_v4((slot7 ^ (c0 << 4)) + (sl >> 2) * 1024, v[0], v[1], v[2], v[3]);
        st_shared_v4((slot7 ^ ((c0 + 1) << 4)) + (sl >> 2) * 1024, v[4], v[5], v[6], v[7]);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(a_full + sa));
      for (int t = 0; t < TEAMS; ++t) ra.next(SA);
    }
    // The run's last segment has no main loop to hide its epilogue behind, and a warp's stores to global memory are
    // slow (tens of cycles each, one per token): the sixteen unpacking warps, idle by now, share it - four to a quarter
    // of the TMEM lanes, each taking every fourth pass of 8 tokens.
    if (n_segments > 0) {
      griddep_wait();
      const SegmentEnd e = epilogue(std::integral_constant<int, 8>{}, n_segments - 1, warp & 3, warp >> 2, 4, nullptr);
      if (e.tail) __threadfence();
      asm volatile("bar.sync 3, 640;" ::: "memory");
    }
  } else if (warp < WARP_EPI) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
    if (warp == WARP_X && lane == 0) {
      Ring rx;
      prefetch_tensormap(&tmap_x);
      griddep_wait();  // the activations come from the kernel before
      int ks = k_lo;
      for (int i = 0; i < n_steps; ++i, rx.next(SX)) {
        const int s = rx.slot;
        mbar_wait(smem_u32(x_empty + s), rx.phase ^ 1, abort_flag, WAIT_X_EMPTY);
        mbar_expect_tx(smem_u32(x_full + s), x_slot_bytes);
#pragma unroll
        for (int u = 0; u < STEP_UNITS; ++u)
          tma_load_2d(smem_u32(sX + s * x_slot_bytes + u * nt * 128), &tmap_x, ks * STEP_ROWS + u * KSTEP, 0, smem_u32(x_full + s));
        if (++ks == S) ks = 0;
      }
    } else if ((warp == WARP_MMA || warp == WARP_MMA + 1) && lane == 0) {
      const int me = warp - WARP_MMA;  // steps me, me + 2, ... of the run; segment s into accumulator me of pair s % 2
      const uint32_t idesc = umma_idesc_bf16(nt, true, false);
      const uint64_t da0 = umma_smem_desc(smem_u32(sA), 1024, 2048), dx0 = umma_smem_desc(smem_u32(sX), 16, 1024);
      const uint32_t x_slot16 = (uint32_t)x_slot_bytes >> 4, x_unit16 = (uint32_t)(nt * 128) >> 4;
      Ring ra, rx;
      if (me) ra.next(SA), rx.next(SX);
      int i = me;
      for (int s = 0; s < n_segments; ++s) {
        const Segment g = segment(s);
        const int i_end = g.i_first + g.k_steps, pair = s & 1;
        const uint32_t acc = tmem + (2 * pair + me) * nt;
        if (s >= 2) {  // the pair is free once the epilogue of the segment before last has read it
          mbar_wait(smem_u32(acc_empty + pair), (uint32_t)((s >> 1) - 1) & 1, abort_flag, WAIT_ACC_EMPTY);
          tc_fence_after();
        }
        uint32_t started = 0;
        for (; i < i_end; i += 2, ra.next(SA), ra.next(SA), rx.next(SX), rx.next(SX)) {
          mbar_wait(smem_u32(a_full + ra.slot), ra.phase, abort_flag, WAIT_A_FULL);
          mbar_wait(smem_u32(x_full + rx.slot), rx.phase, abort_flag, WAIT_X_FULL);
          tc_fence_after();
          const uint64_t da = da0 + (uint32_t)ra.slot * (A_SLOT_BYTES >> 4), dx = dx0 + (uint32_t)rx.slot * x_slot16;
#pragma unroll
          for (int kk = 0; kk < STEP_ROWS / 16; ++kk)
            umma_bf16(acc, da + kk * (4096 >> 4), dx + (kk >> 2) * x_unit16 + (kk & 3) * (32 >> 4), idesc, started | kk);
          started = 1;
          umma_commit(smem_u32(a_empty + ra.slot));
          umma_commit(smem_u32(x_empty + rx.slot));
        }
        umma_commit(smem_u32(acc_full + pair));  // (one arrival per issuer and segment, whether or not it had a step in it)
      }
    }
  } else {
    // ---- the epilogue warps: warp 20 + q reads quarter q of the TMEM lanes (tile rows 32q .. 32q + 31)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    const int qd = warp - WARP_EPI, etid = tid - WARP_EPI * 32;
    griddep_wait();  // the row scales, the residual and the arrival words are the work of kernels before this one
    for (int t = etid; t < nt; t += 128) tok_rstd[t] = p.rstd && t < a.M ? p.rstd[t] : 1.f;
    asm volatile("bar.sync 2, 128;" ::: "memory");
    for (int s = 0; s < n_segments; ++s) {
      const bool last = s == n_segments - 1;
      // (the run's last segment is the unpacking warps' work - they are idle by then, four of them to a quarter;
      // these warps only wait for it and do the bookkeeping)
      const SegmentEnd e = last ? epilogue(std::integral_constant<int, 8>{}, s, qd, 1 << 20, 1, tok_rstd)
                                : epilogue(std::integral_constant<int, 16>{}, s, qd, 0, 1, tok_rstd);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(acc_empty + (s & 1)));  // this warp's quarter of the pair has been read
      if (last || e.tail || e.others) {  // every warp's partial sums are out / have been read: say so, once
        if (e.tail) __threadfence();
        if (last) asm volatile("bar.sync 3, 640;" ::: "memory");
        else asm volatile("bar.sync 2, 128;" ::: "memory");
        if (etid == 0 && e.tail) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.arrived + blockIdx.x), "r"(1u) : "memory");
        if (etid < e.others) p.arrived[blockIdx.x + 1 + etid] = 0;  // read: ready for the next launch
      }
    }
  }
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
  griddep_launch_dependents();
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
  int nt, tmem_cols, tiles, splits, sps, steps, x_slots, a_slots;
  size_t smem;
};

// CTAs of the kernel that are resident at once when launched as clusters of `cluster` (asked of the driver once per
// format and size; the largest ring is assumed - a kernel with tensor memory is alone on its SM whatever it needs)
int resident_ctas(int fmt, int cluster) {
  static int known[2][9] = {};
  int* have = known[fmt == FB_BFP8];
  if (!have[1]) {  // every size at the first call (which is not inside a stream capture: a graph's first run is eager)
    auto kernel = fmt == FB_BFP8 ? linear_tcgen05_kernel<FB_BFP8> : linear_tcgen05_kernel<FB_BFP4>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    for (int n = 1; n <= 8; ++n) {
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3(148, n, 1), cfg.blockDim = dim3(THREADS), cfg.dynamicSmemBytes = 200 * 1024;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1, attr[0].val.clusterDim.y = (unsigned)n, attr[0].val.clusterDim.z = 1;
      cfg.attrs = attr, cfg.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters < 1) clusters = 148 / n, cudaGetLastError();
      have[n] = clusters * n;
    }
  }
  return have[cluster];
}

// slots, mode: an indexed matmul's (mode 1: so many results, more CTAs; mode 2: so many times the steps of K)
Plan make_plan(int fmt, int64_t M, int64_t K, int64_t N, int epilogue, int slots = 1, int mode = 0) {
  Plan pl;
  pl.nt = (int)((M + 15) / 16 * 16);
  pl.tmem_cols = pl.nt <= 16 ? 32 : pl.nt <= 32 ? 64 : pl.nt <= 64 ? 128 : 256;  // two accumulators
  pl.tiles = (int)(epilogue == FB_EPI_SWIGLU ? groups_of(N) / 2 : (groups_of(N) + 1) / 2);
  pl.steps = (int)ceil_div(K, STEP_ROWS) * (mode == 2 ? slots : 1);
  const int64_t ctas_per_split = (int64_t)pl.tiles * (mode == 1 ? slots : 1);
  // K splits (a cluster of up to 8 CTAs per tile): the count with the least modelled time, waves x (a CTA's fixed
  // cost + its steps); SwiGLU's gate/up row pairs must stay inside one CTA's slice of rows
  int best = 1;
  double best_cost = 1e30;
  for (int s = 1; s <= 8; ++s) {
    if (s > 1 && pl.steps / s < 2) break;
    if (epilogue == FB_EPI_SWIGLU && s != 1 && s != 2 && s != 4) continue;
    const int per = (int)ceil_div(pl.steps, s);
    if ((int)ceil_div(pl.steps, per) != s) continue;  // every split gets work
    // (a CTA has its SM to itself; clusters of some sizes - 3, 5, 6, 7 - do not pack the GPCs' SMs fully, and a grid
    // of a few CTAs more than are resident together takes twice the time: ask the driver how many clusters fit)
    const double cost = (double)ceil_div(ctas_per_split * s, resident_ctas(fmt, s)) * (5.0 + (s > 1 ? 1.0 : 0.0) + 0.6 * per);
    if (cost < best_cost) best_cost = cost, best = s;
  }
  pl.splits = best;
  pl.sps = (int)ceil_div(pl.steps, best);
  // Both rings have an even number of slots, so a slot is always consumed by the same one of the two MMA issuers:
  // a parity wait is only sound when the waiter knows that the phase before has completed, and an issuer knows that
  // of the slots it has consumed itself.  (With five A slots the issuer of the odd steps could run a lap ahead of a
  // late team and take the untouched barrier of step 0 for the finished one of step 5.)
  pl.a_slots = TEAMS;  // each team refills its own slot while the tensor core reads the other teams'
  pl.x_slots = pl.nt <= 64 ? 4 : 2;
  // (alignment slack, the rings, the exponent table, two floats per token, the barriers.  Kept tight: up to 32 tokens
  // it stays under 163 KB, the most a CTA gets from the SM's 164 KB shared-memory setting - a byte more and the SM
  // is set to 196 KB, leaving the unpacking warps' loads 60 KB of L1 instead of 92)
  pl.smem = 1024 + (size_t)pl.a_slots * A_SLOT_BYTES + (size_t)pl.x_slots * STEP_UNITS * pl.nt * 128 + 1024 + 2 * 4 * (size_t)pl.nt + 5 * MAX_STAGES * 8 + 64;
  return pl;
}

}  // namespace

bool linear_tcgen05_supports(const LinearArgs& a) {
  return a.K % 8 == 0 && a.ldx % 8 == 0 && (uintptr_t)a.x % 16 == 0 && encode_tiled() != nullptr &&
         (a.epilogue != FB_EPI_SWIGLU || a.N % 128 == 0);
}

// SMs of the current device (the persistent kernel's grid never exceeds it: every CTA must be resident)
static int sm_count() {
  static int known[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
  if (!known[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 1, cudaGetLastError();
    known[dev] = n < MAX_GRID ? n : MAX_GRID;
  }
  return known[dev];
}

static size_t partials_bytes(int64_t M) {
  const int64_t rows = M < 128 ? M : 128, nt = (rows + 15) / 16 * 16;
  return (size_t)MAX_GRID * nt * TILE_N * sizeof(float);
}

int linear_tcgen05_parts(int fmt, int64_t M, int64_t K, int64_t N, int epilogue) {
  if (M < 2 || M > 128 || encode_tiled() == nullptr) return 0;
  const Plan pl = make_plan(fmt, M, K, N, epilogue);
  return pl.tiles * pl.splits;
}

// Measured (32 tokens, bfp8, back to back in a graph): with at least a tile per SM - [4096 x 28672] with SwiGLU 36.6 us
// against the per-tile kernel's 40.5, the [4096 x 128256] output layer 132 against 143, and the same order at 64 and 128
// tokens - the even split of the steps beats whole tiles in waves; with fewer tiles than SMs most tiles are shared by
// several CTAs, whose partial sums go through global memory where the per-tile kernel's clusters use shared memory, and
// the per-tile kernel is ahead (18.8 us against 23.2 for [14336 x 4096]).
bool linear_persistent_wins(const LinearArgs& a) {
  if (a.M < 2 || a.next_norm_w || a.sumsq_in || !linear_tcgen05_supports(a)) return false;
  const int64_t M = a.M < 128 ? a.M : 128;
  const size_t need = WS_BODY_AT + partials_bytes(M) + (a.norm_w ? (size_t)M * a.K * 2 : 0);
  if (!a.workspace || a.workspace_bytes < need) return false;
  return make_plan(a.fmt, M, a.K, a.N, a.epilogue).tiles >= sm_count();
}

size_t linear_tcgen05_workspace(int64_t M, int64_t K, int64_t N) {
  (void)N;
  if (M < 1) return 0;
  return WS_BODY_AT + partials_bytes(M) + (size_t)(M < 128 ? M : 128) * K * 2;
}

// The persistent kernel's grid: the CTA count with the least modelled time - a CTA's fixed cost, its steps, and, where
// tiles are shared between CTAs, the owner's wait and its reads of the other CTAs' partial sums.
static int persistent_grid(int tiles, int steps) {
  const int64_t work = (int64_t)tiles * steps;
  const int most = (int)(work < sm_count() ? work : sm_count());
  int best = 1;
  double best_cost = 1e30;
  for (int g = 1; g <= most; ++g) {
    const int per = (int)ceil_div(work, g);
    const bool shared = work % g != 0 || per % steps != 0;  // some run begins or ends inside a tile
    const double cost = 0.5 * per + (shared ? 1.0 + 0.25 * (double)(ceil_div(steps, per) < g ? ceil_div(steps, per) : g) : 0.0);
    if (cost < best_cost - 1e-9) best_cost = cost, best = g;
  }
  return best;
}

static int run_pass(const LinearArgs& a, const IndexedArgs* ix, cudaStream_t s) {
  const int mode = ix ? ix->mode : 0, slots = ix ? ix->n_slots : 1;
  Plan pl = make_plan(a.fmt, a.M, a.K, a.N, a.epilogue, slots, mode);
  GemmParams p{};
  p.a = a;
  if (ix) {
    p.mode = mode, p.index = ix->index, p.n_experts = ix->n_experts, p.n_slots = slots, p.steps_per_slot = (int)ceil_div(a.K, STEP_ROWS);
    p.expert_bytes = packed_bytes(a.fmt, a.K, a.N), p.x_slot_rows = ix->x_slot_rows, p.out_slot_stride = ix->out_slot_stride;
    p.row_scale = static_cast<const uint16_t*>(ix->row_scale);
  }
  p.nt = pl.nt, p.tmem_cols = pl.tmem_cols, p.splits = pl.splits, p.steps_per_split = pl.sps, p.steps_total = pl.steps;
  p.x_slots = pl.x_slots, p.a_slots = pl.a_slots;
  const void* x = a.x;
  int64_t ldx = a.ldx;
  const size_t shared_tiles = mode == 0 && a.persistent ? partials_bytes(a.M) : 0;
  if (a.norm_w || shared_tiles) {
    const size_t need = WS_BODY_AT + shared_tiles + (a.norm_w ? (size_t)a.M * a.K * 2 : 0);
    if (!a.workspace || a.workspace_bytes < need) {
      set_error("fb_linear: workspace of %zu bytes needed, %zu given (fb_linear_workspace_bytes)", need, a.workspace_bytes);
      return FB_ERR_MEMORY;
    }
  }
  p.sumsq_in = a.sumsq_in, p.sumsq_parts = a.sumsq_parts;
  if (a.norm_w) {
    float* rstd = reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) + WS_RSTD_AT);
    uint16_t* xn = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(a.workspace) + WS_BODY_AT + shared_tiles);
    rms_prepare_kernel<<<(unsigned)a.M, 256, 0, s>>>(static_cast<const uint16_t*>(a.x), a.ldx, static_cast<const uint16_t*>(a.norm_w), a.K,
                                                     a.eps, xn, rstd);
    p.rstd = rstd, x = xn, ldx = a.K;
  }
  CUtensorMap tmap;
  // the activations as TMA sees them: [rows, K]; an indexed matmul's slots add rows (mode 1) or columns (mode 2)
  const cuuint64_t dims[2] = {(cuuint64_t)a.K * (mode == 2 ? slots : 1), (cuuint64_t)(mode == 1 && ix->x_slot_rows ? ix->x_slot_rows * (slots - 1) + a.M : a.M)};
  const cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
  const cuuint32_t box[2] = {KSTEP, (cuuint32_t)pl.nt}, estr[2] = {1, 1};  // 64 bf16 = one 128-byte swizzled row per token
  CUresult rc = encode_tiled()(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    set_error("fb_linear: cuTensorMapEncodeTiled failed (%d) for x [%lld, %lld] stride %lld", (int)rc, (long long)a.M, (long long)a.K, (long long)ldx);
    return FB_ERR_LAUNCH;
  }
  if (mode == 0 && a.persistent) {  // a plain matmul by the persistent kernel: the tiles' steps shared out evenly over the SMs
    auto persistent = a.fmt == FB_BFP8 ? linear_persistent_kernel<FB_BFP8> : linear_persistent_kernel<FB_BFP4>;
    static std::atomic<uint64_t> opted[2];
    if (first_on_device(opted[a.fmt == FB_BFP8])) cudaFuncSetAttribute(persistent, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
    p.splits = 1, p.tiles = pl.tiles, p.work = pl.tiles * pl.steps;
    p.tmem_cols = 4 * pl.nt <= 64 ? 64 : 4 * pl.nt <= 128 ? 128 : 4 * pl.nt <= 256 ? 256 : 512;  // two pairs of accumulators
    p.arrived = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(a.workspace) + WS_ARRIVED_AT);
    p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) + WS_BODY_AT);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(persistent_grid(pl.tiles, pl.steps)), cfg.blockDim = dim3(P_THREADS), cfg.dynamicSmemBytes = pl.smem, cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start while the kernel before it drains
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, persistent, tmap, p) != cudaSuccess) return launch_status("fb_linear (tcgen05 launch)");
    return launch_status("fb_linear (tcgen05)");
  }
  auto kernel = a.fmt == FB_BFP8 ? linear_tcgen05_kernel<FB_BFP8> : linear_tcgen05_kernel<FB_BFP4>;
  static std::atomic<uint64_t> opted_indexed[2];
  if (first_on_device(opted_indexed[a.fmt == FB_BFP8])) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.tiles, pl.splits, mode == 1 ? slots : 1), cfg.blockDim = dim3(THREADS), cfg.dynamicSmemBytes = pl.smem, cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1, attr[0].val.clusterDim.y = pl.splits, attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start while the kernel before it drains
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 2;
  if (cudaLaunchKernelEx(&cfg, kernel, tmap, p) != cudaSuccess) return launch_status("fb_linear (tcgen05 launch)");
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
    if (int rc = run_pass(a, nullptr, s)) return rc;
  }
  return FB_OK;
}

int linear_tcgen05_indexed(const LinearArgs& a, const IndexedArgs& ix, cudaStream_t s) { return run_pass(a, &ix, s); }

}  // namespace fb

int fb::status_word_tcgen05() { return fb::read_and_clear_status_word(); }
