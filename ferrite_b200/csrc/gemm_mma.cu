// fb_linear for 2..32 tokens: the block-float matmul on register-fragment tensor-core MMAs (mma.sync m16n8k16, bf16 in,
// fp32 accumulate), the weights unpacked in registers straight into the MMA's A fragments: no bf16 tile in shared memory.
//
// Why: the tcgen05 kernel writes every unpacked 128x128 bf16 tile into shared memory and the tensor core reads it back;
// at a few tokens that traffic, not HBM, is its ceiling.  Here a warp's 16x16 A tile is one run of 16 output columns
// (two per thread, MMA rows g and g+8) by 16 rows of K, and the tokens are the MMA's 8 columns, so a lane that has
// loaded 4 consecutive rows of a run (64 contiguous bytes, as the GEMV does) holds exactly the values of its own
// fragment registers for eight MMAs.  A fragment register pairs one column's values of two consecutive rows of K; a
// byte permute picks the magnitude and parked-sign bytes of both rows out of their words, the same mask as everywhere
// leaves two bf16 subnormals +-mag * 2^-133, and ONE packed multiply by the pair (2^(top_k - 64), 2^(top_k+1 - 64))
// finishes them: per pair of values a prmt, a lop3 and a mul.  The sums therefore carry a factor 2^-64 that the
// epilogue undoes (the weight's exponent range 2^-62 .. 2^58 is covered exactly; shared exponents beyond it take a
// two-multiply route, smaller values than 2^-62 may lose low bits against a sum they cannot move).
//
// Work split: a CTA of 4 warps owns 128 output columns (two 64-column groups; with SwiGLU the gate's group and its
// up's) and a slice of K; warp w takes the 16-row steps w, w+4, ... of the slice, six of them in flight in a ring of
// shared memory that the warp's lanes fill by cp.async, each lane the bytes it will consume itself (a step's latency,
// not its bytes, is what a warp waits for: with one step in flight a warp needed 1.2 us per step).  The packed bytes
// pass through shared memory once (2 bytes moved per value where an unpacked bf16 tile costs 4.5).  The warps' partial sums meet in shared memory, the K slices of a thread-block cluster (up to 8 CTAs) through
// distributed shared memory, added in rank order (deterministic).  RMSNorm prologue as in the tcgen05 kernel: a small
// kernel writes bf16(x * g) and 1/rms per token, the epilogue applies 1/rms.
#include "bfp_format.cuh"
#include "linear.cuh"
#include "sm100.cuh"

namespace fb {
namespace {

constexpr int MW = 4, MTHREADS = 32 * MW, RED_LD = 132;  // warps per CTA; floats from one token's sums to the next's
constexpr float UNDO_SCALE = 18446744073709551616.f;     // 2^64
constexpr int STAGES = 6;                                // steps a warp keeps in flight (its ring in shared memory)
constexpr int PREFETCH_UNITS = 16;                       // how far ahead of the loads the L2 prefetch runs (64-row units)

template <int FMT>
struct Raw {  // 4 consecutive rows of one run: 64 (bfp8) or 32 (bfp4) bytes, and their shared exponents
  uint4 q[FMT == FB_BFP8 ? 4 : 2];
  uint32_t tops;
};

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {  // 16 bytes past L1
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
// bytes of one step in a warp's ring: mantissa pieces, 32 lanes' exponent words, 32 lanes' activations per token tile
__host__ __device__ constexpr int stage_bytes(int fmt, int nt) { return (fmt == FB_BFP8 ? 4 : 2) * 512 + 128 + nt * 256; }
__host__ __device__ constexpr size_t mma_smem_bytes(int fmt, int nt) {
  const size_t ring = (size_t)MW * STAGES * stage_bytes(fmt, nt), sums = (size_t)MW * 8 * nt * RED_LD * sizeof(float);
  return ring > sums ? ring : sums;
}

__device__ __forceinline__ uint32_t word_of(const uint4& q, int h) { return h == 0 ? q.x : h == 1 ? q.y : h == 2 ? q.z : q.w; }

// The bf16-subnormal pair (row 2*rp, row 2*rp+1) of column c (0..15) of the run: sign on bits 15 / 31, magnitude below.
// `rot` holds the bfp4 words rotated right by a nibble (a column whose nibble is odd starts on a byte there).
template <int FMT>
__device__ __forceinline__ uint32_t pair_of(const Raw<FMT>& r, const uint32_t rot[2][2][2], int rp, int c) {
  if constexpr (FMT == FB_BFP8) {
    const uint32_t w0 = word_of(r.q[2 * rp], c >> 2), w1 = word_of(r.q[2 * rp + 1], c >> 2);
    const int b = bfp8_byte_of_column(c & 3);  // the magnitude's byte; its sign tops the next byte up (cyclically)
    const uint32_t sel = b | ((b + 1) & 3) << 4 | (4 + b) << 8 | (4 + ((b + 1) & 3)) << 12;
    uint32_t v = __byte_perm(w0, w1, sel), m;
    asm("lop3.b32 %0, %1, 0x807F807F, 0, 0xC0;" : "=r"(m) : "r"(v));
    return m;
  } else {
    const int h = c >> 3, p = bfp4_nibble_of_column(c & 7);  // the magnitude's nibble; its sign tops the nibble three up
    const uint32_t w0 = (p & 1) ? rot[rp][0][h] : (h ? r.q[rp].y : r.q[rp].x);
    const uint32_t w1 = (p & 1) ? rot[rp][1][h] : (h ? r.q[rp].w : r.q[rp].z);
    const int b = p >> 1;
    const uint32_t sel = b | ((b + 1) & 3) << 4 | (4 + b) << 8 | (4 + ((b + 1) & 3)) << 12;
    uint32_t v = __byte_perm(w0, w1, sel), m;
    asm("lop3.b32 %0, %1, 0x80078007, 0, 0xC0;" : "=r"(m) : "r"(v));
    return m;
  }
}

__device__ __forceinline__ void mma_bf16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cluster_barrier() {  // every thread of every CTA of the cluster
  __syncwarp();
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float load_from_rank(uint32_t local_addr, uint32_t rank) {  // CTA `rank`'s copy of a shared word
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

struct MmaParams {
  LinearArgs a;       // x already the normalised activations when there is a norm
  const float* rstd;  // 1/rms per token, or null
  int splits;         // K slices = CTAs of a cluster (gridDim.y)
  int steps_per_split, steps_total;  // 16-row steps of K
};

// One 16-row step: 8 MMAs per token tile.  TWO_STEP: some shared exponent of the warp's lies beyond 2^58; the scale is
// then applied as two factors (the first multiply alone would overflow bf16's exponent).
template <int FMT, int NT, bool TWO_STEP>
__device__ __forceinline__ void mma_step(const Raw<FMT>& r, const uint2 xb[NT], float acc[8][NT][4]) {
  constexpr uint32_t LIFT = FMT == FB_BFP8 ? 63 : 67;  // bfp4's 3-bit magnitude stands for 16 times itself
  uint32_t s1[2], s2[2];
#pragma unroll
  for (int rp = 0; rp < 2; ++rp) {
    const uint32_t e2 = __byte_perm(r.tops, 0, rp ? 0x4342 : 0x4140);  // the pair's two exponents in the two halves
    if (!TWO_STEP) {
      s1[rp] = (e2 + LIFT * 0x10001u) << 7;  // bf16 pair 2^(top - 64) (exponent field top + 63)
      s2[rp] = 0;
    } else {
      const int lo = (int)(e2 & 0xFFFFu) + (int)LIFT - 127, hi = (int)(e2 >> 16) + (int)LIFT - 127;  // the powers wanted
      const int la = lo >> 1, ha = hi >> 1;
      s1[rp] = (uint32_t)(la + 127) << 7 | (uint32_t)(ha + 127) << 23;
      s2[rp] = (uint32_t)(lo - la + 127) << 7 | (uint32_t)(hi - ha + 127) << 23;
    }
  }
  uint32_t rot[2][2][2] = {};
  if constexpr (FMT == FB_BFP4) {
#pragma unroll
    for (int rp = 0; rp < 2; ++rp) {
      rot[rp][0][0] = __funnelshift_r(r.q[rp].x, r.q[rp].x, 4), rot[rp][0][1] = __funnelshift_r(r.q[rp].y, r.q[rp].y, 4);
      rot[rp][1][0] = __funnelshift_r(r.q[rp].z, r.q[rp].z, 4), rot[rp][1][1] = __funnelshift_r(r.q[rp].w, r.q[rp].w, 4);
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint32_t a[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // a0: column 2j rows 0,1; a1: column 2j+1 rows 0,1; a2, a3: the same columns' rows 2,3
      const int rp = i >> 1, c = 2 * j + (i & 1);
      a[i] = mul_bf16x2(pair_of<FMT>(r, rot, rp, c), s1[rp]);
      if (TWO_STEP) a[i] = mul_bf16x2(a[i], s2[rp]);
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_bf16(acc[j][nt], a[0], a[1], a[2], a[3], xb[nt].x, xb[nt].y);
  }
}

template <int FMT, int NT>
__global__ void __launch_bounds__(MTHREADS, NT == 4 ? 2 : 3) linear_mma_kernel(const MmaParams p) {
  constexpr int UNIT = unit_bytes(FMT), UNIT_MANT = unit_mant_bytes(FMT), RUN = run_bytes(FMT);
  extern __shared__ __align__(16) float red[];  // the warps' rings, then their sums [MW][8 * NT][RED_LD]
  const LinearArgs& a = p.a;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const bool swiglu = a.epilogue == FB_EPI_SWIGLU;
  const int64_t groups = groups_of(a.N), KS = ksteps_of(a.K);
  // the CTA's two 64-column groups; lanes with g < 4 read the first, the others the second
  const int64_t grp0 = swiglu ? blockIdx.x : 2 * (int64_t)blockIdx.x, grp1 = swiglu ? blockIdx.x + groups / 2 : grp0 + 1;
  const int64_t my_group = g < 4 ? grp0 : grp1;
  const bool live = my_group < groups;
  const int split = blockIdx.y;
  const int s_begin = split * p.steps_per_split, s_end = min(p.steps_total, s_begin + p.steps_per_split);
  const uint8_t* Wp = static_cast<const uint8_t*>(a.W);
  const uint8_t* strip = Wp + (live ? my_group : 0) * KS * UNIT;  // the group's units follow each other along K

  // L2 prefetch of the two strips' slices: the first stretch now, the rest as warp 0 walks (a unit per turn of its)
  const int u_begin = s_begin >> 2, u_end = (s_end + 3) >> 2;
  if (warp == 0 && (lane == 0 || lane == 16) && live && u_begin < u_end) {
    const int n = min(PREFETCH_UNITS, u_end - u_begin);
    bulk_prefetch_l2(strip + (int64_t)u_begin * UNIT, (uint32_t)(n * UNIT));
  }

  float acc[8][NT][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[j][nt][e] = 0.f;

  const uint16_t* x = static_cast<const uint16_t*>(a.x);
  // ---- the warp's private ring of STAGES steps in shared memory, filled by cp.async in 16-byte pieces.  Copies are
  // coalesced: consecutive lanes take consecutive pieces of a run's 256 (bfp8) or 128 (bfp4) contiguous bytes, so an
  // instruction touches 4 whole lines (a lane fetching its own 64 bytes touched 16 to 32 and the load/store unit, not
  // HBM, set the pace).  A lane then reads its fragment's rows from the ring; pieces are stored XOR-swizzled
  // (piece ^ (piece >> 3 & 7)) so that neither the copies nor those reads meet a bank conflict.  Lanes read what other
  // lanes copied: a __syncwarp() after the wait, another before a slot is refilled.
  constexpr int Q = FMT == FB_BFP8 ? 4 : 2, STAGE = stage_bytes(FMT, NT), XI = (NT * 16 + 31) / 32;
  const uint32_t ring = smem_u32(red) + (uint32_t)(warp * STAGES * STAGE);
  const uint8_t* strip0 = Wp + grp0 * KS * UNIT;
  const uint8_t* strip1 = Wp + (grp1 < groups ? grp1 : grp0) * KS * UNIT;  // (a missing second group: any bytes, never stored)
  const uint8_t* wsrc[Q];
  uint32_t wdst[Q];
#pragma unroll
  for (int i = 0; i < Q; ++i) {
    const int pc = i * 32 + lane;
    if (FMT == FB_BFP8) {  // piece = run (0..7) * 16 + row of the step
      const int run8 = pc >> 4;
      wsrc[i] = (run8 < 4 ? strip0 : strip1) + ((run8 & 3) * KSTEP + (pc & 15)) * 16;
    } else {               // piece = run * 8 + pair of rows
      const int run8 = pc >> 3;
      wsrc[i] = (run8 < 4 ? strip0 : strip1) + (run8 & 3) * KSTEP * 8 + (pc & 7) * 16;
    }
    wdst[i] = (uint32_t)((pc ^ ((pc >> 3) & 7)) * 16);
  }
  const uint8_t* esrc = (lane < 4 ? strip0 : strip1) + UNIT_MANT + (lane & 3) * KSTEP;  // lanes 0..7: a run's 16 exponents
  const uint16_t* xsrc[XI];
#pragma unroll
  for (int i = 0; i < XI; ++i) {  // piece = token * 2 + half of the step's 16 activations
    const int pc = i * 32 + lane;
    xsrc[i] = x + (int64_t)min((int64_t)(pc >> 1), a.M - 1) * a.ldx + 8 * (pc & 1);
  }
  auto copy_weights = [&](int step, int slot) {
    const uint32_t dst = ring + (uint32_t)(slot * STAGE);
    const int64_t at = (int64_t)(step >> 2) * UNIT;
#pragma unroll
    for (int i = 0; i < Q; ++i) cp_async_16(dst + wdst[i], wsrc[i] + at + (step & 3) * 16 * RUN);
    if (lane < 8) cp_async_16(dst + (uint32_t)(Q * 512 + lane * 16), esrc + at + (step & 3) * 16);
  };
  auto copy_x = [&](int step, int slot) {
    const uint32_t dst = ring + (uint32_t)(slot * STAGE + Q * 512 + 128);
#pragma unroll
    for (int i = 0; i < XI; ++i)
      if (i * 32 + lane < NT * 16) cp_async_16(dst + (uint32_t)((i * 32 + lane) * 16), xsrc[i] + 16 * (int64_t)step);
  };
  const int s0 = s_begin + warp;
#pragma unroll
  for (int d = 0; d < STAGES; ++d)
    if (s0 + d * MW < s_end) copy_weights(s0 + d * MW, d);
  griddep_wait();  // the weights are nobody's output; the activations are the kernel before's
#pragma unroll
  for (int d = 0; d < STAGES; ++d)
    if (s0 + d * MW < s_end) copy_x(s0 + d * MW, d);
  cp_async_commit();
  int slot = 0;
  for (int s = s0; s < s_end; s += MW) {
    if (s == s0) cp_async_wait<0>(); else cp_async_wait<STAGES - 1>();  // a group per turn: this step's has landed
    __syncwarp();
    const uint32_t src = ring + (uint32_t)(slot * STAGE);
    Raw<FMT> cur;
    uint2 xc[NT];
#pragma unroll
    for (int i = 0; i < Q; ++i) {  // the lane's rows 4t..4t+3 of run g: pieces Q * lane + i
      const int pc = Q * lane + i;
      cur.q[i] = ld_shared_v4(src + (uint32_t)((pc ^ ((pc >> 3) & 7)) * 16));
    }
    cur.tops = ld_shared_u32(src + (uint32_t)(Q * 512 + lane * 4));
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) xc[nt] = ld_shared_v2(src + (uint32_t)(Q * 512 + 128 + (8 * nt + g) * 32 + 8 * t));
    if (warp == 0 && (lane == 0 || lane == 16) && live) {  // warp 0 moves on by one unit (4 steps) per turn
      const int u = (s >> 2) + PREFETCH_UNITS;
      if (u < u_end) bulk_prefetch_l2(strip + (int64_t)u * UNIT, (uint32_t)UNIT);
    }
    // exponents beyond 187 (values of 2^54 and more) do not fit the one-multiply scale: warp-uniform choice
    const uint32_t half = (cur.tops >> 1) & 0x7F7F7F7Fu;
    const bool big = ((half + 0x22222222u) & 0x80808080u) != 0;
    if (__any_sync(0xffffffffu, big)) mma_step<FMT, NT, true>(cur, xc, acc);
    else mma_step<FMT, NT, false>(cur, xc, acc);
    // refill the slot just consumed (its values have gone through the MMAs) with the step STAGES turns ahead
    const int sn = s + STAGES * MW;
    __syncwarp();  // every lane has read the slot
    if (sn < s_end) copy_weights(sn, slot), copy_x(sn, slot);
    cp_async_commit();
    if (++slot == STAGES) slot = 0;
  }
  cp_async_wait<0>();
  __syncthreads();  // the rings are done with: the sums below reuse their memory
  griddep_launch_dependents();

  // ---- the warps' partial sums -> shared memory.  A lane holds, for tokens 8nt + 2t and the next, all 16 columns of
  // run g: acc[j][nt][e] is column 2j of token 8nt + 2t + e, acc[j][nt][2 + e] column 2j + 1.
  float* mine = red + (size_t)warp * (8 * NT) * RED_LD;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float* row = mine + (8 * nt + 2 * t + e) * RED_LD + 16 * g;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        *reinterpret_cast<float4*>(row + 4 * k) = make_float4(acc[2 * k][nt][e], acc[2 * k][nt][2 + e], acc[2 * k + 1][nt][e], acc[2 * k + 1][nt][2 + e]);
    }
  __syncthreads();
  const int M = (int)a.M;
  for (int idx = threadIdx.x; idx < M * 128; idx += MTHREADS) {  // the four warps' sums, in place of warp 0's
    const int at = (idx >> 7) * RED_LD + (idx & 127);
    float v = red[at];
#pragma unroll
    for (int w = 1; w < MW; ++w) v += red[(size_t)w * (8 * NT) * RED_LD + at];
    red[at] = v;
  }
  if (p.splits > 1) cluster_barrier(); else __syncthreads();

  // ---- epilogue: this CTA's share of the outputs; the K slices added in rank order
  const int width = swiglu ? 64 : 128, total = M * width;
  const int share = (total + p.splits - 1) / p.splits, lo = split * share, hi = min(total, lo + share);
  const uint32_t red_addr = smem_u32(red);
  for (int idx = lo + threadIdx.x; idx < hi; idx += MTHREADS) {
    const int tok = swiglu ? idx >> 6 : idx >> 7, c = idx & (width - 1);
    const int at = tok * RED_LD + c;
    float v = 0.f, up = 0.f;
    if (p.splits > 1) {
      for (int r = 0; r < p.splits; ++r) {
        v += load_from_rank(red_addr + 4 * at, r);
        if (swiglu) up += load_from_rank(red_addr + 4 * (at + 64), r);
      }
    } else {
      v = red[at];
      if (swiglu) up = red[at + 64];
    }
    const float scale = p.rstd ? UNDO_SCALE * p.rstd[tok] : UNDO_SCALE;
    v *= scale, up *= scale;
    int64_t n;
    if (swiglu) {
      n = 64 * grp0 + c;
      v = v / (1.f + __expf(-v)) * up;
    } else {
      n = 128 * (int64_t)blockIdx.x + c;
      if (n >= a.N) continue;
      if (a.epilogue == FB_EPI_RESIDUAL) v += bf16_bits_to_float(static_cast<const uint16_t*>(a.residual)[tok * a.ldr + n]);
    }
    if (a.out_dtype == FB_FP32) static_cast<float*>(a.out)[tok * a.ldo + n] = v;
    else static_cast<uint16_t*>(a.out)[tok * a.ldo + n] = (uint16_t)float_to_bf16_bits(v);
  }
  if (p.splits > 1) cluster_barrier();  // no CTA leaves while its sums may still be read
}

// x' = bf16(x * g) and 1/rms per token: the RMSNorm prologue's two factors (the row scale commutes with the matmul)
__global__ void __launch_bounds__(256) mma_rms_prepare_kernel(const uint16_t* __restrict__ x, int64_t ldx, const uint16_t* __restrict__ g,
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
  __shared__ float part[8];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += part[w];
    rstd[t] = rsqrtf(s / (float)K + eps);
  }
}

template <int FMT, int NT>
int launch_mma(MmaParams p, int64_t blocks, cudaStream_t s) {
  auto kernel = linear_mma_kernel<FMT, NT>;
  const size_t smem = mma_smem_bytes(FMT, NT);
  static std::atomic<uint64_t> opted{0};  // the shared-memory opt-in, once per device
  if (first_on_device(opted)) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(MTHREADS), cfg.dynamicSmemBytes = smem, cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1, attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // may start while the kernel before it drains
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  // K slices (= cluster size, 1..8): the count with the least modelled time.  The SMs' load/store and issue rates set
  // the pace, so time goes as the most steps any SM is handed, ceil(CTAs / 148) x a CTA's steps, plus a fixed cost
  // (launch, first loads, the exchange) for every round of CTAs that cannot be resident together.
  static int capacity[9] = {0};  // CTAs resident at once, by cluster size (asked of the driver once)
  int best = 1;
  long best_cost = -1;
  if (!capacity[1]) {  // every size at the first call (not inside a stream capture: a graph's first run is eager)
    for (int n = 1; n <= 8; ++n) {
      int clusters = 0;
      cfg.gridDim = dim3(148, n, 1), attr[0].val.clusterDim.y = (unsigned)n, cfg.numAttrs = 1;
      if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) != cudaSuccess || clusters < 1) clusters = 1, cudaGetLastError();
      capacity[n] = clusters * n;
    }
  }
  for (int n = 1; n <= 8; ++n) {
    const int per = (p.steps_total + n - 1) / n;
    if (n > 1 && (per < 16 || (p.steps_total + per - 1) / per != n)) continue;  // 4 steps a warp at least; no idle slice
    const long ctas = blocks * n;
    const long cost = (ctas + 147) / 148 * per + 24 * ((ctas + capacity[n] - 1) / capacity[n]);
    if (best_cost < 0 || cost <= best_cost) best_cost = cost, best = n;  // a tie: more warps in flight
  }
  p.splits = best;
  p.steps_per_split = (p.steps_total + best - 1) / best;
  cfg.gridDim = dim3((unsigned)blocks, (unsigned)best, 1), attr[0].val.clusterDim.y = (unsigned)best, cfg.numAttrs = 2;
  if (cudaLaunchKernelEx(&cfg, kernel, p) != cudaSuccess) return launch_status("fb_linear (mma launch)");
  return launch_status("fb_linear (mma)");
}

template <int FMT>
int launch_mma_nt(const MmaParams& p, int64_t blocks, cudaStream_t s) {
  if (p.a.M <= 8) return launch_mma<FMT, 1>(p, blocks, s);
  if (p.a.M <= 16) return launch_mma<FMT, 2>(p, blocks, s);
  return launch_mma<FMT, 4>(p, blocks, s);
}

}  // namespace

bool linear_mma_supports(const LinearArgs& a) {
  return a.M >= 1 && a.M <= 32 && a.K % 16 == 0 && a.ldx % 8 == 0 && (uintptr_t)a.x % 16 == 0 &&
         (a.epilogue != FB_EPI_SWIGLU || a.N % 128 == 0);
}

int linear_mma(const LinearArgs& args, cudaStream_t s) {
  MmaParams p{};
  p.a = args;
  if (args.norm_w) {
    const size_t need = WS_BODY_AT + (size_t)args.M * args.K * 2;  // (linear.cuh: row scales at WS_RSTD_AT, the normalised activations after)
    if (!args.workspace || args.workspace_bytes < need) {
      set_error("fb_linear: workspace of %zu bytes needed, %zu given (fb_linear_workspace_bytes)", need, args.workspace_bytes);
      return FB_ERR_MEMORY;
    }
    float* rstd = reinterpret_cast<float*>(static_cast<uint8_t*>(args.workspace) + WS_RSTD_AT);
    uint16_t* xn = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(args.workspace) + WS_BODY_AT);
    mma_rms_prepare_kernel<<<(unsigned)args.M, 256, 0, s>>>(static_cast<const uint16_t*>(args.x), args.ldx,
                                                            static_cast<const uint16_t*>(args.norm_w), args.K, args.eps, xn, rstd);
    p.rstd = rstd, p.a.x = xn, p.a.ldx = args.K;
  }
  const int64_t groups = groups_of(args.N);
  const int64_t blocks = args.epilogue == FB_EPI_SWIGLU ? groups / 2 : (groups + 1) / 2;
  p.steps_total = (int)(args.K / 16);
  return args.fmt == FB_BFP8 ? launch_mma_nt<FB_BFP8>(p, blocks, s) : launch_mma_nt<FB_BFP4>(p, blocks, s);
}

}  // namespace fb
