// Decode attention over a bf16 - or block-float - KV cache: softmax(q k^T / sqrt(hd) + mask) v for one new token per sequence
// (models/llama.py:111-146; ferrite's one-kernel attention Tensor.attend, ferrite/tensor.py:487-516,
// ferrite/compiler.py:1147-1170).  The mask is never materialised: each token carries the first cache row of its
// sequence (`base`) and its place; it sees keys base .. base + place (and, with a sliding window, only the last
// `window` of them), which is what ferrite's places-based mask means.
//
// Bandwidth-bound on the KV read, so the work is laid out to read every key and value row exactly once:
//   CTA = (token, kv head, split of the keys); the kv head's `rep` query heads are the rows of one 16-row MMA tile
//   (grouped-query attention shares each key row among them, as ferrite's batch entry per (kv head, sequence) does);
//   4 warps take 16 keys each of a 64-key tile staged by cp.async (double-buffered, XOR-swizzled rows);
//   q k^T and p v run on mma.sync m16n8k16 (bf16 in, fp32 accumulate) with an online softmax in registers.
// Keys are split across CTAs (flash-decoding) so that few sequences still fill the GPU; a second small kernel
// merges the splits by their running maxima, as ferrite merges its `parts` (ferrite/tensor.py:511-516).
//
// A block-float cache (bfp8 / bfp4 keys and values, models/llama.py:127-128; the reference reads it in place too,
// test/test_sim.py:2081-2107) is a packed matrix [rows, hd] per head: a 64-key tile is one unit of each 64-column group,
// i.e. one or two contiguous pieces of 4352 (2304) bytes.  They are staged raw by cp.async (double-buffered), unpacked
// into the same swizzled bf16 tiles the bf16 cache is copied into, and everything after that is shared - so the result
// is bit for bit that of a bf16 cache holding the same values, with half (a quarter) of the bytes read.
#include "bfp_format.cuh"

namespace fb {

// One CTA serves one ENTRY: up to 16 query rows that share one run of keys (a kv head's query heads for a token; or
// 16 tokens of one head in a prefill).  Entries are numbered e = e0 * E1 + e1 and every operand is addressed by
// two-level strides (in elements), so both the token-major order of a fused decode step and ferrite's
// (kv head, sequence) batch order (models/llama.py:132-135) are read in place.
struct AttnArgs {
  const uint16_t* q;  // row r of entry e at q + e0*q_s0 + e1*q_s1 + r*q_sr
  int64_t q_s0, q_s1, q_sr;
  const uint16_t *k, *v;  // key j of entry e at k + e0*kv_s0 + e1*kv_s1 + (base[e0] + j)*hd
  int64_t kv_s0, kv_s1;
  const int32_t* base;   // [E0] first cache row of a sequence, or null
  int64_t row0;          // added to it (a chunk of one sequence: its first cache row, with no base)
  const int32_t* place;  // row r of entry e sees keys 0..place[e0*p_s0 + e1*p_s1 + r*p_sr]
  int64_t p_s0, p_s1, p_sr;
  int E1, rows;  // rows per entry
  int window;
  float scale_log2;  // log2(e) * scale of the scores
  uint16_t* out;     // like q
  int64_t o_s0, o_s1, o_sr;
  float* part_o;   // [entries * row tiles, splits, 16, hd]
  float* part_ml;  // [entries * row tiles, splits, 16, 2]
  int splits;
  // rows a head's keys have (the cache's rows, or an entry's keys): no key at or past it is read, whatever a place says.
  // block-float cache: k and v point at head 0's packed matrices (bytes), kv_s0 / kv_s1 are in bytes, and a key's
  // cache row is base[e0] + its number, with base[e0] and the split's first key multiples of 64
  int64_t kv_rows;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t r[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t r[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int ATT_THREADS = 128, KEY_TILE = 64;

// byte offset of 16-byte chunk `ch` of row `r` in a tile whose rows are HD bf16 wide (chunks XOR-swizzled by row)
template <int HD>
__device__ __forceinline__ uint32_t tile_off(int r, int ch) { return (uint32_t)(r * HD * 2 + ((ch ^ (r & 7)) << 4)); }

// KVF: 0 for a bf16 cache, FB_BFP8 / FB_BFP4 for a packed one
template <int HD, int KVF>
__global__ void __launch_bounds__(ATT_THREADS) decode_attention_kernel(AttnArgs a) {
  griddep_launch_dependents();
  constexpr int CH = HD / 8;               // 16-byte chunks per row
  constexpr int TILE_BYTES = KEY_TILE * HD * 2;
  constexpr bool PACKED = KVF != 0;
  constexpr int GROUPS = HD / 64, UNIT = PACKED ? unit_bytes(KVF) : 0, RAW_BYTES = GROUPS * UNIT;  // a tile's packed bytes
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;                      // [16][HD] bf16
  uint8_t* sK = sQ + 16 * HD * 2;          // 2 x [64][HD] (packed cache: one, unpacked into before each use)
  uint8_t* sV = sK + (PACKED ? 1 : 2) * TILE_BYTES;
  uint8_t* sRaw = sV + (PACKED ? 1 : 2) * TILE_BYTES;  // packed cache: 2 x (K's, then V's raw tile)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e = blockIdx.x, e0 = e / a.E1, e1 = e % a.E1, split = blockIdx.y, row0 = blockIdx.z * 16;
  const int rep = min(16, a.rows - row0);  // rows of this tile

  // the keys this CTA reads: what its rows can see, cut into `splits` runs of whole tiles
  const int32_t* places = a.place + e0 * a.p_s0 + e1 * a.p_s1 + (int64_t)row0 * a.p_sr;
  int len = 0, least = 0x7fffffff;
  for (int r = 0; r < rep; ++r) {
    const int p = places[r * a.p_sr];
    len = max(len, p + 1), least = min(least, p);
  }
  // a place past its sequence's rows (or a first row outside the cache) reads no key that is not there
  const int64_t seq_first = (a.base ? a.base[e0] : 0) + a.row0;
  const int64_t room = seq_first < 0 ? 0 : a.kv_rows - seq_first;
  len = (int)max((int64_t)0, min((int64_t)len, room));
  int first = a.window > 0 ? max(0, least + 1 - a.window) : 0;
  first -= first % KEY_TILE;  // whole tiles (a packed cache's units); the window's mask hides the keys before it
  const int per = ((len - first + a.splits - 1) / a.splits + KEY_TILE - 1) / KEY_TILE * KEY_TILE;
  const int k0 = first + split * per, k1 = min(len, k0 + per);
  const int n_tiles = k1 > k0 ? (k1 - k0 + KEY_TILE - 1) / KEY_TILE : 0;
  const int64_t kv_off = e0 * a.kv_s0 + e1 * a.kv_s1 + (len > 0 ? seq_first * HD : 0);
  const uint16_t* Kg = a.k + kv_off;
  const uint16_t* Vg = a.v + kv_off;
  const uint16_t* Qg = a.q + e0 * a.q_s0 + e1 * a.q_s1 + (int64_t)row0 * a.q_sr;
  // this thread's two rows (lane/4 and lane/4 + 8) see keys window_lo .. place
  int place_r[2], lo_r[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + 8 * h;
    place_r[h] = r < rep ? places[r * a.p_sr] : -1;
    lo_r[h] = a.window > 0 ? place_r[h] + 1 - a.window : 0;
  }

  // packed: head matrices at k / v + byte offsets; unit u of column group g at (g * KS + u) * UNIT
  const int64_t KS = PACKED ? ksteps_of(a.kv_rows) : 0;
  const uint8_t* Kp = reinterpret_cast<const uint8_t*>(a.k) + e0 * a.kv_s0 + e1 * a.kv_s1;
  const uint8_t* Vp = reinterpret_cast<const uint8_t*>(a.v) + e0 * a.kv_s0 + e1 * a.kv_s1;
  const int64_t row_first = PACKED && len > 0 ? seq_first : 0;
  auto load_tile = [&](int i, int buf) {
    const int key0 = k0 + i * KEY_TILE;
    if (PACKED) {
      const int64_t u = (row_first + key0) / KEY_TILE;
      constexpr int PIECES = RAW_BYTES / 16;
      for (int c = tid; c < 2 * PIECES; c += ATT_THREADS) {
        const int which = c / PIECES, piece = c % PIECES, g = piece / (UNIT / 16), at = piece % (UNIT / 16);
        const uint8_t* src = (which ? Vp : Kp) + (g * KS + u) * UNIT + at * 16;
        cp_async16(smem_addr(sRaw + (buf * 2 + which) * RAW_BYTES) + piece * 16, src);
      }
      cp_async_commit();
      return;
    }
    for (int c = tid; c < KEY_TILE * CH; c += ATT_THREADS) {
      const int r = c / CH, ch = c % CH;
      const int key = min(key0 + r, k1 - 1);  // rows past the end repeat the last key; their scores are masked
      cp_async16(smem_addr(sK + buf * TILE_BYTES) + tile_off<HD>(r, ch), Kg + (int64_t)key * HD + ch * 8);
      cp_async16(smem_addr(sV + buf * TILE_BYTES) + tile_off<HD>(r, ch), Vg + (int64_t)key * HD + ch * 8);
    }
    cp_async_commit();
  };
  if (n_tiles) load_tile(0, 0);

  // the kv head's query heads as rows 0..rep-1 of a 16-row tile, the rest zeros
  for (int c = tid; c < 16 * CH; c += ATT_THREADS) {
    const int r = c / CH, ch = c % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rep) v = *reinterpret_cast<const uint4*>(Qg + r * a.q_sr + ch * 8);
    *reinterpret_cast<uint4*>(sQ + tile_off<HD>(r, ch)) = v;
  }
  __syncthreads();
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int kt = 0; kt < HD / 16; ++kt) {
    const int m = lane >> 3, r = (m & 1) * 8 + (lane & 7), ch = 2 * kt + (m >> 1);
    ldmatrix_x4(smem_addr(sQ) + tile_off<HD>(r, ch), qf[kt]);
  }

  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};  // rows lane/4 and lane/4 + 8

  for (int i = 0; i < n_tiles; ++i) {
    const int buf = i & 1;
    if (i + 1 < n_tiles) load_tile(i + 1, buf ^ 1);
    if (i + 1 < n_tiles) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    if (PACKED) {
      // raw -> bf16 tiles, each warp the 16 keys it multiplies (no other warp reads them: a warp-level sync is enough):
      // a lane per run of 16 (16 bytes + its exponent -> two swizzled 16-byte chunks)
      constexpr int RUNS = HD / 16;
      for (int c = lane; c < 2 * 16 * RUNS; c += 32) {
        const int which = c / (16 * RUNS), run = (c / 16) % RUNS, r = 16 * warp + c % 16;
        const uint8_t* unit = sRaw + (buf * 2 + which) * RAW_BYTES + (run / GROUP_RUNS) * UNIT;
        const int at = (run % GROUP_RUNS) * KSTEP + r;
        const uint32_t top = unit[unit_mant_bytes(KVF) + at];
        uint32_t v[8];
        if (KVF == FB_BFP8) unpack_run8(*reinterpret_cast<const uint4*>(unit + at * 16), top, v);
        else unpack_run4(*reinterpret_cast<const uint2*>(unit + at * 8), top, v);
        uint8_t* tile = which ? sV : sK;
        *reinterpret_cast<uint4*>(tile + tile_off<HD>(r, 2 * run)) = make_uint4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<uint4*>(tile + tile_off<HD>(r, 2 * run + 1)) = make_uint4(v[4], v[5], v[6], v[7]);
      }
      __syncwarp();
    }
    const uint32_t kt_base = smem_addr(sK + (PACKED ? 0 : buf) * TILE_BYTES), vt_base = smem_addr(sV + (PACKED ? 0 : buf) * TILE_BYTES);
    const int krow = 16 * warp;  // this warp's 16 keys of the tile

    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kt = 0; kt < HD / 16; ++kt) {
      uint32_t b[4];
      const int m = lane >> 3, r = krow + (m >> 1) * 8 + (lane & 7), ch = 2 * kt + (m & 1);
      ldmatrix_x4(kt_base + tile_off<HD>(r, ch), b);
      mma_bf16(s[0], qf[kt], b[0], b[1]);
      mma_bf16(s[1], qf[kt], b[2], b[3]);
    }
    // scores -> probabilities under the running maximum of each row
    const int key_first = k0 + i * KEY_TILE + krow + (lane & 3) * 2;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {  // (e: the accumulator's element, not the entry)
        const int key = key_first + nt * 8 + (e & 1);
        const bool seen = key < k1 && key <= place_r[e >> 1] && key >= lo_r[e >> 1];
        s[nt][e] = seen ? s[nt][e] * a.scale_log2 : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
    float corr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      const float m_safe = m_new == -INFINITY ? 0.f : m_new;
      corr[h] = exp2f(m_run[h] - m_safe);  // (-inf - finite = -inf: 0)
      m_run[h] = m_new;
      l_run[h] *= corr[h];
      mx[h] = m_safe;
    }
    uint32_t pf[4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float p0 = exp2f(s[nt][0] - mx[0]), p1 = exp2f(s[nt][1] - mx[0]);
      const float p2 = exp2f(s[nt][2] - mx[1]), p3 = exp2f(s[nt][3] - mx[1]);
      l_run[0] += p0 + p1;
      l_run[1] += p2 + p3;
      pf[2 * nt] = pack_bf16x2(p0, p1);
      pf[2 * nt + 1] = pack_bf16x2(p2, p3);
    }
#pragma unroll
    for (int dt = 0; dt < HD / 8; dt += 2) {
      o[dt][0] *= corr[0], o[dt][1] *= corr[0], o[dt][2] *= corr[1], o[dt][3] *= corr[1];
      o[dt + 1][0] *= corr[0], o[dt + 1][1] *= corr[0], o[dt + 1][2] *= corr[1], o[dt + 1][3] *= corr[1];
      uint32_t b[4];
      const int m = lane >> 3, r = krow + (m & 1) * 8 + (lane & 7), ch = dt + (m >> 1);
      ldmatrix_x4_trans(vt_base + tile_off<HD>(r, ch), b);
      mma_bf16(o[dt], pf, b[0], b[1]);
      mma_bf16(o[dt + 1], pf, b[2], b[3]);
    }
    __syncthreads();  // the buffer is free for the load after next
  }

  // ---- merge the four warps' partial softmaxes (each saw different keys) through shared memory
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  float* so = reinterpret_cast<float*>(sK);           // [4][16][HD]: two tiles' room (packed cache: K's tile and V's)
  float* sml = reinterpret_cast<float*>(PACKED ? sRaw : sV);  // [4][16][2]
#pragma unroll
  for (int dt = 0; dt < HD / 8; ++dt) {
    const int col = dt * 8 + (lane & 3) * 2, r = lane >> 2;
    *reinterpret_cast<float2*>(so + (warp * 16 + r) * HD + col) = make_float2(o[dt][0], o[dt][1]);
    *reinterpret_cast<float2*>(so + (warp * 16 + r + 8) * HD + col) = make_float2(o[dt][2], o[dt][3]);
  }
  if ((lane & 3) == 0) {
    sml[(warp * 16 + (lane >> 2)) * 2] = m_run[0], sml[(warp * 16 + (lane >> 2)) * 2 + 1] = l_run[0];
    sml[(warp * 16 + (lane >> 2) + 8) * 2] = m_run[1], sml[(warp * 16 + (lane >> 2) + 8) * 2 + 1] = l_run[1];
  }
  __syncthreads();
  for (int idx = tid; idx < rep * HD; idx += ATT_THREADS) {
    const int r = idx / HD, d = idx % HD;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, sml[(w * 16 + r) * 2]);
    const float m_safe = m == -INFINITY ? 0.f : m;
    float l = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = exp2f(sml[(w * 16 + r) * 2] - m_safe);
      l += sml[(w * 16 + r) * 2 + 1] * f;
      acc += so[(w * 16 + r) * HD + d] * f;
    }
    if (a.splits == 1) {
      a.out[e0 * a.o_s0 + e1 * a.o_s1 + (int64_t)(row0 + r) * a.o_sr + d] = (uint16_t)float_to_bf16_bits(l > 0.f ? acc / l : 0.f);
    } else {
      const int64_t at = (((int64_t)blockIdx.x * gridDim.z + blockIdx.z) * a.splits + split) * 16 + r;
      a.part_o[at * HD + d] = acc;
      if (d == 0) a.part_ml[at * 2] = m, a.part_ml[at * 2 + 1] = l;
    }
  }
}

// one block per (entry, row): weight each split by exp2(its max - the overall max), sum, divide
template <int HD>
__global__ void __launch_bounds__(HD) attention_combine_kernel(AttnArgs a) {
  griddep_launch_dependents();
  const int e = blockIdx.x / a.rows, row = blockIdx.x % a.rows, d = threadIdx.x;
  const int e0 = e / a.E1, e1 = e % a.E1, tiles = (a.rows + 15) / 16;
  const int64_t first = (((int64_t)e * tiles + row / 16) * a.splits) * 16 + row % 16;
  float m = -INFINITY;
  for (int s = 0; s < a.splits; ++s) m = fmaxf(m, a.part_ml[(first + s * 16) * 2]);
  const float m_safe = m == -INFINITY ? 0.f : m;
  float l = 0.f, acc = 0.f;
  for (int s = 0; s < a.splits; ++s) {
    const float f = exp2f(a.part_ml[(first + s * 16) * 2] - m_safe);
    l += a.part_ml[(first + s * 16) * 2 + 1] * f;
    acc += a.part_o[(first + s * 16) * HD + d] * f;
  }
  a.out[e0 * a.o_s0 + e1 * a.o_s1 + (int64_t)row * a.o_sr + d] = (uint16_t)float_to_bf16_bits(l > 0.f ? acc / l : 0.f);
}

static int pick_splits(int64_t ctas, int64_t max_keys) {
  if (ctas < 1) return 1;
  int64_t want = (4 * 148 + ctas - 1) / ctas;                           // about four CTAs per SM in flight
  const int64_t most = (max_keys + 2 * KEY_TILE - 1) / (2 * KEY_TILE);  // at least two tiles per split
  want = want > most ? most : want;
  return (int)(want < 1 ? 1 : want > 32 ? 32 : want);
}

static size_t attention_workspace(int64_t entries, int rows, int hd, int64_t max_keys, int* splits_out) {
  const int64_t ctas = entries * ((rows + 15) / 16);
  const int splits = pick_splits(ctas, max_keys);
  if (splits_out) *splits_out = splits;
  return splits == 1 ? 0 : (size_t)ctas * splits * 16 * (hd + 2) * sizeof(float);
}

template <int HD, int KVF>
static void launch_one(const AttnArgs& a, dim3 grid, int splits, int64_t entries, cudaStream_t s) {
  const size_t smem = KVF ? (size_t)(16 + 2 * KEY_TILE) * HD * 2 + 4 * (HD / 64) * unit_bytes(KVF ? KVF : FB_BFP8) : (size_t)(16 + 4 * KEY_TILE) * HD * 2;
  static std::atomic<uint64_t> opted{0};  // the shared-memory opt-in, once per device
  if (first_on_device(opted)) cudaFuncSetAttribute(decode_attention_kernel<HD, KVF>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  decode_attention_kernel<HD, KVF><<<grid, ATT_THREADS, smem, s>>>(a);
  if (splits > 1) attention_combine_kernel<HD><<<(unsigned)(entries * a.rows), HD, 0, s>>>(a);
}

static int launch_attention(AttnArgs a, int64_t entries, int hd, int64_t max_keys, void* workspace, size_t workspace_bytes, cudaStream_t s, int kv_fmt = 0) {
  int splits;
  const size_t need = attention_workspace(entries, a.rows, hd, max_keys, &splits);
  if (need && (!workspace || workspace_bytes < need)) {
    set_error("attention: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    return FB_ERR_MEMORY;
  }
  const int tiles = (a.rows + 15) / 16;
  a.splits = splits;
  a.part_o = (float*)workspace;
  a.part_ml = (float*)workspace + (size_t)entries * tiles * splits * 16 * hd;
  dim3 grid((unsigned)entries, (unsigned)splits, (unsigned)tiles);
  if (hd == 128) {
    if (kv_fmt == FB_BFP8) launch_one<128, FB_BFP8>(a, grid, splits, entries, s);
    else if (kv_fmt == FB_BFP4) launch_one<128, FB_BFP4>(a, grid, splits, entries, s);
    else launch_one<128, 0>(a, grid, splits, entries, s);
  } else {
    if (kv_fmt == FB_BFP8) launch_one<64, FB_BFP8>(a, grid, splits, entries, s);
    else if (kv_fmt == FB_BFP4) launch_one<64, FB_BFP4>(a, grid, splits, entries, s);
    else launch_one<64, 0>(a, grid, splits, entries, s);
  }
  return launch_status("attention");
}

}  // namespace fb

extern "C" size_t fb_decode_attention_workspace_bytes(int64_t T, int H, int KV, int hd, int64_t max_keys) {
  if (T < 1 || KV < 1 || H < KV || hd < 1 || max_keys < 1) return 0;  // an empty shape needs nothing (the call itself refuses it)
  return fb::attention_workspace(T * KV, H / KV, hd, max_keys, nullptr);
}

extern "C" int fb_decode_attention(const void* q, int64_t T, int64_t ld_q, int H, int KV, int hd, const void* cache, int64_t cache_rows,
                                   int64_t cache_head_stride, const int32_t* base, const int32_t* place, int64_t max_keys, int window, void* out, int64_t ld_o,
                                   void* workspace, size_t workspace_bytes, void* stream) {
  FB_REQUIRE(q && cache && base && place && out && T >= 1, "fb_decode_attention: null pointer or no tokens");
  FB_REQUIRE(hd == 64 || hd == 128, "fb_decode_attention: heads of 64 or 128 columns (got %d)", hd);
  FB_REQUIRE(KV >= 1 && H % KV == 0 && H / KV <= 16, "fb_decode_attention: up to 16 query heads per key head (got %d / %d)", H, KV);
  FB_REQUIRE(ld_q >= (int64_t)H * hd && ld_o >= (int64_t)H * hd && ld_q % 8 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)cache % 16 == 0,
             "fb_decode_attention: rows of q 16-byte aligned");
  FB_REQUIRE(max_keys >= 1 && max_keys <= cache_rows && window >= 0 && cache_head_stride >= cache_rows * hd, "fb_decode_attention: max_keys within the cache");
  const int rep = H / KV;
  fb::AttnArgs a{};
  a.q = (const uint16_t*)q, a.q_s0 = ld_q, a.q_s1 = (int64_t)rep * hd, a.q_sr = hd;  // entry (token, kv head): its rep query heads
  a.k = (const uint16_t*)cache, a.v = (const uint16_t*)cache + (int64_t)KV * cache_head_stride;
  a.kv_s0 = 0, a.kv_s1 = cache_head_stride, a.base = base, a.kv_rows = cache_rows;
  a.place = place, a.p_s0 = 1, a.p_s1 = 0, a.p_sr = 0;
  a.E1 = KV, a.rows = rep, a.window = window, a.scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  a.out = (uint16_t*)out, a.o_s0 = ld_o, a.o_s1 = (int64_t)rep * hd, a.o_sr = hd;
  return fb::launch_attention(a, T * KV, hd, max_keys, workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" int fb_decode_attention_packed(int cache_fmt, const void* q, int64_t T, int64_t ld_q, int H, int KV, int hd, const void* cache_packed,
                                          int64_t cache_rows, const int32_t* base, const int32_t* place, int64_t max_keys, int window, void* out,
                                          int64_t ld_o, void* workspace, size_t workspace_bytes, void* stream) {
  FB_REQUIRE(cache_fmt == FB_BFP8 || cache_fmt == FB_BFP4, "fb_decode_attention_packed: a bfp8 or bfp4 cache (dtype %d given)", cache_fmt);
  FB_REQUIRE(q && cache_packed && base && place && out && T >= 1, "fb_decode_attention_packed: null pointer or no tokens");
  FB_REQUIRE(hd == 64 || hd == 128, "fb_decode_attention_packed: heads of 64 or 128 columns (got %d)", hd);
  FB_REQUIRE(KV >= 1 && H % KV == 0 && H / KV <= 16, "fb_decode_attention_packed: up to 16 query heads per key head (got %d / %d)", H, KV);
  FB_REQUIRE(ld_q >= (int64_t)H * hd && ld_o >= (int64_t)H * hd && ld_q % 8 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)cache_packed % 16 == 0,
             "fb_decode_attention_packed: rows of q 16-byte aligned");
  FB_REQUIRE(max_keys >= 1 && max_keys <= cache_rows && window >= 0, "fb_decode_attention_packed: max_keys within the cache");
  const int rep = H / KV;
  const int64_t head_bytes = fb::packed_bytes(cache_fmt, cache_rows, hd);
  fb::AttnArgs a{};
  a.q = (const uint16_t*)q, a.q_s0 = ld_q, a.q_s1 = (int64_t)rep * hd, a.q_sr = hd;
  a.k = (const uint16_t*)cache_packed, a.v = (const uint16_t*)((const uint8_t*)cache_packed + KV * head_bytes);
  a.kv_s0 = 0, a.kv_s1 = head_bytes, a.base = base, a.kv_rows = cache_rows;
  a.place = place, a.p_s0 = 1, a.p_s1 = 0, a.p_sr = 0;
  a.E1 = KV, a.rows = rep, a.window = window, a.scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  a.out = (uint16_t*)out, a.o_s0 = ld_o, a.o_s1 = (int64_t)rep * hd, a.o_sr = hd;
  return fb::launch_attention(a, T * KV, hd, max_keys, workspace, workspace_bytes, (cudaStream_t)stream, cache_fmt);
}

extern "C" size_t fb_attend_workspace_bytes(int64_t entries, int64_t rows, int hd, int64_t max_keys) {
  if (entries < 1 || rows < 1 || hd < 1 || max_keys < 1) return 0;
  return fb::attention_workspace(entries, (int)rows, hd, max_keys, nullptr);
}

extern "C" int fb_attend(const void* q, int64_t entries, int64_t rows, int hd, int64_t q_entry_stride, int64_t q_row_stride, const void* k,
                         const void* v, int64_t kv_entry_stride, int64_t kv_rep, int64_t keys, const int32_t* places,
                         int64_t place_entry_stride, int64_t place_row_stride, int window, float scale, void* out, void* workspace,
                         size_t workspace_bytes, void* stream) {
  FB_REQUIRE(q && k && v && places && out && entries >= 1 && rows >= 1 && keys >= 1, "fb_attend: null pointer or empty");
  FB_REQUIRE(hd == 64 || hd == 128, "fb_attend: heads of 64 or 128 columns (got %d)", hd);
  FB_REQUIRE(kv_rep >= 1 && q_row_stride % 8 == 0 && q_entry_stride % 8 == 0 && kv_entry_stride % 8 == 0 && (uintptr_t)q % 16 == 0 &&
                 (uintptr_t)k % 16 == 0 && (uintptr_t)v % 16 == 0,
             "fb_attend: rows 16-byte aligned");
  fb::AttnArgs a{};
  a.q = (const uint16_t*)q, a.q_s0 = q_entry_stride * kv_rep, a.q_s1 = q_entry_stride, a.q_sr = q_row_stride;
  a.k = (const uint16_t*)k, a.v = (const uint16_t*)v, a.kv_s0 = kv_entry_stride, a.kv_s1 = 0, a.base = nullptr, a.kv_rows = keys;  // kv_rep entries share a key matrix
  a.place = places, a.p_s0 = place_entry_stride * kv_rep, a.p_s1 = place_entry_stride, a.p_sr = place_row_stride;
  a.E1 = (int)kv_rep, a.rows = (int)rows, a.window = window, a.scale_log2 = 1.4426950408889634f * scale;
  a.out = (uint16_t*)out, a.o_s0 = rows * hd * kv_rep, a.o_s1 = rows * hd, a.o_sr = hd;
  return fb::launch_attention(a, entries, hd, keys, workspace, workspace_bytes, (cudaStream_t)stream);
}

// A chunk of ONE sequence's prompt: T tokens at places[t] (rising or not), each seeing the sequence's keys up to its own
// place.  An entry is a query head over all the chunk's tokens, 16 tokens a CTA, so a key row is read once per 16
// prompt tokens of a head instead of once per token (what the decode form would cost).
extern "C" size_t fb_prefill_attention_workspace_bytes(int64_t T, int H, int hd, int64_t max_keys) {
  if (T < 1 || H < 1 || hd < 1 || max_keys < 1) return 0;
  return fb::attention_workspace(H, (int)T, hd, max_keys, nullptr);
}

extern "C" int fb_prefill_attention(int cache_fmt, const void* q, int64_t T, int64_t ld_q, int H, int KV, int hd, const void* cache,
                                    int64_t cache_rows, int64_t cache_head_stride, int64_t first_row, const int32_t* places, int64_t max_keys,
                                    int window, void* out, int64_t ld_o, void* workspace, size_t workspace_bytes, void* stream) {
  FB_REQUIRE(cache_fmt == 0 || cache_fmt == FB_BF16 || cache_fmt == FB_BFP8 || cache_fmt == FB_BFP4, "fb_prefill_attention: a bf16, bfp8 or bfp4 cache (dtype %d given)", cache_fmt);
  FB_REQUIRE(q && cache && places && out && T >= 1 && T <= (1 << 20), "fb_prefill_attention: null pointer or no tokens");
  FB_REQUIRE(hd == 64 || hd == 128, "fb_prefill_attention: heads of 64 or 128 columns (got %d)", hd);
  FB_REQUIRE(KV >= 1 && H % KV == 0, "fb_prefill_attention: whole groups of query heads per key head (got %d / %d)", H, KV);
  FB_REQUIRE(ld_q >= (int64_t)H * hd && ld_o >= (int64_t)H * hd && ld_q % 8 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)cache % 16 == 0,
             "fb_prefill_attention: rows of q 16-byte aligned");
  FB_REQUIRE(first_row >= 0 && max_keys >= 1 && first_row + max_keys <= cache_rows && window >= 0, "fb_prefill_attention: the sequence's rows within the cache");
  const bool packed = cache_fmt == FB_BFP8 || cache_fmt == FB_BFP4;
  FB_REQUIRE(!packed || first_row % 64 == 0, "fb_prefill_attention: a sequence's rows start a packed unit (first_row a multiple of 64)");
  FB_REQUIRE(packed || cache_head_stride >= cache_rows * hd, "fb_prefill_attention: heads at least cache_rows rows apart");
  const int rep = H / KV;
  fb::AttnArgs a{};
  a.q = (const uint16_t*)q, a.q_s0 = (int64_t)rep * hd, a.q_s1 = hd, a.q_sr = ld_q;  // entry (key head, query head of its group): a row per token
  if (packed) {
    const int64_t head_bytes = fb::packed_bytes(cache_fmt, cache_rows, hd);
    a.k = (const uint16_t*)cache, a.v = (const uint16_t*)((const uint8_t*)cache + KV * head_bytes), a.kv_s0 = head_bytes;
  } else {
    a.k = (const uint16_t*)cache, a.v = (const uint16_t*)cache + (int64_t)KV * cache_head_stride, a.kv_s0 = cache_head_stride;
  }
  a.kv_s1 = 0, a.base = nullptr, a.row0 = first_row, a.kv_rows = cache_rows;
  a.place = places, a.p_s0 = 0, a.p_s1 = 0, a.p_sr = 1;
  a.E1 = rep, a.rows = (int)T, a.window = window, a.scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  a.out = (uint16_t*)out, a.o_s0 = (int64_t)rep * hd, a.o_s1 = hd, a.o_sr = ld_o;
  return fb::launch_attention(a, H, hd, max_keys, workspace, workspace_bytes, (cudaStream_t)stream, packed ? cache_fmt : 0);
}

// ---- fb_decode_attention with its scratch built into the library -------------------------------------------------
// Some hosts cannot give this library a workspace: a serving process that has handed all of the device's memory to
// its own pool at start-up (weights, KV cache) and forbids any later cudaMalloc, or a binding that has no way to own
// and pass a scratch buffer.  For them the partial sums of the key splits live in this array, which every GPU that
// loads the library holds from load to exit.  All calls on a device share it and it keeps whatever the last call
// left: nothing in it has to start at zero (every split writes all of its rows before the merge reads them), but
// two calls that overlap on the GPU (two streams) would overwrite each other's partial sums.
namespace fb {
constexpr size_t STATIC_SCRATCH_BYTES = 8u << 20;
static __device__ __align__(256) unsigned char g_attention_scratch[STATIC_SCRATCH_BYTES];
static void* g_scratch_ptr[64] = {};  // the array's device address, per device, looked up once
}  // namespace fb

extern "C" size_t fb_decode_attention_static_max_bytes(void) { return fb::STATIC_SCRATCH_BYTES; }

extern "C" int fb_decode_attention_static(const void* q, int64_t T, int64_t ld_q, int H, int KV, int hd, const void* cache, int64_t cache_rows,
                                          int64_t cache_head_stride, const int32_t* base, const int32_t* place, int64_t max_keys, int window,
                                          void* out, int64_t ld_o, void* stream) {
  FB_REQUIRE(T >= 1 && KV >= 1 && H >= 1 && H % KV == 0 && (hd == 64 || hd == 128) && max_keys >= 1,
             "fb_decode_attention_static: at least one token, whole groups of query heads per key head, heads of 64 or 128 columns");
  const size_t need = fb_decode_attention_workspace_bytes(T, H, KV, hd, max_keys);
  FB_REQUIRE(need <= fb::STATIC_SCRATCH_BYTES,
             "fb_decode_attention_static: this call needs %zu bytes of scratch, the built-in array holds %zu: fewer tokens per call, or "
             "fb_decode_attention with a workspace of the caller's",
             need, fb::STATIC_SCRATCH_BYTES);
  int dev = -1;
  if (cudaError_t e = cudaGetDevice(&dev)) {
    fb::set_error("fb_decode_attention_static: cudaGetDevice: %s", cudaGetErrorString(e));
    return FB_ERR_LAUNCH;
  }
  FB_REQUIRE(dev >= 0 && dev < 64, "fb_decode_attention_static: device ordinal %d is beyond the 64 this entry point keeps an address for", dev);
  if (!fb::g_scratch_ptr[dev]) {  // set-up, on the first call on this device: in host code the array's name is not its device address
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, fb::g_attention_scratch);
    if (e != cudaSuccess || !p) {
      fb::set_error("fb_decode_attention_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return FB_ERR_LAUNCH;
    }
    fb::g_scratch_ptr[dev] = p;
  }
  return fb_decode_attention(q, T, ld_q, H, KV, hd, cache, cache_rows, cache_head_stride, base, place, max_keys, window, out, ld_o,
                             fb::g_scratch_ptr[dev], fb::STATIC_SCRATCH_BYTES, stream);
}
