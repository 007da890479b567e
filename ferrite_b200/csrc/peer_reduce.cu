// fb_peer_reduce_add: out = residual + the sum over the ranks of their partial results, in ONE kernel per rank that reads
// the other ranks' partials straight out of their memory over NVLink (plain peer loads; no multicast, no TMA).
//
// It stands where a tensor-parallel block has `all_reduce(partial)` followed by `+ residual` (after o_proj, after
// down_proj or the experts): at decode sizes (tokens x dim bf16, a few hundred KB) a ring or tree collective is all
// latency, and the adding kernel after it is a launch more.  Here every rank
//   1. tells every rank (a release store at system scope into that rank's flag word for it) that its partial of call
//      number e is in place - it was written by the kernel before this one in the stream, into memory every rank maps;
//   2. waits until every rank has told it so (acquire loads of its own flag words, bounded: a rank that never arrives
//      costs ~2 s - or state[3] clock cycles, when that is not 0 -, leaves 201 + its number in state[2] and in the
//      library's status word (fb_status_word), and the call returns with what is there);
//   3. adds the partials in rank order 0, 1, ... in fp32 - the same order on every rank, so all ranks hold bit-identical
//      results and stay in step - adds the residual, rounds once to bf16.
// The call number lives on the device (state[0]) and is advanced by the last CTA to finish, so a recorded graph can
// be replayed: flags only ever grow, and a rank can be at most one call ahead of another (it cannot pass step 2 of
// call e + 1 before that other has entered call e + 1), which is why "flag >= e" is the test.  The partial's buffer of
// a call site may be rewritten once any later call has passed step 2 (every rank has then finished reading it).
#include "sm100.cuh"

namespace fb {

namespace {

constexpr int MAX_RANKS = 8;

struct PeerArgs {
  const uint16_t* partial[MAX_RANKS];  // each rank's partial of this call site (peer-mapped addresses), bf16 [count]
  uint32_t* flags[MAX_RANKS];          // each rank's flag words: flags[r][s] = the last call rank s has entered
  uint32_t* state;                     // this rank's: [0] calls completed, [1] CTAs of the running call that are done,
                                       // [2] 0, or 201 + the rank a wait gave up on, [3] the wait's bound in clocks (0: WAIT_CLOCKS)
  const uint16_t* residual;            // bf16 [count] or null
  uint16_t* out;                       // bf16 [count]
  int64_t count;
  int rank, world;
};

__device__ __forceinline__ void store_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// 16 bytes of another rank's memory (or this rank's): never through the non-coherent path, the same address holds the
// next step's partial
__device__ __forceinline__ uint4 load_peer(const uint16_t* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

enum { WAIT_PEER = 201 };

__global__ void __launch_bounds__(256) peer_reduce_add_kernel(const PeerArgs a) {
  __shared__ uint32_t s_call;
  if (threadIdx.x == 0) {
    const uint32_t e = *reinterpret_cast<volatile uint32_t*>(a.state) + 1;  // this call's number (the last CTA advances it)
    s_call = e;
  }
  __syncthreads();
  const uint32_t e = s_call;
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    store_release_sys(a.flags[threadIdx.x] + a.rank, e);
  }
  // (after a wait has given up once, later calls do not wait again: the caller finds the code in state[2] within seconds)
  if (threadIdx.x < a.world && *reinterpret_cast<volatile uint32_t*>(a.state + 2) == 0) {  // one thread per rank waited for
    const uint32_t* flag = a.flags[a.rank] + threadIdx.x;
    const uint32_t own = *reinterpret_cast<volatile uint32_t*>(a.state + 3);
    const long long limit = own ? (long long)own : WAIT_CLOCKS, start = clock64();
    // (flags only grow; the difference is taken modulo 2^32 so that the count may wrap)
    while ((int32_t)(load_acquire_sys(flag) - e) < 0) {
      if (clock64() - start > limit) {
        atomicCAS(a.state + 2, 0u, (uint32_t)WAIT_PEER + threadIdx.x);  // (the caller reads and clears it)
        atomicCAS(&g_status_word, 0, (int)WAIT_PEER + (int)threadIdx.x);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  const int64_t chunks = a.count / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < chunks; i += (int64_t)gridDim.x * blockDim.x) {
    float acc[8];
    const uint4 r = a.residual ? *reinterpret_cast<const uint4*>(a.residual + 8 * i) : make_uint4(0, 0, 0, 0);
    uint4 v[MAX_RANKS];
#pragma unroll
    for (int s = 0; s < MAX_RANKS; ++s)  // all the ranks' loads are in flight together
      if (s < a.world) v[s] = load_peer(a.partial[s] + 8 * i);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
    for (int s = 0; s < MAX_RANKS; ++s) {
      if (s >= a.world) break;
      const uint32_t w[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += bf16_bits_to_float(w[j] & 0xFFFFu);
        acc[2 * j + 1] += bf16_bits_to_float(w[j] >> 16);
      }
    }
    const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = pack_bf16x2(acc[2 * j] + bf16_bits_to_float(rw[j] & 0xFFFFu), acc[2 * j + 1] + bf16_bits_to_float(rw[j] >> 16));
    *reinterpret_cast<uint4*>(a.out + 8 * i) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  // the last CTA to finish closes the call: every CTA has read state[0] by then
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.state + 1, 1u) == gridDim.x - 1) {
      a.state[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(a.state) = e;
    }
  }
}

}  // namespace

int status_word_peer() { return read_and_clear_status_word(); }

}  // namespace fb

extern "C" int fb_peer_reduce_add(const void* const* partials, void* const* flags, int rank, int world, void* state, int64_t count,
                                  const void* residual, void* out, void* stream) {
  FB_REQUIRE(partials && flags && state && out, "fb_peer_reduce_add: null pointer");
  FB_REQUIRE(world >= 1 && world <= fb::MAX_RANKS && rank >= 0 && rank < world, "fb_peer_reduce_add: rank %d of %d (up to %d ranks)", rank, world, fb::MAX_RANKS);
  FB_REQUIRE(count >= 8 && count % 8 == 0, "fb_peer_reduce_add: whole 16-byte pieces (count %lld)", (long long)count);
  fb::PeerArgs a{};
  for (int r = 0; r < world; ++r) {
    FB_REQUIRE(partials[r] && flags[r] && (uintptr_t)partials[r] % 16 == 0, "fb_peer_reduce_add: rank %d's partial or flags missing or misaligned", r);
    a.partial[r] = static_cast<const uint16_t*>(partials[r]);
    a.flags[r] = static_cast<uint32_t*>(flags[r]);
  }
  FB_REQUIRE((uintptr_t)out % 16 == 0 && (!residual || (uintptr_t)residual % 16 == 0), "fb_peer_reduce_add: misaligned out or residual");
  a.state = static_cast<uint32_t*>(state), a.residual = static_cast<const uint16_t*>(residual), a.out = static_cast<uint16_t*>(out);
  a.count = count, a.rank = rank, a.world = world;
  const int64_t chunks = count / 8;
  const unsigned blocks = (unsigned)(chunks / 256 < 1 ? 1 : chunks / 256 > 148 ? 148 : chunks / 256);
  fb::peer_reduce_add_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(a);
  return fb::launch_status("fb_peer_reduce_add");
}
