/* ferrite_b200: C ABI of the B200 (sm_100a) decode hot path.
 *
 * This is the boundary a host binds instead of ferrite's Tensix code generator: every
 * entry point replaces one device kernel ferrite's `Tensor` launches through
 * `Runtime.launch` (ferrite/runtime.py:373-378).  The reference's own FFI is ctypes to a
 * shared library with plain integer/pointer arguments (ferrite/pci.py:19-31); this header
 * keeps that style: device pointers, sizes, a CUDA stream, an int status.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in `_host`;
 *   - `stream` is a cudaStream_t passed as void*; launches are asynchronous on it and
 *     nothing here synchronises, so a sequence of calls can be captured in a CUDA graph
 *     (the analogue of ferrite's `jit` replay, ferrite/tensor.py:788-810);
 *   - a function returns FB_OK (0) or a negative fb_status; fb_last_error() gives the
 *     reason as text (calling thread's last failure);
 *   - matrices are row-major; `bf16` means the 16-bit pattern ferrite uploads
 *     (round to nearest even, ferrite/tensor.py:56).
 *
 * Packed block-float matrix [K, N] (N a multiple of 16), format FB_BFP8 or FB_BFP4.
 * The values are exactly those of ferrite's block floats (models/gpt2.py:21-32,
 * ferrite/compiler.py:15-20,1631-1684): each run of 16 consecutive columns of one row k
 * shares the largest biased bf16 exponent of the run (`top`), every value keeps a sign and
 * a 7-bit (bfp8) or 3-bit (bfp4) magnitude, value = +-mag * 2^(top-133) (bfp4: mag*16).
 * The footprint is ferrite's too: 1088 / 576 bytes per 1024 values.  The byte ORDER is
 * this library's own (ferrite's is its 32x32 Tensix tile with 16x16 faces): a matrix is a
 * grid of UNITS of 64 rows of K x 64 columns (4 runs); rows and columns are padded with
 * zeros up to whole units (ferrite pads its tiles the same way, ferrite/tensor.py:22-24).
 *     unit (g, s) for column group g = n/64 and row step s = k/64 lies at byte
 *       (g * ceil(K/64) + s) * U,   U = 4352 (bfp8) or 2304 (bfp4);
 *     the units of one column group follow each other along K, so a stretch of K of one
 *     group is one contiguous piece of memory;
 *     inside a unit, for run r = (n/16)%4 and row i = k%64:
 *       mantissas  bfp8: 16 bytes at (r*64 + i)*16, four little-endian 32-bit words of four columns each;
 *                         in word h (columns c0..c3 = 4h..4h+3 of the run):
 *                           byte0 = mag(c0) | sign(c3)<<7   byte1 = mag(c2) | sign(c0)<<7
 *                           byte2 = mag(c1) | sign(c2)<<7   byte3 = mag(c3) | sign(c1)<<7
 *                  bfp4:  8 bytes at (r*64 + i)*8, two words of eight columns each; nibble p (bits 4p..4p+3)
 *                         = mag3(v_p) | sign(v_((p+5) mod 8))<<3 with v_p = column 2*(p%4) + p/4 of the word.
 *                  (A value's sign is parked one byte / three nibbles above its magnitude, cyclically, so a mask of
 *                  the word, or of the word rotated, is two bf16 subnormals mag * 2^-133 with their signs in place;
 *                  two exact multiplications by powers of two then give +-mag * 2^(top-133).)
 *       exponents  one byte at 4*64*(16|8) + r*64 + i.
 *   A zero magnitude is stored without a sign (as ferrite stores it).  fb_unpack_fields
 *   returns (top, sign, mag) per value for checking against the reference model.
 *   A batch of matrices (a mixture's experts) is that many packed matrices back to back,
 *   fb_packed_bytes(fmt, K, N) apart.
 */
#ifndef FERRITE_B200_H
#define FERRITE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  FB_OK = 0,
  FB_ERR_ARG = -1,     /* shape / dtype / alignment misuse: what ferrite asserts on (e.g. tensor.py:122,133-136) */
  FB_ERR_LAUNCH = -2,  /* a CUDA launch or runtime call failed */
  FB_ERR_TIMEOUT = -3, /* a bounded device wait gave up (ferrite: TimeoutError, runtime.py:466-484) */
  FB_ERR_MEMORY = -4   /* a caller-provided workspace is too small (ferrite: MemoryError, runtime.py:445) */
} fb_status;

/* dtype names follow ferrite's Tensor.dtype strings (ferrite/tensor.py:17) */
typedef enum { FB_BF16 = 0, FB_FP32 = 1, FB_INT32 = 2, FB_BFP8 = 3, FB_BFP4 = 4 } fb_dtype;

/* what a matmul fuses after its accumulation */
typedef enum {
  FB_EPI_NONE = 0,
  FB_EPI_SWIGLU = 1,   /* out[t, j] = silu(acc[t, j]) * acc[t, j + N/2]  (models/llama.py:266-275) */
  FB_EPI_RESIDUAL = 2  /* out[t, n] = residual[t, n] + acc[t, n]        (models/llama.py:107-109) */
} fb_epilogue;

int fb_version(void);
const char* fb_last_error(void);
/* Device-side waits are bounded (ferrite gives every wait a timeout, ferrite/chip.py:78-82): a wait that gives up
 * records a non-zero code here and the kernel returns.  Reads and clears it; synchronises with the device. */
int fb_status_word(void);

/* ---- block-float pack / unpack: Tensor.cast("bfp8"|"bfp4") (ferrite/tensor.py:315-320), the packer's
 * bfp8 cast (ferrite/compiler.py:52-70) and bfp4_kernel (ferrite/compiler.py:2038-2072); bit-exact with
 * the numpy model models/gpt2.py:21-32. */
size_t fb_packed_bytes(int fmt, int64_t K, int64_t N);
int fb_quantize(int fmt, const void* src_bf16, int64_t batch, int64_t K, int64_t N, void* dst_packed, void* stream);
/* packed -> bf16 values: what Tensor.tobytes gives for a block float (ferrite/tensor.py:82-107, 718-727) */
int fb_dequantize(int fmt, const void* packed, int64_t batch, int64_t K, int64_t N, void* dst_bf16, void* stream);
/* packed -> top[batch,K,N/16], sign[batch,K,N], mag[batch,K,N] (uint8 each) */
int fb_unpack_fields(int fmt, const void* packed, int64_t batch, int64_t K, int64_t N, uint8_t* top, uint8_t* sign,
                     uint8_t* mag, void* stream);

/* ---- weight matmul: Tensor.matmul with a block-float (or bf16) B (ferrite/tensor.py:443-485,
 * ferrite/compiler.py:699-738), with what models/llama.py computes around it fused in:
 *   x[M, K] bf16 (row stride ldx elements)
 *   optional RMSNorm prologue: h = x * rsqrt(mean(x^2) + eps) * norm_w[K]   (models/llama.py:82-85)
 *   acc = h @ W, fp32 accumulation, W packed [K, N] in `fmt` (FB_BFP8, FB_BFP4 or FB_BF16 row-major)
 *   epilogue (fb_epilogue), out dtype FB_BF16 or FB_FP32 (fp32: the output layer, models/llama.py:479)
 * out is [M, N] (or [M, N/2] after FB_EPI_SWIGLU), row stride ldo elements.
 * M == 1 runs as a bandwidth-bound GEMV on CUDA cores (a CTA per 16 output columns); 2..8 rows of the smaller
 * matrices on tensor-core MMAs whose weight fragments are unpacked in registers; the rest on tcgen05 tensor cores
 * (weight tiles through shared memory, accumulators in TMEM): a CTA per tile of 128 columns (clusters splitting K
 * where the tiles are few), or - with at least a tile per SM and the workspace given - one persistent CTA per SM,
 * the tiles' steps of K shared out evenly (FB_LINEAR_PERSISTENT below).
 * workspace: fb_linear_workspace_bytes(M, K, N) bytes of device scratch (0 / NULL when that is 0):
 * it holds the normalised activations of the RMSNorm prologue between the two kernels of a call, the partial sums of
 * output tiles that several CTAs share, and their arrival counters in the first 18 KB, which every call leaves zero:
 * fb_linear zeroes them itself (in stream order) the first time this process hands it a buffer; nobody else may write
 * there, and a buffer that comes back after other use has to be zeroed by the caller. */
size_t fb_linear_workspace_bytes(int64_t M, int64_t K, int64_t N);
int fb_linear(int fmt, const void* x, int64_t M, int64_t K, int64_t ldx, const void* W, int64_t N, void* out,
              int out_dtype, int64_t ldo, const void* norm_w, float eps, int epilogue, const void* residual,
              int64_t ldr, void* workspace, size_t workspace_bytes, void* stream);

/* Which kernel fb_linear runs (process-wide; for measurements that compare them - results agree within the rounding
 * stated for each).  FB_LINEAR_AUTO (the default) chooses by M as described above; FB_LINEAR_TCGEN05 and
 * FB_LINEAR_GEMV restore the choice without the register-fed kernel (GEMV up to 4 rows when asked for, else one row);
 * FB_LINEAR_MMA sends every shape the register-fed kernel supports (M <= 32, K a multiple of 16) to it, one row too.
 * FB_LINEAR_PERSISTENT runs the tcgen05 path as one persistent CTA per SM, the tiles' steps of K shared out evenly and
 * tiles that several CTAs share summed through the workspace in a fixed order (one row too).
 * FB_LINEAR_GEMV_STREAM runs one row through the streaming GEMV (persistent CTAs fed by bulk copies, each taking an equal
 * stretch of the packed matrix; the output tiles' parts meet in the workspace and are added in a fixed order) or fails
 * with FB_ERR_ARG where its rules do not hold: N a multiple of 64 (128 with SwiGLU), K up to ~13k (the token sits in shared
 * memory as fp32 beside the ring), the workspace given.  Measured slower than the plain GEMV, hence never chosen.
 * The reference has one matmul kernel and no such switch (ferrite/compiler.py:699-738). */
enum fb_linear_kernel { FB_LINEAR_AUTO = 0, FB_LINEAR_TCGEN05 = 1, FB_LINEAR_GEMV = 2, FB_LINEAR_MMA = 3, FB_LINEAR_PERSISTENT = 4, FB_LINEAR_GEMV_STREAM = 5 };
int fb_linear_prefer(int kernel);

/* fb_linear with an RMSNorm handed from the matmul that makes its input to the matmul that consumes it, so that no
 * kernel stands between the two (a decoder block's x + o_proj(...) -> rms -> gate_up, and down_proj -> next block's rms ->
 * qkv: models/llama.py:95-109, 82-85).  No counterpart in the reference, whose fused kernels are generated per tree.
 *   As producer (next_norm_w given; FB_EPI_RESIDUAL or none, out bf16): besides out, xn_out[t, n] = bf16(out[t, n] *
 *   next_norm_w[n]) (rows ld_xn apart) and sumsq_out[part * M + t] = sum over the part's columns of out[t, n]^2, one part
 *   per CTA of the launch: fb_linear_chain_parts(fmt, M, K, N, epilogue) parts (0: this shape cannot chain).
 *   As consumer (sumsq_in given): x is such an xn_out, and the accumulators are scaled by rsqrt(sum of the sumsq_in parts
 *   / K + eps) - what the RMSNorm prologue of fb_linear computes, without its pass over x.
 * A call may be both.  2 <= M <= 128; runs the tcgen05 kernel (a CTA per tile) whatever fb_linear_prefer says. */
int fb_linear_chain_parts(int fmt, int64_t M, int64_t K, int64_t N, int epilogue);
int fb_linear_chained(int fmt, const void* x, int64_t M, int64_t K, int64_t ldx, const void* W, int64_t N, void* out, int out_dtype,
                      int64_t ldo, float eps, int epilogue, const void* residual, int64_t ldr, const float* sumsq_in, int sumsq_parts,
                      const void* next_norm_w, void* xn_out, int64_t ld_xn, float* sumsq_out, void* workspace, size_t workspace_bytes,
                      void* stream);

/* Tensor.matmul(index=) (ferrite/tensor.py:450-460; ferrite/compiler.py:704-706): a mixture of experts' matmul.  W is
 * a batch of n_experts packed [K, N] matrices fb_packed_bytes(fmt, K, N) apart; index[slot] (int32, read on the
 * device, so a replayed step follows its tokens' choices) picks one for each of n_slots slots, and a slot that picks
 * none (index >= n_experts) gives zeros with nothing read.  x: [M <= 128, K] per slot, x_slot_rows rows apart (0: every
 * slot multiplies the same x).  Prologue / epilogue as fb_linear; row_scale_bf16 (optional, [n_slots, M]) multiplies
 * each result row after the epilogue: the experts' weights (models/llama.py:322-324).
 *   sum_slots = 0: one result per slot, out + slot * out_slot_stride elements (what ferrite's batch of entries is);
 *   sum_slots = 1: x is [M, n_slots * K] (slot s's activations in columns s*K..) and the slots' matmuls are summed
 *                  into one [M, N] result in the accumulators: the experts' down projections and their sum over
 *                  the entries (llama.py:324 `.sum(0)`) in one kernel. */
int fb_linear_indexed(int fmt, const void* x, int64_t M, int64_t K, int64_t ldx, int64_t x_slot_rows, const void* W, int64_t N,
                      int n_experts, const int32_t* index, int n_slots, int sum_slots, void* out, int out_dtype, int64_t ldo,
                      int64_t out_slot_stride, const void* norm_w, float eps, int epilogue, const void* residual, int64_t ldr,
                      const void* row_scale_bf16, void* workspace, size_t workspace_bytes, void* stream);

/* ---- the rest of a decode step ------------------------------------------------------------------------- */

/* out[i, :] = table[ids[i], :]: Tensor.gather, the embedding lookup (ferrite/tensor.py:116-126,
 * ferrite/compiler.py:1574-1580).  ids are read on the device (an id outside the table is clamped into it); rows of
 * row_bytes bytes (even; whole 16-byte pieces at 16-byte aligned addresses go 16 bytes at a time). */
int fb_gather_rows(const void* table, int64_t table_rows, int64_t row_bytes, const int32_t* ids, int64_t n, void* out,
                   void* stream);

/* dst[b, ids[i], :] = src[b, i, :] for every matrix b: Tensor.put, gather's inverse (ferrite/tensor.py:128-140,
 * ferrite/compiler.py:1638-1650); of rows put at the same place the later one stays.  Strides in elements. */
int fb_put_rows(void* dst, int64_t ds0, int64_t ds1, int64_t ds2, const void* src, int64_t ss0, int64_t ss1, int64_t ss2,
                const int32_t* ids, int64_t batch, int64_t n, int64_t cols, int64_t dst_rows, int elem_bytes, void* stream);

/* After the fused qkv matmul (models/llama.py:111-128): per head optional RMSNorm of q and k heads by
 * qk_norm[(H+KV)*hd] (Qwen3, llama.py:121-123), RoPE in Hugging Face's half-rotation form with bf16 tables
 * (llama.py:92-93, 351-368), then q heads -> q_out[T, H*hd] and the k and v heads into the cache rows
 * (Tensor.put, ferrite/tensor.py:128-140; ferrite/compiler.py:1638-1650): cache[(k heads, v heads)][rows[t]][:],
 * cache laid out [2*KV, cache_rows, hd] as models/llama.py:506-514.  cos / sin: [places, table_cols] with
 * table_cols = hd (one head's table) or (H + 2*KV)*hd (ferrite's, v's columns 1 and 0).  places[t] picks the
 * table row (clamped into the table's table_rows rows), rows[t] the cache row (place + the sequence's first row,
 * llama.py:443-445; a row outside 0 .. cache_rows-1 is not written: ferrite checks neither, nothing here reads or
 * writes outside what it was given).  cache_head_stride: elements
 * from one head's rows to the next's (cache_rows * hd, or more when the cache is one sequence's part of a larger one,
 * models/llama.py:520-526). */
int fb_rope_kv_write(const void* qkv, int64_t T, int64_t ld_qkv, int H, int KV, int hd, const void* cos, const void* sin,
                     int64_t table_cols, int64_t table_rows, const int32_t* places, const int32_t* rows, const void* qk_norm, float eps,
                     void* q_out, int64_t ld_q, void* cache, int64_t cache_rows, int64_t cache_head_stride, void* stream);

/* softmax(q k^T / sqrt(hd) + mask) v over the bf16 KV cache for one token per sequence: Tensor.attend
 * (ferrite/tensor.py:487-516, ferrite/compiler.py:1147-1170) as models/llama.py:129-146 uses it.  Token t reads
 * cache rows base[t] .. base[t] + place[t] of its kv head (with window > 0 only the last `window` of them);
 * its H/KV query heads share every key row read.  max_keys: an upper bound of place[t] + 1 (it sizes the split
 * of the keys across CTAs, flash-decoding; ferrite's `parts`).  hd is 64 or 128; H/KV <= 16.
 * workspace: fb_decode_attention_workspace_bytes(...) bytes (partial sums of the key splits). */
size_t fb_decode_attention_workspace_bytes(int64_t T, int H, int KV, int hd, int64_t max_keys);
int fb_decode_attention(const void* q, int64_t T, int64_t ld_q, int H, int KV, int hd, const void* cache, int64_t cache_rows,
                        int64_t cache_head_stride, const int32_t* base, const int32_t* place, int64_t max_keys, int window, void* out, int64_t ld_o,
                        void* workspace, size_t workspace_bytes, void* stream);

/* The same two calls over a block-float KV cache (a cache in bfp8 or bfp4: models/llama.py:80,127-128; Tensor.put into a
 * block-float tensor, ferrite/compiler.py:1648-1662; pinned by test/test_sim.py:2081-2107): cache_packed holds 2 KV packed
 * matrices [cache_rows, hd] (fb_packed_bytes each), the keys' heads then the values'.  fb_rope_kv_write_packed rounds
 * each run of 16 of a new row exactly as fb_quantize does; fb_decode_attention_packed unpacks the rows it reads to the
 * same bf16 values a bf16 cache would hold and then computes what fb_decode_attention computes, bit for bit.
 * base[t] (a sequence's first cache row) must be a multiple of 64: a sequence's rows start a packed unit. */
int fb_rope_kv_write_packed(int cache_fmt, const void* qkv, int64_t T, int64_t ld_qkv, int H, int KV, int hd, const void* cos, const void* sin,
                            int64_t table_cols, int64_t table_rows, const int32_t* places, const int32_t* rows, const void* qk_norm, float eps, void* q_out,
                            int64_t ld_q, void* cache_packed, int64_t cache_rows, void* stream);
int fb_decode_attention_packed(int cache_fmt, const void* q, int64_t T, int64_t ld_q, int H, int KV, int hd, const void* cache_packed,
                               int64_t cache_rows, const int32_t* base, const int32_t* place, int64_t max_keys, int window, void* out,
                               int64_t ld_o, void* workspace, size_t workspace_bytes, void* stream);

/* The same attention for a chunk of ONE sequence's prompt (models/llama.py:498-504, forward over a prompt's tokens at
 * once): T tokens at places[t], their keys and values already in the cache rows first_row + place, each token seeing
 * the sequence's keys 0 .. place[t].  A query head's tokens are taken 16 to a CTA, so a key row is read once per 16
 * tokens of a head.  cache_fmt: FB_BF16 (cache as fb_decode_attention takes it) or FB_BFP8 / FB_BFP4 (as
 * fb_decode_attention_packed; first_row a multiple of 64).  max_keys: an upper bound of place[t] + 1. */
size_t fb_prefill_attention_workspace_bytes(int64_t T, int H, int hd, int64_t max_keys);
int fb_prefill_attention(int cache_fmt, const void* q, int64_t T, int64_t ld_q, int H, int KV, int hd, const void* cache, int64_t cache_rows,
                         int64_t cache_head_stride, int64_t first_row, const int32_t* places, int64_t max_keys, int window, void* out,
                         int64_t ld_o, void* workspace, size_t workspace_bytes, void* stream);

/* fb_decode_attention for callers that cannot provide a workspace and must not have one allocated for them (a
 * process whose own pool owns all device memory, a binding with no way to hold a scratch buffer).  It has no
 * counterpart in the reference.  The partial sums of the key splits go into an array built into the library
 * (fb_decode_attention_static_max_bytes() bytes of every GPU that loads it, from load to exit); a call that would
 * need more is refused with FB_ERR_ARG and a message.  No memory is allocated or freed by this call, ever.
 * The first call on a device looks up the array's device address: make that call outside any stream capture.
 * All calls on a device share the array and it keeps the last call's contents; nothing in it needs clearing, but
 * calls that overlap on the GPU (different streams) race on it: keep them on one stream. */
size_t fb_decode_attention_static_max_bytes(void);
int fb_decode_attention_static(const void* q, int64_t T, int64_t ld_q, int H, int KV, int hd, const void* cache, int64_t cache_rows,
                               int64_t cache_head_stride, const int32_t* base, const int32_t* place, int64_t max_keys, int window,
                               void* out, int64_t ld_o, void* stream);

/* The same kernel in ferrite's general form, Tensor.attend (ferrite/tensor.py:487-516): `entries` batch entries of
 * `rows` query rows [rows, hd] (strides in elements), every kv_rep consecutive entries reading one key and one value
 * matrix [keys, hd] (a repeat_interleave read in place, ferrite/tensor.py:210-217), and an int32 place per row
 * (place_row_stride 0: one place for all rows of an entry; place_entry_stride 0: one column of places for all
 * entries): a row sees keys 0..place (the last `window` of them).  Scores are scaled by `scale`.  out: [entries, rows, hd]. */
size_t fb_attend_workspace_bytes(int64_t entries, int64_t rows, int hd, int64_t max_keys);
int fb_attend(const void* q, int64_t entries, int64_t rows, int hd, int64_t q_entry_stride, int64_t q_row_stride, const void* k,
              const void* v, int64_t kv_entry_stride, int64_t kv_rep, int64_t keys, const int32_t* places,
              int64_t place_entry_stride, int64_t place_row_stride, int window, float scale, void* out, void* workspace,
              size_t workspace_bytes, void* stream);

/* x * rsqrt(mean(x^2) + eps) * w, row by row (models/llama.py:82-85), bf16 in and out */
int fb_rmsnorm(const void* x, int64_t rows, int64_t cols, int64_t ldx, const void* w, float eps, void* out, int64_t ldo,
               void* stream);

/* greedy pick: each row's first largest fp32 logit (what models/llama.py:787-795 does on the host with argmax);
 * out_value (optional): the maxima, for picking across vocabulary shards */
int fb_argmax(const void* logits_f32, int64_t rows, int64_t cols, int64_t ld, int32_t* out, float* out_value, void* stream);

/* ---- the mixture-of-experts router (models/llama.py:277-292) ------------------------------------------- */

/* Tensor.topk (ferrite/tensor.py:373-388, ferrite/compiler.py:1716-1731): each row's k <= 64 largest, largest first,
 * the lower column first among equals, -0 equal to 0, compared exactly as stored (dtype FB_BF16 or FB_FP32): the
 * order of numpy's stable argsort (models/llama.py:27).  values (x's dtype) and ids: [rows, k] with row stride ldo;
 * labels (optional, shaped like x): what to report instead of a pick's column.  softmax_weights_bf16 (optional,
 * [rows, k]): the softmax of each row's picked values, the experts' weights (llama.py:287-288). */
int fb_topk(int dtype, const void* x, int64_t rows, int64_t cols, int64_t ldx, int k, const int32_t* labels, void* values,
            int32_t* ids, void* softmax_weights_bf16, int64_t ldo, void* stream);

/* Tensor.touched (ferrite/tensor.py:403-416, ferrite/compiler.py:1898-1905): from ids and bf16 weights [rows, k]
 * (experts below n), experts[min(rows*k, n)]: those some row picks by a weight that is not 0, ascending, then n
 * ("none"); out_bf16[entry, row]: the row's weight for that entry's expert, 0 where it did not pick it.
 * first (0 for the reference's behaviour): experts are counted from it - a rank holding experts first .. first+n-1 of
 * a mixture spread over several GPUs lists only those, numbered from 0, and ignores the picks of other ranks' experts. */
int fb_touched(const int32_t* ids, const void* weights_bf16, int64_t rows, int k, int n, int first, int32_t* experts, void* out_bf16,
               void* stream);

/* Tensor.group (ferrite/tensor.py:389-402, ferrite/compiler.py:1842-1896): a mixture's tokens grouped by expert, from
 * int32 choices [rows, k] (values below n; others are left out).  With t = ceil(rows*k / 32) + min(n, rows*k) tiles of
 * 32 slots and rp = rows rounded up to 32:  order[32 t]: the row each slot holds (0 for none), each value's choices a
 * run of whole tiles, in the choices' own order;  tiles[t]: each tile's value (n past those used: "none" to a matmul
 * that picks by them);  places[k * rp]: run j holds, for each row, the slot of its choice j.  One kernel. */
int fb_group(const int32_t* ids, int64_t rows, int k, int n, int32_t* order, int32_t* tiles, int32_t* places, void* stream);

/* ---- the general operator surface (ferrite/tensor.py:292-372, 443-485), for expressions that are not one of the
 * fused kernels above.  Strides are in elements for (batch, row, col); a stride of 0 broadcasts.  *_host arguments
 * are host arrays read during the call. */

/* One fused elementwise expression (ferrite fuses a tree into one kernel, ferrite/compiler.py:699-738).  The
 * expression is a postfix program of n_ops (op, arg) pairs: op 0 pushes input `arg`, op 1 pushes consts_host[position];
 * 10.. are binary (add sub mul max cmplt cmpne keep drop div min), 30.. unary (exp log sin cos sqrt recip relu exp2
 * log2 round-to-bf16 trunc neg).  Computed in fp32, rounded once at the store. */
int fb_elementwise(int n_ops, const int32_t* program_host, const float* consts_host, int n_inputs, const void* const* inputs_host,
                   const int64_t* strides_host, const int32_t* dtypes_host, void* out, const int64_t* out_strides_host,
                   int out_dtype, int64_t batch, int64_t rows, int64_t cols, void* stream);

/* sum or max along one axis, kept as 1 (Tensor.sum / Tensor.max, ferrite/tensor.py:359-368) */
int fb_reduce(int is_max, const void* in, const int64_t* in_strides_host, int in_dtype, int64_t batch, int64_t rows, int64_t cols,
              int axis, void* out, const int64_t* out_strides_host, int out_dtype, void* stream);

/* C[b] = A[b] @ B[b] for bf16 / fp32 operands by strides (a transposed B is a stride swap, a batch stride of 0
 * repeats a matrix): Tensor.matmul without a block-float B (ferrite/tensor.py:443-485); fp32 accumulation. */
int fb_matmul(const void* a, const int64_t* a_strides_host, int a_dtype, const void* b, const int64_t* b_strides_host, int b_dtype,
              void* c, const int64_t* c_strides_host, int c_dtype, int64_t batch, int64_t M, int64_t N, int64_t K, void* stream);

/* ---- several GPUs -------------------------------------------------------------------------------------- */

/* out = residual + sum over the ranks of their partials, bf16 [count], one kernel per rank reading the other ranks'
 * partials out of their memory over NVLink (plain peer loads).  No counterpart in the reference, which drives one chip
 * (ferrite/runtime.py:304-311); it stands where a tensor-parallel block all-reduces o_proj's / down_proj's / the
 * experts' partial sums and adds the residual (models/llama.py:95-109).
 * partials[r], flags[r]: HOST arrays of `world` device addresses, valid on this GPU, of rank r's partial for this call
 * site and of rank r's flag words (`world` uint32, zero before the first call); every rank passes the same buffers in
 * the same order and makes the same sequence of calls.  state: 4 uint32 of this GPU, zero before the first call
 * ([0] counts the calls; [2] holds 201 + r after a bounded wait for rank r gave up, else 0; [3]: the wait's bound in
 * clock cycles, 0 for the default of about two seconds).  The partial of a call site may be overwritten once a later
 * call has passed its wait (every rank has then finished reading it).  count: a multiple of 8.
 * All ranks add in rank order, so their results are bit-identical. */
int fb_peer_reduce_add(const void* const* partials, void* const* flags, int rank, int world, void* state, int64_t count,
                       const void* residual, void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FERRITE_B200_H */
