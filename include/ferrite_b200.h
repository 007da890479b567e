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
 *       mantissas  bfp8: 16 bytes at (r*64 + i)*16, byte j = sign<<7 | mag for column 16*(n/16) + j;
 *                  bfp4:  8 bytes at (r*64 + i)*8 read as two little-endian 32-bit words;
 *                         nibble p (bits 4p..4p+3) of word h holds column 8h + 2*(p%4) + p/4
 *                         of the run as the excess-8 code 8 + (sign ? -mag : mag);
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
 * M <= 4 runs as a bandwidth-bound GEMV on CUDA cores; larger M on tcgen05 tensor cores.
 * workspace: fb_linear_workspace_bytes(M, K, N) bytes of device scratch (0 / NULL when that is 0):
 * it holds the normalised activations of the RMSNorm prologue between the two kernels of a call. */
size_t fb_linear_workspace_bytes(int64_t M, int64_t K, int64_t N);
int fb_linear(int fmt, const void* x, int64_t M, int64_t K, int64_t ldx, const void* W, int64_t N, void* out,
              int out_dtype, int64_t ldo, const void* norm_w, float eps, int epilogue, const void* residual,
              int64_t ldr, void* workspace, size_t workspace_bytes, void* stream);

/* ---- the rest of a decode step ------------------------------------------------------------------------- */

/* out[i, :] = table[ids[i], :]: Tensor.gather, the embedding lookup (ferrite/tensor.py:116-126,
 * ferrite/compiler.py:1574-1580).  ids are read on the device; rows of row_bytes bytes (a multiple of 16). */
int fb_gather_rows(const void* table, int64_t table_rows, int64_t row_bytes, const int32_t* ids, int64_t n, void* out,
                   void* stream);

/* After the fused qkv matmul (models/llama.py:111-128): per head optional RMSNorm of q and k heads by
 * qk_norm[(H+KV)*hd] (Qwen3, llama.py:121-123), RoPE in Hugging Face's half-rotation form with bf16 tables
 * (llama.py:92-93, 351-368), then q heads -> q_out[T, H*hd] and the k and v heads into the cache rows
 * (Tensor.put, ferrite/tensor.py:128-140; ferrite/compiler.py:1638-1650): cache[(k heads, v heads)][rows[t]][:],
 * cache laid out [2*KV, cache_rows, hd] as models/llama.py:506-514.  cos / sin: [places, table_cols] with
 * table_cols = hd (one head's table) or (H + 2*KV)*hd (ferrite's, v's columns 1 and 0).  places[t] picks the
 * table row, rows[t] the cache row (place + the sequence's first row, llama.py:443-445). */
int fb_rope_kv_write(const void* qkv, int64_t T, int64_t ld_qkv, int H, int KV, int hd, const void* cos, const void* sin,
                     int64_t table_cols, const int32_t* places, const int32_t* rows, const void* qk_norm, float eps,
                     void* q_out, int64_t ld_q, void* cache, int64_t cache_rows, void* stream);

/* softmax(q k^T / sqrt(hd) + mask) v over the bf16 KV cache for one token per sequence: Tensor.attend
 * (ferrite/tensor.py:487-516, ferrite/compiler.py:1147-1170) as models/llama.py:129-146 uses it.  Token t reads
 * cache rows base[t] .. base[t] + place[t] of its kv head (with window > 0 only the last `window` of them);
 * its H/KV query heads share every key row read.  max_keys: an upper bound of place[t] + 1 (it sizes the split
 * of the keys across CTAs, flash-decoding; ferrite's `parts`).  hd is 64 or 128; H/KV <= 16.
 * workspace: fb_decode_attention_workspace_bytes(...) bytes (partial sums of the key splits). */
size_t fb_decode_attention_workspace_bytes(int64_t T, int H, int KV, int hd, int64_t max_keys);
int fb_decode_attention(const void* q, int64_t T, int64_t ld_q, int H, int KV, int hd, const void* cache, int64_t cache_rows,
                        const int32_t* base, const int32_t* place, int64_t max_keys, int window, void* out, int64_t ld_o,
                        void* workspace, size_t workspace_bytes, void* stream);

/* x * rsqrt(mean(x^2) + eps) * w, row by row (models/llama.py:82-85), bf16 in and out */
int fb_rmsnorm(const void* x, int64_t rows, int64_t cols, int64_t ldx, const void* w, float eps, void* out, int64_t ldo,
               void* stream);

/* greedy pick: each row's first largest fp32 logit (what models/llama.py:787-795 does on the host with argmax) */
int fb_argmax(const void* logits_f32, int64_t rows, int64_t cols, int64_t ld, int32_t* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FERRITE_B200_H */
