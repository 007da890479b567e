// The general half of ferrite's Tensor surface: whatever expression a model writes that is not one of the fused
// decode kernels still runs on the device, through four small kernels:
//   fb_elementwise  a fused elementwise expression over up to 8 broadcast inputs (ferrite fuses an expression tree
//                   into one kernel, ferrite/compiler.py:699-738); the expression arrives as a postfix program and
//                   every thread evaluates it on a small register stack in fp32, rounding once at the store
//   fb_reduce       sum / max along one axis (ferrite/tensor.py:359-372)
//   fb_matmul       batched matmul of bf16 / fp32 operands with arbitrary strides (a transposed B is a stride swap)
//   fb_topk, fb_touched  the router's integer kernels live in router.cu
// None of these is on the timed decode path except the router's small matmul.
#include "common.cuh"

namespace fb {

constexpr int EW_MAX_INPUTS = 8, EW_MAX_OPS = 48, EW_STACK = 12;

enum EwOp {
  EW_LOAD = 0, EW_CONST = 1,
  EW_ADD = 10, EW_SUB, EW_MUL, EW_MAX, EW_CMPLT, EW_CMPNE, EW_KEEP, EW_DROP, EW_DIV, EW_MIN,
  EW_EXP = 30, EW_LOG, EW_SIN, EW_COS, EW_SQRT, EW_RECIP, EW_RELU, EW_EXP2, EW_LOG2, EW_BF16, EW_TRUNC, EW_NEG
};

struct EwOperand {
  const void* ptr;
  int64_t s[3];  // strides in elements for (batch, row, col); 0 broadcasts
  int dtype;
};

struct EwArgs {
  EwOperand in[EW_MAX_INPUTS];
  EwOperand out;
  int64_t batch, rows, cols;
  int n_ops;
  int16_t op[EW_MAX_OPS];
  int16_t arg[EW_MAX_OPS];
  float consts[EW_MAX_OPS];
};

__device__ __forceinline__ float load_as_float(const EwOperand& o, int64_t b, int64_t r, int64_t c) {
  const int64_t at = b * o.s[0] + r * o.s[1] + c * o.s[2];
  if (o.dtype == FB_BF16) return bf16_bits_to_float(static_cast<const uint16_t*>(o.ptr)[at]);
  if (o.dtype == FB_FP32) return static_cast<const float*>(o.ptr)[at];
  return (float)static_cast<const int32_t*>(o.ptr)[at];
}

__global__ void __launch_bounds__(256) elementwise_kernel(const __grid_constant__ EwArgs a) {
  griddep_launch_dependents();
  const int64_t total = a.batch * a.rows * a.cols;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t c = i % a.cols, r = (i / a.cols) % a.rows, b = i / (a.cols * a.rows);
    float st[EW_STACK];
    int sp = 0;
    for (int k = 0; k < a.n_ops; ++k) {
      const int op = a.op[k];
      if (op == EW_LOAD) { st[sp++] = load_as_float(a.in[a.arg[k]], b, r, c); continue; }
      if (op == EW_CONST) { st[sp++] = a.consts[k]; continue; }
      if (op >= EW_EXP) {
        float x = st[sp - 1];
        switch (op) {
          case EW_EXP: x = expf(x); break;
          case EW_LOG: x = logf(x); break;
          case EW_SIN: x = sinf(x); break;
          case EW_COS: x = cosf(x); break;
          case EW_SQRT: x = sqrtf(x); break;
          case EW_RECIP: x = 1.f / x; break;
          case EW_RELU: x = fmaxf(x, 0.f); break;
          case EW_EXP2: x = exp2f(x); break;
          case EW_LOG2: x = log2f(x); break;
          case EW_BF16: x = bf16_bits_to_float(float_to_bf16_bits(x)); break;
          case EW_TRUNC: x = truncf(x); break;
          case EW_NEG: x = -x; break;
        }
        st[sp - 1] = x;
        continue;
      }
      const float y = st[--sp], x = st[sp - 1];
      float z = 0.f;
      switch (op) {
        case EW_ADD: z = x + y; break;
        case EW_SUB: z = x - y; break;
        case EW_MUL: z = x * y; break;
        case EW_DIV: z = x / y; break;
        case EW_MAX: z = fmaxf(x, y); break;
        case EW_MIN: z = fminf(x, y); break;
        case EW_CMPLT: z = x < y ? 1.f : 0.f; break;
        case EW_CMPNE: z = x != y ? 1.f : 0.f; break;
        case EW_KEEP: z = x != 0.f ? y : 0.f; break;  // y where x is set
        case EW_DROP: z = x != 0.f ? 0.f : y; break;  // y where x is not
      }
      st[sp - 1] = z;
    }
    const float v = st[0];
    const int64_t at = b * a.out.s[0] + r * a.out.s[1] + c * a.out.s[2];
    if (a.out.dtype == FB_BF16) static_cast<uint16_t*>(const_cast<void*>(a.out.ptr))[at] = (uint16_t)float_to_bf16_bits(v);
    else if (a.out.dtype == FB_FP32) static_cast<float*>(const_cast<void*>(a.out.ptr))[at] = v;
    else static_cast<int32_t*>(const_cast<void*>(a.out.ptr))[at] = (int32_t)v;
  }
}

// out[o] = fold over `len` elements `step` apart starting at in[o's place]; one warp per output element
struct ReduceArgs {
  EwOperand in, out;
  int64_t outer[3];  // the output's (batch, rows, cols)
  int64_t len, step;
  int is_max;
};
__global__ void __launch_bounds__(256) reduce_kernel(const __grid_constant__ ReduceArgs a) {
  const int64_t total = a.outer[0] * a.outer[1] * a.outer[2];
  const int64_t o = blockIdx.x * (int64_t)(blockDim.x / 32) + threadIdx.x / 32;
  if (o >= total) return;
  const int lane = threadIdx.x & 31;
  const int64_t c = o % a.outer[2], r = (o / a.outer[2]) % a.outer[1], b = o / (a.outer[2] * a.outer[1]);
  const int64_t start = b * a.in.s[0] + r * a.in.s[1] + c * a.in.s[2];
  auto value = [&](int64_t i) {
    const int64_t at = start + i * a.step;
    if (a.in.dtype == FB_BF16) return bf16_bits_to_float(static_cast<const uint16_t*>(a.in.ptr)[at]);
    if (a.in.dtype == FB_FP32) return static_cast<const float*>(a.in.ptr)[at];
    return (float)static_cast<const int32_t*>(a.in.ptr)[at];
  };
  // four loads in flight a lane (a long row is otherwise one L2 round trip per element), each with its own partial
  float part[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) part[u] = a.is_max ? -INFINITY : 0.f;
  int64_t i = lane;
  for (; i + 96 < a.len; i += 128) {
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = value(i + 32 * u);
#pragma unroll
    for (int u = 0; u < 4; ++u) part[u] = a.is_max ? fmaxf(part[u], v[u]) : part[u] + v[u];
  }
  for (; i < a.len; i += 32) part[0] = a.is_max ? fmaxf(part[0], value(i)) : part[0] + value(i);
  float acc = a.is_max ? fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])) : (part[0] + part[1]) + (part[2] + part[3]);
  acc = a.is_max ? warp_max(acc) : warp_sum(acc);
  if (lane == 0) {
    const int64_t at = b * a.out.s[0] + r * a.out.s[1] + c * a.out.s[2];
    if (a.out.dtype == FB_BF16) static_cast<uint16_t*>(const_cast<void*>(a.out.ptr))[at] = (uint16_t)float_to_bf16_bits(acc);
    else if (a.out.dtype == FB_FP32) static_cast<float*>(const_cast<void*>(a.out.ptr))[at] = acc;
    else static_cast<int32_t*>(const_cast<void*>(a.out.ptr))[at] = (int32_t)acc;
  }
}

// C[b] = A[b] @ B[b], 16 x 16 tiles through shared memory, fp32 accumulate; operands by strides
struct MatmulArgs {
  EwOperand a, b, c;  // strides (batch, row, col); a batch stride of 0 repeats the matrix
  int64_t batch, M, N, K;
};
__global__ void __launch_bounds__(256) matmul_kernel(const __grid_constant__ MatmulArgs g) {
  __shared__ float sa[16][17], sb[16][17];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t bz = blockIdx.z, row = blockIdx.y * 16 + ty, col = blockIdx.x * 16 + tx;
  float acc = 0.f;
  for (int64_t k0 = 0; k0 < g.K; k0 += 16) {
    sa[ty][tx] = row < g.M && k0 + tx < g.K ? load_as_float(g.a, bz, row, k0 + tx) : 0.f;
    sb[ty][tx] = col < g.N && k0 + ty < g.K ? load_as_float(g.b, bz, k0 + ty, col) : 0.f;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) acc = fmaf(sa[ty][k], sb[k][tx], acc);
    __syncthreads();
  }
  if (row < g.M && col < g.N) {
    const int64_t at = bz * g.c.s[0] + row * g.c.s[1] + col * g.c.s[2];
    if (g.c.dtype == FB_BF16) static_cast<uint16_t*>(const_cast<void*>(g.c.ptr))[at] = (uint16_t)float_to_bf16_bits(acc);
    else static_cast<float*>(const_cast<void*>(g.c.ptr))[at] = acc;
  }
}

// The same for a result of few elements and a long K (a router's logits: 64 x 8 over 4096): a warp per element of C
// strides over K, so that the whole GPU works on it instead of a handful of tiles walking K one after another.
__global__ void __launch_bounds__(256) matmul_skinny_kernel(const __grid_constant__ MatmulArgs g) {
  const int64_t o = blockIdx.x * (int64_t)(blockDim.x / 32) + threadIdx.x / 32;
  if (o >= g.batch * g.M * g.N) return;
  const int lane = threadIdx.x & 31;
  const int64_t col = o % g.N, row = (o / g.N) % g.M, bz = o / (g.N * g.M);
  float part[4] = {0.f, 0.f, 0.f, 0.f};
  int64_t k = lane;
  for (; k + 96 < g.K; k += 128) {
    float x[4], y[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) x[u] = load_as_float(g.a, bz, row, k + 32 * u), y[u] = load_as_float(g.b, bz, k + 32 * u, col);
#pragma unroll
    for (int u = 0; u < 4; ++u) part[u] = fmaf(x[u], y[u], part[u]);
  }
  for (; k < g.K; k += 32) part[0] = fmaf(load_as_float(g.a, bz, row, k), load_as_float(g.b, bz, k, col), part[0]);
  const float acc = warp_sum((part[0] + part[1]) + (part[2] + part[3]));
  if (lane == 0) {
    const int64_t at = bz * g.c.s[0] + row * g.c.s[1] + col * g.c.s[2];
    if (g.c.dtype == FB_BF16) static_cast<uint16_t*>(const_cast<void*>(g.c.ptr))[at] = (uint16_t)float_to_bf16_bits(acc);
    else static_cast<float*>(const_cast<void*>(g.c.ptr))[at] = acc;
  }
}

static bool fill_operand(EwOperand& o, const void* ptr, const int64_t* strides, int dtype) {
  o.ptr = ptr, o.dtype = dtype;
  for (int i = 0; i < 3; ++i) o.s[i] = strides[i];
  return ptr != nullptr && (dtype == FB_BF16 || dtype == FB_FP32 || dtype == FB_INT32);
}

}  // namespace fb

// program_host: n_ops pairs (op, arg); consts_host[k] is the value an EW_CONST at position k pushes.
// inputs_host / strides_host / dtypes_host: n_inputs device pointers, 3 strides each, dtypes.
extern "C" int fb_elementwise(int n_ops, const int32_t* program_host, const float* consts_host, int n_inputs, const void* const* inputs_host,
                              const int64_t* strides_host, const int32_t* dtypes_host, void* out, const int64_t* out_strides_host,
                              int out_dtype, int64_t batch, int64_t rows, int64_t cols, void* stream) {
  FB_REQUIRE(n_ops >= 1 && n_ops <= fb::EW_MAX_OPS && n_inputs >= 0 && n_inputs <= fb::EW_MAX_INPUTS, "fb_elementwise: %d ops over %d inputs: at most %d and %d",
             n_ops, n_inputs, fb::EW_MAX_OPS, fb::EW_MAX_INPUTS);
  FB_REQUIRE(batch >= 1 && rows >= 1 && cols >= 1 && out, "fb_elementwise: empty result");
  fb::EwArgs a{};
  for (int i = 0; i < n_inputs; ++i)
    FB_REQUIRE(fb::fill_operand(a.in[i], inputs_host[i], strides_host + 3 * i, dtypes_host[i]), "fb_elementwise: input %d: null or not bf16/fp32/int32", i);
  FB_REQUIRE(fb::fill_operand(a.out, out, out_strides_host, out_dtype), "fb_elementwise: bad output");
  int depth = 0;
  for (int k = 0; k < n_ops; ++k) {
    const int op = program_host[2 * k];
    a.op[k] = (int16_t)op, a.arg[k] = (int16_t)program_host[2 * k + 1], a.consts[k] = consts_host ? consts_host[k] : 0.f;
    depth += op <= fb::EW_CONST ? 1 : op >= fb::EW_EXP ? 0 : -1;
    FB_REQUIRE(depth >= 1 && depth <= fb::EW_STACK && (op != fb::EW_LOAD || (a.arg[k] >= 0 && a.arg[k] < n_inputs)), "fb_elementwise: malformed program at op %d", k);
  }
  FB_REQUIRE(depth == 1, "fb_elementwise: the program leaves %d values", depth);
  a.batch = batch, a.rows = rows, a.cols = cols, a.n_ops = n_ops;
  const int64_t total = batch * rows * cols;
  const unsigned blocks = (unsigned)(fb::ceil_div(total, 256) > 148 * 16 ? 148 * 16 : fb::ceil_div(total, 256));
  fb::elementwise_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(a);
  return fb::launch_status("fb_elementwise");
}

extern "C" int fb_reduce(int is_max, const void* in, const int64_t* in_strides_host, int in_dtype, int64_t batch, int64_t rows, int64_t cols,
                         int axis, void* out, const int64_t* out_strides_host, int out_dtype, void* stream) {
  FB_REQUIRE(axis >= 0 && axis <= 2 && batch >= 1 && rows >= 1 && cols >= 1, "fb_reduce: axis 0, 1 or 2 of a non-empty tensor");
  fb::ReduceArgs a{};
  FB_REQUIRE(fb::fill_operand(a.in, in, in_strides_host, in_dtype) && fb::fill_operand(a.out, out, out_strides_host, out_dtype), "fb_reduce: bad operand");
  const int64_t shape[3] = {batch, rows, cols};
  for (int i = 0; i < 3; ++i) a.outer[i] = i == axis ? 1 : shape[i];
  a.len = shape[axis], a.step = in_strides_host[axis], a.is_max = is_max;
  const int64_t total = a.outer[0] * a.outer[1] * a.outer[2];
  fb::reduce_kernel<<<(unsigned)fb::ceil_div(total, 8), 256, 0, (cudaStream_t)stream>>>(a);
  return fb::launch_status("fb_reduce");
}

extern "C" int fb_matmul(const void* a, const int64_t* a_strides_host, int a_dtype, const void* b, const int64_t* b_strides_host, int b_dtype,
                         void* c, const int64_t* c_strides_host, int c_dtype, int64_t batch, int64_t M, int64_t N, int64_t K, void* stream) {
  FB_REQUIRE(batch >= 1 && M >= 1 && N >= 1 && K >= 1 && batch <= 65535, "fb_matmul: empty or too large a batch");
  fb::MatmulArgs g{};
  FB_REQUIRE(fb::fill_operand(g.a, a, a_strides_host, a_dtype) && fb::fill_operand(g.b, b, b_strides_host, b_dtype) &&
                 fb::fill_operand(g.c, c, c_strides_host, c_dtype) && a_dtype != FB_INT32 && b_dtype != FB_INT32 && c_dtype != FB_INT32,
             "fb_matmul: operands are bf16 or fp32 (the FPU multiplies floats, ferrite/tensor.py:466)");
  g.batch = batch, g.M = M, g.N = N, g.K = K;
  dim3 grid((unsigned)fb::ceil_div(N, 16), (unsigned)fb::ceil_div(M, 16), (unsigned)batch);
  if ((int64_t)grid.x * grid.y * grid.z < 148 && K >= 512 && batch * M * N <= 148 * 64)  // few tiles, long K: a warp per element
    fb::matmul_skinny_kernel<<<(unsigned)fb::ceil_div(batch * M * N, 8), 256, 0, (cudaStream_t)stream>>>(g);
  else
    fb::matmul_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(g);
  return fb::launch_status("fb_matmul");
}
