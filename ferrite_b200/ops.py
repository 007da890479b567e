"""Thin typed wrappers over the C ABI: torch tensors own the device memory, every call is one or two
kernel launches on torch's current CUDA stream.  No arithmetic happens in Python or in torch here."""
import torch

from . import _lib
from ._lib import BF16, BFP4, BFP8, FP32, check, lib

_TORCH = {"bf16": torch.bfloat16, "fp32": torch.float32, "int32": torch.int32}

KERNELS = [0]  # kernels of this library launched so far by this process (every wrapper below counts its own)


def count(n=1):
    KERNELS[0] += n


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


class Packed:
    """A batch of block-float matrices [batch, K, N] on the device (include/ferrite_b200.h says how the bytes lie)."""

    def __init__(self, fmt, batch, K, N, data):
        self.fmt, self.batch, self.K, self.N, self.data = fmt, batch, K, N, data

    @property
    def code(self):
        return _lib.DTYPES[self.fmt]

    @property
    def matrix_bytes(self):
        return lib().fb_packed_bytes(self.code, self.K, self.N)

    def matrix(self, e):
        """Matrix e of the batch, in place."""
        n = self.matrix_bytes
        return Packed(self.fmt, 1, self.K, self.N, self.data[e * n:(e + 1) * n])


def quantize(x, fmt):
    """bf16 [K, N] or [batch, K, N] -> Packed (Tensor.cast to a block float, ferrite/tensor.py:315-320)."""
    assert x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous(), "a contiguous bf16 CUDA tensor"
    batch, K, N = (1, *x.shape) if x.dim() == 2 else x.shape
    n = lib().fb_packed_bytes(_lib.DTYPES[fmt], K, N)
    assert n, f"{tuple(x.shape)} to {fmt}: columns in runs of 16"
    data = torch.empty(batch * n, dtype=torch.uint8, device=x.device)
    check(lib().fb_quantize(_lib.DTYPES[fmt], x.data_ptr(), batch, K, N, data.data_ptr(), _stream()))
    count()
    return Packed(fmt, batch, K, N, data)


def dequantize(p):
    """Packed -> bf16 [batch, K, N]: the values, each exactly a bf16."""
    out = torch.empty(p.batch, p.K, p.N, dtype=torch.bfloat16, device=p.data.device)
    check(lib().fb_dequantize(p.code, p.data.data_ptr(), p.batch, p.K, p.N, out.data_ptr(), _stream()))
    return out


def unpack_fields(p):
    """Packed -> (top [batch,K,N/16], sign [batch,K,N], mag [batch,K,N]) uint8."""
    dev = p.data.device
    top = torch.empty(p.batch, p.K, p.N // 16, dtype=torch.uint8, device=dev)
    sign = torch.empty(p.batch, p.K, p.N, dtype=torch.uint8, device=dev)
    mag = torch.empty_like(sign)
    check(lib().fb_unpack_fields(p.code, p.data.data_ptr(), p.batch, p.K, p.N, top.data_ptr(), sign.data_ptr(), mag.data_ptr(), _stream()))
    return top, sign, mag


_WORKSPACES = {}
_RETIRED = []  # scratch buffers a larger one has replaced: a recorded CUDA graph may still hold their addresses


def _scratch(table, device, nbytes, least):
    """The device's buffer of one kind of scratch: zeroed when made, replaced by a larger one when a call needs more.
    The one it replaces is kept alive for good: a step recorded by `jit` replays kernels that were given its address."""
    have = table.get(device)
    if have is None or have.numel() < nbytes:
        if have is not None:
            _RETIRED.append(have)
        have = table[device] = torch.zeros(max(nbytes, least), dtype=torch.uint8, device=device)
    return have


def linear_workspace(device, nbytes):
    """The device's scratch buffer for fb_linear (the normalised activations of a fused RMSNorm, the partial tiles and
    arrival counters of tiles shared by several CTAs): one per device, zeroed when made (the counters start at 0 and
    every call leaves them 0).  Calls on one stream run in order, so they can share it."""
    return _scratch(_WORKSPACES, device, nbytes, 64 << 20) if nbytes else None


def linear(x, w, out=None, out_dtype="bf16", norm_w=None, eps=1e-5, epilogue="none", residual=None, workspace=None):
    """x [M, K] bf16 @ w (Packed, one matrix) with the fused RMSNorm prologue / SwiGLU or residual epilogue."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and w.batch == 1 and x.shape[1] == w.K, \
        f"{tuple(x.shape)} @ [{w.K}, {w.N}]"
    M, K = x.shape
    epi = {"none": _lib.EPI_NONE, "swiglu": _lib.EPI_SWIGLU, "residual": _lib.EPI_RESIDUAL}[epilogue]
    cols = w.N // 2 if epilogue == "swiglu" else w.N
    if out is None:
        out = torch.empty(M, cols, dtype=_TORCH[out_dtype], device=x.device)
    assert out.shape == (M, cols) and out.stride(1) == 1 and out.dtype == _TORCH[out_dtype]
    if workspace is None:
        workspace = linear_workspace(x.device, lib().fb_linear_workspace_bytes(M, K, w.N))
    check(lib().fb_linear(w.code, x.data_ptr(), M, K, x.stride(0), w.data.data_ptr(), w.N, out.data_ptr(), _lib.DTYPES[out_dtype],
                          out.stride(0), _ptr(norm_w), eps, epi, _ptr(residual), residual.stride(0) if residual is not None else 0,
                          _ptr(workspace), workspace.numel() if workspace is not None else 0, _stream()))
    count(1 if M <= 1 else -(-M // 128) * (2 if norm_w is not None else 1))  # the GEMV, or GEMM passes (+ the norm's)
    return out


def chain_parts(w, M, epilogue="none"):
    """How many parts the sums of squares of fb_linear_chained's result come in for this shape; 0: it cannot hand a norm on."""
    epi = {"none": _lib.EPI_NONE, "swiglu": _lib.EPI_SWIGLU, "residual": _lib.EPI_RESIDUAL}[epilogue]
    return lib().fb_linear_chain_parts(w.code, M, w.K, w.N, epi)


def linear_chained(x, w, out=None, out_dtype="bf16", eps=1e-5, epilogue="none", residual=None, norm_in=None, next_norm_w=None):
    """fb_linear_chained: x @ w with an RMSNorm taken over from the matmul before (norm_in = (sumsq, parts): x is that
    matmul's xn) and / or handed on to the one after (next_norm_w: returns (out, xn, sumsq, parts) instead of out)."""
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and w.batch == 1 and x.shape[1] == w.K
    M = x.shape[0]
    epi = {"none": _lib.EPI_NONE, "swiglu": _lib.EPI_SWIGLU, "residual": _lib.EPI_RESIDUAL}[epilogue]
    cols = w.N // 2 if epilogue == "swiglu" else w.N
    if out is None:
        out = torch.empty(M, cols, dtype=_TORCH[out_dtype], device=x.device)
    xn = sumsq = None
    parts = 0
    if next_norm_w is not None:
        parts = chain_parts(w, M, epilogue)
        assert parts, "this shape cannot hand a norm on"
        xn = torch.empty(M, w.N, dtype=torch.bfloat16, device=x.device)
        sumsq = torch.empty(parts, M, dtype=torch.float32, device=x.device)
    check(lib().fb_linear_chained(w.code, x.data_ptr(), M, w.K, x.stride(0), w.data.data_ptr(), w.N, out.data_ptr(), _lib.DTYPES[out_dtype], out.stride(0),
                                  eps, epi, _ptr(residual), residual.stride(0) if residual is not None else 0,
                                  _ptr(norm_in[0]) if norm_in else None, norm_in[1] if norm_in else 0, _ptr(next_norm_w), _ptr(xn),
                                  xn.stride(0) if xn is not None else 0, _ptr(sumsq), None, 0, _stream()))
    count()
    return (out, xn, sumsq, parts) if next_norm_w is not None else out


def gather_rows(table, ids, out=None):
    """table[ids] for a 2-D table and an int32 vector of ids on the device (Tensor.gather)."""
    assert table.dim() == 2 and table.is_contiguous() and ids.dtype == torch.int32 and ids.dim() == 1
    if out is None:
        out = torch.empty(ids.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    check(lib().fb_gather_rows(table.data_ptr(), table.shape[0], table.shape[1] * table.element_size(), ids.data_ptr(), ids.numel(),
                               out.data_ptr(), _stream()))
    count()
    return out


def rope_kv_write(qkv, cos, sin, places, rows, cache, H, KV, hd, q_out=None, qk_norm=None, eps=1e-5):
    """RoPE (and Qwen3's q/k norm) on a fused qkv [T, (H+2KV)*hd]; q -> q_out [T, H*hd], k and v into cache
    [2*KV, cache_rows, hd] at rows (a bf16 tensor, or a Packed block-float batch of 2*KV matrices [cache_rows, hd])."""
    T = qkv.shape[0]
    assert qkv.dtype == torch.bfloat16 and qkv.shape[1] == (H + 2 * KV) * hd and qkv.stride(1) == 1
    if isinstance(cache, Packed):
        assert cache.batch == 2 * KV and cache.N == hd and places.dtype == torch.int32 and rows.dtype == torch.int32
        if q_out is None:
            q_out = torch.empty(T, H * hd, dtype=torch.bfloat16, device=qkv.device)
        check(lib().fb_rope_kv_write_packed(cache.code, qkv.data_ptr(), T, qkv.stride(0), H, KV, hd, cos.data_ptr(), sin.data_ptr(), cos.shape[-1],
                                            cos.shape[0], places.data_ptr(), rows.data_ptr(), _ptr(qk_norm), eps, q_out.data_ptr(), q_out.stride(0),
                                            cache.data.data_ptr(), cache.K, _stream()))
        count()
        return q_out
    assert cache.dtype == torch.bfloat16 and cache.shape[0] == 2 * KV and cache.shape[2] == hd and cache.stride(2) == 1 and cache.stride(1) == hd
    assert places.dtype == torch.int32 and rows.dtype == torch.int32 and places.numel() == T and rows.numel() == T
    assert cos.shape == sin.shape and cos.is_contiguous() and sin.is_contiguous() and cos.dtype == torch.bfloat16
    if q_out is None:
        q_out = torch.empty(T, H * hd, dtype=torch.bfloat16, device=qkv.device)
    check(lib().fb_rope_kv_write(qkv.data_ptr(), T, qkv.stride(0), H, KV, hd, cos.data_ptr(), sin.data_ptr(), cos.shape[-1], cos.shape[0], places.data_ptr(),
                                 rows.data_ptr(), _ptr(qk_norm), eps, q_out.data_ptr(), q_out.stride(0), cache.data_ptr(), cache.shape[1], cache.stride(0), _stream()))
    count()
    return q_out


_ATT_WS = {}


def decode_attention(q, cache, base, place, H, KV, hd, max_keys, window=0, out=None):
    """One token per sequence: token t attends cache rows base[t] .. base[t] + place[t] of its kv head."""
    T = q.shape[0]
    packed = isinstance(cache, Packed)  # a block-float cache: sequences start at multiples of 64 rows (base)
    assert q.dtype == torch.bfloat16 and q.shape[1] == H * hd and q.stride(1) == 1
    assert (cache.batch == 2 * KV and cache.N == hd) if packed else (cache.stride(2) == 1 and cache.stride(1) == hd)
    assert base.dtype == torch.int32 and place.dtype == torch.int32 and base.numel() == T and place.numel() == T
    if out is None:
        out = torch.empty(T, H * hd, dtype=torch.bfloat16, device=q.device)
    need = lib().fb_decode_attention_workspace_bytes(T, H, KV, hd, max_keys)
    ws = attention_workspace(q.device, need)
    if packed:
        check(lib().fb_decode_attention_packed(cache.code, q.data_ptr(), T, q.stride(0), H, KV, hd, cache.data.data_ptr(), cache.K, base.data_ptr(),
                                               place.data_ptr(), max_keys, window, out.data_ptr(), out.stride(0), _ptr(ws) if need else None,
                                               ws.numel() if need else 0, _stream()))
    else:
        check(lib().fb_decode_attention(q.data_ptr(), T, q.stride(0), H, KV, hd, cache.data_ptr(), cache.shape[1], cache.stride(0), base.data_ptr(),
                                        place.data_ptr(), max_keys, window, out.data_ptr(), out.stride(0), _ptr(ws) if need else None,
                                        ws.numel() if need else 0, _stream()))
    count(2 if need else 1)  # the attention kernel, and the merge of its key splits
    return out


def prefill_attention(q, cache, first_row, places, H, KV, hd, max_keys, window=0, out=None):
    """A chunk of one sequence's prompt: token t (at places[t]) attends the cache rows first_row .. first_row + places[t]
    of its kv head; 16 tokens of a query head share every key row read."""
    T = q.shape[0]
    packed = isinstance(cache, Packed)
    assert q.dtype == torch.bfloat16 and q.shape[1] == H * hd and q.stride(1) == 1 and places.dtype == torch.int32 and places.numel() == T
    assert (cache.batch == 2 * KV and cache.N == hd) if packed else (cache.stride(2) == 1 and cache.stride(1) == hd)
    if out is None:
        out = torch.empty(T, H * hd, dtype=torch.bfloat16, device=q.device)
    need = lib().fb_prefill_attention_workspace_bytes(T, H, hd, max_keys)
    ws = attention_workspace(q.device, need)
    check(lib().fb_prefill_attention(cache.code if packed else BF16, q.data_ptr(), T, q.stride(0), H, KV, hd, cache.data.data_ptr() if packed else cache.data_ptr(),
                                     cache.K if packed else cache.shape[1], 0 if packed else cache.stride(0), first_row, places.data_ptr(), max_keys, window,
                                     out.data_ptr(), out.stride(0), _ptr(ws) if need else None, ws.numel() if need else 0, _stream()))
    count(2 if need else 1)
    return out


def rmsnorm(x, w, eps=1e-5, out=None):
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and w.numel() == x.shape[1]
    if out is None:
        out = torch.empty_like(x)
    check(lib().fb_rmsnorm(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), w.data_ptr(), eps, out.data_ptr(), out.stride(0), _stream()))
    count()
    return out


def argmax(logits, out=None, values=None):
    """Each row's first largest fp32 logit's column (int32); values: an fp32 vector that receives the maxima."""
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1
    if out is None:
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    check(lib().fb_argmax(logits.data_ptr(), logits.shape[0], logits.shape[1], logits.stride(0), out.data_ptr(), _ptr(values), _stream()))
    count()
    return out


def attention_workspace(device, nbytes):
    """The device's scratch for the attention kernels' key splits (a larger one replaces it when a call needs more;
    the replaced one stays alive for the recorded steps that hold its address)."""
    return _scratch(_ATT_WS, device, nbytes, 16 << 20) if nbytes else None


def linear_indexed(x, w, index, out, sum_slots=False, x_slot_rows=0, out_slot_stride=0, M=None, out_dtype="bf16", norm_w=None, eps=1e-5,
                   epilogue="none", residual=None, row_scale=None):
    """A mixture of experts' matmul: x [M, K] (or n_slots of them, or [M, n_slots * K] with sum_slots) by the matrices
    of the batch w (Packed) that index (int32 [n_slots], on the device) picks; see fb_linear_indexed."""
    M = x.shape[0] if M is None else M
    n_slots = index.numel()
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and index.dtype == torch.int32 and index.is_contiguous()
    epi = {"none": _lib.EPI_NONE, "swiglu": _lib.EPI_SWIGLU, "residual": _lib.EPI_RESIDUAL}[epilogue]
    ws = linear_workspace(x.device, lib().fb_linear_workspace_bytes(max(M, 5), w.K, w.N)) if norm_w is not None else None
    check(lib().fb_linear_indexed(w.code, x.data_ptr(), M, w.K, x.stride(0), x_slot_rows, w.data.data_ptr(), w.N, w.batch, index.data_ptr(), n_slots,
                                  int(sum_slots), out.data_ptr(), _lib.DTYPES[out_dtype], out.stride(-2), out_slot_stride, _ptr(norm_w), eps, epi,
                                  _ptr(residual), residual.stride(0) if residual is not None else 0, _ptr(row_scale), _ptr(ws),
                                  ws.numel() if ws is not None else 0, _stream()))
    count(2 if norm_w is not None else 1)
    return out
