"""Thin typed wrappers over the C ABI: torch tensors own the device memory, every call is one or two
kernel launches on torch's current CUDA stream.  No arithmetic happens in Python or in torch here."""
import torch

from . import _lib
from ._lib import BF16, BFP4, BFP8, FP32, check, lib

_TORCH = {"bf16": torch.bfloat16, "fp32": torch.float32, "int32": torch.int32}


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


def linear_workspace(device, nbytes):
    """The device's scratch buffer for fb_linear (split-K partial tiles, tile counters, the normalised
    activations): one per device, zeroed when made (the counters start at 0 and every call leaves them 0),
    grown when a call needs more.  Calls on one stream run in order, so they can share it."""
    if not nbytes:
        return None
    have = _WORKSPACES.get(device)
    if have is None or have.numel() < nbytes:
        have = _WORKSPACES[device] = torch.zeros(max(nbytes, 64 << 20), dtype=torch.uint8, device=device)
    return have


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
    return out
