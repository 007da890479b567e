"""ctypes binding of include/ferrite_b200.h.

The shared library is the product's only compute path: if it is missing this module raises (there is
no CPU or PyTorch fallback).  Build it with `python -m ferrite_b200.build` (needs nvcc).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libferrite_b200.so")

BF16, FP32, INT32, BFP8, BFP4 = 0, 1, 2, 3, 4
DTYPES = {"bf16": BF16, "fp32": FP32, "int32": INT32, "bfp8": BFP8, "bfp4": BFP4}
EPI_NONE, EPI_SWIGLU, EPI_RESIDUAL = 0, 1, 2
LINEAR_AUTO, LINEAR_TCGEN05, LINEAR_GEMV, LINEAR_MMA, LINEAR_PERSISTENT, LINEAR_GEMV_STREAM = 0, 1, 2, 3, 4, 5  # fb_linear_prefer

_p, _i, _i64, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_size_t

# name -> (restype, argtypes); one entry per declaration in include/ferrite_b200.h
SIGNATURES = {
    "fb_version": (_i, []),
    "fb_last_error": (ctypes.c_char_p, []),
    "fb_status_word": (_i, []),
    "fb_packed_bytes": (_sz, [_i, _i64, _i64]),
    "fb_quantize": (_i, [_i, _p, _i64, _i64, _i64, _p, _p]),
    "fb_dequantize": (_i, [_i, _p, _i64, _i64, _i64, _p, _p]),
    "fb_unpack_fields": (_i, [_i, _p, _i64, _i64, _i64, _p, _p, _p, _p]),
    "fb_linear_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "fb_linear_prefer": (_i, [_i]),
    "fb_linear": (_i, [_i, _p, _i64, _i64, _i64, _p, _i64, _p, _i, _i64, _p, _f, _i, _p, _i64, _p, _sz, _p]),
    "fb_linear_chain_parts": (_i, [_i, _i64, _i64, _i64, _i]),
    "fb_linear_chained": (_i, [_i, _p, _i64, _i64, _i64, _p, _i64, _p, _i, _i64, _f, _i, _p, _i64, _p, _i, _p, _p, _i64, _p, _p, _sz, _p]),
    "fb_linear_indexed": (_i, [_i, _p, _i64, _i64, _i64, _i64, _p, _i64, _i, _p, _i, _i, _p, _i, _i64, _i64, _p, _f, _i, _p, _i64, _p, _p, _sz, _p]),
    "fb_gather_rows": (_i, [_p, _i64, _i64, _p, _i64, _p, _p]),
    "fb_put_rows": (_i, [_p, _i64, _i64, _i64, _p, _i64, _i64, _i64, _p, _i64, _i64, _i64, _i64, _i, _p]),
    "fb_rope_kv_write": (_i, [_p, _i64, _i64, _i, _i, _i, _p, _p, _i64, _i64, _p, _p, _p, _f, _p, _i64, _p, _i64, _i64, _p]),
    "fb_decode_attention_workspace_bytes": (_sz, [_i64, _i, _i, _i, _i64]),
    "fb_decode_attention": (_i, [_p, _i64, _i64, _i, _i, _i, _p, _i64, _i64, _p, _p, _i64, _i, _p, _i64, _p, _sz, _p]),
    "fb_decode_attention_static_max_bytes": (_sz, []),
    "fb_decode_attention_static": (_i, [_p, _i64, _i64, _i, _i, _i, _p, _i64, _i64, _p, _p, _i64, _i, _p, _i64, _p]),
    "fb_prefill_attention_workspace_bytes": (_sz, [_i64, _i, _i, _i64]),
    "fb_prefill_attention": (_i, [_i, _p, _i64, _i64, _i, _i, _i, _p, _i64, _i64, _i64, _p, _i64, _i, _p, _i64, _p, _sz, _p]),
    "fb_attend_workspace_bytes": (_sz, [_i64, _i64, _i, _i64]),
    "fb_attend": (_i, [_p, _i64, _i64, _i, _i64, _i64, _p, _p, _i64, _i64, _i64, _p, _i64, _i64, _i, _f, _p, _p, _sz, _p]),
    "fb_topk": (_i, [_i, _p, _i64, _i64, _i64, _i, _p, _p, _p, _p, _i64, _p]),
    "fb_touched": (_i, [_p, _p, _i64, _i, _i, _i, _p, _p, _p]),
    "fb_group": (_i, [_p, _i64, _i, _i, _p, _p, _p, _p]),
    "fb_elementwise": (_i, [_i, _p, _p, _i, _p, _p, _p, _p, _p, _i, _i64, _i64, _i64, _p]),
    "fb_reduce": (_i, [_i, _p, _p, _i, _i64, _i64, _i64, _i, _p, _p, _i, _p]),
    "fb_matmul": (_i, [_p, _p, _i, _p, _p, _i, _p, _p, _i, _i64, _i64, _i64, _i64, _p]),
    "fb_rmsnorm": (_i, [_p, _i64, _i64, _i64, _p, _f, _p, _i64, _p]),
    "fb_argmax": (_i, [_p, _i64, _i64, _i64, _p, _p, _p]),
    "fb_rope_kv_write_packed": (_i, [_i, _p, _i64, _i64, _i, _i, _i, _p, _p, _i64, _i64, _p, _p, _p, _f, _p, _i64, _p, _i64, _p]),
    "fb_decode_attention_packed": (_i, [_i, _p, _i64, _i64, _i, _i, _i, _p, _i64, _p, _p, _i64, _i, _p, _i64, _p, _sz, _p]),
    "fb_peer_reduce_add": (_i, [_p, _p, _i, _i, _p, _i64, _p, _p, _p]),
}


class FerriteError(RuntimeError):
    pass


_lib = None


def lib():
    """The loaded library (loads it on first use)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is not built: run `python -m ferrite_b200.build` (the CUDA library is the only compute path)")
        _lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype, fn.argtypes = res, args
    return _lib


_RAISES = {-1: AssertionError, -2: FerriteError, -3: TimeoutError, -4: MemoryError}


def check(status):
    """0 passes; a negative fb_status raises what ferrite raises for the same misuse: AssertionError for a
    bad shape or dtype, MemoryError, TimeoutError (ferrite/tensor.py asserts; ferrite/runtime.py:445,476)."""
    if status != 0:
        raise _RAISES.get(status, FerriteError)(lib().fb_last_error().decode())
