"""Compile oracle/bfp_oracle.c into oracle/_build/libbfp_oracle.so (gcc, OpenMP).  Test infrastructure only."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_build", "libbfp_oracle.so")


def build(force=False):
    src = os.path.join(HERE, "bfp_oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(LIB), exist_ok=True)
        subprocess.run(["gcc", "-O3", "-fopenmp", "-shared", "-fPIC", src, "-o", LIB], check=True)
    return LIB


def bfp_values(a, fmt):
    """oracle.bfp.bfp(a, fmt) as float32, by the C restatement (rows of whole runs of 16)."""
    import ctypes
    import numpy as np
    lib = ctypes.CDLL(build())
    a = np.ascontiguousarray(a, np.float32)
    out = np.empty_like(a)
    rows = a.size // a.shape[-1]
    lib.bfp_values(a.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_int64(rows), ctypes.c_int64(a.shape[-1]),
                   ctypes.c_int(8 if fmt == "bfp8" else 4))
    return out


if __name__ == "__main__":
    print(build(force=True))
