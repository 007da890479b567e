"""Compile csrc/*.cu for sm_100a into lib/libferrite_b200.so with nvcc (in-tree, no JIT cache).

    python -m ferrite_b200.build            # build if sources are newer than the library
    python -m ferrite_b200.build --force
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "lib", "libferrite_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xptxas", "-v"]


def sources():
    return sorted(f for f in os.listdir(SRC) if f.endswith(".cu"))


def stale():
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(SRC, f) for f in os.listdir(SRC)] + [os.path.join(HERE, "..", "include", "ferrite_b200.h")]
    return any(os.path.getmtime(d) > built for d in deps)


def compile_one(name):
    obj = os.path.join(OBJ, name[:-3] + ".o")
    hdrs = [os.path.join(SRC, f) for f in os.listdir(SRC) if f.endswith((".cuh", ".h"))] + [os.path.join(HERE, "..", "include", "ferrite_b200.h")]
    newest = max(os.path.getmtime(p) for p in [os.path.join(SRC, name)] + hdrs)
    if os.path.exists(obj) and os.path.getmtime(obj) > newest:
        return name, ""
    r = subprocess.run([NVCC, *FLAGS, "-c", os.path.join(SRC, name), "-o", obj], capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError(f"nvcc failed on {name}:\n{r.stdout}\n{r.stderr}")
    return name, r.stderr


def build(force=False, verbose=False):
    if not force and not stale():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        logs = list(pool.map(compile_one, sources()))
    if verbose:
        for name, log in logs:
            print(f"== {name}\n{log}")
    objs = [os.path.join(OBJ, f[:-3] + ".o") for f in sources()]
    r = subprocess.run([NVCC, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a"], capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
