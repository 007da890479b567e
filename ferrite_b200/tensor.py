"""Lazy tensors on a B200: the drop-in for `ferrite.tensor` (Tensor, jit) on the decode path.

The operator surface is ferrite's (ferrite/tensor.py:14-817): batch x rows x cols tensors of bf16, fp32, int32, bfp8 or
bfp4 whose ops build a tree; `realize` turns the tree into kernel launches.  Below the method signatures nothing is
ferrite's: storage is a torch CUDA tensor (ownership and views only), every computation is one of this package's
sm_100a kernels reached through the C ABI (ferrite_b200/_lib.py), launched on torch's current stream, and the planner
maps the trees a Llama block builds onto the fused kernels:

    x * rsqrt(mean(x*x) + eps) * w  feeding a block-float matmul   -> RMSNorm prologue of fb_linear
    silu(mm[:, :m]) * mm[:, m:]                                      -> SwiGLU epilogue of fb_linear
    x + mm                                                           -> residual epilogue of fb_linear
    any other elementwise tree                                       -> one fb_elementwise launch (postfix program)

There is no CPU path: without the CUDA library the import of `_lib` raises.
`jit` replays a recorded step as one CUDA graph (ferrite/tensor.py:788-810 replays a recorded block of launches).
"""
import array
import math

import numpy as np
import torch

from . import _lib, ops
from ._lib import check, lib

BFP = ("bfp8", "bfp4")
_TORCH = {"bf16": torch.bfloat16, "fp32": torch.float32, "int32": torch.int32}
_NAME = {v: k for k, v in _TORCH.items()}
# Whether the planner hands an RMSNorm from the matmul that makes its input to the matmul that consumes it
# (fb_linear_chained) instead of running the norm's preparation as a kernel of its own.  Off: measured on the 8B-shape
# step it saves 64 launches and still costs time (5.21 ms against 5.01): the preparation kernel hides behind the next
# matmul's set-up, while the hand-over adds a pass at the end of the producing matmul and a sum over its 128 parts.
CHAIN_NORMS = False
FIDELITY = 4  # accepted and ignored, as the numpy reference ignores it (models/llama.py:33): products are exact here

# elementwise opcodes of fb_elementwise (include/ferrite_b200.h)
_BINARY = {"add": 10, "sub": 11, "mul": 12, "max": 13, "cmplt": 14, "cmpne": 15, "keep": 16, "drop": 17, "div": 18, "min": 19}
_UNARY = {"exp": 30, "log": 31, "sin": 32, "cos": 33, "sqrt": 34, "recip": 35, "relu": 36, "exp2": 37, "log2": 38, "round_bf16": 39,
          "trunc": 40, "neg": 41}
_ELEMENTWISE = set(_BINARY) | set(_UNARY) | {"cast"}
_MAX_OPS, _MAX_INPUTS, _MAX_STACK = 48, 8, 12


class Runtime:
    """What ferrite's Runtime is to its Tensors (ferrite/runtime.py:304-505), on a CUDA device: launches are queued on
    a stream in order and only reading back waits; `wait` has a timeout in the sense that every device-side wait of the
    kernels is bounded and reports through the status word."""

    def __init__(self, device=0):
        assert torch.cuda.is_available(), "ferrite_b200 needs a CUDA device: there is no CPU path"
        self.device = torch.device("cuda", device) if not isinstance(device, torch.device) else device
        torch.cuda.set_device(self.device)
        lib()
        self.numbers, self.launches, self.names = {}, 0, []

    def launched(self, name, kernels=0):
        """One op queued; kernels: how many kernels it launched that no ops.* wrapper has counted already."""
        ops.count(kernels)
        self.launches += 1
        if len(self.names) < 4096:
            self.names.append(name)

    def wait(self, timeout=None):
        torch.cuda.synchronize(self.device)
        code = lib().fb_status_word()
        if code:
            raise TimeoutError(f"a device-side wait gave up (code {code})")

    def profile(self, since=0):
        """(name, launches) of the kernels launched after launch number `since`, most frequent first."""
        counts = {}
        for n in self.names[since:]:
            counts[n] = counts.get(n, 0) + 1
        return sorted(counts.items(), key=lambda kv: -kv[1])


def _strides3(buf):
    return [int(s) for s in buf.stride()]


class Tensor:
    """batch x rows x cols of bf16, fp32, int32, bfp8 or bfp4 (ferrite/tensor.py:15-29); realized (it has storage) or
    an op on other tensors not yet computed."""

    def __init__(self, rt, rows, cols, op=None, srcs=(), batch=1, dtype="bf16", buf=None, packed=None, owner=None, args=None):
        self.rt, self.rows, self.cols, self.batch, self.op, self.srcs, self.dtype = rt, rows, cols, batch, op, srcs, dtype
        self.args, self.owner, self.buf, self.packed = args or {}, owner, buf, packed
        self.requires_grad, self.grad = False, None
        if op is None and buf is None and packed is None:
            if dtype in BFP:
                n = lib().fb_packed_bytes(_lib.DTYPES[dtype], rows, cols)
                assert n, f"a block float's columns come in runs of 16, not {cols}"
                self.packed = ops.Packed(dtype, batch, rows, cols, torch.empty(batch * n, dtype=torch.uint8, device=rt.device))
            else:
                self.buf = torch.empty(batch, rows, cols, dtype=_TORCH[dtype], device=rt.device)

    @property
    def shape(self):
        return (self.batch, self.rows, self.cols)

    def __hash__(self):
        return id(self)

    # ---------------------------------------------------------------- in and out

    @classmethod
    def full(cls, rt, rows, cols, value, dtype="bf16"):
        return cls.of(rt, [[value] * cols for _ in range(rows)], dtype)

    @classmethod
    def of(cls, rt, data, dtype="bf16"):
        """From a list of rows of numbers, or a list of those (a batch), rounded to dtype (bf16: to nearest even)."""
        a = np.asarray(data, dtype=np.int32 if dtype == "int32" else np.float32)
        a = a.reshape((1,) * (3 - a.ndim) + a.shape)
        host = torch.from_numpy(np.ascontiguousarray(a))
        return cls(rt, a.shape[1], a.shape[2], batch=a.shape[0], dtype=dtype, buf=host.to(_TORCH[dtype]).to(rt.device))

    @classmethod
    def frombytes(cls, rt, rows, cols, data, batch=1, dtype="bf16"):
        """From dtype's values in row-major order (little-endian), matrix after matrix (ferrite/tensor.py:60-80)."""
        assert dtype not in BFP, "a block float is made on the chip, by cast"
        raw = np.frombuffer(memoryview(data).cast("B"), dtype=np.uint8)
        size = {"bf16": 2, "fp32": 4, "int32": 4}[dtype]
        assert len(raw) == size * batch * rows * cols, f"{len(raw)} bytes for {batch} x {rows} x {cols} of {dtype}"
        view = {"bf16": np.int16, "fp32": np.float32, "int32": np.int32}[dtype]
        host = torch.from_numpy(raw.view(view).reshape(batch, rows, cols).copy())
        if dtype == "bf16":
            host = host.view(torch.bfloat16)
        return cls(rt, rows, cols, batch=batch, dtype=dtype, buf=host.to(rt.device))

    def tobytes(self):
        """dtype's values in row-major order, a block float's as bf16 (ferrite/tensor.py:82-107).  Waits."""
        t = self.realize()
        buf = ops.dequantize(t.packed) if t.dtype in BFP else t.buf
        host = buf.contiguous().cpu()
        code = lib().fb_status_word()
        if code:
            raise TimeoutError(f"a device-side wait gave up (code {code})")
        if host.dtype == torch.bfloat16:
            host = host.view(torch.int16)
        return host.numpy().tobytes()

    def tolist(self):
        raw = self.tobytes()
        if self.dtype == "bf16" or self.dtype in BFP:
            raw = array.array("I", [b << 16 for b in array.array("H", raw)]).tobytes()
        values = array.array("i" if self.dtype == "int32" else "f", raw).tolist()
        m = [[values[(b * self.rows + r) * self.cols:(b * self.rows + r + 1) * self.cols] for r in range(self.rows)] for b in range(self.batch)]
        return m if self.batch > 1 else m[0]

    def numpy(self):
        """The values as a numpy array of shape (batch, rows, cols): float32 (bf16 and block floats widened) or int32."""
        kind = np.int32 if self.dtype == "int32" else np.float32
        raw = self.tobytes()
        if self.dtype == "bf16" or self.dtype in BFP:
            return (np.frombuffer(raw, np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(self.shape)
        return np.frombuffer(raw, kind).reshape(self.shape)

    # ---------------------------------------------------------------- building the tree

    def _lazy(self, op, srcs, shape, dtype, **args):
        return Tensor(self.rt, shape[1], shape[2], op, tuple(srcs), shape[0], dtype, args=args)

    def _view(self, buf):
        """A realized tensor over `buf`, a torch view of this one's storage (shares it; writes go through)."""
        return Tensor(self.rt, buf.shape[1], buf.shape[2], batch=buf.shape[0], dtype=self.dtype, buf=buf, owner=self.owner or self)

    def _unary(self, op):
        if self.dtype == "int32" and op != "relu":
            return self.float()._unary(op)
        return self._lazy(op, (self,), self.shape, self.dtype)

    def _binop(self, op, x, reverse=False):
        """numpy's broadcasting: shapes match, or one side has 1 where the other does not; different dtypes meet in
        fp32 (ferrite/tensor.py:305-314).  A Python number is a constant of the expression."""
        if isinstance(x, Tensor):
            assert all(n == m or 1 in (n, m) for n, m in zip(self.shape, x.shape)), f"cannot broadcast {self.shape} with {x.shape}"
            shape = tuple(map(max, self.shape, x.shape))
            dtype = self.dtype if self.dtype == x.dtype else "fp32"
        else:
            shape, dtype = self.shape, "fp32" if self.dtype == "int32" and isinstance(x, float) else self.dtype
        if dtype == "int32" and op in ("mul", "div"):
            dtype = "int32"  # computed through fp32, exact below 2^24 (as ferrite's)
        a, b = (x, self) if reverse else (self, x)
        return self._lazy(op, (a, b), shape, dtype)

    def cast(self, dtype):
        if dtype == self.dtype:
            return self
        return self._lazy("cast", (self,), self.shape, dtype)

    def float(self): return self.cast("fp32")
    def bfloat16(self): return self.cast("bf16")
    def exp2(self): return self._unary("exp2")
    def log2(self): return self._unary("log2")
    def sin(self): return self._unary("sin")
    def cos(self): return self._unary("cos")
    def sqrt(self): return self._unary("sqrt")
    def reciprocal(self): return self._unary("recip")
    def exp(self): return self._unary("exp")
    def log(self): return self._unary("log")
    def relu(self): return self._unary("relu")
    def rsqrt(self): return self.sqrt().reciprocal()
    def maximum(self, x): return self._binop("max", x)
    def minimum(self, x): return self._binop("min", x)
    def __add__(self, x): return self._binop("add", x)
    def __sub__(self, x): return self._binop("sub", x)
    def __mul__(self, x): return self._binop("mul", x)
    def __rsub__(self, x): return self._binop("sub", x, True)
    __radd__, __rmul__ = __add__, __mul__
    def __truediv__(self, x): return self * (1 / x) if isinstance(x, (int, float)) else self * x.reciprocal()
    def __rtruediv__(self, x): return self.reciprocal() * x
    def __neg__(self): return 0 - self if self.dtype == "int32" else self * -1
    def __lt__(self, x): return self._binop("cmplt", x)
    def __gt__(self, x): return self._binop("cmplt", x, True)
    def __ge__(self, x): return 1 - (self < x)
    def __le__(self, x): return 1 - (self > x)
    def ne(self, x): return self._binop("cmpne", x)
    def eq(self, x): return 1 - self.ne(x)
    __ne__, __eq__ = ne, eq
    def sigmoid(self): return (1 + (-self).exp()).reciprocal()
    def silu(self): return self * self.sigmoid()

    def where(self, x, y):
        """x where self is not 0, else y (ferrite/tensor.py:343-346)."""
        return self._binop("keep", x) + self._binop("drop", y)

    def gelu(self):  # GPT-2's tanh form (ferrite/tensor.py:355-357)
        k = 2 * math.sqrt(2 / math.pi)
        return self * (1 + (self * (self * self * (-0.044715 * k) - k)).exp()).reciprocal()

    def delta(self, *args, **kwargs):
        """Gated DeltaNet's recurrence (ferrite/tensor.py): on the reference's surface, not on the decode path built here."""
        raise NotImplementedError("Tensor.delta (Gated DeltaNet) is outside the decode path this library covers")

    def sum(self, axis=None): return self._reduce("sum", axis)
    def max(self, axis=None): return self._reduce("max", axis)

    def _reduce(self, f, axis):
        """numpy's, keeping the axis as 1 (ferrite/tensor.py:361-368)."""
        if axis is None:
            return self._reduce(f, 0)._reduce(f, 1)._reduce(f, 2)
        axis %= 3
        shape = tuple(1 if ax == axis else s for ax, s in enumerate(self.shape))
        return self if shape == self.shape else self._lazy("reduce_" + f, (self,), shape, self.dtype, axis=axis)

    def mean(self, axis=None):
        s = self.sum(axis)
        return s * (math.prod(s.shape) / math.prod(self.shape))

    def softmax(self, axis=-1):
        e = (self - self.max(axis)).exp()
        return e / e.sum(axis)

    def log_softmax(self, axis=-1):
        m = self - self.max(axis)
        return m - m.exp().sum(axis).log()

    def layernorm(self, axis=-1, eps=1e-5):
        c = self - self.mean(axis)
        return c * ((c * c).mean(axis) + eps).rsqrt()

    # ---------------------------------------------------------------- movement: views of the storage where torch has one

    def __getitem__(self, key):
        """x[b]; x[rows, cols] of every matrix; x[batch, rows, cols], with slices (ferrite/tensor.py:149-165).  A slice
        of a matmul not yet computed stays part of the tree, so that SwiGLU's halves fuse into the matmul."""
        if isinstance(key, int):
            return self.realize()._view(self.buf[key:key + 1])
        assert isinstance(key, tuple) and len(key) in (2, 3) and all(isinstance(k, slice) for k in key), "x[b], x[rows, cols] or x[batch, rows, cols]"
        key = (slice(None),) * (3 - len(key)) + tuple(key)
        ranges = [range(*k.indices(n)) for k, n in zip(key, self.shape)]
        assert all(len(r) for r in ranges), f"an empty slice of {self.shape}"
        if self.op == "matmul" and all(r.step == 1 for r in ranges) and len(ranges[0]) == self.batch and len(ranges[1]) == self.rows:
            return self._lazy("cols", (self,), (self.batch, self.rows, len(ranges[2])), self.dtype, start=ranges[2].start)
        t = self.realize()
        if any(r.step < 0 for r in ranges):  # torch has no negative strides: flip through a gather of indices
            buf = t.buf
            for ax, r in enumerate(ranges):
                buf = buf.index_select(ax, torch.tensor(list(r), device=buf.device))
            return t._view(buf)
        return t._view(t.buf[key])

    def reshape(self, *shape):
        shape = (1,) * (3 - len(shape)) + tuple(shape)
        assert math.prod(shape) == math.prod(self.shape), f"cannot reshape {self.shape} to {shape}"
        if shape == self.shape:
            return self
        t = self.realize()
        try:
            return t._view(t.buf.view(shape))
        except RuntimeError:  # not expressible by strides: a copy, made by the elementwise kernel
            return (t + 0).realize().reshape(*shape)

    def permute(self, *order):
        assert sorted(order) == [0, 1, 2]
        t = self.realize()
        return t._view(t.buf.permute(*order))

    @property
    def T(self):
        return self.permute(0, 2, 1)

    def expand(self, *shape):
        shape = (1,) * (3 - len(shape)) + tuple(shape)
        assert all(n in (m, 1) for n, m in zip(self.shape, shape)), f"cannot expand {self.shape} to {shape}"
        t = self.realize()
        return t._view(t.buf.expand(*shape))

    def pad(self, widths):
        """Zeros around: (before, after) for each of the last len(widths) axes (ferrite/tensor.py:194-199)."""
        widths = ((0, 0),) * (3 - len(widths)) + tuple(widths)
        t = self.realize()
        shape = [n + w[0] + w[1] for n, w in zip(self.shape, widths)]
        out = Tensor(self.rt, shape[1], shape[2], batch=shape[0], dtype=self.dtype)
        _fill(out, 0)
        out[tuple(slice(w[0], w[0] + n) for n, w in zip(self.shape, widths))].assign(t)
        return out

    def cat(self, *xs, axis=0):
        ts, axis = [t.realize() for t in (self, *xs)], axis % 3
        shape = list(self.shape)
        shape[axis] = sum(t.shape[axis] for t in ts)
        out, at = Tensor(self.rt, shape[1], shape[2], batch=shape[0], dtype=self.dtype), 0
        for t in ts:
            key = [slice(None)] * 3
            key[axis] = slice(at, at + t.shape[axis])
            out[tuple(key)].assign(t)
            at += t.shape[axis]
        return out

    def repeat_interleave(self, n):
        """Each matrix n times over along the batch (ferrite/tensor.py:210-217).  Attention reads the repeat in place
        (entry b uses matrix b // n); anything else that needs its values gets a copy."""
        t = self.realize()
        return self._lazy("repeat", (t,), (t.batch * n, t.rows, t.cols), t.dtype, n=n)

    def split(self, n, axis=2):
        """The matrix cut into n equal parts along axis as a batch of n, in place (ferrite/tensor.py:219-232)."""
        assert axis in (1, 2)
        t = self.realize()
        if axis == 2:
            assert t.batch == 1 and t.cols % n == 0, "equal parts of one matrix"
            return t._view(t.buf.view(t.rows, n, t.cols // n).permute(1, 0, 2))
        assert t.rows % n == 0, "equal parts"
        if t.batch == 1:
            return t._view(t.buf.view(n, t.rows // n, t.cols))
        return t._view(t.buf.unflatten(1, (n, t.rows // n)).flatten(0, 1))

    def merge(self):
        """The batch side by side as one matrix, the inverse of split (ferrite/tensor.py:234-240)."""
        t = self.realize()
        out = Tensor(self.rt, t.rows, t.batch * t.cols, dtype=t.dtype)
        out.split(t.batch).assign(t)
        return out

    def assign(self, x):
        """x's value into this tensor's storage, in place (ferrite/tensor.py:273-283)."""
        assert self.op is None and (x.shape, x.dtype) == (self.shape, self.dtype), "a tensor or view, its own shape and dtype"
        if x.op is not None and x.op in _ELEMENTWISE:
            _run_elementwise(x, into=self)
            x.op, x.srcs, x.buf = None, (), self.buf
        else:
            _copy(x.realize(), self)
        return self

    # ---------------------------------------------------------------- rows by index

    def gather(self, ids):
        """Rows ids of this matrix: an embedding lookup (ferrite/tensor.py:116-126)."""
        if not isinstance(ids, Tensor):  # a list of rows: a constant of the program, uploaded once (a recorded step meets it again)
            key = ("rows", tuple(int(i) for i in ids))
            assert all(0 <= i < self.rows for i in key[1])
            if key not in self.rt.numbers:
                self.rt.numbers[key] = Tensor.of(self.rt, [list(key[1])], "int32")
            ids = self.rt.numbers[key]
        assert self.batch == 1 and ids.dtype == "int32" and ids.shape[:2] == (1, 1), "rows of a matrix, by a row of int32"
        t, ids = self.realize(), ids.realize()
        table = t.buf[0] if t.buf[0].is_contiguous() else t.buf[0].contiguous()
        out = Tensor(self.rt, ids.cols, self.cols, dtype=self.dtype)
        ops.gather_rows(table, ids.buf.reshape(-1), out.buf[0])
        self.rt.launched("gather")
        return out

    def put(self, ids, x):
        """x's rows into rows ids of each matrix of this tensor, in place (ferrite/tensor.py:128-140); a later
        duplicate wins."""
        assert ids.dtype == "int32" and ids.shape[:2] == (1, 1) and ids.cols == x.rows, "rows of x, by a row of int32 places"
        assert (x.batch, x.cols) == (self.batch, self.cols) and x.dtype == self.dtype, f"{x.shape} {x.dtype} into {self.shape} {self.dtype}"
        t, x, ids = self.realize(), x.realize(), ids.realize()
        check(lib().fb_put_rows(t.buf.data_ptr(), *_strides3(t.buf), x.buf.data_ptr(), *_strides3(x.buf), ids.buf.data_ptr(), t.batch, x.rows, t.cols,
                                t.rows, t.buf.element_size(), ops._stream()))
        self.rt.launched("put", 1)
        return self

    # ---------------------------------------------------------------- matmul, attention, the router

    def __matmul__(self, x):
        return self.matmul(x)

    def matmul(self, x, dtype=None, fidelity=None, index=None):
        """Matrix by matrix through a batch, summed in fp32 and written as dtype: bf16, or fp32 if either operand is,
        unless said (ferrite/tensor.py:443-485).  x may be a block float when self is bf16.  index: an int32 (rows, k)
        tensor picking, for batch entry b of the result, which of x's matrices to multiply by (a mixture of experts'
        choice); an entry picking none (x.batch or more) is zeros."""
        assert "int32" not in (self.dtype, x.dtype), "the FPU multiplies floats"
        assert self.cols == x.rows, f"{self.shape} @ {x.shape}"
        if index is not None:
            assert index.dtype == "int32" and self.dtype == "bf16" and self.batch in (1, index.rows * index.cols), \
                f"{self.shape} @ {x.shape} picked by {index.shape} {index.dtype}"
            return self._lazy("matmul", (self, x, index), (index.rows * index.cols, self.rows, x.cols), dtype or "bf16")
        assert self.batch == x.batch or 1 in (self.batch, x.batch), f"{self.shape} @ {x.shape}"
        dtype = dtype or ("fp32" if "fp32" in (self.dtype, x.dtype) else "bf16")
        return self._lazy("matmul", (self, x), (max(self.batch, x.batch), self.rows, x.cols), dtype)

    def attend(self, k, v, places, window=0, fidelity=None, parts=None):
        """softmax(self @ k^T + mask) @ v in one kernel (ferrite/tensor.py:487-516): self a batch of queries, k and v
        the keys and values for each (a repeat is read in place), places (int32, a column per entry or one for all):
        each row's last key; with a window, only the last `window` keys.  bf16 keys and values."""
        rep = k.args.get("n", 1) if k.op == "repeat" else 1
        assert (v.args.get("n", 1) if v.op == "repeat" else 1) == rep and self.batch == k.batch == v.batch
        assert self.dtype == "bf16" and k.dtype == v.dtype == "bf16", "bf16 queries, keys and values (a block-float cache is read by attend_cache)"
        assert self.cols == k.cols == v.cols and self.cols in (64, 128) and k.rows == v.rows, "heads of 64 or 128 columns"
        assert places.rows == self.rows and places.batch in (1, self.batch) and places.cols == 1 and places.dtype == "int32", \
            f"{self.shape} by {k.shape}, {places.shape}"
        q, places = self.realize(), places.realize()
        kb = (k.srcs[0] if k.op == "repeat" else k).realize().buf
        vb = (v.srcs[0] if v.op == "repeat" else v).realize().buf
        if q.buf.stride(2) != 1 or q.buf.stride(1) % 8 or q.buf.stride(0) % 8:
            q = (q + 0).realize()
        kb, vb = (b if b.stride(2) == 1 and b.stride(1) == self.cols else b.contiguous() for b in (kb, vb))
        assert kb.stride(0) == vb.stride(0), "keys and values laid out alike"
        out = Tensor(self.rt, self.rows, self.cols, batch=self.batch)
        need = lib().fb_attend_workspace_bytes(self.batch, self.rows, self.cols, k.rows)
        ws = ops.attention_workspace(self.rt.device, need)
        check(lib().fb_attend(q.buf.data_ptr(), self.batch, self.rows, self.cols, q.buf.stride(0), q.buf.stride(1), kb.data_ptr(), vb.data_ptr(),
                              kb.stride(0), rep, k.rows, places.buf.data_ptr(), places.buf.stride(0) if places.batch > 1 else 0,
                              places.buf.stride(1), window or 0, 1.0, out.buf.data_ptr(), ops._ptr(ws), ws.numel() if ws is not None else 0,
                              ops._stream()))
        self.rt.launched("attention", 2 if need else 1)
        return out

    def topk(self, k, parts=1, labels=None):
        """Along each row, largest first: (values, int32 indices), the first column of equals first
        (ferrite/tensor.py:373-388).  parts: each row cut into so many parts, each part's k best side by side."""
        cols = self.cols // parts
        assert self.dtype in ("bf16", "fp32") and k <= min(cols, 64) and parts * cols == self.cols, "bf16 or fp32, k of at most 64, whole parts"
        assert labels is None or (labels.dtype == "int32" and labels.shape == self.shape and parts == 1), "labels: int32, x's shape"
        x = self.realize()
        if not x.buf.is_contiguous():
            x = (x + 0).realize()
        labels = None if labels is None else labels.realize()
        if labels is not None and not labels.buf.is_contiguous():
            labels = (labels + 0).realize()
        values = Tensor(self.rt, x.rows, parts * k, batch=x.batch, dtype=x.dtype)
        ids = Tensor(self.rt, x.rows, parts * k, batch=x.batch, dtype="int32")
        # a row of `parts` parts is `parts` rows of one part each: one launch for all of them
        check(lib().fb_topk(_lib.DTYPES[x.dtype], x.buf.data_ptr(), x.batch * x.rows * parts, cols, cols, k, ops._ptr(labels.buf) if labels is not None else None,
                            values.buf.data_ptr(), ids.buf.data_ptr(), None, k, ops._stream()))
        if parts > 1:  # (the parts' first columns: a constant, uploaded once - a recorded step meets it again)
            key = ("topk parts", parts, cols, k)
            if key not in self.rt.numbers:
                self.rt.numbers[key] = Tensor.of(self.rt, [[p * cols for p in range(parts) for _ in range(k)]], "int32")
            ids = (ids + self.rt.numbers[key]).realize()
        self.rt.launched("topk", 1)
        return values, ids

    def group(self, n):
        """A mixture of experts' tokens grouped by expert, from int32 choices (rows x k, values below n), as three int32
        tensors (ferrite/tensor.py:389-402): order, a row of 32 t slots in which each value's choices have a run of whole
        tiles of 32, each slot the row it holds (0 for none); tiles, a column of t, each tile's value (n past those
        used); places, a row of k runs of the rows rounded up to 32, run j holding the slot of each row's choice j."""
        assert self.dtype == "int32" and self.batch == 1 and self.cols <= 32, "a matrix of int32 choices, at most 32 a row"
        x = self.realize()
        x = x if x.buf.is_contiguous() else (x + 0).realize()
        rows, k = self.rows, self.cols
        t, rp = -(-rows * k // 32) + min(n, rows * k), -(-rows // 32) * 32
        order, tiles, places = Tensor(self.rt, 1, 32 * t, dtype="int32"), Tensor(self.rt, t, 1, dtype="int32"), Tensor(self.rt, 1, k * rp, dtype="int32")
        check(lib().fb_group(x.buf.data_ptr(), rows, k, n, order.buf.data_ptr(), tiles.buf.data_ptr(), places.buf.data_ptr(), ops._stream()))
        self.rt.launched("group", 1)
        return order, tiles, places

    def touched(self, n, weights, first=0):
        """The experts some row picks by a weight that is not 0, each once, ascending, then n (none); and each entry's
        weight from each row (ferrite/tensor.py:403-416).  first: count the experts from it (a rank's run of a mixture's
        experts: only those are listed, numbered from 0)."""
        assert self.dtype == "int32" and weights.dtype == "bf16" and self.shape == weights.shape and self.batch == 1 and self.cols <= 32
        x, w = self.realize(), weights.realize()
        x = x if x.buf.is_contiguous() else (x + 0).realize()
        w = w if w.buf.is_contiguous() else (w + 0).realize()
        slots = min(self.rows * self.cols, n)
        experts, out = Tensor(self.rt, slots, 1, dtype="int32"), Tensor(self.rt, self.rows, 1, batch=slots)
        check(lib().fb_touched(x.buf.data_ptr(), w.buf.data_ptr(), self.rows, self.cols, n, first, experts.buf.data_ptr(), out.buf.data_ptr(), ops._stream()))
        self.rt.launched("touched", 1)
        return experts, out

    # ---------------------------------------------------------------- a decode step's two fused kernels

    def rope_put(self, cos, sin, places, rows, cache, heads, kv, qk_norm=None, eps=1e-5):
        """self: a fused q, k, v projection [1, tokens, (heads + 2 kv) hd].  One kernel does what models/llama.py:119-128
        spells as split, (Qwen3's norm of each q and k head,) rope, merge and put: q's heads turned by RoPE come back as
        [1, tokens, heads hd]; k's (turned) and v's go into `cache` ([2 kv, size, hd]) at `rows`.  cos / sin: tables with
        a row for each place, one head wide or as wide as self; places, rows: int32 rows read on the device."""
        hd = cache.cols
        qkv = self.realize()
        assert qkv.batch == 1 and qkv.cols == (heads + 2 * kv) * hd and cache.batch == 2 * kv and cache.dtype in ("bf16",) + tuple(BFP), \
            f"{qkv.shape} into a cache {cache.shape}"
        assert places.dtype == rows.dtype == "int32" and places.cols == rows.cols == qkv.rows, "a place and a cache row per token"
        cos, sin, places, rows = (t.realize() for t in (cos, sin, places, rows))
        qb = qkv.buf[0] if qkv.buf.stride(2) == 1 else (qkv + 0).realize().buf[0]
        out = Tensor(self.rt, qkv.rows, heads * hd)
        assert cache.dtype in BFP or (cache.buf.stride(2) == 1 and cache.buf.stride(1) == hd), "a cache's rows lie one after another"
        ops.rope_kv_write(qb, cos.buf[0], sin.buf[0], places.buf.reshape(-1), rows.buf.reshape(-1), cache.packed if cache.dtype in BFP else cache.buf, heads, kv, hd, q_out=out.buf[0],
                          qk_norm=None if qk_norm is None else qk_norm.realize().buf, eps=eps)
        self.rt.launched("rope put")
        return out

    def attend_cache(self, cache, base, last, kv, length=None, window=0, chunk=False):
        """self: [1, tokens, heads hd], each token's query heads.  Token t attends the cache rows base[t] .. base[t] +
        last[t] of every kv head (the last `window` of them, if any), its heads / kv query heads sharing each key row
        read: attention as models/llama.py:129-146 runs it on the chip (Tensor.attend with places), without the views,
        the repeat and the regrouping moves in between.  length: the most keys a token can see (it sizes the split of
        the keys over the GPU).  chunk: the tokens are one sequence's (a prompt's chunk, its first cache row 0): a query
        head's tokens then share each key row read, 16 at a time, instead of every token reading the keys anew."""
        hd = cache.cols
        q = self.realize()
        heads = q.cols // hd
        assert q.batch == 1 and q.cols % hd == 0 and heads % kv == 0 and cache.batch == 2 * kv, f"{q.shape} over a cache {cache.shape}"
        base, last = base.realize(), last.realize()
        out = Tensor(self.rt, q.rows, q.cols)
        if chunk:
            ops.prefill_attention(q.buf[0], cache.packed if cache.dtype in BFP else cache.buf, 0, last.buf.reshape(-1), heads, kv, hd,
                                  max_keys=min(length or cache.rows, cache.rows), window=window or 0, out=out.buf[0])
            self.rt.launched("attention")
            return out
        ops.decode_attention(q.buf[0], cache.packed if cache.dtype in BFP else cache.buf, base.buf.reshape(-1), last.buf.reshape(-1), heads, kv, hd,
                             max_keys=min(length or cache.rows, cache.rows),
                             window=window or 0, out=out.buf[0])
        self.rt.launched("attention")
        return out

    def greedy(self, values=None):
        """Each row's first largest logit's column, int32 [1, 1, rows], picked on the device (the reference reads the
        logits back and takes numpy's argmax, models/llama.py:787-795): fp32 logits of one matrix."""
        x = self.realize()
        assert x.dtype == "fp32" and x.batch == 1 and x.buf.stride(2) == 1, "a matrix of fp32 logits"
        out = Tensor(self.rt, 1, x.rows, dtype="int32")
        ops.argmax(x.buf[0], out.buf.reshape(-1), None if values is None else values.buf.reshape(-1))
        self.rt.launched("argmax")
        return out

    # ---------------------------------------------------------------- computing the tree

    def realize(self, into=None):
        """Compute it now, into storage of its own or into `into`'s (ferrite/tensor.py:247-272).  Returns it, realized."""
        if self.op is None:
            if into is not None:
                _copy(self, into)
            return self
        _realize(self, into)
        return self


# -------------------------------------------------------------------- the planner

def _done(t, buf=None, packed=None):
    """t is computed: it now owns storage and forgets how it was made."""
    t.buf, t.packed, t.op, t.srcs = buf, packed, None, ()


def _realize(t, into=None):
    op = t.op
    if op in _ELEMENTWISE:
        if op == "cast" and t.dtype in BFP:
            src = t.srcs[0].cast("bf16").realize()
            buf = src.buf if src.buf.is_contiguous() else (src + 0).realize().buf
            _done(t, packed=ops.quantize(buf if t.batch > 1 else buf[0], t.dtype))
            t.rt.launched("cast " + t.dtype)
            return
        if op == "cast" and t.srcs[0].dtype in BFP:
            src = t.srcs[0].realize()
            bf = Tensor(t.rt, t.rows, t.cols, batch=t.batch, buf=ops.dequantize(src.packed))
            _done(t, buf=bf.buf if t.dtype == "bf16" else bf.cast(t.dtype).realize().buf)
            return
        if _fused_linear(t, into):
            return
        if _run_rmsnorm(t, into):
            return
        _run_elementwise(t, into)
    elif op == "reduce_sum" and t.args["axis"] == 0 and _match_experts(t.srcs[0]):
        _run_experts(t, _match_experts(t.srcs[0]), None, into)
    elif op in ("reduce_sum", "reduce_max"):
        src, axis = t.srcs[0].realize(), t.args["axis"]
        out = into or Tensor(t.rt, t.rows, t.cols, batch=t.batch, dtype=t.dtype)
        i64 = lambda v: (ctypes_i64 * 3)(*v)
        check(lib().fb_reduce(int(op == "reduce_max"), src.buf.data_ptr(), i64(_strides3(src.buf)), _lib.DTYPES[src.dtype], *src.shape, axis,
                              out.buf.data_ptr(), i64(_strides3(out.buf)), _lib.DTYPES[out.dtype], ops._stream()))
        t.rt.launched(f"{op}{axis}", 1)
        _done(t, buf=out.buf)
    elif op == "matmul":
        _run_matmul(t, into)
    elif op == "cols":  # a run of columns of a matmul, read on its own: the whole matmul, then a view
        mm = t.srcs[0].realize()
        start = t.args["start"]
        _done(t, buf=mm.buf[:, :, start:start + t.cols])
        t.owner = mm
        if into is not None:
            _copy(t, into)
    elif op == "repeat":
        src, n = t.srcs[0].realize(), t.args["n"]
        out = Tensor(t.rt, t.rows, t.cols, batch=t.batch, dtype=t.dtype)
        for b in range(src.batch):
            _copy(src._view(src.buf[b:b + 1].expand(n, src.rows, src.cols)), out._view(out.buf[b * n:(b + 1) * n]))
        _done(t, buf=out.buf)
    else:
        raise NotImplementedError(f"no kernel for {op}")
    if into is not None and t.buf is not into.buf and op not in ("cols",):
        _copy(t, into)


import ctypes  # noqa: E402

ctypes_i64 = ctypes.c_int64


def _is_const(x, value=None):
    return isinstance(x, (int, float)) and (value is None or x == value)


def _match_rms(t):
    """(x, w, eps) if t is x * rsqrt(mean(x * x) + eps) * w as models/llama.py:82-85 writes RMSNorm, else None."""
    if not isinstance(t, Tensor) or t.op != "mul":
        return None
    for n, w in (t.srcs, t.srcs[::-1]):
        if not (isinstance(w, Tensor) and w.op is None and w.shape == (1, 1, t.cols) and isinstance(n, Tensor) and n.op == "mul"):
            continue
        for x, r in (n.srcs, n.srcs[::-1]):
            if not (isinstance(r, Tensor) and r.op == "recip" and isinstance(x, Tensor)):
                continue
            root = r.srcs[0]
            if root.op != "sqrt" or root.srcs[0].op != "add":
                continue
            mean, eps = root.srcs[0].srcs
            if not (_is_const(eps) and isinstance(mean, Tensor) and mean.op == "mul" and _is_const(mean.srcs[1])):
                continue
            total = mean.srcs[0]
            if not (isinstance(total, Tensor) and total.op == "reduce_sum" and total.args["axis"] == 2 and abs(mean.srcs[1] * x.cols - 1) < 1e-6):
                continue
            sq = total.srcs[0]
            if sq.op == "mul" and sq.srcs[0] is x and sq.srcs[1] is x:
                return x, w, float(eps)
    return None


def _run_rmsnorm(t, into):
    """t as one fb_rmsnorm call where its tree is an RMSNorm of bf16 rows that no matmul takes in as its prologue (a
    mixture's router and experts both read the normed rows; the output layer of a single sequence reads its last)."""
    found = _match_rms(t) if t.dtype == "bf16" and t.batch == 1 else None
    if not found or found[0].dtype != "bf16" or found[0].shape != t.shape:
        return False
    x, w, eps = found
    x = x.realize()
    if x.buf.stride(2) != 1 or (into is not None and into.buf.stride(2) != 1):
        return False
    out = into if into is not None else Tensor(t.rt, t.rows, t.cols)
    ops.rmsnorm(x.buf[0], w.realize().buf.reshape(-1), eps, out=out.buf[0])
    t.rt.launched("rmsnorm")
    _done(t, buf=out.buf)
    return True


def _match_silu_of(g):
    """The tensor a if g is a * sigmoid(a) as Tensor.silu builds it, else None."""
    if not isinstance(g, Tensor) or g.op != "mul":
        return None
    for a, s in (g.srcs, g.srcs[::-1]):
        if not (isinstance(s, Tensor) and s.op == "recip" and isinstance(a, Tensor)):
            continue
        plus = s.srcs[0]
        if plus.op != "add":
            continue
        for e, one in (plus.srcs, plus.srcs[::-1]):
            if _is_const(one, 1) and isinstance(e, Tensor) and e.op == "exp":
                neg = e.srcs[0]
                if neg.op == "mul" and neg.srcs[0] is a and _is_const(neg.srcs[1], -1):
                    return a
    return None


def _packed_matmul(t):
    """(a, w) if t is a matmul, not yet computed, of one bf16 matrix by one block-float matrix, else None."""
    if isinstance(t, Tensor) and t.op == "matmul" and len(t.srcs) == 2 and t.srcs[1].dtype in BFP and t.srcs[1].batch == 1 and t.srcs[0].batch == 1 \
            and t.srcs[0].dtype == "bf16":
        return t.srcs
    return None


def _fused_linear(t, into, hand_on=None):
    """t as one fb_linear call with an epilogue, where its tree is a block's SwiGLU or residual add; else False.
    hand_on: the weight of the RMSNorm the result goes through next (see _linear): only a residual add takes it."""
    if t.op == "mul" and t.dtype == "bf16":  # silu(mm[:, :m]) * mm[:, m:]
        for g, u in (t.srcs, t.srcs[::-1]):
            gate = _match_silu_of(g)
            if gate is None or not isinstance(u, Tensor) or gate.op != "cols" or u.op != "cols":
                continue
            mm = gate.srcs[0]
            if u.srcs[0] is mm and _packed_matmul(mm) and mm.dtype == "bf16" and gate.args["start"] == 0 and u.args["start"] == gate.cols \
                    and 2 * gate.cols == mm.cols and mm.cols % 32 == 0:
                _linear(t, mm, "swiglu", None, into)
                return True
    if t.op == "add" and t.dtype == "bf16":  # x + the experts' sum
        for x, y in (t.srcs, t.srcs[::-1]):
            if isinstance(x, Tensor) and isinstance(y, Tensor) and y.op == "reduce_sum" and y.args["axis"] == 0 and x.shape == t.shape:
                found = _match_experts(y.srcs[0])
                if found:
                    _run_experts(t, found, x, into)
                    return True
    if t.op == "add" and t.dtype == "bf16":  # x + mm
        for x, mm in (t.srcs, t.srcs[::-1]):
            if isinstance(x, Tensor) and _packed_matmul(mm) and x.shape == mm.shape == t.shape and x.dtype == "bf16" and mm.dtype == "bf16":
                _linear(t, mm, "residual", x, into, hand_on)
                return True
    return False


def _linear(t, mm, epilogue, residual, into, hand_on=None):
    """fb_linear for the matmul mm (with its RMSNorm prologue, if its A is one) and the epilogue, into t.

    An RMSNorm between two block-float matmuls costs no kernel of its own where the first can hand it to the second
    (fb_linear_chained): when mm's A is rms(x) and x is a residual add of a block-float matmul not yet computed, that
    matmul is run with this norm's weight (hand_on) and leaves, beside x, x * g in bf16 and the rows' sums of squares;
    mm then reads those.  x is computed either way, for whoever else reads it (the next residual add)."""
    a, w = mm.srcs
    rms = _match_rms(a)
    x, norm_w, eps = rms if rms else (a, None, 0.0)
    w = w.realize()
    taken = None  # (x * g, sums of squares, parts) left by the matmul that made x
    # (9 rows and more: fewer go to the register-fed kernel, which takes no norm over)
    if CHAIN_NORMS and rms and x.op == "add" and x.dtype == "bf16" and x.batch == 1 and 9 <= x.rows <= 128:
        norm_w = norm_w.realize()
        if norm_w.buf.is_contiguous() and _fused_linear(x, None, hand_on=norm_w):
            taken = x.args.pop("handed", {}).get(id(norm_w))
    x = x.realize()
    res = None
    if residual is not None:
        residual = residual.realize()
        res = residual.buf[0] if residual.buf.stride(2) == 1 else (residual + 0).realize().buf[0]
    out = into if into is not None and into.buf.stride(2) == 1 else Tensor(t.rt, t.rows, t.cols, dtype=t.dtype)
    name = "linear " + w.dtype + (" rms" if rms else "") + ("" if epilogue == "none" else " " + epilogue)
    give = hand_on is not None and epilogue == "residual" and t.dtype == "bf16" and 9 <= t.rows <= 128 and ops.chain_parts(w.packed, t.rows, epilogue)
    if taken or give:
        xb = taken[0] if taken else (x.buf[0] if x.buf.stride(2) == 1 and x.buf.stride(1) % 8 == 0 else (x + 0).realize().buf[0])
        if rms and not taken:  # (a norm that nobody handed over: computed on its own, then the chained call reads plain rows)
            xb = ops.rmsnorm(xb, norm_w.buf.reshape(-1), eps)
        got = ops.linear_chained(xb, w.packed, out=out.buf[0], out_dtype=t.dtype, eps=eps, epilogue=epilogue, residual=res,
                                 norm_in=taken[1:] if taken else None, next_norm_w=hand_on.buf if give else None)
        if give:
            t.args = dict(t.args, handed={id(hand_on): (got[1], got[2], got[3])})
        t.rt.launched(name + " chained")
        _done(t, buf=out.buf)
        return
    xb = x.buf[0] if x.buf.stride(2) == 1 and x.buf.stride(1) % 8 == 0 else (x + 0).realize().buf[0]
    ops.linear(xb, w.packed, out=out.buf[0], out_dtype=t.dtype, norm_w=None if norm_w is None else norm_w.realize().buf, eps=eps, epilogue=epilogue, residual=res)
    t.rt.launched(name)
    _done(t, buf=out.buf)


def _run_matmul(t, into):
    if _packed_matmul(t):
        return _linear(t, t, "none", None, into)
    if len(t.srcs) == 3:
        return _run_indexed_matmul(t, into)
    a, b = t.srcs[0].realize(), t.srcs[1]
    if b.dtype in BFP:  # a batch of block floats, or an fp32 A: by the values, through the general kernel
        b = b.cast("bf16")
    b = b.realize()
    out = into or Tensor(t.rt, t.rows, t.cols, batch=t.batch, dtype=t.dtype)
    i64 = lambda buf, batch: (ctypes_i64 * 3)(*([0] + _strides3(buf)[1:] if batch == 1 and t.batch > 1 else _strides3(buf)))
    check(lib().fb_matmul(a.buf.data_ptr(), i64(a.buf, a.batch), _lib.DTYPES[a.dtype], b.buf.data_ptr(), i64(b.buf, b.batch), _lib.DTYPES[b.dtype],
                          out.buf.data_ptr(), i64(out.buf, t.batch), _lib.DTYPES[out.dtype], t.batch, t.rows, t.cols, a.cols, ops._stream()))
    t.rt.launched("matmul", 1)
    _done(t, buf=out.buf)


def _indexed_packed(t):
    """(a, w, index) if t is a matmul, not yet computed, picking block-float matrices by an index, else None."""
    if isinstance(t, Tensor) and t.op == "matmul" and len(t.srcs) == 3 and t.srcs[1].dtype in BFP and t.srcs[0].dtype == "bf16":
        return t.srcs
    return None


def _match_experts(t):
    """A mixture's touched experts as models/llama.py:317-324 writes them for a decode step:
    (glu(x[:, :, :m], x[:, :, m:]) * weights).matmul(down, index=picks) with x = h.matmul(gate_up, index=picks).
    Returns (h, gate_up, down, picks, weights or None), else None."""
    found = _indexed_packed(t)
    if not found:
        return None
    a, down, picks = found
    weights = None
    if isinstance(a, Tensor) and a.op == "mul":
        for g, w in (a.srcs, a.srcs[::-1]):
            if isinstance(w, Tensor) and w.op is None and w.shape == (t.batch, t.rows, 1) and w.dtype == "bf16" and isinstance(g, Tensor) and g.op == "mul":
                a, weights = g, w
                break
    if not (isinstance(a, Tensor) and a.op == "mul"):
        return None
    for g, u in (a.srcs, a.srcs[::-1]):
        gate = _match_silu_of(g)
        if gate is None or not isinstance(u, Tensor) or gate.op != "cols" or u.op != "cols" or u.srcs[0] is not gate.srcs[0]:
            continue
        first = _indexed_packed(gate.srcs[0])
        if first and first[2] is picks and first[0].batch == 1 and gate.args["start"] == 0 and u.args["start"] == gate.cols \
                and 2 * gate.cols == first[1].cols and first[1].cols % 128 == 0 and gate.cols == down.rows and gate.cols % 64 == 0 and t.rows <= 128:
            return first[0], first[1], down, picks, weights
    return None


def _run_experts(t, found, residual, into):
    """Two kernels for a mixture's decode step: every touched expert's gate_up with SwiGLU and its tokens' weights into
    act [tokens, entries * m]; then the experts' downs summed over the entries in the accumulators (+ the residual)."""
    h, gate_up, down, picks, weights = found
    rms = _match_rms(h)
    x, norm_w, eps = rms if rms else (h, None, 0.0)
    x, picks = x.realize(), picks.realize()
    xb = x.buf[0] if x.buf.stride(2) == 1 and x.buf.stride(1) % 8 == 0 else (x + 0).realize().buf[0]
    slots, m, rows = picks.rows * picks.cols, down.rows, x.rows
    idx = picks.buf.reshape(-1) if picks.buf.is_contiguous() else (picks + 0).realize().buf.reshape(-1)
    act = Tensor(t.rt, rows, slots * m)
    scale = None
    if weights is not None:
        scale = weights.buf if weights.buf.is_contiguous() else (weights + 0).realize().buf
    ops.linear_indexed(xb, gate_up.realize().packed, idx, act.buf[0], out_slot_stride=m, norm_w=None if norm_w is None else norm_w.buf, eps=eps,
                       epilogue="swiglu", row_scale=scale)
    res = None
    if residual is not None:
        residual = residual.realize()
        res = residual.buf[0] if residual.buf.stride(2) == 1 else (residual + 0).realize().buf[0]
    out = into if into is not None and into.buf.stride(2) == 1 else Tensor(t.rt, t.rows, t.cols, dtype=t.dtype)
    ops.linear_indexed(act.buf[0], down.realize().packed, idx, out.buf[0], sum_slots=True, out_dtype=t.dtype,
                       epilogue="residual" if res is not None else "none", residual=res)
    t.rt.launched("experts " + gate_up.dtype)
    _done(t, buf=out.buf)


def _run_indexed_matmul(t, into):
    """Tensor.matmul(index=) on its own: one result per entry (ferrite/tensor.py:450-460); block-float matrices."""
    a, w, picks = t.srcs
    assert w.dtype in BFP and t.rows <= 128, "picked matrices are block floats here, for up to 128 rows"
    rms = _match_rms(a) if a.batch == 1 else None
    x, norm_w, eps = rms if rms else (a, None, 0.0)
    x, picks = x.realize(), picks.realize()
    if not (x.buf.is_contiguous() and x.cols % 8 == 0):
        x = (x + 0).realize()
    idx = picks.buf.reshape(-1) if picks.buf.is_contiguous() else (picks + 0).realize().buf.reshape(-1)
    out = into if into is not None and into.buf.is_contiguous() else Tensor(t.rt, t.rows, t.cols, batch=t.batch, dtype=t.dtype)
    ops.linear_indexed(x.buf.reshape(-1, x.cols), w.realize().packed, idx, out.buf, M=t.rows, x_slot_rows=0 if x.batch == 1 else t.rows,
                       out_slot_stride=t.rows * t.cols, out_dtype=t.dtype, norm_w=None if norm_w is None else norm_w.buf, eps=eps)
    t.rt.launched("matmul index " + w.dtype)
    _done(t, buf=out.buf)


def _program(t, inputs, code, consts, depth=1):
    """Append the postfix program of the elementwise tree under t; realized tensors become inputs."""
    if not isinstance(t, Tensor):
        code.append((1, 0)), consts.append(float(t))
        return depth
    if t.op not in _ELEMENTWISE or (t.op == "cast" and (t.dtype in BFP or t.srcs[0].dtype in BFP)) or len(code) > _MAX_OPS - 8 \
            or (len(inputs) >= _MAX_INPUTS - 1 and t.op is not None) or depth > _MAX_STACK - 2:
        leaf = t.realize()
        for i, u in enumerate(inputs):
            if u is leaf:
                break
        else:
            inputs.append(leaf)
            i = len(inputs) - 1
        code.append((0, i)), consts.append(0.0)
        return depth
    if t.op == "cast":
        most = _program(t.srcs[0], inputs, code, consts, depth)
        if t.dtype == "bf16":
            code.append((_UNARY["round_bf16"], 0)), consts.append(0.0)
        elif t.dtype == "int32":
            code.append((_UNARY["trunc"], 0)), consts.append(0.0)
        return most
    if t.op in _UNARY:
        most = _program(t.srcs[0], inputs, code, consts, depth)
        code.append((_UNARY[t.op], 0)), consts.append(0.0)
        return most
    most = max(_program(t.srcs[0], inputs, code, consts, depth), _program(t.srcs[1], inputs, code, consts, depth + 1))
    code.append((_BINARY[t.op], 0)), consts.append(0.0)
    return most


def _run_elementwise(t, into=None):
    inputs, code, consts = [], [], []
    _program(t, inputs, code, consts)
    assert len(code) <= _MAX_OPS and len(inputs) <= _MAX_INPUTS, "an expression too large for one kernel even after splitting"
    out = into if into is not None else Tensor(t.rt, t.rows, t.cols, batch=t.batch, dtype=t.dtype)
    n = len(inputs)
    prog = (ctypes.c_int32 * (2 * len(code)))(*[v for pair in code for v in pair])
    cst = (ctypes.c_float * len(code))(*consts)
    ptrs = (ctypes.c_void_p * max(n, 1))(*[u.buf.data_ptr() for u in inputs])
    strides = (ctypes_i64 * (3 * max(n, 1)))(*[s for u in inputs for s in _strides3(u.buf.expand(t.shape))])
    dtypes = (ctypes.c_int32 * max(n, 1))(*[_lib.DTYPES[u.dtype] for u in inputs])
    check(lib().fb_elementwise(len(code), prog, cst, n, ptrs, strides, dtypes, out.buf.data_ptr(), (ctypes_i64 * 3)(*_strides3(out.buf)),
                               _lib.DTYPES[out.dtype], *t.shape, ops._stream()))
    t.rt.launched("elementwise", 1)
    _done(t, buf=out.buf)


def _copy(src, dst):
    """src's values into dst's storage (same shape; strides free), by the elementwise kernel."""
    assert src.shape == dst.shape, f"{src.shape} into {dst.shape}"
    _run_elementwise(src._lazy("add", (src, 0), src.shape, dst.dtype), into=dst)


def _fill(t, value):
    _run_elementwise(t._lazy("add", (value, 0), t.shape, t.dtype), into=t)


def jit(f):
    """f, a function of tensors that returns one, run from a recording (ferrite/tensor.py:788-810): its first call runs
    as any would, its second is recorded as a CUDA graph (the storage it takes kept from then on), and each later call
    copies its inputs into the second call's and replays the graph: nothing is planned, launched one by one or
    allocated again.  Its inputs keep their shapes and dtypes; it may not read back; its result is the same tensor
    every call, written again by the next."""
    state = {"calls": 0}

    def run(*xs):
        state["calls"] += 1
        if state["calls"] == 1:
            return f(*xs).realize()
        if state["calls"] == 2:
            inputs = [x.realize() for x in xs]
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):  # (other threads, NCCL's watchdog, may touch CUDA meanwhile)
                out = f(*inputs).realize()
            graph.replay()
            state.update(inputs=inputs, graph=graph, out=out)
            return out
        for x, to in zip(xs, state["inputs"]):
            assert (x.shape, x.dtype) == (to.shape, to.dtype), f"{x.shape} {x.dtype} where the recording had {to.shape} {to.dtype}"
            if x is not to:
                to.buf.copy_(x.realize().buf, non_blocking=True)
        state["graph"].replay()
        return state["out"]

    return run
