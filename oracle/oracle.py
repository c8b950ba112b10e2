"""numpy front end of the CPU oracle (oracle.c).  TEST INFRASTRUCTURE ONLY.

`Ref` mirrors the crate's `Tensor` API (src/tensor.rs:418-644 and the op front-ends) eagerly
on the host: math goes through oracle.c (double evaluation, one rounding per op), views and
moves are numpy views/copies (bit-exact by construction).  Element types: float32, float16,
and bfloat16 kept as uint16 bit patterns with `bf16=True`.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

F32, F16, BF16 = 0, 1, 2
(OP_EXP, OP_EXP2, OP_LOG, OP_LOG2, OP_SQR, OP_SQRT, OP_SIN, OP_COS, OP_TAN, OP_ASIN, OP_ACOS,
 OP_ATAN, OP_SINH, OP_COSH, OP_TANH, OP_ASINH, OP_ACOSH, OP_ATANH, OP_ABS, OP_NEG) = range(20)
OP_ADD_C, OP_SUB_C, OP_RSUB_C, OP_MUL_C, OP_DIV_C, OP_RDIV_C = range(32, 38)
OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_POW = range(64, 69)
OP_SUM, OP_MAX, OP_MIN, OP_PRODUCT = range(96, 100)
UNARY_NAMES = ["exp", "exp2", "log", "log2", "sqr", "sqrt", "sin", "cos", "tan", "asin", "acos", "atan",
               "sinh", "cosh", "tanh", "asinh", "acosh", "atanh", "abs", "neg"]


def build():
    subprocess.run(["make", "-s", "-C", HERE, "liboracle.so"], check=True)
    return os.path.join(HERE, "liboracle.so")


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(os.path.join(HERE, "oracle.c")):
            build()
        _LIB = C.CDLL(path)
        _LIB.orc_fast_sum_exp.restype = C.c_float
        _LIB.orc_ulp_diff_f32.restype = C.c_int64
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype=None):
    """C-contiguous array that keeps rank 0 (np.ascontiguousarray would make it rank 1)."""
    return np.asarray(a, dtype=dtype, order="C")


def _code(a, bf16):
    if bf16:
        return BF16
    return F16 if a.dtype == np.float16 else F32


class Ref:
    def __init__(self, a, bf16=False):
        a = np.asarray(a)
        if bf16:
            assert a.dtype == np.uint16
        elif a.dtype not in (np.float32, np.float16):
            a = a.astype(np.float32)
        self.a = a
        self.bf16 = bf16

    # ---- plumbing ----
    @property
    def shape(self):
        return tuple(self.a.shape)

    @property
    def code(self):
        return _code(self.a, self.bf16)

    def _like(self, a, code=None):
        return Ref(a, bf16=(self.bf16 if code is None else code == BF16))

    def numpy(self):
        return _c(self.a)

    def _unary(self, op):
        x = _c(self.a)
        out = np.empty_like(x)
        lib().orc_unary(op, self.code, _p(x), _p(out), C.c_int64(x.size))
        return self._like(out)

    def _scalar(self, op, c):
        x = _c(self.a)
        out = np.empty_like(x)
        lib().orc_scalar(op, self.code, _p(x), C.c_float(c), _p(out), C.c_int64(x.size))
        return self._like(out)

    def _binary(self, o, op):
        assert self.shape == o.shape and self.code == o.code
        x, y = _c(self.a), _c(o.a)
        out = np.empty_like(x)
        lib().orc_binary(op, self.code, _p(x), _p(y), _p(out), C.c_int64(x.size))
        return self._like(out)

    # ---- operators ----
    def __add__(self, o):
        return self._binary(o, OP_ADD) if isinstance(o, Ref) else self._scalar(OP_ADD_C, o)

    __radd__ = __add__

    def __sub__(self, o):
        return self._binary(o, OP_SUB) if isinstance(o, Ref) else self._scalar(OP_SUB_C, o)

    def __rsub__(self, o):
        return self._scalar(OP_RSUB_C, o)

    def __mul__(self, o):
        return self._binary(o, OP_MUL) if isinstance(o, Ref) else self._scalar(OP_MUL_C, o)

    __rmul__ = __mul__

    def __truediv__(self, o):
        return self._binary(o, OP_DIV) if isinstance(o, Ref) else self._scalar(OP_DIV_C, o)

    def __rtruediv__(self, o):
        return self._scalar(OP_RDIV_C, o)

    def __neg__(self):
        return self._unary(OP_NEG)

    def pow(self, o):
        return self._binary(o, OP_POW)

    def cast(self, code):
        x = _c(self.a)
        out = np.empty(x.shape, dtype=np.float32 if code == F32 else (np.float16 if code == F16 else np.uint16))
        lib().orc_cast(self.code, code, _p(x), _p(out), C.c_int64(x.size))
        return Ref(out, bf16=code == BF16)

    # ---- reduce / matmul ----
    def reduce(self, op, axis):
        x = _c(self.a)
        outer = int(np.prod(x.shape[:axis], dtype=np.int64))
        k = x.shape[axis]
        inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
        out = np.empty(x.shape[:axis] + x.shape[axis + 1:], dtype=x.dtype)
        lib().orc_reduce(op, self.code, _p(x), _p(out), C.c_int64(outer), C.c_int64(k), C.c_int64(inner))
        return self._like(out)

    def sum(self, axis):
        return self.reduce(OP_SUM, axis)

    def max(self, axis):
        return self.reduce(OP_MAX, axis)

    def min(self, axis):
        return self.reduce(OP_MIN, axis)

    def product(self, axis):
        return self.reduce(OP_PRODUCT, axis)

    def mat_mul(self, o):
        x, y = _c(self.a), _c(o.a)
        batch = x.shape[0] if x.ndim == 3 else 1
        M, K, N = x.shape[-2], x.shape[-1], y.shape[-1]
        out = np.empty(x.shape[:-1] + (N,), dtype=x.dtype)
        lib().orc_matmul(self.code, _p(x), _p(y), _p(out), C.c_int64(batch), C.c_int64(M), C.c_int64(N), C.c_int64(K))
        return self._like(out)

    # ---- views / moves: src/map_layout.rs:41-98, src/resize.rs:121-144, src/slice_assign.rs ----
    def slice(self, ranges):
        return self._like(self.a[tuple(slice(s, e) for s, e in ranges)])

    def transpose(self, a, b):
        return self._like(np.swapaxes(self.a, a, b))

    def broadcast_axis(self, axis, size):
        x = np.expand_dims(self.a, axis)
        shape = list(x.shape)
        shape[axis] = size
        return self._like(np.broadcast_to(x, shape))

    def broadcast(self, out_shape):
        new_dim = 0
        while new_dim < self.a.ndim and self.a.shape[new_dim] == out_shape[new_dim]:
            new_dim += 1
        assert tuple(self.a.shape[new_dim:]) == tuple(out_shape[new_dim + 1:])
        return self.broadcast_axis(new_dim, out_shape[new_dim])

    def expand(self, out_shape):
        return self._like(np.broadcast_to(self.a, out_shape))

    def resize(self, new_shape):
        out = np.zeros(new_shape, dtype=self.a.dtype)
        out[tuple(slice(0, s) for s in self.a.shape)] = self.a
        return self._like(out)

    def reshape(self, new_shape):
        return self._like(_c(self.a).reshape(new_shape))

    def slice_assign(self, ranges, value):
        out = np.array(self.a, copy=True)
        out[tuple(slice(s, e) for s, e in ranges)] = value.a
        return self._like(out)

    @staticmethod
    def cat(parts, dim):
        return parts[0]._like(np.concatenate([p.a for p in parts], axis=dim))

    def narrow(self, axis, start, length):
        return self.slice([(start, start + length) if i == axis else (0, s) for i, s in enumerate(self.shape)])

    def unsqueeze(self, axis):
        return self._like(np.expand_dims(_c(self.a), axis))

    # ---- composites: src/composite/*.rs ----
    def silu(self):
        return self / (1.0 + (-self).exp())

    def layer_norm(self, weight, eps):
        last = self.a.ndim - 1
        h = self.shape[last]
        f = self.cast(F32)
        norm = f.sqr().sum(last) / float(h)
        normed = f / (norm + eps).sqrt().broadcast_axis(last, h)
        w = weight
        for i in range(last):
            w = w.broadcast_axis(i, self.shape[i])
        return normed.cast(self.code) * w

    def softmax(self):
        e = self.exp()
        return e / e.sum(0).broadcast_axis(0, self.shape[0])

    def softmax_last_dim(self):
        last = self.a.ndim - 1
        h = self.shape[last]
        e = (self - self.max(last).broadcast_axis(last, h)).exp()
        return e / e.sum(last).broadcast_axis(last, h)

    def rope(self, cos, sin):
        heads, seq, d = self.shape
        c = Ref.cat([cos, cos], 1).narrow(0, 0, seq).broadcast_axis(0, heads)
        s = Ref.cat([sin, sin], 1).narrow(0, 0, seq).broadcast_axis(0, heads)
        x1, x2 = self.narrow(2, 0, d // 2), self.narrow(2, d // 2, d - d // 2)
        rot = Ref.cat([-x2, x1], 2)
        return self * c + rot * s


for _i, _name in enumerate(UNARY_NAMES):
    if _name != "neg":
        setattr(Ref, _name, (lambda op: lambda self: self._unary(op))(_i))


def arange(start, end, step=1.0, dtype=np.float32):
    """src/composite/arange.rs:8-23: accumulate in the element type."""
    vals = []
    cur, e, st = dtype(start), dtype(end), dtype(step)
    while (cur < e) if st >= 0 else (cur > e):
        vals.append(cur)
        cur = dtype(cur + st)
    return Ref(np.array(vals, dtype=dtype))


def ulp_diff_f32(got, ref):
    """Elementwise distance in units in the last place (NaN matches NaN)."""
    g = _c(got, dtype=np.float32).view(np.int32).astype(np.int64)
    r = _c(ref, dtype=np.float32).view(np.int32).astype(np.int64)
    g = np.where(g < 0, -(2 ** 31) - g, g)
    r = np.where(r < 0, -(2 ** 31) - r, r)
    d = np.abs(g - r)
    both_nan = np.isnan(got) & np.isnan(ref)
    one_nan = np.isnan(got) ^ np.isnan(ref)
    d = np.where(both_nan, 0, d)
    d = np.where(one_nan, 2 ** 40, d)
    return d


def ulp_diff_f16(got, ref):
    g = _c(got, dtype=np.float16).view(np.int16).astype(np.int64)
    r = _c(ref, dtype=np.float16).view(np.int16).astype(np.int64)
    g = np.where(g < 0, -(2 ** 15) - g, g)
    r = np.where(r < 0, -(2 ** 15) - r, r)
    d = np.abs(g - r)
    gn, rn = np.isnan(got.astype(np.float32)), np.isnan(ref.astype(np.float32))
    d = np.where(gn & rn, 0, d)
    d = np.where(gn ^ rn, 2 ** 40, d)
    return d
