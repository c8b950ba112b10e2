"""ctypes binding of libwgf.so (include/wgf.h) and a thin `Tensor` mirror of the crate's
`Tensor<R, D>` API (src/tensor.rs:418-644) for tests and benchmarks.

Everything here goes through the C ABI.  There is no CPU implementation behind it: without
the library, or without a GPU, calls raise.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libwgf.so")
MAX_RANK = 8

F32, F16, BF16 = 0, 1, 2
_NP = {F32: np.float32, F16: np.float16, BF16: np.uint16}

# opcodes (include/wgf.h)
(OP_EXP, OP_EXP2, OP_LOG, OP_LOG2, OP_SQR, OP_SQRT, OP_SIN, OP_COS, OP_TAN, OP_ASIN, OP_ACOS,
 OP_ATAN, OP_SINH, OP_COSH, OP_TANH, OP_ASINH, OP_ACOSH, OP_ATANH, OP_ABS, OP_NEG) = range(20)
OP_ADD_C, OP_SUB_C, OP_RSUB_C, OP_MUL_C, OP_DIV_C, OP_RDIV_C = range(32, 38)
OP_CAST = 48
OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_POW = range(64, 69)
OP_SUM, OP_MAX, OP_MIN, OP_PRODUCT = range(96, 100)
UNARY_NAMES = ["exp", "exp2", "log", "log2", "sqr", "sqrt", "sin", "cos", "tan", "asin", "acos", "atan",
               "sinh", "cosh", "tanh", "asinh", "acosh", "atanh", "abs", "neg"]

STATUS = {0: "OK", 1: "SHAPE", 2: "DTYPE", 3: "RANK", 4: "OOM", 5: "CUDA", 6: "NCCL", 7: "TIMEOUT",
          8: "INVALID_HANDLE", 9: "INVALID_ARGUMENT", 10: "COMPILE", 11: "UNSUPPORTED"}


class WgfError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"WGF_ERR_{STATUS.get(code, code)}: {msg}")
        self.code = code
        self.status = STATUS.get(code, str(code))


class TensorDesc(C.Structure):
    _fields_ = [("buf", C.c_void_p), ("dtype", C.c_uint32), ("rank", C.c_uint32), ("offset", C.c_int64),
                ("shape", C.c_int64 * MAX_RANK), ("stride", C.c_int64 * MAX_RANK)]


class EwOp(C.Structure):
    _fields_ = [("opcode", C.c_uint16), ("out_dtype", C.c_uint16), ("imm", C.c_float)]


_lib = None


def lib():
    """Loads libwgf.so (built by build.py).  Fails loudly when it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python {os.path.join(HERE, 'build.py')}` first")
        os.environ.setdefault("WGF_KERNEL_CACHE", os.path.join(HERE, "_jit_cache"))
        _lib = C.CDLL(LIB_PATH)
        _lib.wgf_last_error.restype = C.c_char_p
    return _lib


def check(status):
    if status != 0:
        raise WgfError(status, lib().wgf_last_error().decode(errors="replace"))


def _i64(seq):
    seq = [int(v) for v in seq]
    return (C.c_int64 * max(len(seq), 1))(*seq)


class Device:
    """Device::new (src/device.rs:14-32).  ordinal -1 = compile-only device (no GPU)."""

    def __init__(self, ordinal=0):
        self.h = C.c_void_p()
        check(lib().wgf_device_create(C.c_int32(ordinal), C.byref(self.h)))
        self.ordinal = ordinal

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.wgf_device_release(self.h)
            self.h = None

    def sync(self):
        check(lib().wgf_device_sync(self.h))

    def set_timing(self, on):
        check(lib().wgf_device_set_timing(self.h, C.c_int32(1 if on else 0)))

    @property
    def launch_count(self):
        v = C.c_uint64()
        check(lib().wgf_device_launch_count(self.h, C.byref(v)))
        return v.value

    @property
    def compile_count(self):
        v = C.c_uint64()
        check(lib().wgf_device_compile_count(self.h, C.byref(v)))
        return v.value

    def memory(self):
        a, b = C.c_uint64(), C.c_uint64()
        check(lib().wgf_device_memory(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def info(self):
        sm, st = C.c_int32(), C.c_void_p()
        check(lib().wgf_device_info(self.h, C.byref(sm), C.byref(st)))
        return sm.value, st.value

    def tensor(self, data, dtype=None):
        return Tensor.new(self, data, dtype)

    def tensor_pinned(self, pinned, dtype=None):
        """Asynchronous upload from a PinnedArray: returns at once; keep the array unchanged until a
        synchronising call has returned."""
        a = pinned.array
        if dtype is None:
            dtype = F16 if a.dtype == np.float16 else F32
        out = C.c_void_p()
        check(lib().wgf_tensor_from_host_pinned(self.h, C.c_uint32(dtype), C.c_uint32(a.ndim), _i64(a.shape),
                                                C.c_void_p(pinned.ptr.value), C.byref(out)))
        return Tensor(self, out)

    def record(self):
        """`with dev.record() as s:` captures every kernel queued inside the block as one schedule
        (wgf_schedule_begin / _end); afterwards `s.launch()` replays them with one call."""
        return Schedule(self)

    def arange(self, start, end, step=1.0, dtype=F32):
        out = C.c_void_p()
        check(lib().wgf_tensor_arange(self.h, C.c_uint32(dtype), C.c_float(start), C.c_float(end),
                                      C.c_float(step), C.byref(out)))
        return Tensor(self, out)


class Tensor:
    """Handle on a lazy graph node.  Python operators mirror the crate's operator impls."""

    def __init__(self, dev, handle):
        self.dev = dev
        self.h = handle

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.wgf_tensor_release(self.h)
            self.h = None

    # ---- construction / introspection -------------------------------------------------
    @staticmethod
    def new(dev, data, dtype=None):
        a = np.asarray(data)
        if dtype is None:
            dtype = F16 if a.dtype == np.float16 else F32
        if dtype == BF16:
            a = np.ascontiguousarray(a, dtype=np.uint16)
        else:
            a = np.ascontiguousarray(a, dtype=_NP[dtype])
        out = C.c_void_p()
        check(lib().wgf_tensor_from_host(dev.h, C.c_uint32(dtype), C.c_uint32(a.ndim), _i64(a.shape),
                                         a.ctypes.data_as(C.c_void_p), C.byref(out)))
        return Tensor(dev, out)

    def _info(self):
        dt, rk = C.c_uint32(), C.c_uint32()
        shp = (C.c_int64 * MAX_RANK)()
        check(lib().wgf_tensor_info(self.h, C.byref(dt), C.byref(rk), shp))
        return dt.value, tuple(shp[i] for i in range(rk.value))

    @property
    def shape(self):
        return self._info()[1]

    @property
    def dtype(self):
        return self._info()[0]

    @property
    def rank(self):
        return len(self.shape)

    def clone(self):
        out = C.c_void_p()
        check(lib().wgf_tensor_clone(self.h, C.byref(out)))
        return Tensor(self.dev, out)

    def release(self):
        """Drops this handle now (Rust's move semantics: `t + 1.0` consumes `t`)."""
        if self.h:
            check(lib().wgf_tensor_release(self.h))
            self.h = None

    # ---- helpers ----------------------------------------------------------------------
    def _un(self, fn, *args):
        out = C.c_void_p()
        check(fn(self.h, *args, C.byref(out)))
        return Tensor(self.dev, out)

    def unary(self, op):
        return self._un(lib().wgf_tensor_unary, C.c_uint32(op))

    def scalar(self, op, c):
        return self._un(lib().wgf_tensor_scalar, C.c_uint32(op), C.c_float(c))

    def binary(self, other, op):
        out = C.c_void_p()
        check(lib().wgf_tensor_binary(self.h, other.h, C.c_uint32(op), C.byref(out)))
        return Tensor(self.dev, out)

    # ---- operators (src/element_wise.rs:197-651, src/pair_wise.rs:205-489) --------------
    def __add__(self, o):
        return self.binary(o, OP_ADD) if isinstance(o, Tensor) else self.scalar(OP_ADD_C, o)

    __radd__ = __add__

    def __sub__(self, o):
        return self.binary(o, OP_SUB) if isinstance(o, Tensor) else self.scalar(OP_SUB_C, o)

    def __rsub__(self, o):
        return self.scalar(OP_RSUB_C, o)

    def __mul__(self, o):
        return self.binary(o, OP_MUL) if isinstance(o, Tensor) else self.scalar(OP_MUL_C, o)

    __rmul__ = __mul__

    def __truediv__(self, o):
        return self.binary(o, OP_DIV) if isinstance(o, Tensor) else self.scalar(OP_DIV_C, o)

    def __rtruediv__(self, o):
        return self.scalar(OP_RDIV_C, o)

    def __neg__(self):
        return self.unary(OP_NEG)

    def pow(self, o):
        return self.binary(o, OP_POW)

    def cast(self, dtype):
        return self._un(lib().wgf_tensor_cast, C.c_uint32(dtype))

    # ---- reductions / matmul -----------------------------------------------------------
    def reduce(self, op, axis):
        return self._un(lib().wgf_tensor_reduce, C.c_uint32(op), C.c_uint32(axis))

    def sum(self, axis):
        return self.reduce(OP_SUM, axis)

    def max(self, axis):
        return self.reduce(OP_MAX, axis)

    def min(self, axis):
        return self.reduce(OP_MIN, axis)

    def product(self, axis):
        return self.reduce(OP_PRODUCT, axis)

    def mat_mul(self, o):
        out = C.c_void_p()
        check(lib().wgf_tensor_matmul(self.h, o.h, C.byref(out)))
        return Tensor(self.dev, out)

    # ---- views / moves -----------------------------------------------------------------
    def slice(self, ranges):
        return self._un(lib().wgf_tensor_slice, _i64([r[0] for r in ranges]), _i64([r[1] for r in ranges]))

    def transpose(self, a, b):
        return self._un(lib().wgf_tensor_transpose, C.c_uint32(a), C.c_uint32(b))

    def broadcast(self, out_shape):
        return self._un(lib().wgf_tensor_broadcast, C.c_uint32(len(out_shape)), _i64(out_shape))

    def broadcast_axis(self, axis, size):
        return self._un(lib().wgf_tensor_broadcast_axis, C.c_uint32(axis), C.c_int64(size))

    def expand(self, out_shape):
        return self._un(lib().wgf_tensor_expand, _i64(out_shape))

    def resize(self, new_shape):
        return self._un(lib().wgf_tensor_resize, _i64(new_shape))

    def reshape(self, new_shape):
        return self._un(lib().wgf_tensor_reshape, C.c_uint32(len(new_shape)), _i64(new_shape))

    def slice_assign(self, ranges, value):
        out = C.c_void_p()
        check(lib().wgf_tensor_slice_assign(self.h, _i64([r[0] for r in ranges]), _i64([r[1] for r in ranges]),
                                            value.h, C.byref(out)))
        return Tensor(self.dev, out)

    @staticmethod
    def cat(parts, dim):
        arr = (C.c_void_p * len(parts))(*[p.h for p in parts])
        out = C.c_void_p()
        check(lib().wgf_tensor_cat(arr, C.c_uint32(len(parts)), C.c_uint32(dim), C.byref(out)))
        return Tensor(parts[0].dev, out)

    def narrow(self, axis, start, length):
        return self._un(lib().wgf_tensor_narrow, C.c_uint32(axis), C.c_int64(start), C.c_int64(length))

    def unsqueeze(self, axis):
        return self._un(lib().wgf_tensor_unsqueeze, C.c_uint32(axis))

    # ---- composites --------------------------------------------------------------------
    def silu(self):
        return self._un(lib().wgf_tensor_silu)

    def layer_norm(self, weight, eps):
        out = C.c_void_p()
        check(lib().wgf_tensor_layer_norm(self.h, weight.h, C.c_float(eps), C.byref(out)))
        return Tensor(self.dev, out)

    rms_norm = layer_norm

    def softmax(self):
        return self._un(lib().wgf_tensor_softmax)

    def softmax_last_dim(self):
        return self._un(lib().wgf_tensor_softmax_last_dim)

    def rope(self, cos, sin):
        out = C.c_void_p()
        check(lib().wgf_tensor_rope(self.h, cos.h, sin.h, C.byref(out)))
        return Tensor(self.dev, out)

    def llama_block(self, weights, norm1, norm2, cos, sin, mask, n_heads, eps=1e-5):
        """Llama-style decoder block forward; weights = [Wq, Wk, Wv, Wo, Wg, Wu, Wd], each [out, in].
        mask: additive [seq, seq] tensor, or None for causal attention through the fused kernel."""
        arr = (C.c_void_p * 7)(*[w.h for w in weights])
        out = C.c_void_p()
        check(lib().wgf_tensor_llama_block(self.h, arr, norm1.h, norm2.h, cos.h, sin.h, mask.h if mask is not None else None,
                                           C.c_uint32(n_heads), C.c_float(eps), C.byref(out)))
        return Tensor(self.dev, out)

    def attention(self, k, v, mask=None, causal=False, scale=None):
        """softmax(scale * self k^T + mask) v for [batch*heads, seq, head_dim] tensors (wgf_tensor_attention)."""
        if scale is None:
            scale = 1.0 / float(np.sqrt(self.shape[-1]))
        out = C.c_void_p()
        check(lib().wgf_tensor_attention(self.h, k.h, v.h, mask.h if mask is not None else None, C.c_int32(1 if causal else 0),
                                         C.c_float(scale), C.byref(out)))
        return Tensor(self.dev, out)

    def all_reduce(self, comm, op=OP_SUM):
        out = C.c_void_p()
        check(lib().wgf_tensor_all_reduce(self.h, comm.h, C.c_uint32(op), C.byref(out)))
        return Tensor(self.dev, out)

    # ---- materialisation ---------------------------------------------------------------
    def materialize(self):
        check(lib().wgf_tensor_materialize(self.h))
        return self

    @staticmethod
    def materialize_all(tensors):
        """One request for several tensors: a whole-tensor reduction among them rides along in the
        row kernel of another one over the same index space (wgf_tensor_materialize_many)."""
        arr = (C.c_void_p * len(tensors))(*[t.h for t in tensors])
        check(lib().wgf_tensor_materialize_many(arr, C.c_uint32(len(tensors))))
        return tensors

    def desc(self):
        d = TensorDesc()
        check(lib().wgf_tensor_desc_of(self.h, C.byref(d)))
        return d

    def as_slice(self):
        """Tensor::as_slice (src/tensor.rs:551-554): resolves the graph and downloads."""
        dt, shape = self._info()
        out = np.empty(shape, dtype=_NP[dt])
        check(lib().wgf_tensor_download(self.h, out.ctypes.data_as(C.c_void_p), C.c_uint64(out.nbytes)))
        return out

    def write(self, data):
        """New contents for a materialised, contiguous tensor, written into the buffer it already
        has (the way to feed the inputs of a recorded schedule)."""
        dt, shape = self._info()
        a = np.ascontiguousarray(data, dtype=_NP[dt])
        if tuple(a.shape) != tuple(shape):
            raise ValueError(f"shape {a.shape} does not match the tensor's {tuple(shape)}")
        d = self.desc()
        try:
            want = [int(np.prod(shape[i + 1:], dtype=np.int64)) for i in range(len(shape))]
            if any(shape[i] > 1 and d.stride[i] != want[i] for i in range(len(shape))):
                raise ValueError("write needs a contiguous tensor")
            check(lib().wgf_buffer_upload(C.c_void_p(d.buf), C.c_uint64(d.offset * a.itemsize),
                                          a.ctypes.data_as(C.c_void_p), C.c_uint64(a.nbytes)))
        finally:
            lib().wgf_buffer_release(C.c_void_p(d.buf))
        return self

    def download_into(self, out):
        check(lib().wgf_tensor_download(self.h, out.ctypes.data_as(C.c_void_p), C.c_uint64(out.nbytes)))
        return out

    def all_timing_information(self):
        n = C.c_uint32()
        check(lib().wgf_tensor_timing(self.h, None, C.c_uint32(0), C.byref(n)))
        arr = (C.c_uint64 * max(n.value, 1))()
        check(lib().wgf_tensor_timing(self.h, arr, C.c_uint32(n.value), C.byref(n)))
        return [arr[i] for i in range(n.value)]

    def timing_labels(self):
        """Kernel names matching all_timing_information(), in launch order."""
        need = C.c_uint64()
        check(lib().wgf_tensor_timing_labels(self.h, None, C.c_uint64(0), C.byref(need)))
        buf = C.create_string_buffer(need.value)
        check(lib().wgf_tensor_timing_labels(self.h, buf, C.c_uint64(need.value), C.byref(need)))
        return [s for s in buf.value.decode().split("\n") if s]

    def graphvis(self):
        need = C.c_uint64()
        check(lib().wgf_tensor_graphviz(self.h, None, C.c_uint64(0), C.byref(need)))
        buf = C.create_string_buffer(need.value)
        check(lib().wgf_tensor_graphviz(self.h, buf, C.c_uint64(need.value), C.byref(need)))
        return buf.value.decode()

    def graph_size(self):
        n = C.c_uint64()
        check(lib().wgf_tensor_graph_size(self.h, C.byref(n)))
        return n.value


for _i, _name in enumerate(UNARY_NAMES):
    if _name == "neg":
        continue
    setattr(Tensor, _name, (lambda op: lambda self: self.unary(op))(_i))


class PinnedArray:
    """numpy array over page-locked host memory (wgf_host_alloc)."""

    def __init__(self, shape, dtype):
        self.nbytes = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
        self.ptr = C.c_void_p()
        check(lib().wgf_host_alloc(C.c_uint64(self.nbytes), C.byref(self.ptr)))
        buf = (C.c_char * max(self.nbytes, 1)).from_address(self.ptr.value)
        self.array = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape, dtype=np.int64))).reshape(shape)

    def __del__(self):
        if getattr(self, "ptr", None) and _lib is not None:
            self.array = None
            _lib.wgf_host_free(self.ptr)
            self.ptr = None


class Schedule:
    """A recorded schedule (wgf_schedule_*): the kernels of the materialisations made inside the
    `with` block, replayed by `launch()`.  Inputs are tensors created before the block; feed them
    with `Tensor.write`.  Tensors materialised inside hold the values of the latest launch."""

    def __init__(self, dev):
        self.dev = dev
        self.h = None

    def __enter__(self):
        check(lib().wgf_schedule_begin(self.dev.h))
        return self

    def __exit__(self, exc_type, exc, tb):
        h = C.c_void_p()
        status = lib().wgf_schedule_end(self.dev.h, C.byref(h))
        if exc_type is None:
            check(status)
            self.h = h
        elif status == 0:
            lib().wgf_schedule_destroy(h)
        return False

    def launch(self):
        check(lib().wgf_schedule_launch(self.h))

    @property
    def kernel_count(self):
        v = C.c_uint64()
        check(lib().wgf_schedule_kernel_count(self.h, C.byref(v)))
        return v.value

    def destroy(self):
        if self.h:
            check(lib().wgf_schedule_destroy(self.h))
            self.h = None

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.wgf_schedule_destroy(self.h)
            self.h = None


def shard_range(n_units, world, rank):
    b, e = C.c_int64(), C.c_int64()
    check(lib().wgf_shard_range(C.c_int64(n_units), C.c_int32(world), C.c_int32(rank), C.byref(b), C.byref(e)))
    return b.value, e.value


class Comm:
    def __init__(self, dev, world, rank, unique_id):
        self.h = C.c_void_p()
        idb = (C.c_uint8 * 128).from_buffer_copy(bytes(unique_id))
        check(lib().wgf_comm_create(dev.h, C.c_int32(world), C.c_int32(rank), idb, C.byref(self.h)))

    @staticmethod
    def unique_id():
        idb = (C.c_uint8 * 128)()
        check(lib().wgf_comm_unique_id(idb))
        return bytes(idb)

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.wgf_comm_release(self.h)
            self.h = None
