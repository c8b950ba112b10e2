"""The kernel-level entry points (the seams where the crate's Untyped*Kernel::run_with_query bodies
would call in) checked against the CPU oracle."""
import ctypes as C

import numpy as np
import pytest

from conftest import seeded

pytestmark = pytest.mark.gpu


class Buf:
    """A device buffer + row-major descriptor made through wgf_buffer_*."""

    def __init__(self, wgf, dev, array):
        self.wgf, self.dev = wgf, dev
        a = np.ascontiguousarray(array)
        self.h = C.c_void_p()
        wgf.check(wgf.lib().wgf_buffer_alloc(dev.h, C.c_uint64(max(a.nbytes, 1)), C.c_int32(0), C.byref(self.h)))
        wgf.check(wgf.lib().wgf_buffer_upload(self.h, C.c_uint64(0), a.ctypes.data_as(C.c_void_p), C.c_uint64(a.nbytes)))
        self.dtype = wgf.F16 if a.dtype == np.float16 else wgf.F32
        self.shape = a.shape

    def desc(self, shape=None, strides=None, offset=0):
        shape = self.shape if shape is None else shape
        if strides is None:
            strides, acc = [], 1
            for s in reversed(shape):
                strides.insert(0, acc)
                acc *= s
        d = self.wgf.TensorDesc()
        d.buf, d.dtype, d.rank, d.offset = self.h.value, self.dtype, len(shape), offset
        for i, (s, st) in enumerate(zip(shape, strides)):
            d.shape[i], d.stride[i] = s, st
        return d

    def release(self):
        self.wgf.check(self.wgf.lib().wgf_buffer_release(self.h))


def fetch(wgf, desc, np_dtype):
    """Downloads the (row-major, offset 0) result described by `desc` and releases its buffer."""
    shape = tuple(desc.shape[i] for i in range(desc.rank))
    out = np.empty(shape, np_dtype)
    wgf.check(wgf.lib().wgf_buffer_download(C.c_void_p(desc.buf), C.c_uint64(desc.offset * out.itemsize),
                                            out.ctypes.data_as(C.c_void_p), C.c_uint64(out.nbytes)))
    wgf.check(wgf.lib().wgf_buffer_release(C.c_void_p(desc.buf)))
    return out


def chain(wgf, ops):
    arr = (wgf.EwOp * max(len(ops), 1))()
    for i, (op, imm, dt) in enumerate(ops):
        arr[i].opcode, arr[i].imm, arr[i].out_dtype = op, imm, dt
    return arr, len(ops)


def test_launch_elementwise_chain_and_inplace(wgf, dev, orc):
    x = seeded(0, 10).standard_normal((33, 70)).astype(np.float32)
    b = Buf(wgf, dev, x)
    ops, n = chain(wgf, [(wgf.OP_MUL_C, 2.0, 0), (wgf.OP_ADD_C, 1.0, 0), (wgf.OP_SIN, 0, 0)])
    out, timing = wgf.TensorDesc(), C.c_void_p()
    d = b.desc()
    wgf.check(wgf.lib().wgf_launch_elementwise(dev.h, C.byref(d), ops, C.c_uint32(n), C.c_int32(0), C.byref(out), C.byref(timing)))
    # the timing handle is read later (PerformanceQueries, src/query.rs:78-112): the launch did not wait
    ns, count = C.c_uint64(), C.c_uint32()
    wgf.check(wgf.lib().wgf_timing_kernel_count(timing, C.byref(count)))
    wgf.check(wgf.lib().wgf_timing_elapsed_ns(timing, C.byref(ns)))
    wgf.check(wgf.lib().wgf_timing_release(timing))
    assert out.buf != d.buf and ns.value > 0 and count.value == 1
    ref = (orc.Ref(x) * 2.0 + 1.0).sin().numpy()
    got = fetch(wgf, out, np.float32)
    assert orc.ulp_diff_f32(got, ref).max() <= 2
    # in place: same buffer comes back, its reference count went up by one
    ops, n = chain(wgf, [(wgf.OP_ADD_C, 1.0, 0)])
    wgf.check(wgf.lib().wgf_launch_elementwise(dev.h, C.byref(d), ops, C.c_uint32(n), C.c_int32(1), C.byref(out), None))
    assert out.buf == d.buf
    np.testing.assert_array_equal(fetch(wgf, out, np.float32), x + 1)
    # strided view as input (a column slice): new contiguous output
    v = b.desc(shape=(33, 10), strides=(70, 1), offset=5)
    ops, n = chain(wgf, [(wgf.OP_CAST, 0, wgf.F16)])
    wgf.check(wgf.lib().wgf_launch_elementwise(dev.h, C.byref(v), ops, C.c_uint32(n), C.c_int32(0), C.byref(out), None))
    np.testing.assert_array_equal(fetch(wgf, out, np.float16), (x + 1)[:, 5:15].astype(np.float16))
    b.release()


def test_launch_pairwise_with_prologues_and_epilogue(wgf, dev, orc):
    g = seeded(0, 11)
    x, y = g.standard_normal((5, 6, 40)).astype(np.float32), g.standard_normal((6, 40)).astype(np.float32)
    bx, by = Buf(wgf, dev, x), Buf(wgf, dev, y)
    dx, dy = bx.desc(), by.desc(shape=(5, 6, 40), strides=(0, 40, 1))     # y broadcast over axis 0
    pa, na = chain(wgf, [(wgf.OP_ADD_C, 1.0, 0)])
    pb, nb = chain(wgf, [(wgf.OP_MUL_C, 2.0, 0)])
    po, no = chain(wgf, [(wgf.OP_SUB_C, 1.0, 0)])
    out = wgf.TensorDesc()
    wgf.check(wgf.lib().wgf_launch_pairwise(dev.h, C.byref(dx), C.byref(dy), pa, C.c_uint32(na), pb, C.c_uint32(nb),
                                            C.c_uint32(wgf.OP_ADD), po, C.c_uint32(no), C.byref(out), None))
    np.testing.assert_array_equal(fetch(wgf, out, np.float32), ((x + 1) + (y[None] * 2)) - 1)
    bx.release()
    by.release()


@pytest.mark.parametrize("axis", [0, 1, 2])
def test_launch_reduce(axis, wgf, dev, orc):
    x = seeded(0, 12).standard_normal((9, 130, 17)).astype(np.float32)
    b = Buf(wgf, dev, x)
    d = b.desc()
    pre, npre = chain(wgf, [(wgf.OP_SQR, 0, 0)])
    post, npost = chain(wgf, [(wgf.OP_SQRT, 0, 0)])
    out = wgf.TensorDesc()
    wgf.check(wgf.lib().wgf_launch_reduce(dev.h, C.byref(d), C.c_uint32(axis), pre, C.c_uint32(npre),
                                          C.c_uint32(wgf.OP_SUM), post, C.c_uint32(npost), C.byref(out), None))
    got = fetch(wgf, out, np.float32)
    ref = np.sqrt((x.astype(np.float64) ** 2).sum(axis))
    assert got.shape == ref.shape and np.max(np.abs(got - ref) / ref) <= 1e-5
    b.release()


def test_launch_matmul_resize_slice_assign(wgf, dev, orc):
    g = seeded(4, 0)
    a, bm = g.standard_normal((37, 50)).astype(np.float32), g.standard_normal((50, 21)).astype(np.float32)
    ba, bb = Buf(wgf, dev, a), Buf(wgf, dev, bm)
    da, db, out = ba.desc(), bb.desc(), wgf.TensorDesc()
    wgf.check(wgf.lib().wgf_launch_matmul(dev.h, C.byref(da), C.byref(db), C.c_uint32(wgf.F32), C.byref(out), None))
    got = fetch(wgf, out, np.float32)
    ref = a.astype(np.float64) @ bm.astype(np.float64)
    assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) <= 1e-4
    # transposed view of a as left operand: strides are honoured (the crate ignores them, src/matmul.rs:96-117)
    dat = ba.desc(shape=(50, 37), strides=(1, 50))
    bc = Buf(wgf, dev, g.standard_normal((37, 8)).astype(np.float32))
    dc = bc.desc()
    wgf.check(wgf.lib().wgf_launch_matmul(dev.h, C.byref(dat), C.byref(dc), C.c_uint32(wgf.F32), C.byref(out), None))
    got = fetch(wgf, out, np.float32)
    # resize: zero-filled larger tensor with the input in its leading box (src/resize.rs:121-130)
    ns = (C.c_int64 * 2)(40, 64)
    fs = (C.c_int64 * 2)(37, 50)
    wgf.check(wgf.lib().wgf_launch_resize(dev.h, C.byref(da), C.c_uint32(2), ns, fs, C.byref(out), None))
    big = fetch(wgf, out, np.float32)
    want = np.zeros((40, 64), np.float32)
    want[:37, :50] = a
    np.testing.assert_array_equal(big, want)
    # reshape through the same entry point (new_shape == fill_shape, src/resize.rs:132-144)
    ns = (C.c_int64 * 1)(37 * 50)
    wgf.check(wgf.lib().wgf_launch_resize(dev.h, C.byref(da), C.c_uint32(1), ns, ns, C.byref(out), None))
    np.testing.assert_array_equal(fetch(wgf, out, np.float32), a.reshape(-1))
    # slice_assign writes into the target's buffer (src/slice_assign.rs:68-72)
    val = Buf(wgf, dev, np.full((3, 4), 7.0, np.float32))
    dv = val.desc()
    st, en = (C.c_int64 * 2)(2, 5), (C.c_int64 * 2)(5, 9)
    wgf.check(wgf.lib().wgf_launch_slice_assign(dev.h, C.byref(da), st, en, C.byref(dv), None))
    ba.wgf.check(wgf.lib().wgf_buffer_retain(ba.h))
    da2 = ba.desc()
    now = fetch(wgf, da2, np.float32)
    want = a.copy()
    want[2:5, 5:9] = 7.0
    np.testing.assert_array_equal(now, want)
    for b in (ba, bb, bc, val):
        b.release()


def test_buffer_use_count_and_bad_descriptors(wgf, dev):
    b = Buf(wgf, dev, np.zeros(16, np.float32))
    n = C.c_int64()
    wgf.check(wgf.lib().wgf_buffer_use_count(b.h, C.byref(n)))
    assert n.value == 1
    t = C.c_void_p()
    d = b.desc()
    wgf.check(wgf.lib().wgf_tensor_from_desc(dev.h, C.byref(d), C.byref(t)))
    wgf.check(wgf.lib().wgf_buffer_use_count(b.h, C.byref(n)))
    assert n.value == 2                       # the graph leaf holds a reference (src/tensor.rs:413-415)
    wgf.check(wgf.lib().wgf_tensor_release(t))
    wgf.check(wgf.lib().wgf_buffer_use_count(b.h, C.byref(n)))
    assert n.value == 1
    bad = b.desc(shape=(4, 8), strides=(8, 1))   # reaches past the 16 elements
    out = wgf.TensorDesc()
    ops, k = chain(wgf, [(wgf.OP_EXP, 0, 0)])
    rc = wgf.lib().wgf_launch_elementwise(dev.h, C.byref(bad), ops, C.c_uint32(k), C.c_int32(0), C.byref(out), None)
    assert wgf.STATUS[rc] == "INVALID_ARGUMENT"
    assert wgf.STATUS[wgf.lib().wgf_buffer_release(None)] == "INVALID_HANDLE"
    b.release()


def test_matmul_accumulator_type_and_async_upload(wgf, dev):
    """The accumulator of wgf_launch_matmul is f32 for every element type: asking for another one is
    refused, not ignored.  wgf_buffer_upload_async copies from page-locked memory without waiting and
    hands back a handle that can be waited for and gives the copy time."""
    g = seeded(4, 11)
    a, bm = g.standard_normal((64, 64)).astype(np.float16), g.standard_normal((64, 64)).astype(np.float16)
    ba, bb = Buf(wgf, dev, a), Buf(wgf, dev, bm)
    da, db, out = ba.desc(), bb.desc(), wgf.TensorDesc()
    rc = wgf.lib().wgf_launch_matmul(dev.h, C.byref(da), C.byref(db), C.c_uint32(wgf.F16), C.byref(out), None)
    assert wgf.STATUS[rc] == "UNSUPPORTED"
    rc = wgf.lib().wgf_launch_matmul(dev.h, C.byref(da), C.byref(db), C.c_uint32(77), C.byref(out), None)
    assert wgf.STATUS[rc] == "DTYPE"
    timing = C.c_void_p()
    wgf.check(wgf.lib().wgf_launch_matmul(dev.h, C.byref(da), C.byref(db), C.c_uint32(wgf.F32), C.byref(out), C.byref(timing)))
    ns = C.c_uint64()
    wgf.check(wgf.lib().wgf_timing_elapsed_ns(timing, C.byref(ns)))
    wgf.check(wgf.lib().wgf_timing_release(timing))
    got = fetch(wgf, out, np.float16).astype(np.float64)
    ref = a.astype(np.float64) @ bm.astype(np.float64)
    assert ns.value > 0 and np.max(np.abs(got - ref)) / np.max(np.abs(ref)) <= 1e-2
    # asynchronous upload into the middle of a buffer
    n = 1 << 20
    pin = wgf.PinnedArray((n,), np.float32)
    pin.array[...] = g.standard_normal(n, dtype=np.float32)
    buf = C.c_void_p()
    wgf.check(wgf.lib().wgf_buffer_alloc(dev.h, C.c_uint64(8 * n), C.c_int32(1), C.byref(buf)))
    done = C.c_void_p()
    wgf.check(wgf.lib().wgf_buffer_upload_async(buf, C.c_uint64(4 * n), C.c_void_p(pin.ptr.value), C.c_uint64(4 * n), C.byref(done)))
    wgf.check(wgf.lib().wgf_timing_wait(done))
    wgf.check(wgf.lib().wgf_timing_elapsed_ns(done, C.byref(ns)))
    wgf.check(wgf.lib().wgf_timing_release(done))
    back = np.empty(2 * n, np.float32)
    wgf.check(wgf.lib().wgf_buffer_download(buf, C.c_uint64(0), back.ctypes.data_as(C.c_void_p), C.c_uint64(8 * n)))
    wgf.check(wgf.lib().wgf_buffer_release(buf))
    assert ns.value > 0 and not back[:n].any() and np.array_equal(back[n:], pin.array)
    pageable = np.zeros(16, np.float32)
    wgf.check(wgf.lib().wgf_buffer_alloc(dev.h, C.c_uint64(64), C.c_int32(0), C.byref(buf)))
    rc = wgf.lib().wgf_buffer_upload_async(buf, C.c_uint64(0), pageable.ctypes.data_as(C.c_void_p), C.c_uint64(64), None)
    wgf.check(wgf.lib().wgf_buffer_release(buf))
    assert wgf.STATUS[rc] == "INVALID_ARGUMENT"
