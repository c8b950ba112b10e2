"""wgf_full_reduce_f32_noalloc: the full-tensor reduction for callers of this library that cannot
let a compute call reach the device allocator (real-time loops that rule out calls of unbounded
latency, embedders whose device-memory budget is fixed up front).  Its scratch is a fixed array
inside the library image, so it is checked here against the regular entry point, which takes its
scratch from the device pool -- same inputs, two calls in a row (the array keeps what the first call
left behind) -- and against float64 numpy; reduction tolerance 1e-5 relative.

Collected last on purpose: a failure here cannot hide the result of any other test."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NONE = 0xFFFFFFFF
F32_MAX = np.float32(3.40282e38)


def _noalloc(wgf, dev, x_desc, n, pre, red, out_desc, offset_elems=0):
    lib = wgf.lib()
    xp, op = C.c_void_p(), C.c_void_p()
    wgf.check(lib.wgf_buffer_device_ptr(C.c_void_p(x_desc.buf), C.byref(xp), None))
    wgf.check(lib.wgf_buffer_device_ptr(C.c_void_p(out_desc.buf), C.byref(op), None))
    _, stream = dev.info()
    lib.wgf_full_reduce_f32_noalloc.argtypes = [C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
    return lib.wgf_full_reduce_f32_noalloc(C.c_void_p(xp.value + 4 * offset_elems), C.c_uint64(n), C.c_uint32(pre),
                                           C.c_uint32(red), op, C.c_void_p(stream))


def free_device_memory(ordinal):
    """cudaMemGetInfo of the device: what ANY allocation on it, pooled or not, would lower."""
    import torch
    return torch.cuda.mem_get_info(ordinal)[0]


def numpy_reduce(x, pre, red, wgf):
    v = x.astype(np.float64)
    v = {wgf.OP_EXP: np.exp, wgf.OP_SQR: np.square, wgf.OP_ABS: np.abs}.get(pre, lambda a: a)(v)
    if v.size == 0:   # the reduction's identity
        return {wgf.OP_SUM: 0.0, wgf.OP_PRODUCT: 1.0, wgf.OP_MAX: -float(F32_MAX), wgf.OP_MIN: float(F32_MAX)}[red]
    return float({wgf.OP_SUM: np.sum, wgf.OP_PRODUCT: np.prod, wgf.OP_MAX: np.max, wgf.OP_MIN: np.min}[red](v))


def close(got, want, red, wgf):
    if red in (wgf.OP_MAX, wgf.OP_MIN):
        return np.float32(got) == np.float32(want)
    return abs(got - want) <= 1e-5 * abs(want)


def test_matches_pooled_reduce_and_float64_twice_in_a_row(wgf, dev):
    g = np.random.Generator(np.random.PCG64(0xB2000000 + 16 * 2 + 7))
    a = g.standard_normal((1500, 1031)).astype(np.float32)          # ragged length: 1 546 500 elements
    b = (g.standard_normal(4099) * 0.5).astype(np.float32)
    p = (1 + 1e-3 * g.standard_normal(3000)).astype(np.float32)     # a product that stays near 1
    cases = [(a, wgf.OP_EXP, wgf.OP_SUM, lambda t: t.exp()), (b, NONE, wgf.OP_MAX, lambda t: t),
             (a, wgf.OP_SQR, wgf.OP_SUM, lambda t: t.sqr()), (b, wgf.OP_ABS, wgf.OP_MIN, lambda t: t.abs()),
             (p, NONE, wgf.OP_PRODUCT, lambda t: t), (b[:3], NONE, wgf.OP_SUM, lambda t: t)]
    out_t = dev.tensor(np.zeros(1, np.float32))
    out_desc = out_t.desc()
    free_device_memory(dev.ordinal)                                 # sets up the measuring side's own context first
    for x, pre, red, chain in cases:
        t = dev.tensor(x.reshape(-1))
        d = t.desc()
        want = float(chain(t).reduce(red, 0).as_slice())            # the existing entry point (scratch from the pool)
        exact = numpy_reduce(x, pre, red, wgf)
        # The first launch of a kernel variant lets the driver load its code (CUDA loads kernels
        # lazily, and that takes device memory once); it is made here, before the memory is watched.
        wgf.check(_noalloc(wgf, dev, d, x.size, pre, red, out_desc))
        for _ in range(2):                                          # two calls in a row share the fixed scratch
            dev.sync()
            free_before = free_device_memory(dev.ordinal)
            wgf.check(_noalloc(wgf, dev, d, x.size, pre, red, out_desc))
            dev.sync()
            assert free_device_memory(dev.ordinal) >= free_before   # nothing was taken from the device
            got = float(out_t_download(wgf, dev, out_desc))
            assert close(got, want, red, wgf), (got, want)
            assert close(got, exact, red, wgf), (got, exact)
        if x.size > 8:
            # unaligned start (pointer 4 bytes past a 16-byte boundary) and short input
            wgf.check(_noalloc(wgf, dev, d, x.size - 3, pre, red, out_desc, offset_elems=1))
            got = float(out_t_download(wgf, dev, out_desc))
            assert close(got, numpy_reduce(x.reshape(-1)[1:x.size - 2], pre, red, wgf), red, wgf)
        # nothing to reduce: the identity of the reduction
        wgf.check(_noalloc(wgf, dev, d, 0, pre, red, out_desc))
        assert close(float(out_t_download(wgf, dev, out_desc)), numpy_reduce(x[:0], pre, red, wgf), red, wgf)
        lib_release(wgf, d)
    lib_release(wgf, out_desc)


def test_second_gpu_has_its_own_scratch_address(wgf, dev):
    """The array's device address is looked up once per GPU, with that GPU current: a call whose
    input lives on GPU 1 after one on GPU 0 must use GPU 1's copy of the array."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    g = np.random.Generator(np.random.PCG64(0xB2000000 + 16 * 2 + 8))
    x = g.standard_normal(1 << 20).astype(np.float32)
    devices = [dev, wgf.Device(1)]
    for _ in range(2):
        for d in devices:
            t, o = d.tensor(x), d.tensor(np.zeros(1, np.float32))
            td, od = t.desc(), o.desc()
            wgf.check(_noalloc(wgf, d, td, x.size, wgf.OP_SQR, wgf.OP_SUM, od))
            got = float(out_t_download(wgf, d, od))
            assert abs(got - numpy_reduce(x, wgf.OP_SQR, wgf.OP_SUM, wgf)) <= 1e-5 * got
            lib_release(wgf, td)
            lib_release(wgf, od)


def test_rejects_what_it_cannot_do(wgf, dev):
    t = dev.tensor(np.ones(16, np.float32))
    d, o = t.desc(), dev.tensor(np.zeros(1, np.float32)).desc()
    rc = _noalloc(wgf, dev, d, (1 << 31) + 1, NONE, wgf.OP_SUM, o)
    assert wgf.STATUS[rc] == "UNSUPPORTED" and b"maximum" in wgf.lib().wgf_last_error()
    assert wgf.STATUS[_noalloc(wgf, dev, d, 16, wgf.OP_SIN, wgf.OP_SUM, o)] == "INVALID_ARGUMENT"
    assert wgf.STATUS[_noalloc(wgf, dev, d, 16, NONE, wgf.OP_ADD, o)] == "INVALID_ARGUMENT"
    lib_release(wgf, d)
    lib_release(wgf, o)


def out_t_download(wgf, dev, desc):
    host = np.zeros(1, np.float32)
    wgf.check(wgf.lib().wgf_buffer_download(C.c_void_p(desc.buf), C.c_uint64(0), host.ctypes.data_as(C.c_void_p),
                                            C.c_uint64(4)))
    return host[0]


def lib_release(wgf, desc):
    wgf.check(wgf.lib().wgf_buffer_release(C.c_void_p(desc.buf)))
