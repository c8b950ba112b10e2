"""wgf_full_reduce_f32_noalloc: the full-tensor reduction for callers that cannot allocate
(work issued inside a CUDA stream capture, real-time loops, embedders with a fixed device-memory
budget).  Its scratch is a fixed array inside the library, so it is checked here against the
regular entry point, which takes its scratch from the device pool: same inputs, two calls in a
row (the array keeps what the first call left behind), reduction tolerance 1e-5 relative.

Collected last on purpose: a failure here cannot hide the result of any other test."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NONE = 0xFFFFFFFF


def _noalloc(wgf, dev, x_desc, n, pre, red, out_desc, offset_elems=0):
    lib = wgf.lib()
    xp, op = C.c_void_p(), C.c_void_p()
    wgf.check(lib.wgf_buffer_device_ptr(C.c_void_p(x_desc.buf), C.byref(xp), None))
    wgf.check(lib.wgf_buffer_device_ptr(C.c_void_p(out_desc.buf), C.byref(op), None))
    _, stream = dev.info()
    lib.wgf_full_reduce_f32_noalloc.argtypes = [C.c_void_p, C.c_uint64, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]
    return lib.wgf_full_reduce_f32_noalloc(C.c_void_p(xp.value + 4 * offset_elems), C.c_uint64(n), C.c_uint32(pre),
                                           C.c_uint32(red), op, C.c_void_p(stream))


def test_matches_pooled_reduce_twice_in_a_row(wgf, dev):
    g = np.random.Generator(np.random.PCG64(0xB2000000 + 16 * 2 + 7))
    a = g.standard_normal((1500, 1031)).astype(np.float32)          # ragged length: 1 546 500 elements
    b = (g.standard_normal(4099) * 0.5).astype(np.float32)
    cases = [(a, wgf.OP_EXP, wgf.OP_SUM, lambda t: t.exp()), (b, NONE, wgf.OP_MAX, lambda t: t),
             (a, wgf.OP_SQR, wgf.OP_SUM, lambda t: t.sqr()), (b, wgf.OP_ABS, wgf.OP_MIN, lambda t: t.abs())]
    out_t = dev.tensor(np.zeros(1, np.float32))
    out_desc = out_t.desc()
    mem_before = dev.memory()
    for x, pre, red, chain in cases:
        t = dev.tensor(x.reshape(-1))
        d = t.desc()
        # the existing entry point (scratch from the pool)
        want = float(chain(t).reduce(red, 0).as_slice())
        for _ in range(2):  # two calls in a row share the fixed scratch
            reserved = dev.memory()[0]
            wgf.check(_noalloc(wgf, dev, d, x.size, pre, red, out_desc))
            got = float(out_t_download(wgf, dev, out_desc))
            assert dev.memory()[0] == reserved            # the pool did not grow: nothing was allocated
            if red in (wgf.OP_MAX, wgf.OP_MIN):
                assert got == want
            else:
                assert abs(got - want) <= 1e-5 * abs(want)
        # unaligned start (pointer 4 bytes past a 16-byte boundary) and short input
        wgf.check(_noalloc(wgf, dev, d, x.size - 3, pre, red, out_desc, offset_elems=1))
        got = float(out_t_download(wgf, dev, out_desc))
        want2 = float(chain(dev.tensor(x.reshape(-1)[1:x.size - 2])).reduce(red, 0).as_slice())
        assert got == want2 if red in (wgf.OP_MAX, wgf.OP_MIN) else abs(got - want2) <= 1e-5 * abs(want2)
        lib_release(wgf, d)
    lib_release(wgf, out_desc)
    assert mem_before[0] >= 0


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
