"""CUDA path vs CPU oracle on identical seeded inputs.  Tolerances: element-wise <= 2 ulp f32
(<= 1 ulp f16), casts / moves / index ops bit-exact, reductions 1e-5 relative."""
import numpy as np
import pytest

from conftest import seeded

pytestmark = pytest.mark.gpu

ULP = 2


def ulps(orc, got, ref):
    return int(orc.ulp_diff_f32(got, ref).max()) if got.size else 0


def assert_ulp(orc, got, ref, tol=ULP):
    assert got.shape == ref.shape and got.dtype == ref.dtype
    if got.dtype == np.float16:
        d = orc.ulp_diff_f16(got, ref)
    else:
        d = orc.ulp_diff_f32(got, ref)
    worst = int(d.max()) if d.size else 0
    assert worst <= tol, f"max ulp distance {worst} > {tol} at {np.unravel_index(d.argmax(), d.shape)}"


def assert_rel(got, ref, tol):
    g, r = got.astype(np.float64), ref.astype(np.float64)
    err = np.abs(g - r) / np.maximum(np.abs(r), 1e-30)
    assert err.max() <= tol, f"max relative error {err.max():.3e} > {tol}"


UNARY_DOMAIN = {
    "exp": (-10, 10), "exp2": (-10, 10), "log": (1e-3, 100), "log2": (1e-3, 100), "sqr": (-100, 100),
    "sqrt": (0, 100), "sin": (-20, 20), "cos": (-20, 20), "tan": (-1.5, 1.5), "asin": (-1, 1),
    "acos": (-1, 1), "atan": (-50, 50), "sinh": (-8, 8), "cosh": (-8, 8), "tanh": (-5, 5),
    "asinh": (-100, 100), "acosh": (1, 100), "atanh": (-0.99, 0.99), "abs": (-5, 5),
}


@pytest.mark.parametrize("name", sorted(UNARY_DOMAIN))
def test_unary_f32(name, dev, orc):
    lo, hi = UNARY_DOMAIN[name]
    x = (seeded(0, 1).random(40003, dtype=np.float32) * (hi - lo) + lo).astype(np.float32)
    got = getattr(dev.tensor(x), name)().as_slice()
    ref = getattr(orc.Ref(x), name)().numpy()
    assert_ulp(orc, got, ref)


@pytest.mark.parametrize("name", sorted(UNARY_DOMAIN))
def test_unary_f16(name, dev, orc):
    lo, hi = UNARY_DOMAIN[name]
    x = (seeded(0, 2).random(4099, dtype=np.float32) * (hi - lo) + lo).astype(np.float16)
    got = getattr(dev.tensor(x), name)().as_slice()
    ref = getattr(orc.Ref(x), name)().numpy()
    assert_ulp(orc, got, ref, 1)


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_scalar_and_binary_exact(dtype, dev, orc):
    g = seeded(0, 3)
    x = (g.standard_normal((37, 129)) * 3).astype(dtype)
    y = (g.standard_normal((37, 129)) * 3 + 0.1).astype(dtype)
    for f in (lambda t: t + 1.7, lambda t: t - 0.3, lambda t: 2.5 - t, lambda t: t * 1.1, lambda t: t / 3.0,
              lambda t: 7.0 / t):
        np.testing.assert_array_equal(f(dev.tensor(x)).as_slice(), f(orc.Ref(x)).numpy())
    for f in (lambda a, b: a + b, lambda a, b: a - b, lambda a, b: a * b, lambda a, b: a / b):
        np.testing.assert_array_equal(f(dev.tensor(x), dev.tensor(y)).as_slice(), f(orc.Ref(x), orc.Ref(y)).numpy())
    xa, ya = np.abs(x) + dtype(0.1), y
    assert_ulp(orc, dev.tensor(xa).pow(dev.tensor(ya)).as_slice(), orc.Ref(xa).pow(orc.Ref(ya)).numpy(), 2 if dtype == np.float32 else 1)


def test_cast_round_trip_bit_exact(wgf, dev, orc):
    g = seeded(3, 0)
    x = np.concatenate([g.standard_normal(100000).astype(np.float32),
                        (g.standard_normal(1000) * 1e-6).astype(np.float32),
                        np.float32([0, -0.0, 65504, 65519.9, 65520, 1e9, -1e9, np.inf, -np.inf, 6e-8, 2.9e-8, 3e-8])])
    h = dev.tensor(x).cast(wgf.F16)
    np.testing.assert_array_equal(h.as_slice().view(np.uint16), orc.Ref(x).cast(orc.F16).numpy().view(np.uint16))
    before = dev.launch_count
    rt = dev.tensor(x).cast(wgf.F16).cast(wgf.F32).as_slice()
    assert dev.launch_count - before == 1  # both casts in one kernel
    np.testing.assert_array_equal(rt.view(np.uint32), orc.Ref(x).cast(orc.F16).cast(orc.F32).numpy().view(np.uint32))
    b = dev.tensor(x).cast(wgf.BF16).as_slice()
    np.testing.assert_array_equal(b, orc.Ref(x).cast(orc.BF16).numpy())


def c1_chain(x):
    return ((x * 2.0 + 1.0).sin().cos() * 0.5) + (-(x * x)).exp()


def test_config1_fused_chain(dev, orc):
    """f32 [1024,1024] uniform[-1,1]; y = cos(sin(x*2+1))*0.5 + exp(-x*x): one kernel, x read once."""
    x = (seeded(1, 0).random((1024, 1024), dtype=np.float32) * 2 - 1).astype(np.float32)
    t = dev.tensor(x)
    before = dev.launch_count
    got = c1_chain(t).as_slice()
    assert dev.launch_count - before == 1
    assert_ulp(orc, got, c1_chain(orc.Ref(x)).numpy())
    # written with sqr() instead of x*x
    got2 = (((t * 2.0 + 1.0).sin().cos() * 0.5) + (-(t.sqr())).exp()).as_slice()
    np.testing.assert_array_equal(got, got2)


@pytest.mark.parametrize("shape", [(1,), (7,), (255,), (257,), (2049,), (3, 5), (9, 8), (8, 255), (257, 9), (2, 3, 5),
                                   (4, 8, 16), (7, 9, 257), (2, 3, 4, 5), (0,), (3, 0, 4)])
def test_shapes_and_views(shape, dev, orc):
    g = seeded(0, 4)
    x = g.standard_normal(shape).astype(np.float32)
    f = lambda t: (t * 1.5 + 0.25).tanh()
    np.testing.assert_array_equal(f(dev.tensor(x)).as_slice(), f(orc.Ref(x)).numpy()) if x.size == 0 else \
        assert_ulp(orc, f(dev.tensor(x)).as_slice(), f(orc.Ref(x)).numpy())
    r = len(shape)
    if x.size and r >= 2:
        for a in range(r):
            for b in range(a + 1, r):
                got = f(dev.tensor(x).transpose(a, b)).as_slice()
                assert_ulp(orc, got, f(orc.Ref(x).transpose(a, b)).numpy())
        rng = [(s // 3, s - s // 4) for s in shape]
        got = f(dev.tensor(x).slice(rng)).as_slice()
        assert_ulp(orc, got, f(orc.Ref(x).slice(rng)).numpy())


def test_config3_pairwise_broadcast(wgf, dev, orc):
    """silu(a*1.5) + b*c with b broadcast over axis 0 and c over axis 1 (reduced sizes for the oracle)."""
    A, B, H = 6, 20, 1024
    a = seeded(3, 0).standard_normal((A, B, H)).astype(np.float32)
    b = (seeded(3, 1).random((B, H), dtype=np.float32) * 2 - 1).astype(np.float32)
    c = seeded(3, 2).random((A, H), dtype=np.float32)
    ta, tb, tc = dev.tensor(a), dev.tensor(b), dev.tensor(c)
    before = dev.launch_count
    got = ((ta * 1.5).silu() + tb.broadcast((A, B, H)) * tc.broadcast((A, B, H))).as_slice()
    assert dev.launch_count - before == 1
    ra, rb, rc = orc.Ref(a), orc.Ref(b), orc.Ref(c)
    silu_ref, bc_ref = (ra * 1.5).silu(), rb.broadcast((A, B, H)) * rc.broadcast((A, B, H))
    ref = (silu_ref + bc_ref).numpy()
    # Every op is within 2 ulp of the oracle on its own inputs, but the final add can cancel:
    # the bound is 2 ulp of the result plus 2 ulp of the larger addend.
    eps = np.float64(2.0 ** -23)
    # the addends: silu within its own chain bound of 6 ulp (below), b*c exactly rounded; then one rounding of the sum
    bound = eps * (np.abs(ref.astype(np.float64)) + 6 * np.abs(silu_ref.numpy().astype(np.float64)) + np.abs(bc_ref.numpy().astype(np.float64)))
    assert np.all(np.abs(got.astype(np.float64) - ref) <= bound)
    assert np.mean(orc.ulp_diff_f32(got, ref) <= 2) > 0.9
    # transposed (permute 1,0,2) view of a, b and c permuted alike
    before = dev.launch_count
    got_t = ((ta.transpose(0, 1) * 1.5).silu() + tb.broadcast_axis(1, A) * tc.broadcast_axis(0, B)).as_slice()
    assert dev.launch_count - before == 1
    np.testing.assert_array_equal(got_t, np.ascontiguousarray(got.transpose(1, 0, 2)))
    # inner-axis transpose: exercises the strided load path
    got_i = ((ta.transpose(1, 2) * 1.5).silu()).as_slice()
    # silu is five ops deep (mul, neg, exp, add, div); each is within 2 ulp on its own inputs: exp uses up
    # to 2 (carried through the add with weight e / (1 + e) < 1), the quotient -- whose divisor is that
    # approximate value -- is taken with div.full.f32, up to 2 more, plus the roundings of mul and add
    assert_ulp(orc, got_i, (ra.transpose(1, 2) * 1.5).silu().numpy(), 6)
    # size-1 expansion form of the same broadcast
    got_e = ((ta * 1.5).silu() + tb.reshape((1, B, H)).expand((A, B, H)) * tc.reshape((A, 1, H)).expand((A, B, H))).as_slice()
    np.testing.assert_array_equal(got_e, got)


@pytest.mark.parametrize("shape", [(5,), (1000,), (33, 7), (7, 33), (64, 256), (3, 4096), (200, 1000), (4, 5, 6), (3, 17, 129),
                                   (2, 3, 4, 5)])
@pytest.mark.parametrize("op", ["sum", "max", "min", "product"])
def test_reduce_every_axis(shape, op, dev, orc):
    g = seeded(2, 5)
    x = g.standard_normal(shape).astype(np.float32)
    if op == "product":
        x = (1 + 0.01 * x).astype(np.float32)
    for axis in range(len(shape)):
        got = getattr(dev.tensor(x), op)(axis).as_slice()
        ref = getattr(orc.Ref(x), op)(axis).numpy()
        if op in ("max", "min"):
            np.testing.assert_array_equal(got, ref)
        else:
            g64 = got.astype(np.float64)
            scale = np.abs(x).astype(np.float64).sum(axis) if op == "sum" else np.abs(ref.astype(np.float64))
            assert np.all(np.abs(g64 - ref) <= 1e-5 * np.maximum(scale, 1e-30))


def test_reduce_fusion_and_views(dev, orc):
    g = seeded(2, 6)
    x = g.standard_normal((130, 514)).astype(np.float32)
    t, r = dev.tensor(x), orc.Ref(x)
    before = dev.launch_count
    got = ((t * 2.0 + 1.0).sqr().sum(1) / 514.0 + 1e-5).sqrt().as_slice()
    assert dev.launch_count - before == 1  # prologue and epilogue fused into the reduce
    assert_rel(got, ((r * 2.0 + 1.0).sqr().sum(1) / 514.0 + 1e-5).sqrt().numpy(), 1e-5)
    # reduce of views: slice with offset (the crate drops the offset, src/reduce.rs:351-352), transpose
    s = [(3, 100), (10, 500)]
    assert_rel(t.slice(s).sum(1).as_slice(), r.slice(s).sum(1).numpy(), 1e-4)
    np.testing.assert_array_equal(t.slice(s).max(0).as_slice(), r.slice(s).max(0).numpy())
    np.testing.assert_array_equal(t.transpose(0, 1).max(1).as_slice(), r.transpose(0, 1).max(1).numpy())
    # f16: fp32 accumulation, one rounding
    h = x[:64, :256].astype(np.float16)
    got = dev.tensor(h).sum(1).as_slice()
    ref = orc.Ref(h).sum(1).numpy()
    assert np.all(orc.ulp_diff_f16(got, ref) <= 1)
    # the crate's identity for max is -3.40282e38, not -inf (src/reduce.rs:640)
    m = dev.tensor(np.full((4, 8), -np.inf, np.float32)).max(1).as_slice()
    np.testing.assert_array_equal(m, np.full((4,), np.float32(-3.40282e38)))


def test_full_tensor_sum_is_one_kernel(dev, orc):
    x = seeded(2, 0).standard_normal((512, 1024)).astype(np.float32)
    t = dev.tensor(x)
    before = dev.launch_count
    got = t.exp().sum(0).sum(0).as_slice()
    assert dev.launch_count - before == 1
    ref = np.exp(x.astype(np.float64)).sum()
    assert got.shape == () and abs(float(got) - ref) <= 1e-5 * ref
    # 1-D long vector, odd length
    v = seeded(2, 1).standard_normal(1000003).astype(np.float32)
    got = dev.tensor(v).sum(0).as_slice()
    assert abs(float(got) - v.astype(np.float64).sum()) <= 1e-5 * np.abs(v).astype(np.float64).sum()


@pytest.mark.parametrize("rows,h", [(3, 2), (5, 7), (64, 128), (33, 1000), (16, 4096), (4, 8192), (2, 20000)])
def test_rms_norm_and_softmax_rows(rows, h, dev, orc):
    x = seeded(2, 0).standard_normal((rows, h)).astype(np.float32)
    w = (1 + 0.1 * seeded(2, 1).standard_normal(h)).astype(np.float32)
    t, tw = dev.tensor(x), dev.tensor(w)
    r, rw = orc.Ref(x), orc.Ref(w)
    before = dev.launch_count
    got = t.layer_norm(tw, 1e-5).as_slice()
    assert dev.launch_count - before == 1
    ref = r.layer_norm(rw, 1e-5).numpy()
    assert_rel(got, ref, 2e-6 * 8)
    before = dev.launch_count
    sm = t.softmax_last_dim().as_slice()
    assert dev.launch_count - before == 1
    sref = r.softmax_last_dim().numpy()
    assert np.max(np.abs(sm.astype(np.float64) - sref) / sref.max()) <= 1e-5
    assert_rel(sm, sref, 1e-4)
    before = dev.launch_count
    both = t.layer_norm(tw, 1e-5).softmax_last_dim().as_slice()
    assert dev.launch_count - before == 1  # RmsNorm -> softmax: one pass over the row
    bref = r.layer_norm(rw, 1e-5).softmax_last_dim().numpy()
    assert_rel(both, bref, 1e-4)
    np.testing.assert_allclose(both.astype(np.float64).sum(1), 1.0, atol=1e-5)


def test_softmax_rank1_and_rank3(dev, orc):
    x = seeded(2, 2).standard_normal(1000).astype(np.float32)
    assert_rel(dev.tensor(x).softmax().as_slice(), orc.Ref(x).softmax().numpy(), 1e-5)
    y = seeded(2, 3).standard_normal((3, 5, 130)).astype(np.float32)
    assert_rel(dev.tensor(y).softmax_last_dim().as_slice(), orc.Ref(y).softmax_last_dim().numpy(), 1e-4)
    h = y.astype(np.float16)
    w = np.ones(130, np.float16)
    got = dev.tensor(h).layer_norm(dev.tensor(w), 1e-5).as_slice()
    ref = orc.Ref(h).layer_norm(orc.Ref(w), 1e-5).numpy()
    assert np.all(orc.ulp_diff_f16(got, ref) <= 1)


def test_moves_bit_exact(wgf, dev, orc):
    g = seeded(3, 5)
    x = g.standard_normal((6, 10, 14)).astype(np.float32)
    t, r = dev.tensor(x), orc.Ref(x)
    eq = lambda a, b: np.testing.assert_array_equal(a.as_slice().view(np.uint32), b.numpy().view(np.uint32))
    eq(t.resize((8, 10, 20)), r.resize((8, 10, 20)))
    eq(t.reshape((60, 14)), r.reshape((60, 14)))
    eq(t.transpose(0, 2).reshape((14, 60)), r.transpose(0, 2).reshape((14, 60)))
    eq(t.slice([(1, 5), (2, 9), (3, 11)]).reshape((4 * 7 * 8,)), r.slice([(1, 5), (2, 9), (3, 11)]).reshape((4 * 7 * 8,)))
    v = g.standard_normal((2, 3, 4)).astype(np.float32)
    eq(t.slice_assign([(1, 3), (4, 7), (5, 9)], dev.tensor(v)), r.slice_assign([(1, 3), (4, 7), (5, 9)], orc.Ref(v)))
    eq(t, r)  # slice_assign must not write into a tensor that is still held
    for dim in range(3):
        eq(wgf.Tensor.cat([t, t * 2.0, -t], dim), orc.Ref.cat([r, r * 2.0, -r], dim))
    eq(t.narrow(1, 2, 5), r.narrow(1, 2, 5))
    eq(t.unsqueeze(1), r.unsqueeze(1))
    eq(t.unsqueeze(3), r.unsqueeze(3))
    h = x.astype(np.float16)
    th, rh = dev.tensor(h), orc.Ref(h)
    np.testing.assert_array_equal(wgf.Tensor.cat([th, th], 2).as_slice().view(np.uint16), orc.Ref.cat([rh, rh], 2).numpy().view(np.uint16))
    np.testing.assert_array_equal(th.transpose(0, 1).reshape((60, 14)).as_slice().view(np.uint16),
                                  rh.transpose(0, 1).reshape((60, 14)).numpy().view(np.uint16))


def test_rope(dev, orc):
    heads, seq, d = 4, 24, 64
    x = seeded(5, 0).standard_normal((heads, seq, d)).astype(np.float32)
    pos = np.arange(32, dtype=np.float32)[:, None]
    inv = (1.0 / (10000 ** (np.arange(0, d, 2, dtype=np.float32) / d)))[None, :]
    ang = (pos * inv).astype(np.float32)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    got = dev.tensor(x).rope(dev.tensor(cos), dev.tensor(sin)).as_slice()
    ref = orc.Ref(x).rope(orc.Ref(cos), orc.Ref(sin)).numpy()
    np.testing.assert_array_equal(got, ref)
    # against the textbook rotate-half form in float64
    c = np.concatenate([cos, cos], 1)[:seq][None].astype(np.float64)
    s = np.concatenate([sin, sin], 1)[:seq][None].astype(np.float64)
    rot = np.concatenate([-x[..., d // 2:], x[..., :d // 2]], -1).astype(np.float64)
    np.testing.assert_allclose(got, x * c + rot * s, rtol=0, atol=1e-5)


def test_memoised_and_inplace(wgf, dev, orc):
    x = seeded(0, 7).standard_normal((64, 64)).astype(np.float32)
    t = dev.tensor(x)
    e = t.exp()
    a = (e + 1.0).as_slice()
    b = (e * 2.0).as_slice()
    r = orc.Ref(x).exp()
    assert_ulp(orc, a, (r + 1.0).numpy())
    assert_ulp(orc, b, (r * 2.0).numpy())
    np.testing.assert_array_equal(t.as_slice(), x)
    # a chain of materialised steps with dropped handles reuses buffers in place
    import ctypes as C

    def device_ptr(t):
        d = t.desc()
        p = C.c_void_p()
        wgf.check(wgf.lib().wgf_buffer_device_ptr(C.c_void_p(d.buf), C.byref(p), None))
        wgf.check(wgf.lib().wgf_buffer_release(C.c_void_p(d.buf)))   # drop the extra reference again
        return p.value

    cur = dev.tensor(x)
    cur.materialize()
    ptrs = [device_ptr(cur)]
    for _ in range(5):
        nxt = cur + 1.0
        cur.release()
        nxt.materialize()
        cur = nxt
        ptrs.append(device_ptr(cur))
    assert len(set(ptrs)) == 1, ptrs                  # every step wrote into the same buffer
    np.testing.assert_array_equal(cur.as_slice(), ((((x + 1) + 1) + 1) + 1) + 1)
    # ... but never into a buffer whose tensor is still held
    held = dev.tensor(x)
    y = held + 1.0
    y.materialize()
    assert device_ptr(y) != device_ptr(held)
    np.testing.assert_array_equal(held.as_slice(), x)


def test_pinned_async_upload(wgf, dev, orc):
    x = np.abs(seeded(0, 8).standard_normal((300, 1000))).astype(np.float32)   # positive: no cancellation in the sums
    pins =[wgf.PinnedArray(x.shape, np.float32) for _ in range(2)]
    outs = []
    for k in range(4):                       # uploads overlap the previous round's kernels and downloads
        pins[k % 2].array[...] = x + k
        t = dev.tensor_pinned(pins[k % 2])
        outs.append(((t * 2.0).sum(1), k))
        got = outs[-1][0].as_slice()         # synchronises: the pinned array may be rewritten afterwards
        ref = (orc.Ref(x + k) * 2.0).sum(1).numpy()
        assert_rel(got, ref, 1e-5)
    with pytest.raises(wgf.WgfError):        # pageable memory is refused, not copied synchronously
        class Fake:
            array = x
            ptr = type("P", (), {"value": x.ctypes.data})()
        dev.tensor_pinned(Fake())


def test_timing_and_graphviz(dev):
    x = dev.tensor(np.ones((10, 10, 20), np.float32))
    y = x.sum(0).sum(0).sum(0)          # examples/hello.rs:15-22
    assert float(y.as_slice()) == 2000.0
    times = y.all_timing_information()
    assert len(times) >= 1 and all(t > 0 for t in times)
    assert "digraph" in y.graphvis()


def test_errors_do_not_abort(wgf, dev):
    a, b = dev.tensor(np.zeros((2, 3), np.float32)), dev.tensor(np.zeros((3, 2), np.float32))
    with pytest.raises(wgf.WgfError) as e:
        a + b
    assert e.value.status == "SHAPE"
    with pytest.raises(wgf.WgfError):
        a.mat_mul(a)
    with pytest.raises(wgf.WgfError):
        a.sum(2)
    with pytest.raises(wgf.WgfError):
        a + dev.tensor(np.zeros((2, 3), np.float16))
    with pytest.raises(wgf.WgfError):
        a.narrow(1, 2, 5)
    with pytest.raises(wgf.WgfError):
        wgf.Device(99)


@pytest.mark.parametrize("shape", [(300, 1000), (8192, 512), (7, 33), (5, 6, 64), (1, 4096)])
def test_reductions_riding_along_match_the_oracle(shape, wgf, dev, orc):
    """materialize_all: whole-tensor reductions computed inside the row kernel of a tensor requested
    with them.  Same values as the separate kernels (reductions: 1e-5 relative)."""
    g = seeded(2, 7)
    x = g.standard_normal(shape, dtype=np.float32)
    w = (1.0 + 0.1 * g.standard_normal(shape[-1])).astype(np.float32)
    tx, tw = dev.tensor(x), dev.tensor(w)
    y = tx.layer_norm(tw, 1e-5).softmax_last_dim() if len(shape) == 2 else tx.softmax_last_dim()
    s, m, q = tx.exp(), tx, tx * tx
    for _ in shape:
        s, m, q = s.sum(0), m.max(0), q.sum(0)
    before = dev.launch_count
    wgf.Tensor.materialize_all([y, s, m, q])
    assert dev.launch_count - before == 1
    rx, rw = orc.Ref(x), orc.Ref(w)
    ry = rx.layer_norm(rw, 1e-5).softmax_last_dim() if len(shape) == 2 else rx.softmax_last_dim()
    assert_rel(y.as_slice(), ry.numpy(), 1e-4)
    x64 = x.astype(np.float64)
    assert_rel(s.as_slice(), np.float32(np.exp(x64).sum()), 1e-5)
    assert float(m.as_slice()) == float(x.max())
    assert_rel(q.as_slice(), np.float32((x64 * x64).sum()), 1e-5)
    # the same requests one by one give the same answers
    s2 = tx.exp()
    for _ in shape:
        s2 = s2.sum(0)
    assert_rel(s2.as_slice(), s.as_slice(), 1e-5)


def test_reduction_riding_along_f16_and_all_results_cached(wgf, dev, orc):
    g = seeded(2, 8)
    x = g.standard_normal((96, 256), dtype=np.float32).astype(np.float16)
    tx = dev.tensor(x)
    y, mx = tx.softmax_last_dim(), tx.max(1).max(0)
    wgf.Tensor.materialize_all([mx, y])
    before = dev.launch_count
    assert float(mx.as_slice()) == float(x.max())
    d = orc.ulp_diff_f16(y.as_slice(), orc.Ref(x).softmax_last_dim().numpy())
    assert int(d.max()) <= 2
    assert dev.launch_count == before          # both were computed by the one request


def bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def test_bf16_elementwise_reduce_and_cast(wgf, dev, orc):
    """bf16 tensors (u16 bit patterns on both sides): + - * / exact, transcendental <= 1 ulp of bf16,
    reductions and casts through the same kernels as f16."""
    g = seeded(3, 5)
    x, y = bf16_bits(g.standard_normal((37, 200)) * 3), bf16_bits(g.standard_normal((37, 200)) * 3 + 4)
    tx, ty = dev.tensor(x, dtype=wgf.BF16), dev.tensor(y, dtype=wgf.BF16)
    rx, ry = orc.Ref(x, bf16=True), orc.Ref(y, bf16=True)
    for f in (lambda a, b: a + b, lambda a, b: a - b, lambda a, b: a * b, lambda a, b: a / b, lambda a, b: a * 1.5 + 0.25,
              lambda a, b: (a + b) * (a - b) / (b + 3.0)):
        np.testing.assert_array_equal(f(tx, ty).as_slice(), f(rx, ry).numpy())

    def bf_ulps(got, ref):      # distance in bf16 steps: the patterns are sign-magnitude
        a, b = got.astype(np.int32), ref.astype(np.int32)
        a = np.where(a & 0x8000, -(a & 0x7FFF), a)
        b = np.where(b & 0x8000, -(b & 0x7FFF), b)
        return np.abs(a - b)
    for name in ("exp", "tanh", "sqrt", "sin"):
        arg = bf16_bits(np.abs(g.standard_normal(4099)) * 2) if name == "sqrt" else bf16_bits(g.standard_normal(4099) * 2)
        got = getattr(dev.tensor(arg, dtype=wgf.BF16), name)().as_slice()
        ref = getattr(orc.Ref(arg, bf16=True), name)().numpy()
        assert int(bf_ulps(got, ref).max()) <= 1, name
    got = tx.max(1).as_slice()
    np.testing.assert_array_equal(got, rx.max(1).numpy())
    s = (tx.cast(wgf.F32).sum(0)).as_slice()
    assert_rel(s, rx.cast(orc.F32).sum(0).numpy(), 1e-5)
    np.testing.assert_array_equal(tx.cast(wgf.F32).cast(wgf.BF16).as_slice(), x)      # round trip is the identity
    f = g.standard_normal(10000).astype(np.float32)
    np.testing.assert_array_equal(dev.tensor(f).cast(wgf.BF16).as_slice(), bf16_bits(f))  # round to nearest even


@pytest.mark.parametrize("shape", [(2, 3, 2, 2, 3, 4), (2, 1, 3, 2, 2, 1, 2, 5), (3, 2, 2, 2, 2, 2, 2, 2)])
def test_rank_6_to_8(shape, dev, orc):
    """Ranks up to 8 (the C ABI's limit; the crate instantiates ranks up to 6): element-wise on permuted views,
    reductions over inner, middle and outer axes, broadcast along a middle axis."""
    g = seeded(3, 6)
    x = g.standard_normal(shape, dtype=np.float32)
    y = g.standard_normal(shape, dtype=np.float32)
    r = len(shape)
    tx, ty, rx, ry = dev.tensor(x), dev.tensor(y), orc.Ref(x), orc.Ref(y)
    got = (tx.transpose(0, r - 1).transpose(1, r - 2) * 2.0 + ty.transpose(0, r - 1).transpose(1, r - 2)).as_slice()
    ref = (rx.transpose(0, r - 1).transpose(1, r - 2) * 2.0 + ry.transpose(0, r - 1).transpose(1, r - 2)).numpy()
    np.testing.assert_array_equal(got, ref)
    for axis in (0, r // 2, r - 1):
        assert_rel(tx.sum(axis).as_slice(), rx.sum(axis).numpy(), 1e-5 * 10)      # sums of signed values: looser, relative to the result
        np.testing.assert_array_equal(tx.max(axis).as_slice(), rx.max(axis).numpy())
    mid = r // 2
    red = tx.max(mid)
    back = red.broadcast_axis(mid, shape[mid])
    np.testing.assert_array_equal((tx - back).as_slice(), (rx - rx.max(mid).broadcast_axis(mid, shape[mid])).numpy())


def test_joint_request_edge_cases(wgf, dev):
    wgf.Tensor.materialize_all([])                                   # nothing to do
    x = dev.tensor(np.arange(12, dtype=np.float32).reshape(3, 4))
    s = x.sum(0).sum(0)
    before = dev.launch_count
    wgf.Tensor.materialize_all([s, s, x])                            # duplicates and an already materialised tensor
    assert dev.launch_count - before == 1
    assert float(s.as_slice()) == 66.0
    e = dev.tensor(np.zeros((0, 8), np.float32))
    y, t = e.softmax_last_dim(), e.sum(0).sum(0)
    wgf.Tensor.materialize_all([y, t])                               # empty index space: the reduction is the identity
    assert y.as_slice().shape == (0, 8) and float(t.as_slice()) == 0.0


@pytest.mark.parametrize("case", ["2d", "3d_12", "3d_02", "ragged", "f16", "two_staged_and_broadcast"])
def test_transposed_operands_staged_through_shared_memory(case, wgf, dev, orc):
    """Operands that are contiguous along another axis than the output, large enough (>= 65536 elements)
    for the shared-memory-staged kernel (one launch) or, where its alignment rules fail, for the
    transposing copy in front of the plain kernel (two launches): bit-exact (only + - * here), ragged
    tile edges included."""
    g = seeded(3, 7)
    if case == "2d":
        x, y = g.standard_normal((300, 700), dtype=np.float32), g.standard_normal((700, 300), dtype=np.float32)
        build = lambda X, Y: X.transpose(0, 1) * 2.0 + Y
    elif case == "3d_12":
        x, y = g.standard_normal((64, 130, 257), dtype=np.float32), g.standard_normal((64, 257, 130), dtype=np.float32)
        build = lambda X, Y: (X.transpose(1, 2) - Y) * X.transpose(1, 2)
    elif case == "3d_02":
        x, y = g.standard_normal((96, 20, 72), dtype=np.float32), g.standard_normal((72, 20, 96), dtype=np.float32)
        build = lambda X, Y: X.transpose(0, 2) + Y * 0.5
    elif case == "ragged":
        x, y = g.standard_normal((1001, 77), dtype=np.float32), g.standard_normal((77, 1001), dtype=np.float32)
        build = lambda X, Y: X.transpose(0, 1) * Y
    elif case == "f16":
        x = g.standard_normal((256, 300, 40), dtype=np.float32).astype(np.float16)
        y = g.standard_normal((40, 300, 256), dtype=np.float32).astype(np.float16)
        build = lambda X, Y: X.transpose(0, 2) * 2.0 + Y
    else:
        x, y = g.standard_normal((32, 256, 512), dtype=np.float32), g.standard_normal((256, 512), dtype=np.float32)
        # a and the broadcast b are both read through their transposes; c stays a broadcast along the new inner axis
        build = lambda X, Y: X.transpose(1, 2) * 1.5 + Y.broadcast((32, 256, 512)).transpose(1, 2)
    tx, ty = dev.tensor(x), dev.tensor(y)
    before = dev.launch_count
    got = build(tx, ty).as_slice()
    # the staged variant wants 4-byte elements and extents / strides that allow 16-byte loads along the
    # transposed operand's contiguous axis; otherwise that operand is transposed by a copy first
    expected = {"3d_12": 2, "ragged": 2, "f16": 2}.get(case, 1)
    assert dev.launch_count - before == expected
    ref = build(orc.Ref(x), orc.Ref(y)).numpy()
    np.testing.assert_array_equal(got, ref)


@pytest.mark.parametrize("lo,hi", [(-3.0, 3.0), (45.0, 70.0), (-85.0, -60.0), (-20.0, 20.0)])   # the sums stay finite in f32
def test_exp_that_only_feeds_a_sum_stays_inside_the_reduction_bound(lo, hi, wgf, dev):
    """sum(exp(x)) computes its exponentials with the two-instruction form (nothing but the sum can
    see them); the sums must hold the 1e-5 bound of reductions over the whole range of exp, alone,
    per row, and riding along in a row kernel."""
    x = (seeded(2, 9).random((512, 1024), dtype=np.float32) * (hi - lo) + lo).astype(np.float32)
    e = np.exp(x.astype(np.float64))
    t = dev.tensor(x)
    assert_rel(t.exp().sum(0).sum(0).as_slice(), np.float64(e.sum()), 1e-5)
    assert_rel(t.exp().sum(1).as_slice(), e.sum(1), 1e-5)
    assert_rel(t.exp().sum(0).as_slice(), e.sum(0), 1e-5)
    y, s = t.softmax_last_dim(), t.exp().sum(0).sum(0)
    wgf.Tensor.materialize_all([y, s])
    assert_rel(s.as_slice(), np.float64(e.sum()), 1e-5)
    # an exp that is also an output keeps the 2-ulp function
    both = t.exp()
    tot = both.sum(1)
    wgf.Tensor.materialize_all([both, tot])
    assert np.array_equal(both.as_slice(), dev.tensor(x).exp().as_slice())


@pytest.mark.parametrize("inner", ["tanh", "sin", "cos"])
def test_sine_and_cosine_of_bounded_values(inner, dev, orc):
    """sin / cos whose argument is a tanh, sine or cosine use the polynomial for [-1, 1] (no range
    reduction).  4 Mi arguments per inner function -- every binade down to 1e-30 on both sides, the
    values that saturate tanh, a dense stretch around the ends of the interval -- checked against
    float64 applied to the VERY float the fused kernel saw (the inner function materialised on its
    own is the same code): 2 ulp, the bound of every transcendental here."""
    g = seeded(1, 40)
    mant = g.random(1 << 21, dtype=np.float32) + 1
    expo = g.integers(-100, 5, 1 << 21).astype(np.float32)
    x = np.concatenate([mant * np.exp2(expo), -(mant * np.exp2(expo)),
                        g.uniform(-1.6, 1.6, 1 << 19).astype(np.float32),
                        np.array([0.0, -0.0, 1.0, -1.0, 20.0, -20.0, np.pi / 2, -np.pi / 2, np.inf, -np.inf, np.nan], np.float32)])
    t = dev.tensor(x)
    u = getattr(t, inner)().as_slice()                       # the bounded value, as the fused kernel computes it
    assert np.all((np.abs(u) <= 1) | np.isnan(u))
    for outer in ("sin", "cos"):
        before = dev.launch_count
        got = getattr(getattr(t, inner)(), outer)().as_slice()
        assert dev.launch_count - before == 1
        want = getattr(np, outer)(u.astype(np.float64)).astype(np.float32)
        ok = ~np.isnan(want)
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert_ulp(orc, got[ok], want[ok], tol=2)
        # and against the full-range function on the same values (a separate, unfused graph)
        plain = getattr(dev.tensor(u), outer)().as_slice()
        assert_ulp(orc, got[ok], plain[ok], tol=2)
