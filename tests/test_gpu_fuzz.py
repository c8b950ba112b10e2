"""Randomised graphs (seeded) through the whole stack -- lazy graph, fusion resolver, generated kernels --
against the CPU oracle evaluating the same expression op by op.  Only exactly-rounded operations are
drawn (+ - * with tensors and constants, neg, abs, sqr, max/min reductions, views, moves), so fused and
unfused evaluation must agree BIT FOR BIT; sums are drawn too and checked at 1e-5 relative to sum|x|."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

DIMS = [1, 2, 3, 5, 8, 9, 33, 64]


class Pair:
    """The same value in both worlds."""

    def __init__(self, t, r, exact=True):
        self.t, self.r, self.exact = t, r, exact

    @property
    def shape(self):
        return self.r.shape


def leaf(dev, orc, g, shape, dtype):
    a = (g.integers(-8, 9, size=shape) / 4.0).astype(dtype)     # small dyadic values: products stay exact-ish
    return Pair(dev.tensor(a), orc.Ref(a))


def random_view(g, p):
    shape = p.shape
    r = len(shape)
    kind = g.integers(0, 4)
    if kind == 0 and r >= 2:
        a, b = g.choice(r, 2, replace=False)
        return Pair(p.t.transpose(int(a), int(b)), p.r.transpose(int(a), int(b)), p.exact)
    if kind == 1 and r >= 1 and all(s >= 2 for s in shape):
        rng = [(int(g.integers(0, s // 2)), int(g.integers(s // 2 + 1, s + 1))) for s in shape]
        return Pair(p.t.slice(rng), p.r.slice(rng), p.exact)
    if kind == 2 and r <= 3:
        axis, size = int(g.integers(0, r + 1)), int(g.choice([1, 2, 5]))
        return Pair(p.t.broadcast_axis(axis, size), p.r.broadcast_axis(axis, size), p.exact)
    return p


def random_unary(g, p):
    k = g.integers(0, 7)
    c = float(g.integers(-4, 5)) / 2.0
    if k == 0:
        return Pair(p.t + c, p.r + c, p.exact)
    if k == 1:
        return Pair(c - p.t, c - p.r, p.exact)
    if k == 2:
        return Pair(p.t * c, p.r * c, p.exact)
    if k == 3:
        return Pair(-p.t, -p.r, p.exact)
    if k == 4:
        return Pair(p.t.abs(), p.r.abs(), p.exact)
    if k == 5:
        return Pair(p.t.sqr(), p.r.sqr(), p.exact)
    return Pair(p.t - c, p.r - c, p.exact)


def random_binary(g, p, q):
    k = g.integers(0, 3)
    ex = p.exact and q.exact
    if k == 0:
        return Pair(p.t + q.t, p.r + q.r, ex)
    if k == 1:
        return Pair(p.t - q.t, p.r - q.r, ex)
    return Pair(p.t * q.t, p.r * q.r, ex)


def random_reduce(g, p):
    axis = int(g.integers(0, len(p.shape)))
    k = g.integers(0, 3)
    if k == 0:
        return Pair(p.t.max(axis), p.r.max(axis), p.exact)
    if k == 1:
        return Pair(p.t.min(axis), p.r.min(axis), p.exact)
    return Pair(p.t.sum(axis), p.r.sum(axis), False)


def random_move(g, wgf, orc, p):
    shape = p.shape
    k = g.integers(0, 3)
    if k == 0:
        n = int(np.prod(shape))
        return Pair(p.t.reshape((n,)), p.r.reshape((n,)), p.exact)
    if k == 1:
        dim = int(g.integers(0, len(shape)))
        return Pair(wgf.Tensor.cat([p.t, p.t], dim), orc.Ref.cat([p.r, p.r], dim), p.exact)
    new = tuple(s + int(g.integers(0, 3)) for s in shape)
    return Pair(p.t.resize(new), p.r.resize(new), p.exact)


@pytest.mark.parametrize("seed", range(60))
def test_random_graph(seed, wgf, dev, orc):
    g = np.random.Generator(np.random.PCG64(0xF00D + seed))
    dtype = np.float32 if seed % 4 else np.float16
    rank = int(g.integers(1, 5))
    shape = tuple(int(g.choice(DIMS)) for _ in range(rank))
    pool = [leaf(dev, orc, g, shape, dtype) for _ in range(int(g.integers(1, 4)))]
    cur = pool[0]
    for _ in range(int(g.integers(2, 9))):
        k = g.integers(0, 10)
        if k < 4:
            cur = random_unary(g, cur)
        elif k < 6:
            other = pool[int(g.integers(0, len(pool)))]
            if other.shape == cur.shape:
                cur = random_binary(g, cur, other)
            else:
                cur = random_unary(g, cur)
        elif k < 7:
            v = random_view(g, cur)
            # a view changes the shape: later binary ops pair it with itself
            cur = v
            pool = [cur]
        elif k < 8 and len(cur.shape) >= 1 and np.prod(cur.shape) > 0:
            cur = random_reduce(g, cur)
            pool = [cur]
            if len(cur.shape) == 0:
                break
        elif k < 9 and 1 <= len(cur.shape) and np.prod(cur.shape) < 20000:
            cur = random_move(g, wgf, orc, cur)
            pool = [cur]
        else:
            cur = random_binary(g, cur, random_unary(g, cur))
    got = cur.t.as_slice()
    ref = cur.r.numpy()
    assert got.shape == ref.shape and got.dtype == ref.dtype
    if cur.exact:
        np.testing.assert_array_equal(got, ref)
    else:
        scale = np.maximum(np.abs(ref.astype(np.float64)), 1.0)
        tol = 1e-5 if dtype == np.float32 else 2e-3
        assert np.all(np.abs(got.astype(np.float64) - ref.astype(np.float64)) <= tol * scale * 64)
