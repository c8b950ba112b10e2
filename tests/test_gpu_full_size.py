"""Parity at the benchmark's own sizes.  The oracle works row by row, so a full-size result is checked
on rows sampled over the whole row range (first, last, tile and CTA boundaries, random ones); what has
an exact or cheap full statement (casts, the whole-tensor sum, matmul through a projection) is checked
on every element.  Tolerances as everywhere: element-wise 2 ulp f32 per op, reductions 1e-5, f32
matmul 1e-4, 16-bit matmul / attention 1e-2 and the 16-bit decoder block 2e-2 norm-wise."""
import numpy as np
import pytest

from conftest import seeded

pytestmark = pytest.mark.gpu


def sampled(n, count, seed):
    """`count` indices of range(n): both ends, the neighbours of powers of two, the rest random."""
    fixed = {0, 1, n - 1, n - 2, n // 2, n // 2 - 1}
    for p in (127, 128, 129, 255, 256, 1023, 1024, 4095, 4096):
        if p < n:
            fixed.add(p)
    g = np.random.Generator(np.random.PCG64(seed))
    while len(fixed) < count:
        fixed.add(int(g.integers(0, n)))
    return np.array(sorted(i for i in fixed if 0 <= i < n))


def rel(got, ref):
    g, r = got.astype(np.float64), ref.astype(np.float64)
    return float(np.max(np.abs(g - r) / np.maximum(np.abs(r), 1e-30)))


def normwise(got, ref):
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(np.asarray(got, dtype=np.float64) - ref)) / max(np.max(np.abs(ref)), 1e-30))


def test_config2_rows_and_full_sum_at_8192x4096(wgf, dev, orc):
    """RmsNorm -> softmax rows of f32 [8192,4096] against the oracle on 96 sampled rows, and
    sum(exp(x)) of all 33 554 432 elements against float64; asked for one by one and as the joint
    request of the benchmark step (one kernel, the sum riding along)."""
    R, H = 8192, 4096
    x = seeded(2, 0).standard_normal((R, H), dtype=np.float32)
    w = (1 + 0.1 * seeded(2, 1).standard_normal(H)).astype(np.float32)
    rows = sampled(R, 96, 1)
    ref_w = orc.Ref(w)
    ref_norm = orc.Ref(x[rows]).layer_norm(ref_w, 1e-5)
    ref_y = ref_norm.softmax_last_dim().numpy()
    s_ref = np.exp(x.astype(np.float64)).sum()
    t, tw = dev.tensor(x), dev.tensor(w)
    norm = t.layer_norm(tw, 1e-5).as_slice()
    assert rel(norm[rows], ref_norm.numpy()) <= 2e-6 * 8
    y = t.layer_norm(tw, 1e-5).softmax_last_dim().as_slice()
    assert rel(y[rows], ref_y) <= 1e-4
    assert np.max(np.abs(y[rows].astype(np.float64) - ref_y) / ref_y.max(axis=1, keepdims=True)) <= 1e-5
    np.testing.assert_allclose(y.astype(np.float64).sum(1), 1.0, atol=1e-5)      # every row, not only the sampled
    s = float(t.exp().sum(0).sum(0).as_slice())
    assert abs(s - s_ref) <= 1e-5 * s_ref
    before = dev.launch_count
    y2, s2 = t.layer_norm(tw, 1e-5).softmax_last_dim(), t.exp().sum(0).sum(0)
    wgf.Tensor.materialize_all([y2, s2])
    assert dev.launch_count - before == 1
    np.testing.assert_array_equal(y2.as_slice(), y)
    assert abs(float(s2.as_slice()) - s_ref) <= 1e-5 * s_ref
    # reductions over either axis at this size (1e-5 relative to the sum of magnitudes)
    for axis in (0, 1):
        got = t.sum(axis).as_slice().astype(np.float64)
        ref = x.astype(np.float64).sum(axis)
        assert np.max(np.abs(got - ref) / np.abs(x).astype(np.float64).sum(axis)) <= 1e-5
        np.testing.assert_array_equal(t.max(axis).as_slice(), x.max(axis))


def test_config3_pairwise_broadcast_at_64x512x1024(wgf, dev, orc):
    """silu(a*1.5) + b*c on a = f32 [64,512,1024], b broadcast over axis 0, c over axis 1: the plain
    form, the permute(1,0,2) form and the inner-axis transpose (staged through shared memory),
    each on 128 sampled (i, j) rows against the oracle; cast round trip bit-exact on everything."""
    A, B, H = 64, 512, 1024
    a = seeded(3, 0).standard_normal((A, B, H), dtype=np.float32)
    b = (seeded(3, 1).random((B, H), dtype=np.float32) * 2 - 1).astype(np.float32)
    c = seeded(3, 2).random((A, H), dtype=np.float32)
    ta, tb, tc = dev.tensor(a), dev.tensor(b), dev.tensor(c)
    flat = sampled(A * B, 128, 2)
    ii, jj = flat // B, flat % B
    silu_ref = (orc.Ref(a[ii, jj]) * 1.5).silu()
    bc_ref = orc.Ref(b[jj]) * orc.Ref(c[ii])
    ref = (silu_ref + bc_ref).numpy()
    # every op within 2 ulp on its own inputs: the silu chain (mul, neg, exp, add, div.full) within 6 ulp
    # of its value, b*c exactly rounded; the final add can cancel, so the bound is on the addends
    eps = np.float64(2.0 ** -23)
    bound = eps * (np.abs(ref.astype(np.float64)) + 6 * np.abs(silu_ref.numpy().astype(np.float64)) + np.abs(bc_ref.numpy().astype(np.float64)))

    before = dev.launch_count
    got = ((ta * 1.5).silu() + tb.broadcast((A, B, H)) * tc.broadcast((A, B, H))).as_slice()
    assert dev.launch_count - before == 1
    assert np.all(np.abs(got[ii, jj].astype(np.float64) - ref) <= bound)
    before = dev.launch_count
    got_t = ((ta.transpose(0, 1) * 1.5).silu() + tb.broadcast_axis(1, A) * tc.broadcast_axis(0, B)).as_slice()
    assert dev.launch_count - before == 1
    assert got_t.shape == (B, A, H)
    np.testing.assert_array_equal(got_t, np.ascontiguousarray(got.transpose(1, 0, 2)))     # all elements
    # a read through transpose(1,2): [64,1024,512]; silu alone (five ops deep, two of them to 2 ulp: 6 ulp)
    got_i = (ta.transpose(1, 2) * 1.5).silu().as_slice()
    assert got_i.shape == (A, H, B)
    ref_i = (orc.Ref(a[ii, jj]) * 1.5).silu().numpy()
    assert int(orc.ulp_diff_f32(np.ascontiguousarray(got_i[ii, :, jj]), ref_i).max()) <= 6
    # the inner-transposed pairwise form: a^T(1,2) with b^T, c broadcast along the new inner axis
    got_p = ((ta.transpose(1, 2) * 1.5).silu() + tb.transpose(0, 1).broadcast_axis(0, A)
             * tc.broadcast_axis(2, B)).as_slice()
    np.testing.assert_array_equal(got_p, np.ascontiguousarray(got.transpose(0, 2, 1)))
    # casts f32 -> f16 -> f32 over all 33 554 432 elements, one kernel, bit-exact (RNE)
    before = dev.launch_count
    rt = ta.cast(wgf.F16).cast(wgf.F32).as_slice()
    assert dev.launch_count - before == 1
    np.testing.assert_array_equal(rt.view(np.uint32), a.astype(np.float16).astype(np.float32).view(np.uint32))


def test_config1_chain_at_16384x4096(dev, orc):
    """The C1 chain on a tensor larger than L2, sampled rows against the oracle (2 ulp of the result
    plus 2 ulp of the larger addend of the final add)."""
    R, H = 16384, 4096
    x = (seeded(1, 0).random((R, H), dtype=np.float32) * 2 - 1).astype(np.float32)
    rows = sampled(R, 48, 3)
    t = dev.tensor(x)
    got = (((t * 2.0 + 1.0).sin().cos() * 0.5) + (-(t * t)).exp()).as_slice()
    r = orc.Ref(x[rows])
    left, right = (r * 2.0 + 1.0).sin().cos() * 0.5, (-(r * r)).exp()
    ref = (left + right).numpy()
    eps = np.float64(2.0 ** -23)
    bound = 2 * eps * (np.abs(ref.astype(np.float64)) + np.maximum(np.abs(left.numpy()), np.abs(right.numpy())))
    assert np.all(np.abs(got[rows].astype(np.float64) - ref) <= bound)


@pytest.mark.parametrize("kind", ["f32", "f16"])
def test_config4_every_tile_through_a_projection(kind, wgf, dev):
    """4096^3: for every block of 256 columns, C[:, blk] v against A (B[:, blk] v) in float64 for three
    random v.  Every entry of C takes part, so every tile of the banded persistent schedule and of
    the cut last wave is covered: entry-wise rounding shows as its typical relative size (2^-12 for
    an f16 result, 1e-6 for f32), a tile off by a relative e as about e."""
    import dense_ref
    n = 4096
    g = seeded(4, 0)
    a = (g.random((n, n), dtype=np.float32) * 2 - 1)
    b = (g.random((n, n), dtype=np.float32) * 2 - 1)
    if kind == "f16":
        a, b = a.astype(np.float16), b.astype(np.float16)
    c = dev.tensor(a).mat_mul(dev.tensor(b)).as_slice().astype(np.float64)
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    assert dense_ref.matmul_projection_error(c, a, b) <= (1e-3 if kind == "f16" else 1e-5)
    # and the per-entry bound on rows of every one of the 16 tile rows, and on whole columns
    rows = np.array([r * 256 + o for r in range(16) for o in (0, 77, 255)])
    tol = 1e-2 if kind == "f16" else 1e-4
    assert normwise(c[rows], a64[rows] @ b64) <= tol
    cols = np.array([k * 256 + o for k in range(16) for o in (1, 130)])
    assert normwise(c[:, cols], a64 @ b64[:, cols]) <= tol


@pytest.mark.parametrize("causal", [True, False])
def test_attention_at_seq_2048(causal, wgf, dev):
    import dense_ref
    g = seeded(5, 8)
    q, k, v = (g.standard_normal((4, 2048, 128), dtype=np.float32).astype(np.float16) for _ in range(3))
    before = dev.launch_count
    out = dev.tensor(q).attention(dev.tensor(k), dev.tensor(v), causal=causal).as_slice()
    assert dev.launch_count - before == 1
    assert normwise(out, dense_ref.attention(q, k, v, causal, 1 / np.sqrt(128))) <= 1e-2


def test_attention_many_heads_at_seq_2048_sampled(wgf, dev):
    """[256, 2048, 128] (the decoder block's 8 x 32 heads): more work items than CTAs, so the
    persistent schedule wraps; heads sampled over the whole range against float64."""
    import dense_ref
    g = seeded(5, 9)
    n = 256
    q, k, v = (g.standard_normal((n, 2048, 128), dtype=np.float32).astype(np.float16) for _ in range(3))
    out = dev.tensor(q).attention(dev.tensor(k), dev.tensor(v), causal=True).as_slice()
    heads = [0, 1, 73, 74, 147, 148, 149, 200, 255]
    ref = dense_ref.attention(q[heads], k[heads], v[heads], True, 1 / np.sqrt(128))
    assert normwise(out[heads], ref) <= 1e-2
    assert np.isfinite(out.astype(np.float32)).all()


def llama_inputs(Bg, S, Hd, heads, inter):
    g = np.random.Generator(np.random.PCG64(0xB2000000 + 16 * 5))
    h16 = lambda a: a.astype(np.float16)
    shapes = [(Hd, Hd)] * 4 + [(inter, Hd), (inter, Hd), (Hd, inter)]
    W = [h16(g.standard_normal(s, dtype=np.float32) * 0.02) for s in shapes]
    n1 = h16(1 + 0.1 * g.standard_normal(Hd))
    n2 = h16(1 + 0.1 * g.standard_normal(Hd))
    D = Hd // heads
    pos = np.arange(S, dtype=np.float32)[:, None]
    inv = (1.0 / (10000.0 ** (np.arange(0, D, 2, dtype=np.float32) / D)))[None, :]
    cos, sin = h16(np.cos(pos * inv)), h16(np.sin(pos * inv))
    x = h16(np.random.Generator(np.random.PCG64(0xB2000000 + 16 * 5 + 1)).standard_normal((Bg, S, Hd), dtype=np.float32))
    return x, W, n1, n2, cos, sin


def test_llama_block_at_8x2048x4096_sampled_tokens(wgf, dev):
    """The decoder block at the benchmark shape (hidden 4096, 32 heads, MLP 11008, batch 8, seq 2048,
    weights N(0, 0.02)), fused causal attention; tokens of the first and the last batch element
    against float64 (only those elements' keys and values are needed)."""
    import dense_ref
    Bg, S, Hd, heads, inter = 8, 2048, 4096, 32, 11008
    x, W, n1, n2, cos, sin = llama_inputs(Bg, S, Hd, heads, inter)
    out = dev.tensor(x).llama_block([dev.tensor(w) for w in W], dev.tensor(n1), dev.tensor(n2), dev.tensor(cos),
                                    dev.tensor(sin), None, heads, 1e-5).as_slice()
    assert out.shape == (Bg, S, Hd) and np.isfinite(out.astype(np.float32)).all()
    tokens = np.array([0, 1, 127, 128, 129, 1000, 1023, 1024, 2046, 2047])
    for bi in (0, Bg - 1):
        ref = dense_ref.llama_block_tokens(x[bi], W, n1, n2, cos, sin, heads, 1e-5, tokens)
        err = np.max(np.abs(out[bi, tokens].astype(np.float64) - ref)) / np.max(np.abs(ref))
        assert err <= 2e-2, (bi, err)
    # the batch elements are independent: the block of element 3 alone gives the same bits
    alone = dev.tensor(x[3:4]).llama_block([dev.tensor(w) for w in W], dev.tensor(n1), dev.tensor(n2), dev.tensor(cos),
                                           dev.tensor(sin), None, heads, 1e-5).as_slice()
    np.testing.assert_array_equal(alone[0], out[3])
