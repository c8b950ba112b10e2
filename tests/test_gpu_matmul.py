"""MatMul family vs the mathematical definition (double accumulation): f32 within 1e-4, f16 / bf16
within 1e-2, both norm-wise (max |got - ref| / max |ref|).  The crate's own kernel is only right up
to 8x8 (src/matmul.rs:31-39, 131-141) and ignores strides, so its output is not the oracle here."""
import numpy as np
import pytest

from conftest import seeded

pytestmark = pytest.mark.gpu


def normwise(got, ref):
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.max(np.abs(np.asarray(got, dtype=np.float64) - ref)) / max(np.max(np.abs(ref)), 1e-30))


def bf16_round(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return u.astype(np.uint16)


def bf16_to_f32(u):
    return (u.astype(np.uint32) << 16).view(np.float32)


def make(dev, wgf, a, kind):
    if kind == "f32":
        return dev.tensor(a.astype(np.float32)), a.astype(np.float32).astype(np.float64)
    if kind == "f16":
        h = a.astype(np.float16)
        return dev.tensor(h), h.astype(np.float64)
    u = bf16_round(a)
    return dev.tensor(u, dtype=wgf.BF16), bf16_to_f32(u).astype(np.float64)


def result(t, kind):
    out = t.as_slice()
    return bf16_to_f32(out) if kind == "bf16" else out


TOL = {"f32": 1e-4, "f16": 1e-2, "bf16": 1e-2}

SHAPES = [(1, 1, 1), (3, 5, 7), (8, 8, 8), (9, 9, 9), (37, 50, 21), (64, 64, 64), (100, 100, 100), (128, 256, 64),
          (129, 257, 72), (256, 512, 128), (300, 520, 200), (512, 1024, 256), (1024, 128, 1024)]


@pytest.mark.parametrize("kind", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", SHAPES)
def test_matmul_row_major(shape, kind, wgf, dev):
    M, N, K = shape
    g = seeded(4, 1)
    a = (g.random((M, K)) * 2 - 1)
    b = (g.random((K, N)) * 2 - 1)
    ta, ra = make(dev, wgf, a, kind)
    tb, rb = make(dev, wgf, b, kind)
    got = result(ta.mat_mul(tb), kind)
    assert got.shape == (M, N)
    assert normwise(got, ra @ rb) <= TOL[kind]


@pytest.mark.parametrize("kind", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("shape", [(5, 6, 7), (128, 256, 64), (200, 392, 136), (512, 512, 512)])
def test_matmul_transposed_and_sliced_operands(shape, kind, wgf, dev):
    """Strides and offsets are honoured (the crate reads operands as if contiguous, src/matmul.rs:96-117)."""
    M, N, K = shape
    g = seeded(4, 2)
    a = g.random((M, K)) * 2 - 1
    bt = g.random((N, K)) * 2 - 1            # B given as its transpose: b = bt^T
    ta, ra = make(dev, wgf, a, kind)
    tbt, rbt = make(dev, wgf, bt, kind)
    got = result(ta.mat_mul(tbt.transpose(0, 1)), kind)
    assert normwise(got, ra @ rbt.T) <= TOL[kind]
    at = np.ascontiguousarray(a.T)
    tat, rat = make(dev, wgf, at, kind)
    got = result(tat.transpose(0, 1).mat_mul(tbt.transpose(0, 1)), kind)   # A column-major
    assert normwise(got, rat.T @ rbt.T) <= TOL[kind]
    if M > 8 and K > 16:
        sa = ta.slice([(3, M - 1), (8, K)])                                   # offset view of A
        sb = tbt.transpose(0, 1).slice([(8, K), (0, N)])
        got = result(sa.mat_mul(sb), kind)
        assert normwise(got, ra[3:M - 1, 8:] @ rbt.T[8:, :]) <= TOL[kind]


@pytest.mark.parametrize("kind", ["f32", "f16", "bf16"])
def test_matmul_batched(kind, wgf, dev):
    g = seeded(4, 3)
    for (B, M, K, N) in [(3, 5, 7, 4), (4, 128, 64, 256), (5, 96, 40, 72)]:
        a = g.random((B, M, K)) * 2 - 1
        b = g.random((B, K, N)) * 2 - 1
        ta, ra = make(dev, wgf, a, kind)
        tb, rb = make(dev, wgf, b, kind)
        got = result(ta.mat_mul(tb), kind)
        assert got.shape == (B, M, N)
        assert normwise(got, ra @ rb) <= TOL[kind]


@pytest.mark.parametrize("kind", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("m", [1, 2, 4, 8, 3])
def test_skinny_gemv(m, kind, wgf, dev):
    g = seeded(4, 4)
    K, N = 1024, 2752
    a = g.random((m, K)) * 2 - 1
    b = g.random((K, N)) * 2 - 1
    ta, ra = make(dev, wgf, a, kind)
    tb, rb = make(dev, wgf, b, kind)
    assert normwise(result(ta.mat_mul(tb), kind), ra @ rb) <= TOL[kind]
    bt = np.ascontiguousarray(b.T)
    tbt, rbt = make(dev, wgf, bt, kind)
    assert normwise(result(ta.mat_mul(tbt.transpose(0, 1)), kind), ra @ rbt.T) <= TOL[kind]


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("shape", [(1024, 1024, 512), (1536, 1000, 320), (512, 768, 2048), (2304, 256, 200),
                                   (4864, 1024, 128), (5120, 1100, 192)])
def test_matmul_leftover_tiles_cut_along_n(shape, kind, wgf, dev):
    """Tile counts that leave at most half a wave of 256 x 256 tiles over (or are less than half a
    wave altogether): the CTA-pair kernel cuts those tiles into two 256 x 128 units.  Ragged N
    makes one of the two halves partly or wholly empty."""
    M, N, K = shape
    g = seeded(4, 5)
    a = g.random((M, K)) * 2 - 1
    b = g.random((K, N)) * 2 - 1
    ta, ra = make(dev, wgf, a, kind)
    tb, rb = make(dev, wgf, b, kind)
    ref = ra @ rb
    assert normwise(result(ta.mat_mul(tb), kind), ref) <= TOL[kind]
    bt = np.ascontiguousarray(b.T)
    tbt, rbt = make(dev, wgf, bt, kind)
    assert normwise(result(ta.mat_mul(tbt.transpose(0, 1)), kind), ref) <= TOL[kind]


def test_config4_full_sizes(wgf, dev):
    """Full benchmark sizes; checked on sampled rows against float64 (size-independent: any row is as good as another)."""
    g = seeded(4, 0)
    n = 4096
    a = (g.random((n, n), dtype=np.float32) * 2 - 1)
    b = (g.random((n, n), dtype=np.float32) * 2 - 1)
    rows = [0, 1, 127, 128, 2047, 4095]
    for kind in ("f32", "f16"):
        ta, ra = make(dev, wgf, a, kind)
        tb, rb = make(dev, wgf, b, kind)
        got = result(ta.mat_mul(tb), kind)
        ref = ra[rows] @ rb
        assert normwise(got[rows], ref) <= TOL[kind]
        # linearity: (2A)B == 2(AB) exactly in binary floating point
        got2 = result((ta * 2.0).mat_mul(tb), kind)
        np.testing.assert_array_equal(got2[rows], got[rows] * 2)
    # batched f16 [32,1024,128] x [32,128,1024]
    a3 = (g.random((32, 1024, 128), dtype=np.float32) * 2 - 1)
    b3 = (g.random((32, 128, 1024), dtype=np.float32) * 2 - 1)
    ta, ra = make(dev, wgf, a3, "f16")
    tb, rb = make(dev, wgf, b3, "f16")
    got = result(ta.mat_mul(tb), "f16")
    for z in (0, 17, 31):
        assert normwise(got[z], ra[z] @ rb[z]) <= 1e-2
    # decode GEMV f16 [1,4096] x [4096,11008]
    x = (g.random((1, 4096), dtype=np.float32) * 2 - 1)
    w = (g.random((4096, 11008), dtype=np.float32) * 2 - 1)
    tx, rx = make(dev, wgf, x, "f16")
    tw, rw = make(dev, wgf, w, "f16")
    assert normwise(result(tx.mat_mul(tw), "f16"), rx @ rw) <= 1e-2


def silu64(g):
    return g / (1 + np.exp(-g))


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("shape", [(256, 128, 64), (512, 384, 256), (1024, 1000, 192), (2304, 640, 128), (300, 256, 128)])
def test_matmul_epilogues_give_the_bits_of_the_separate_kernels(shape, kind, wgf, dev, monkeypatch):
    """`product + t`, `t + product` and `silu(a bg) * (a bu)` run inside the tensor-core kernel's
    epilogue (one launch each); with WGF_NO_MATMUL_EPILOGUE=1 the same graphs run as separate kernels.
    Both must give the same bits, and both must be within the 16-bit matmul bound of float64."""
    M, N, K = shape
    g = seeded(4, 6)
    a, w, w2 = g.random((M, K)) * 2 - 1, g.random((N, K)) * 2 - 1, g.random((N, K)) * 2 - 1
    r = g.standard_normal((M, N))
    ta, ra = make(dev, wgf, a, kind)
    tw, rw = make(dev, wgf, w, kind)
    tw2, rw2 = make(dev, wgf, w2, kind)
    tr, rr = make(dev, wgf, r, kind)
    graphs = {
        "residual": (lambda: tr + ta.mat_mul(tw.transpose(0, 1)), rr + ra @ rw.T),
        "residual, product first": (lambda: ta.mat_mul(tw.transpose(0, 1)) + tr, rr + ra @ rw.T),
        "silu_mul": (lambda: ta.mat_mul(tw.transpose(0, 1)).silu() * ta.mat_mul(tw2.transpose(0, 1)), silu64(ra @ rw.T) * (ra @ rw2.T)),
        "silu_mul, up first": (lambda: ta.mat_mul(tw2.transpose(0, 1)) * ta.mat_mul(tw.transpose(0, 1)).silu(), silu64(ra @ rw.T) * (ra @ rw2.T)),
    }
    for name, (build, ref) in graphs.items():
        monkeypatch.delenv("WGF_NO_MATMUL_EPILOGUE", raising=False)
        before = dev.launch_count
        fused = build().materialize()
        n_fused = dev.launch_count - before
        monkeypatch.setenv("WGF_NO_MATMUL_EPILOGUE", "1")
        before = dev.launch_count
        apart = build().materialize()
        n_apart = dev.launch_count - before
        monkeypatch.delenv("WGF_NO_MATMUL_EPILOGUE")
        got, want = fused.as_slice(), apart.as_slice()
        # (300 rows: the second 128-row half of the CTA pair's tile would be mostly padding, the pair
        # kernel leaves such products to the one-CTA kernel, which has no epilogues)
        assert (n_fused == 1 or M == 300) and n_apart >= 2, (name, n_fused, n_apart)
        np.testing.assert_array_equal(got.view(np.uint16), want.view(np.uint16), err_msg=name)
        assert normwise(result(fused, kind), ref) <= (2e-2 if kind == "bf16" else 1e-2), name


def test_matmul_epilogues_batched_row_major_and_views(wgf, dev, monkeypatch):
    """The same with a batch axis, with B given row-major [K, N], and with a residual that is a
    strided view; a product that something else also reads is not fused away."""
    g = seeded(4, 7)
    B, M, N, K = 3, 256, 256, 128
    a, b, r = g.random((B, M, K)) * 2 - 1, g.random((B, K, N)) * 2 - 1, g.standard_normal((B, M, 2 * N))
    ta, ra = make(dev, wgf, a, "f16")
    tb, rb = make(dev, wgf, b, "f16")
    tr, rr = make(dev, wgf, r, "f16")
    view = tr.slice([(0, B), (0, M), (N // 2, N // 2 + N)])
    before = dev.launch_count
    fused = (ta.mat_mul(tb) + view).materialize()
    assert dev.launch_count - before == 1
    monkeypatch.setenv("WGF_NO_MATMUL_EPILOGUE", "1")
    apart = (ta.mat_mul(tb) + view).as_slice()
    monkeypatch.delenv("WGF_NO_MATMUL_EPILOGUE")
    np.testing.assert_array_equal(fused.as_slice().view(np.uint16), apart.view(np.uint16))
    assert normwise(fused.as_slice(), ra @ rb + rr[:, :, N // 2:N // 2 + N]) <= 1e-2
    # the product is held by a handle: it has to exist on its own, so nothing is folded into its kernel
    prod = ta.mat_mul(tb)
    both = prod + view
    before = dev.launch_count
    both.materialize()
    assert dev.launch_count - before == 2
    np.testing.assert_array_equal(both.as_slice().view(np.uint16), apart.view(np.uint16))
    assert normwise(prod.as_slice(), ra @ rb) <= 1e-2


def test_two_devices_in_one_process_each_run_the_tcgen05_kernels(wgf, dev):
    """Function attributes (the opt-in to large dynamic shared memory) and the occupancy figures the
    launchers keep are per GPU: a second wgf_device in the same process must set up its own.  The
    pair kernel, the single-CTA kernel and the fused attention run on GPU 0, GPU 1 and GPU 0 again."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import dense_ref
    g = seeded(4, 90)
    a = (g.random((512, 384)) * 2 - 1).astype(np.float16)
    b = (g.random((384, 640)) * 2 - 1).astype(np.float16)
    small_a = a[:96, :64].copy()                      # below the pair kernel's shape: the single-CTA kernel
    q, k, v = [(g.standard_normal((2, 256, 128)) * 0.5).astype(np.float16) for _ in range(3)]
    for d in (dev, wgf.Device(1), dev):
        got = d.tensor(a).mat_mul(d.tensor(b)).as_slice()
        assert normwise(got, a.astype(np.float64) @ b.astype(np.float64)) <= 1e-2
        got = d.tensor(small_a).mat_mul(d.tensor(b[:64])).as_slice()
        assert normwise(got, small_a.astype(np.float64) @ b[:64].astype(np.float64)) <= 1e-2
        got = d.tensor(q).attention(d.tensor(k), d.tensor(v), causal=True).as_slice()
        assert normwise(got, dense_ref.attention(q, k, v, True, 128 ** -0.5)) <= 2e-2


@pytest.mark.parametrize("shape", [(2100, 4420, 260), (4096, 2560, 512), (2, 2100, 2304, 264)])
def test_f32_wide_tile_kernel_on_ragged_shapes(shape, wgf, dev):
    """Large f32 products take the 128x256-tile kernel (cp.async ring); M, N and K that are not
    multiples of the tile (zero-filled pieces on three edges, a short last k tile) and a batch."""
    g = seeded(4, 70)
    if len(shape) == 4:
        B, M, N, K = shape
        a = (g.random((B, M, K), dtype=np.float32) * 2 - 1)
        b = (g.random((B, K, N), dtype=np.float32) * 2 - 1)
    else:
        M, N, K = shape
        a = (g.random((M, K), dtype=np.float32) * 2 - 1)
        b = (g.random((K, N), dtype=np.float32) * 2 - 1)
    t = dev.tensor(a).mat_mul(dev.tensor(b))       # per-kernel timing is on by default: the labels name the kernel
    got = t.as_slice()
    assert "sgemm_wide" in t.timing_labels()
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert normwise(got, ref) <= 1e-5
