"""Fused tensor-core attention (wgf_tensor_attention; the crate has no attention op) against a float64
numpy statement of softmax(scale * q k^T [causal]) v, and against the same request run as
mat_mul / softmax_last_dim / mat_mul through an explicit mask.  16-bit inputs, fp32 accumulation:
the bound is 1e-2 norm-wise, as for 16-bit matmul."""
import numpy as np
import pytest

from conftest import seeded

pytestmark = pytest.mark.gpu


def bf16_round(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(u):
    return (u.astype(np.uint32) << 16).view(np.float32)


def reference(q, k, v, causal, scale):
    q, k, v = (a.astype(np.float64) for a in (q, k, v))
    s = q @ k.transpose(0, 2, 1) * scale
    if causal:
        sq, sk = s.shape[1:]
        s = np.where(np.arange(sk)[None, :] <= np.arange(sq)[:, None], s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    return (p / p.sum(-1, keepdims=True)) @ v


def normwise(got, ref):
    return float(np.max(np.abs(got.astype(np.float64) - ref)) / np.max(np.abs(ref)))


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("n,seq", [(1, 128), (3, 256), (2, 640), (150, 128), (5, 1024)])
def test_fused_attention_f16(n, seq, causal, wgf, dev):
    g = seeded(5, 3)
    q, k, v = (g.standard_normal((n, seq, 128), dtype=np.float32).astype(np.float16) for _ in range(3))
    tq, tk, tv = dev.tensor(q), dev.tensor(k), dev.tensor(v)
    before = dev.launch_count
    out = tq.attention(tk, tv, causal=causal).as_slice()
    assert dev.launch_count - before == 1                     # one kernel; the scores never reach memory
    assert out.shape == (n, seq, 128) and out.dtype == np.float16
    assert normwise(out, reference(q, k, v, causal, 1 / np.sqrt(128))) <= 1e-2


def test_fused_attention_large_scores_and_scale(wgf, dev):
    """Rows whose scores span a wide range (the max-subtraction matters), and a caller-given scale."""
    g = seeded(5, 4)
    q, k, v = (g.standard_normal((4, 384, 128), dtype=np.float32) for _ in range(3))
    q = (q * 6).astype(np.float16)
    k = (k * 6).astype(np.float16)
    v = v.astype(np.float16)
    out = dev.tensor(q).attention(dev.tensor(k), dev.tensor(v), causal=True, scale=0.25).as_slice()
    assert np.isfinite(out.astype(np.float32)).all()
    assert normwise(out, reference(q, k, v, True, 0.25)) <= 1e-2


def test_fused_attention_growing_maxima(wgf, dev):
    """Keys whose norm grows along the sequence: the row maxima keep growing from key tile to key
    tile, so the one-pass kernel has to rescale its accumulators again and again."""
    g = seeded(5, 6)
    n, seq = 3, 1024
    q = g.standard_normal((n, seq, 128), dtype=np.float32)
    k = g.standard_normal((n, seq, 128), dtype=np.float32) * (1 + 7 * np.arange(seq, dtype=np.float32) / seq)[None, :, None]
    # every query looks a little along every key direction it will meet, so later keys score higher
    q = (q + 0.5 * np.sign(k.mean(axis=1, keepdims=True))).astype(np.float16)
    k = (k + 0.5 * np.sign(k.mean(axis=1, keepdims=True)) * (1 + 7 * np.arange(seq, dtype=np.float32) / seq)[None, :, None]).astype(np.float16)
    v = g.standard_normal((n, seq, 128), dtype=np.float32).astype(np.float16)
    for causal in (True, False):
        out = dev.tensor(q).attention(dev.tensor(k), dev.tensor(v), causal=causal, scale=0.5).as_slice()
        assert np.isfinite(out.astype(np.float32)).all()
        assert normwise(out, reference(q, k, v, causal, 0.5)) <= 1e-2


@pytest.mark.parametrize("variant", ["WGF_ATT_TWO_PASS=1", "WGF_ATT_SINGLE=1", "WGF_ATT_SMEM_P=1", "WGF_ATT_MODE=0", "WGF_ATT_MODE=1"])
@pytest.mark.parametrize("n,seq", [(3, 256), (2, 640), (5, 1024)])
def test_fused_attention_other_kernel_variants(n, seq, variant, wgf, dev, monkeypatch):
    """The kernel forms kept beside the default: P through shared memory (two query tiles per CTA, one
    pass or two; one query tile per CTA), and the ways the softmax warps of the default kernel can go
    over the scores (one sweep from registers, two sweeps over tensor memory)."""
    name, value = variant.split("=")
    monkeypatch.setenv(name, value)
    g = seeded(5, 7)
    q, k, v = (g.standard_normal((n, seq, 128), dtype=np.float32) for _ in range(3))
    q, k, v = (q * 3).astype(np.float16), (k * 3).astype(np.float16), v.astype(np.float16)
    for causal in (True, False):
        out = dev.tensor(q).attention(dev.tensor(k), dev.tensor(v), causal=causal).as_slice()
        assert normwise(out, reference(q, k, v, causal, 1 / np.sqrt(128))) <= 1e-2


def test_fused_attention_bf16_and_strided_views(wgf, dev):
    g = seeded(5, 5)
    n, seq = 6, 256
    raw = [g.standard_normal((n, seq, 128), dtype=np.float32) for _ in range(3)]
    u = [bf16_round(a) for a in raw]
    t = [dev.tensor(a, dtype=wgf.BF16) for a in u]
    out = bf16_to_f32(t[0].attention(t[1], t[2], causal=True).as_slice())
    ref = reference(*[bf16_to_f32(a) for a in u], True, 1 / np.sqrt(128))
    assert normwise(out, ref) <= 1e-2
    # q, k, v as views of one [seq, n, 3, 128] tensor (heads interleaved the way a fused QKV projection leaves them)
    packed = g.standard_normal((seq, n, 3, 128), dtype=np.float32).astype(np.float16)
    tp = dev.tensor(packed.reshape(seq, n, 384))
    parts = [tp.narrow(2, 128 * i, 128).transpose(0, 1) for i in range(3)]          # [n, seq, 128], row stride n * 384
    out = parts[0].attention(parts[1], parts[2], causal=True).as_slice()
    pq, pk, pv = (np.ascontiguousarray(packed[:, :, i, :].transpose(1, 0, 2)) for i in range(3))
    assert normwise(out, reference(pq, pk, pv, True, 1 / np.sqrt(128))) <= 1e-2


def test_attention_other_shapes_run_as_primitives(wgf, dev):
    """Head dimension 64, f32, ragged sequence lengths or an explicit mask: mat_mul, softmax, mat_mul."""
    g = seeded(5, 6)
    n, seq, d = 3, 100, 64
    q, k, v = (g.standard_normal((n, seq, d), dtype=np.float32) for _ in range(3))
    mask = np.where(np.arange(seq)[None, :] <= np.arange(seq)[:, None], 0.0, -np.inf).astype(np.float32)
    tq, tk, tv = dev.tensor(q), dev.tensor(k), dev.tensor(v)
    out = tq.attention(tk, tv, mask=dev.tensor(mask)).as_slice()
    assert normwise(out, reference(q, k, v, True, 1 / np.sqrt(d))) <= 1e-4
    out = tq.attention(tk, tv).as_slice()                       # no mask, not causal
    assert normwise(out, reference(q, k, v, False, 1 / np.sqrt(d))) <= 1e-4
    with pytest.raises(wgf.WgfError) as e:                      # causal without a mask needs the fused shapes
        tq.attention(tk, tv, causal=True)
    assert e.value.status == "UNSUPPORTED"
    # an explicit mask on fusable shapes takes the primitive path and agrees with the fused kernel
    h = [g.standard_normal((2, 256, 128), dtype=np.float32).astype(np.float16) for _ in range(3)]
    th = [dev.tensor(a) for a in h]
    m16 = np.where(np.arange(256)[None, :] <= np.arange(256)[:, None], 0.0, -np.inf).astype(np.float16)
    a = th[0].attention(th[1], th[2], mask=dev.tensor(m16)).as_slice()
    b = th[0].attention(th[1], th[2], causal=True).as_slice()
    assert normwise(a, b.astype(np.float64)) <= 1e-2


def test_llama_block_without_mask_uses_fused_attention(wgf, dev):
    from test_gpu_llama_block import reference_block
    g = seeded(5, 7)
    B, S, Hd, heads, inter = 2, 256, 512, 4, 1376
    D = Hd // heads
    h16 = lambda a: a.astype(np.float16)
    x = h16(g.standard_normal((B, S, Hd)))
    shapes = [(Hd, Hd)] * 4 + [(inter, Hd), (inter, Hd), (Hd, inter)]
    W = [h16(g.standard_normal(s) * 0.02 * (8 if i < 4 else 4)) for i, s in enumerate(shapes)]
    n1, n2 = h16(1 + 0.1 * g.standard_normal(Hd)), h16(1 + 0.1 * g.standard_normal(Hd))
    pos = np.arange(S, dtype=np.float32)[:, None]
    inv = (1.0 / (10000.0 ** (np.arange(0, D, 2, dtype=np.float32) / D)))[None, :]
    cos, sin = h16(np.cos(pos * inv)), h16(np.sin(pos * inv))
    mask = np.where(np.arange(S)[None, :] <= np.arange(S)[:, None], 0.0, -np.inf).astype(np.float16)
    args = lambda: ([dev.tensor(w) for w in W], dev.tensor(n1), dev.tensor(n2), dev.tensor(cos), dev.tensor(sin))
    before = dev.launch_count
    fused = dev.tensor(x).llama_block(*args(), None, heads, 1e-5).as_slice()
    n_fused = dev.launch_count - before
    before = dev.launch_count
    masked = dev.tensor(x).llama_block(*args(), dev.tensor(mask), heads, 1e-5).as_slice()
    n_masked = dev.launch_count - before
    assert n_fused < n_masked
    ref = reference_block(x, W, n1, n2, cos, sin, mask, heads, 1e-5)
    for out in (fused, masked):
        assert np.max(np.abs(out.astype(np.float64) - ref)) / np.max(np.abs(ref)) <= 2e-2
