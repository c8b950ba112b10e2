"""Llama-style decoder block (a composition of the primitives; the crate has no model code) against a
float64 numpy statement of the same math on a reduced shape.  f16 weights and activations: the bound
is 2e-2 norm-wise (matmul chain in f16 with fp32 accumulation)."""
import numpy as np
import pytest

from conftest import seeded

pytestmark = pytest.mark.gpu


def reference_block(x, W, n1, n2, cos, sin, mask, heads, eps):
    B, S, Hd = x.shape
    D = Hd // heads
    f = lambda a: a.astype(np.float64)
    x = f(x)

    def rms(t, w):
        return t / np.sqrt((t * t).mean(-1, keepdims=True) + eps) * f(w)

    def split(t):
        return t.reshape(B, S, heads, D).transpose(0, 2, 1, 3)

    def rope(t):
        c = np.concatenate([f(cos), f(cos)], 1)[:S][None, None]
        s = np.concatenate([f(sin), f(sin)], 1)[:S][None, None]
        rot = np.concatenate([-t[..., D // 2:], t[..., :D // 2]], -1)
        return t * c + rot * s

    wq, wk, wv, wo, wg, wu, wd = [f(w) for w in W]
    a = rms(x, n1)
    q, k, v = rope(split(a @ wq.T)), rope(split(a @ wk.T)), split(a @ wv.T)
    sc = q @ k.transpose(0, 1, 3, 2) / np.sqrt(D) + f(mask)[None, None]
    sc = sc - sc.max(-1, keepdims=True)
    p = np.exp(sc)
    p = p / p.sum(-1, keepdims=True)
    ctx = (p @ v).transpose(0, 2, 1, 3).reshape(B, S, Hd)
    h = x + ctx @ wo.T
    b = rms(h, n2)
    g = b @ wg.T
    return h + ((g / (1 + np.exp(-g))) * (b @ wu.T)) @ wd.T


@pytest.mark.parametrize("B,S,Hd,heads,inter", [(2, 64, 256, 4, 688), (1, 128, 512, 4, 1376)])
def test_llama_block_matches_float64(B, S, Hd, heads, inter, wgf, dev):
    g = seeded(5, 0)
    D = Hd // heads
    h16 = lambda a: a.astype(np.float16)
    x = h16(g.standard_normal((B, S, Hd)))
    shapes = [(Hd, Hd)] * 4 + [(inter, Hd), (inter, Hd), (Hd, inter)]
    W = [h16(g.standard_normal(s) * 0.02 * (8 if i < 4 else 4)) for i, s in enumerate(shapes)]
    n1 = h16(1 + 0.1 * g.standard_normal(Hd))
    n2 = h16(1 + 0.1 * g.standard_normal(Hd))
    pos = np.arange(S, dtype=np.float32)[:, None]
    inv = (1.0 / (10000.0 ** (np.arange(0, D, 2, dtype=np.float32) / D)))[None, :]
    cos, sin = h16(np.cos(pos * inv)), h16(np.sin(pos * inv))
    mask = np.where(np.arange(S)[None, :] <= np.arange(S)[:, None], 0.0, -np.inf).astype(np.float16)

    t = dev.tensor(x)
    before = dev.launch_count
    out = t.llama_block([dev.tensor(w) for w in W], dev.tensor(n1), dev.tensor(n2), dev.tensor(cos), dev.tensor(sin),
                        dev.tensor(mask), heads, 1e-5).as_slice()
    launches = dev.launch_count - before
    ref = reference_block(x, W, n1, n2, cos, sin, mask, heads, 1e-5)
    err = np.max(np.abs(out.astype(np.float64) - ref)) / np.max(np.abs(ref))
    assert out.shape == (B, S, Hd) and np.isfinite(out.astype(np.float32)).all()
    assert err <= 2e-2, err
    assert launches < 60
    # causality: changing the last token must not change the outputs of earlier tokens
    x2 = x.copy()
    x2[:, -1, :] += np.float16(1.0)
    out2 = dev.tensor(x2).llama_block([dev.tensor(w) for w in W], dev.tensor(n1), dev.tensor(n2), dev.tensor(cos),
                                      dev.tensor(sin), dev.tensor(mask), heads, 1e-5).as_slice()
    np.testing.assert_array_equal(out2[:, :-1], out[:, :-1])
