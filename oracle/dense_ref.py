"""float64 numpy statements of the tensor-core ops at full size: the Llama-style decoder block and
causal attention for sampled tokens of a large input, and a matmul check that covers every tile
through projections.  TEST INFRASTRUCTURE ONLY (the checker of tests/ and of bench.py's
`check` keys); nothing in the product may import it.

The crate has no model code (its composites stop at rms-norm, softmax, silu and rope:
src/composite/rms_norm.rs:8-15, softmax.rs:4-10, silu.rs:4-7, rope.rs:13-22); the block is those
composites around matmuls:
    h   = x + Wo . attn(rope(Wq . n1), rope(Wk . n1), Wv . n1),   n1 = rms_norm(x, w1, eps)
    out = h + Wd . (silu(Wg . n2) * (Wu . n2)),                   n2 = rms_norm(h, w2, eps)
Causal attention of one token needs the keys and values of its own batch element only, so the
reference for a handful of tokens of a [8, 2048, 4096] input costs two [2048,4096]x[4096,4096]
products per sampled batch element instead of the whole block.
"""
import numpy as np


def _f(a):
    return np.asarray(a).astype(np.float64)


def rms_norm(t, w, eps):
    return t / np.sqrt((t * t).mean(-1, keepdims=True) + eps) * _f(w)


def rope_rows(t, cos, sin, positions):
    """t [..., len(positions), D]; cos/sin [S, D/2] (rotate-half form)."""
    d = t.shape[-1]
    c = np.concatenate([_f(cos), _f(cos)], 1)[positions]
    s = np.concatenate([_f(sin), _f(sin)], 1)[positions]
    rot = np.concatenate([-t[..., d // 2:], t[..., :d // 2]], -1)
    return t * c + rot * s


def llama_block_tokens(xb, W, n1, n2, cos, sin, heads, eps, tokens):
    """Rows `tokens` of the block's output for ONE batch element xb [S, hidden], causal attention.
    W = [Wq, Wk, Wv, Wo, Wg, Wu, Wd], each [out, in]."""
    S, Hd = xb.shape
    D = Hd // heads
    tokens = np.asarray(tokens)
    x = _f(xb)
    wq, wk, wv, wo, wg, wu, wd = [_f(w) for w in W]
    a = rms_norm(x, n1, eps)
    allpos = np.arange(S)
    k = rope_rows((a @ wk.T).reshape(S, heads, D).transpose(1, 0, 2), cos, sin, allpos)     # [heads, S, D]
    v = (a @ wv.T).reshape(S, heads, D).transpose(1, 0, 2)
    q = rope_rows((a[tokens] @ wq.T).reshape(len(tokens), heads, D).transpose(1, 0, 2), cos, sin, tokens)
    sc = q @ k.transpose(0, 2, 1) / np.sqrt(D)                                             # [heads, T, S]
    sc = np.where(allpos[None, None, :] <= tokens[None, :, None], sc, -np.inf)
    sc = sc - sc.max(-1, keepdims=True)
    p = np.exp(sc)
    p = p / p.sum(-1, keepdims=True)
    ctx = (p @ v).transpose(1, 0, 2).reshape(len(tokens), Hd)
    h = x[tokens] + ctx @ wo.T
    b = rms_norm(h, n2, eps)
    g = b @ wg.T
    return h + ((g / (1 + np.exp(-g))) * (b @ wu.T)) @ wd.T


def attention(q, k, v, causal, scale):
    """softmax(scale * q k^T [causal]) v for [n, S, D] arrays."""
    q, k, v = _f(q), _f(k), _f(v)
    s = q @ k.transpose(0, 2, 1) * scale
    if causal:
        sq, sk = s.shape[1:]
        s = np.where(np.arange(sk)[None, :] <= np.arange(sq)[:, None], s, -np.inf)
    s = s - s.max(-1, keepdims=True)
    p = np.exp(s)
    return (p / p.sum(-1, keepdims=True)) @ v


def matmul_projection_error(c, a, b, block=256, vectors=3, seed=0):
    """Largest error of C's column blocks projected on random vectors, relative to the largest
    projection: for every block of `block` columns, C[:, blk] v against A (B[:, blk] v) in float64.
    Every entry of C takes part at O(n^2) cost.  The rounding errors of the entries of a row are
    independent, so they grow like sqrt(block) in a projection while the reference grows the same
    way: the result is the typical relative error of an ENTRY (about 2^-12 for an f16 result), and a
    tile whose entries are off by a relative e shows as about e."""
    a64, b64, c64 = _f(a), _f(b), _f(c)
    n = b64.shape[1]
    g = np.random.Generator(np.random.PCG64(seed))
    worst, scale = 0.0, 0.0
    for j0 in range(0, n, block):
        v = g.standard_normal((min(block, n - j0), vectors))
        ref = a64 @ (b64[:, j0:j0 + block] @ v)
        got = c64[:, j0:j0 + block] @ v
        worst = max(worst, float(np.max(np.abs(got - ref))))
        scale = max(scale, float(np.max(np.abs(ref))))
    return worst / max(scale, 1e-300)
