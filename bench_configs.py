"""Times every benchmark configuration on one GPU and prints one JSON object per row.

Run as  python bench.py --workload configs [--rows TEXT]  (one GPU; --rows keeps the rows whose name
contains TEXT, e.g. "C2", "attention", "matmul f16").  Each row builds its lazy graph afresh every
iteration, materialises it with per-kernel timestamps on (the crate's own method: timestamp queries
around each dispatch, benches/elementwise.rs:42-43) and reports, per iteration, the median over the
iterations of the summed kernel times.  Inputs larger than the 126 MB L2 are reused as they are;
smaller inputs rotate through enough copies to exceed L2 ("cold") and are also timed on one copy
("warm").  `bytes` / `flop` are the algorithmic figures of the row, so GB/s and TFLOP/s are
algorithmic too.  Beside that, `back_to_back_us` is the time per materialisation when the same
launches follow one another with nothing between them (stream_time_row).
"""
import collections
import json

import numpy as np

SEED = 0xB2000000


def rng(config, index):
    return np.random.Generator(np.random.PCG64(SEED + 16 * config + index))


def uniform(g, shape, lo, hi):
    return (g.random(shape, dtype=np.float32) * (hi - lo) + lo).astype(np.float32)


def normal(g, shape, mu=0.0, sigma=1.0):
    return (g.standard_normal(shape, dtype=np.float32) * sigma + mu).astype(np.float32)


class Row:
    def __init__(self, name, build, nbytes=None, flop=None, variants=1, custom=None):
        self.name, self.build, self.nbytes, self.flop, self.variants = name, build, nbytes, flop, variants
        self.custom = custom          # a row that measures itself: returns the fields of its JSON object


def time_row(dev, row, iters, warmup):
    # A tensor reports the timestamps of every kernel its (merged) graph has run so far, the
    # inputs' earlier iterations included: one iteration's share is the growth of the total.
    per_iter, labels = [], None
    total_before, labels_before = 0, collections.Counter()
    for i in range(warmup + iters):
        t = row.build(i % row.variants)
        if row.variants > 1:
            probe = row.build(i % row.variants)
            total_before = sum(probe.all_timing_information())
            labels_before = collections.Counter(probe.timing_labels())
            probe.release()
        t.materialize()
        dev.sync()
        total = sum(t.all_timing_information())
        names = collections.Counter(t.timing_labels())
        if i >= warmup:
            per_iter.append(total - total_before)
            if labels is None:
                labels = dict(names - labels_before)
        total_before, labels_before = total, names
        t.release()
    per_iter.sort()
    return per_iter[len(per_iter) // 2] * 1e-3, per_iter[0] * 1e-3, labels


def stream_time_row(dev, row, budget_s=0.03):
    """The same materialisation as a STREAM of launches with nothing between them: `reps` of them
    recorded once as a schedule (one CUDA graph) and replayed until about `budget_s` of device time
    has passed; wall clock around the replays with the device drained on both sides, divided by the
    number of materialisations.  An event pair around a single launch adds about 2.5 us of event
    handling to it (10 % of a 25 us kernel); back to back that cost is not there, and neither is the
    host's (a replay costs the host one graph launch per `reps` materialisations).  Returns
    microseconds per materialisation, or None where the row cannot be recorded."""
    import time
    reps = max(row.variants, 8)
    dev.set_timing(False)
    sched = None
    try:
        with dev.record() as sched:
            for k in range(reps):
                t = row.build(k % row.variants)
                t.materialize()
                t.release()
        dev.sync()
        sched.launch()
        dev.sync()
        t0 = time.perf_counter()
        sched.launch()
        dev.sync()
        once = max(time.perf_counter() - t0, 1e-6)
        n = max(3, min(400, int(budget_s / once)))
        t0 = time.perf_counter()
        for _ in range(n):
            sched.launch()
        dev.sync()
        us = (time.perf_counter() - t0) / (n * reps) * 1e6
        # tens of milliseconds of tensor-core work back to back leave the GPU at its power cap: give it a
        # moment, or the next row's single launches are timed at the clocks this row ended with
        time.sleep(0.3)
        return us
    except Exception:
        return None
    finally:
        if sched is not None and getattr(sched, "h", None):
            sched.destroy()
        dev.set_timing(True)


# Each group allocates its inputs only when one of its rows is wanted.
def group_c1(wgf, dev):
    """Fused element-wise chain y = cos(sin(x*2+1))*0.5 + exp(-x*x)."""
    x1 = [dev.tensor(uniform(rng(1, k), (1024, 1024), -1, 1)) for k in range(64)]   # 256 MiB of inputs for the cold run

    def chain(x):
        return (x * 2.0 + 1.0).sin().cos() * 0.5 + (-(x * x)).exp()
    xb = dev.tensor(uniform(rng(1, 100), (8192, 4096), -1, 1))

    def host_cost(passes=200):
        """Wall-clock per materialisation of the small chain (the kernel itself takes a few
        microseconds): built and resolved every time, against one replay of a recorded schedule."""
        import time
        dev.set_timing(False)
        chain(x1[0]).materialize()
        dev.sync()
        t0 = time.perf_counter()
        for _ in range(passes):
            chain(x1[0]).materialize()
        dev.sync()
        eager = (time.perf_counter() - t0) / passes
        with dev.record() as s:
            y = chain(x1[0]).materialize()
        dev.sync()
        t0 = time.perf_counter()
        for _ in range(passes):
            s.launch()
        dev.sync()
        replay = (time.perf_counter() - t0) / passes
        y.release()
        s.destroy()
        dev.set_timing(True)
        return {"eager_us_per_pass": round(eager * 1e6, 2), "replay_us_per_pass": round(replay * 1e6, 2),
                "passes": passes, "bytes": 8388608, "replay_gbs": round(8388608 / replay / 1e9, 1)}

    return [Row("C1 chain f32 [1024,1024] wall clock per pass, resolved each time vs recorded schedule", None,
                custom=host_cost),
            Row("C1 chain f32 [1024,1024] cold", lambda k: chain(x1[k]), nbytes=8388608, variants=64),
            Row("C1 chain f32 [1024,1024] warm", lambda k: chain(x1[0]), nbytes=8388608),
            Row("C1' chain f32 [8192,4096]", lambda k: chain(xb), nbytes=2 * 134217728),
            Row("C1 x*2+1 f32 [8192,4096]", lambda k: xb * 2.0 + 1.0, nbytes=2 * 134217728)]


def group_c2(wgf, dev):
    """Row-wise RmsNorm / softmax and reductions of f32 [8192,4096]."""
    x2 = dev.tensor(normal(rng(2, 0), (8192, 4096)))
    w2 = dev.tensor(normal(rng(2, 1), (4096,), 1.0, 0.1))
    normed = x2.layer_norm(w2, 1e-5)
    normed.materialize()

    class Both:
        """RmsNorm->softmax and sum(exp(x)) requested together: one kernel."""

        def __init__(self):
            self.y = x2.layer_norm(w2, 1e-5).softmax_last_dim()
            self.s = x2.exp().sum(0).sum(0)

        def materialize(self):
            wgf.Tensor.materialize_all([self.y, self.s])

        def all_timing_information(self):
            return self.y.all_timing_information()

        def timing_labels(self):
            return self.y.timing_labels()

        def release(self):
            self.y.release()
            self.s.release()

    return [Row("C2a RmsNorm rows f32 [8192,4096]", lambda k: x2.layer_norm(w2, 1e-5), nbytes=268451840),
            Row("C2b softmax rows f32 [8192,4096]", lambda k: normed.softmax_last_dim(), nbytes=268435456),
            Row("C2ab RmsNorm->softmax f32 [8192,4096]", lambda k: x2.layer_norm(w2, 1e-5).softmax_last_dim(), nbytes=268451840),
            Row("C2ab+c RmsNorm->softmax with sum(exp(x)) riding along", lambda k: Both(), nbytes=268451844),
            Row("C2c sum(exp(x)) f32 [8192,4096]", lambda k: x2.exp().sum(0).sum(0), nbytes=134217728),
            Row("C2 sum(x) all f32 [8192,4096]", lambda k: x2.sum(0).sum(0), nbytes=134217728),
            Row("C2 sum(x, axis 1) f32 [8192,4096]", lambda k: x2.sum(1), nbytes=134217728 + 32768),
            Row("C2 max(x, axis 1) f32 [8192,4096]", lambda k: x2.max(1), nbytes=134217728 + 32768),
            Row("C2 sum(x, axis 0) f32 [8192,4096]", lambda k: x2.sum(0), nbytes=134217728 + 16384)]


def group_c3(wgf, dev):
    """Pair-wise with broadcast operands, transposed views, casts."""
    a = dev.tensor(normal(rng(3, 0), (64, 512, 1024)))
    b = dev.tensor(uniform(rng(3, 1), (512, 1024), -1, 1))
    c = dev.tensor(uniform(rng(3, 2), (64, 1024), 0, 1))
    bv = b.broadcast((64, 512, 1024))
    cv = c.broadcast_axis(1, 512)
    at, bt, ct = a.transpose(0, 1), bv.transpose(0, 1), cv.transpose(0, 1)
    a12, b12, c12 = a.transpose(1, 2), bv.transpose(1, 2), cv.transpose(1, 2)
    a2 = dev.tensor(normal(rng(3, 3), (64, 512, 1024)))
    ah, a2h = a.cast(wgf.F16), a2.cast(wgf.F16)
    ah.materialize(), a2h.materialize()
    return [Row("C3a silu(a*1.5)+b*c f32 [64,512,1024]", lambda k: (a * 1.5).silu() + bv * cv, nbytes=270794752),
            Row("C3b same, operands permuted (1,0,2)", lambda k: (at * 1.5).silu() + bt * ct, nbytes=270794752),
            Row("C3b' same, a.transpose(1,2): strided inner axis", lambda k: (a12 * 1.5).silu() + b12 * c12, nbytes=270794752),
            Row("C3c cast f32->f16->f32 [64,512,1024]", lambda k: a.cast(wgf.F16).cast(wgf.F32), nbytes=268435456),
            Row("C3 cast f32->f16 [64,512,1024]", lambda k: a.cast(wgf.F16), nbytes=134217728 + 67108864),
            Row("C3 reshape of a.transpose(1,2) (gather) f32", lambda k: a12.reshape((64 * 1024, 512)), nbytes=268435456),
            Row("C3 a+b f32 [64,512,1024]", lambda k: a + a2, nbytes=3 * 134217728),
            Row("C3 a+b f16 [64,512,1024]", lambda k: ah + a2h, nbytes=3 * 67108864),
            Row("C3 silu(a)*b f16 [64,512,1024]", lambda k: ah.silu() * a2h, nbytes=3 * 67108864),
            Row("C3 softmax rows f16 [64*512,1024]", lambda k: ah.softmax_last_dim(), nbytes=2 * 67108864)]


def group_c4(wgf, dev):
    """MatMul: square f32 / f16, batched f16, decode GEMV."""
    n = 4096
    af = dev.tensor(uniform(rng(4, 0), (n, n), -1, 1))
    bf = dev.tensor(uniform(rng(4, 1), (n, n), -1, 1))
    ah, bh = af.cast(wgf.F16), bf.cast(wgf.F16)
    ah.materialize(), bh.materialize()
    a3 = dev.tensor(uniform(rng(4, 2), (32, 1024, 128), -1, 1).astype(np.float16))
    b3 = dev.tensor(uniform(rng(4, 3), (32, 128, 1024), -1, 1).astype(np.float16))
    xv = dev.tensor(uniform(rng(4, 4), (1, 4096), -1, 1).astype(np.float16))
    wv = dev.tensor(uniform(rng(4, 5), (4096, 11008), -1, 1).astype(np.float16))
    wt = dev.tensor(uniform(rng(4, 6), (11008, 4096), -1, 1).astype(np.float16))
    return [Row("C4a matmul f32 4096^3", lambda k: af.mat_mul(bf), flop=2 * n ** 3),
            Row("C4b matmul f16 4096^3", lambda k: ah.mat_mul(bh), flop=2 * n ** 3),
            Row("C4b matmul f16 4096^3, B transposed view", lambda k: ah.mat_mul(bh.transpose(0, 1)), flop=2 * n ** 3),
            Row("C4c batched f16 [32,1024,128]x[32,128,1024]", lambda k: a3.mat_mul(b3), nbytes=83886080, flop=8589934592),
            Row("C4d GEMV f16 [1,4096]x[4096,11008]", lambda k: xv.mat_mul(wv), nbytes=90207744),
            Row("C4d GEMV f16, weight stored [11008,4096]", lambda k: xv.mat_mul(wt.transpose(0, 1)), nbytes=90207744)]


def group_c5(wgf, dev):
    """Pieces of the Llama block at its full shape: fused causal attention, rope, SiLU gate."""
    g = rng(5, 8)
    bh, s, d = 256, 2048, 128
    q, k, v = (dev.tensor(normal(g, (bh, s, d)).astype(np.float16)) for _ in range(3))
    pos = np.arange(s, dtype=np.float32)[:, None]
    inv = (1.0 / (10000.0 ** (np.arange(0, d, 2, dtype=np.float32) / d)))[None, :]
    cos, sin = dev.tensor(np.cos(pos * inv).astype(np.float16)), dev.tensor(np.sin(pos * inv).astype(np.float16))
    gate, up = (dev.tensor(normal(g, (16384, 11008)).astype(np.float16)) for _ in range(2))
    xt = dev.tensor(normal(g, (16384, 4096)).astype(np.float16))
    wq, wu, wd, wg = (dev.tensor((normal(g, shape) * 0.02).astype(np.float16))
                      for shape in ((4096, 4096), (11008, 4096), (4096, 11008), (11008, 4096)))
    causal_flop = 4 * bh * s * s * d // 2          # QK^T and PV, the masked half not counted
    return [Row("C5 attention f16 causal [256,2048,128]", lambda i: q.attention(k, v, causal=True), flop=causal_flop),
            Row("C5 attention f16 full [256,2048,128]", lambda i: q.attention(k, v), flop=2 * causal_flop),
            Row("C5 rope f16 [256,2048,128]", lambda i: q.rope(cos, sin), nbytes=2 * bh * s * d * 2),
            Row("C5 silu(gate)*up f16 [16384,11008]", lambda i: gate.silu() * up, nbytes=3 * 16384 * 11008 * 2),
            # the block's projections: 16384 tokens against weights stored [out, in]
            Row("C5 projection f16 [16384,4096] x W^T [4096,4096]", lambda i: xt.mat_mul(wq.transpose(0, 1)),
                flop=2 * 16384 * 4096 * 4096),
            Row("C5 up projection f16 [16384,4096] x W^T [11008,4096]", lambda i: xt.mat_mul(wu.transpose(0, 1)),
                flop=2 * 16384 * 4096 * 11008),
            Row("C5 down projection f16 [16384,11008] x W^T [4096,11008]", lambda i: gate.mat_mul(wd.transpose(0, 1)),
                flop=2 * 16384 * 4096 * 11008),
            # the same products with the element-wise step that follows them done in the GEMM's epilogue
            Row("C5 gate and up in one GEMM: silu(x Wg^T) * (x Wu^T) f16", lambda i: xt.mat_mul(wg.transpose(0, 1)).silu() * xt.mat_mul(wu.transpose(0, 1)),
                flop=4 * 16384 * 4096 * 11008),
            Row("C5 down projection with the residual add in its epilogue f16", lambda i: xt + gate.mat_mul(wd.transpose(0, 1)),
                flop=2 * 16384 * 4096 * 11008)]


GROUPS = [("C1", group_c1), ("C2", group_c2), ("C3", group_c3), ("C4", group_c4), ("C5", group_c5)]


def run(wgf, dev, peak_gbs, peak_tflops, iters=30, warmup=5, only=None, emit=print, stream=True, peak_tflops_sustained=None):
    dev.set_timing(True)
    results = []
    for prefix, make in GROUPS:
        if only and not (only.startswith(prefix) or not only.startswith("C")):
            continue
        rows = [r for r in make(wgf, dev) if not only or only in r.name]
        for row in rows:
            if row.custom:
                r = {"row": row.name, **row.custom()}
                results.append(r)
                emit(json.dumps(r))
                continue
            med, best, labels = time_row(dev, row, iters, warmup)
            med = max(med, 1e-9)          # the compile-only device records no time
            r = {"row": row.name, "kernels": labels, "median_us": round(med, 2), "best_us": round(best, 2)}
            stream_us = stream_time_row(dev, row) if stream else None
            if stream_us:
                r["back_to_back_us"] = round(stream_us, 2)
                if row.nbytes:
                    r["back_to_back_frac_hbm"] = round(row.nbytes / stream_us / 1e3 / peak_gbs, 3)
                elif row.flop and "f32" in row.name:
                    r["back_to_back_frac_ffma_peak"] = round(row.flop / stream_us / 1e6 / 74.5, 3)
                elif row.flop:
                    # tensor-core kernels launched back to back for tens of milliseconds run under the
                    # power cap: the denominator is the cuBLAS figure measured the same way
                    r["back_to_back_tflops"] = round(row.flop / stream_us / 1e6, 1)
                    r["back_to_back_frac_bf16_sustained"] = round(row.flop / stream_us / 1e6 / (peak_tflops_sustained or peak_tflops), 3)
            if row.nbytes:
                r["gbs"] = round(row.nbytes / med / 1e3, 1)
                r["frac_hbm"] = round(row.nbytes / med / 1e3 / peak_gbs, 3)
            if row.flop:
                r["tflops"] = round(row.flop / med / 1e6, 1)
                if not row.nbytes and "f32" in row.name:
                    # FFMA peak: 148 SMs x 128 lanes x 2 flop at the 1965 MHz maximum clock
                    r["frac_ffma_peak"] = round(row.flop / med / 1e6 / 74.5, 3)
                elif not row.nbytes:
                    r["frac_bf16_peak"] = round(row.flop / med / 1e6 / peak_tflops, 3)
            results.append(r)
            emit(json.dumps(r))
        del rows
    dev.set_timing(False)
    return results
