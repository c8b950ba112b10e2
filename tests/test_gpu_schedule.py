"""Recorded schedules (wgf_schedule_*): a materialisation captured once and replayed must give,
for new input data, exactly the bits that an ordinary materialisation gives."""
import numpy as np
import pytest

from conftest import seeded

pytestmark = pytest.mark.gpu


def rows_and_sum(x, w):
    return x.layer_norm(w, 1e-5).softmax_last_dim(), x.exp().sum(0).sum(0)


def test_replay_matches_eager_for_new_inputs(wgf, dev):
    g = seeded(40, 0)
    xs = [g.standard_normal((512, 1024), dtype=np.float32) for _ in range(3)]
    wv = g.standard_normal(1024, dtype=np.float32)
    x, w = dev.tensor(xs[0]), dev.tensor(wv)
    before = dev.launch_count
    with dev.record() as s:
        y, t = rows_and_sum(x, w)
        wgf.Tensor.materialize_all([y, t])
        z = (y * 3.0 + t.broadcast_axis(0, 1024).broadcast_axis(0, 512)).materialize()       # needs both results of the first kernel
    assert s.kernel_count == dev.launch_count - before == 2
    for data in xs:                            # xs[0] again first: the values of the recording itself
        x.write(data)
        s.launch()
        got_y, got_t, got_z = y.as_slice(), t.as_slice(), z.as_slice()
        ex, ew = dev.tensor(data), dev.tensor(wv)
        ey, et = rows_and_sum(ex, ew)
        wgf.Tensor.materialize_all([ey, et])
        ez = ey * 3.0 + et.broadcast_axis(0, 1024).broadcast_axis(0, 512)
        assert np.array_equal(got_y, ey.as_slice())
        assert np.array_equal(got_t, et.as_slice())
        assert np.array_equal(got_z, ez.as_slice())
    s.destroy()


def test_values_are_there_after_the_recording(wgf, dev):
    """wgf_schedule_end runs the schedule once: tensors materialised while recording read like
    any materialised tensor."""
    a = seeded(41, 0).standard_normal((300, 77), dtype=np.float32)
    x = dev.tensor(a)
    with dev.record() as s:
        y = (x * 2.0 - 1.0).sum(1).materialize()
    ref = (dev.tensor(a) * 2.0 - 1.0).sum(1).as_slice()
    assert np.array_equal(y.as_slice(), ref)
    s.destroy()
    assert np.array_equal(y.as_slice(), ref)   # the tensor outlives the schedule


def test_schedule_memory_is_not_handed_out_while_it_lives(wgf, dev):
    """Intermediates of a recording are freed inside it; the pool must not give their blocks to
    anyone else, or a replay would write over the new owner's data."""
    g = seeded(42, 0)
    a = g.standard_normal((1024, 1024), dtype=np.float32)
    x = dev.tensor(a)
    with dev.record() as s:
        h = (x.exp().materialize() * 0.5).materialize()      # first result is released below
        y = h.sum(0).materialize()
    h.release()
    # same sizes as the schedule's blocks: the pool would reuse them if it had them
    others = [dev.tensor(np.full((1024, 1024), float(i), np.float32)) for i in range(4)]
    grown = [(o + 0.0).materialize() for o in others]
    for _ in range(3):
        s.launch()
    for i, o in enumerate(grown):
        assert np.array_equal(o.as_slice(), np.full((1024, 1024), float(i), np.float32))
    ref = (dev.tensor(a).exp() * 0.5).sum(0).as_slice()
    assert np.array_equal(y.as_slice(), ref)
    s.destroy()


def test_matmul_and_attention_replay(wgf, dev, orc):
    """Tensor-core kernels (TMA descriptors by value, split-K scratch and flags, ticketed
    finishes) inside a schedule, replayed with new operands."""
    g = seeded(43, 0)
    M, K, N = 512, 1024, 768

    def operands():
        return ((g.standard_normal((M, K), dtype=np.float32) * 0.1).astype(np.float16),
                (g.standard_normal((K, N), dtype=np.float32) * 0.1).astype(np.float16),
                (g.standard_normal((4, 256, 128), dtype=np.float32)).astype(np.float16))

    a0, b0, q0 = operands()
    a, b, q = dev.tensor(a0), dev.tensor(b0), dev.tensor(q0)
    with dev.record() as s:
        c = a.mat_mul(b).materialize()
        v = a.narrow(0, 0, 1).mat_mul(b).materialize()     # GEMV with a ticketed finish
        o = q.attention(q, q, causal=True).materialize()
    for _ in range(2):
        a1, b1, q1 = operands()
        a.write(a1), b.write(b1), q.write(q1)
        s.launch()
        ea, eb, eq = dev.tensor(a1), dev.tensor(b1), dev.tensor(q1)
        assert np.array_equal(c.as_slice(), ea.mat_mul(eb).as_slice())
        assert np.array_equal(v.as_slice(), ea.narrow(0, 0, 1).mat_mul(eb).as_slice())
        assert np.array_equal(o.as_slice(), eq.attention(eq, eq, causal=True).as_slice())
        ref = a1.astype(np.float64) @ b1.astype(np.float64)
        assert np.abs(c.as_slice().astype(np.float64) - ref).max() / np.abs(ref).max() <= 1e-2
    s.destroy()


def test_kernels_first_met_while_recording(wgf, dev):
    """A kernel that has to be generated, compiled and loaded in the middle of a recording."""
    a = seeded(44, 0).standard_normal((64, 1000), dtype=np.float32)
    x = dev.tensor(a)
    compiles = dev.compile_count
    with dev.record() as s:
        # an op chain no other test builds, on a shape no other test uses
        y = ((x * 1.25).cos().abs() + x.tanh()).max(1).materialize()
    assert dev.compile_count > compiles
    x.write(a * 0.5)
    s.launch()
    e = dev.tensor(a * 0.5)
    assert np.array_equal(y.as_slice(), ((e * 1.25).cos().abs() + e.tanh()).max(1).as_slice())
    s.destroy()


def test_replay_of_a_long_chain_and_its_host_time(wgf, dev):
    """What the schedule is for: a chain of small kernels is bound by the host's per-kernel cost;
    the replay queues them with one call."""
    import time
    a = seeded(45, 0).standard_normal((256, 256), dtype=np.float32)
    x = dev.tensor(a)

    def chain(t):
        for i in range(24):
            t = t.sum(0).broadcast((256, 256)) * 0.00390625 + t     # column reduction + element-wise kernel
        return t

    dev.set_timing(False)
    try:
        chain(x).materialize()                         # compile everything first
        dev.sync()
        t0 = time.perf_counter()
        for _ in range(20):
            chain(x).materialize()
        dev.sync()
        eager = (time.perf_counter() - t0) / 20
        with dev.record() as s:
            y = chain(x).materialize()
        dev.sync()
        t0 = time.perf_counter()
        for _ in range(20):
            s.launch()
        dev.sync()
        replay = (time.perf_counter() - t0) / 20
    finally:
        dev.set_timing(True)
    assert np.array_equal(y.as_slice(), chain(dev.tensor(a)).as_slice())
    # the two times are printed, not asserted on: wall-clock time on a shared host is not a correctness property
    print(f"\n{s.kernel_count} kernels: eager {eager * 1e6:.0f} us, replay {replay * 1e6:.0f} us per pass")
    s.destroy()


def test_schedule_keeps_the_inputs_it_reads_and_its_own_buffers(wgf, dev):
    """A replay reads the addresses of the tensors that existed before the recording and writes the
    addresses of the ones made inside it.  So (a) the schedule keeps an input alive after the caller
    has dropped its handle -- the pool must not hand the block to someone else -- and (b) a result of
    the recording never donates its buffer to a later in-place op, whose tensor the next replay
    would overwrite."""
    g = seeded(45, 0)
    a = g.standard_normal((512, 1024), dtype=np.float32)
    wv = g.standard_normal((512, 1024), dtype=np.float32)
    x, w = dev.tensor(a), dev.tensor(wv)
    with dev.record() as s:
        y = ((x * w).tanh() + w).materialize()
    want = ((dev.tensor(a) * dev.tensor(wv)).tanh() + dev.tensor(wv)).as_slice()
    assert np.array_equal(y.as_slice(), want)
    # (a) drop the weight's handle, then allocate tensors of the same size: without the schedule's
    # reference one of them would get w's block
    w.release()
    junk = [dev.tensor(g.standard_normal((512, 1024), dtype=np.float32)) for _ in range(4)]
    b = g.standard_normal((512, 1024), dtype=np.float32)
    x.write(b)
    s.launch()
    want_b = ((dev.tensor(b) * dev.tensor(wv)).tanh() + dev.tensor(wv)).as_slice()
    assert np.array_equal(y.as_slice(), want_b)
    # (b) y is consumed by an op that could run in place (y's handle is dropped, nothing else reads it)
    z = y * 2.0
    y.release()
    z.materialize()
    z_first = z.as_slice()
    assert np.array_equal(z_first, want_b * np.float32(2.0))
    x.write(a)
    s.launch()                                   # writes y's buffer again
    dev.sync()
    assert np.array_equal(z.as_slice(), z_first)  # z did not move into it
    del junk
    s.destroy()
