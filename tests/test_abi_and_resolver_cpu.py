"""CPU-only checks: the C ABI library loads and exports everything include/wgf.h declares; the
graph, the fusion resolver and the generated kernels are exercised on the compile-only device
(ordinal -1: every kernel is generated and compiled for sm_100a, nothing is executed)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "wgf.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(wgf_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(wgf):
    lib = wgf.lib()
    names = declared_functions()
    assert len(names) >= 60
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, f"declared in wgf.h but not exported: {missing}"
    assert lib.wgf_abi_version() == 2


def test_no_gpu_means_error_not_fallback(wgf):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(wgf.WgfError) as e:
        wgf.Device(0)
    assert e.value.status == "CUDA"


def test_compile_only_device_refuses_download(wgf, drydev):
    t = drydev.tensor(np.ones((4, 4), np.float32)) + 1.0
    t.materialize()
    with pytest.raises(wgf.WgfError):
        t.as_slice()


def launches(dev, build):
    before = dev.launch_count
    t = build()
    t.materialize()
    return dev.launch_count - before


def test_fusion_decisions(wgf, drydev):
    d = drydev
    x = d.tensor(np.zeros((64, 512), np.float32))
    w = d.tensor(np.zeros((512,), np.float32))
    y = d.tensor(np.zeros((64, 512), np.float32))
    # chains and DAGs of element-wise / pair-wise nodes: one kernel (src/compute_graph/resolve.rs:63-136)
    assert launches(d, lambda: (x + 1.0) * 2.0) == 1
    assert launches(d, lambda: (x + 1.0) + (y * 2.0)) == 1
    assert launches(d, lambda: ((x * 2.0 + 1.0).sin().cos() * 0.5) + (-(x * x)).exp()) == 1
    assert launches(d, lambda: (x + y) * (x - y) / (y + 3.0)) == 1         # pair-wise of pair-wise
    # reduce with prologue and epilogue (resolve.rs:164-196)
    assert launches(d, lambda: (x + 1.0).sum(1) + 1.0) == 1
    assert launches(d, lambda: (x + 1.0).sum(0) * 2.0) == 1
    # reduce -> broadcast -> pair-wise patterns: one row kernel
    assert launches(d, lambda: x.layer_norm(w, 1e-5)) == 1
    assert launches(d, lambda: x.softmax_last_dim()) == 1
    assert launches(d, lambda: x.layer_norm(w, 1e-5).softmax_last_dim()) == 1
    # same-op reduce chain over all axes folds into one full reduction
    assert launches(d, lambda: x.exp().sum(0).sum(0)) == 1
    assert launches(d, lambda: x.max(1).max(0)) == 1
    # different ops do not fold
    assert launches(d, lambda: x.max(1).sum(0)) == 2
    # matmul, resize, slice_assign never fuse (resolve.rs:138-154, 210-244)
    assert launches(d, lambda: (x.mat_mul(y.transpose(0, 1)) + 1.0)) == 2
    # views are free
    assert launches(d, lambda: x.transpose(0, 1).slice([(0, 100), (3, 60)]) + 1.0) == 1
    # a reshape of row-major data is a view; of a transposed view it is one gather
    assert launches(d, lambda: x.reshape((128, 256))) == 0
    assert launches(d, lambda: x.transpose(0, 1).reshape((128, 256))) == 1


def test_whole_tensor_reductions_ride_along_in_a_row_kernel(wgf, drydev):
    """materialize_all: reductions of a whole tensor to a scalar requested together with a row-fused
    tensor over the same index space cost no kernel of their own (the crate's README lists fusing
    parallel reduce ops as an open item, README.md:20)."""
    d = drydev
    x = d.tensor(np.zeros((64, 512), np.float32))
    w = d.tensor(np.zeros((512,), np.float32))
    z = d.tensor(np.zeros((32, 512), np.float32))

    def count(build):
        before = d.launch_count
        ts = build()
        wgf.Tensor.materialize_all(ts)
        again = d.launch_count
        wgf.Tensor.materialize_all(ts)            # everything is cached now
        assert d.launch_count == again
        return again - before

    assert count(lambda: [x.layer_norm(w, 1e-5).softmax_last_dim(), x.exp().sum(0).sum(0)]) == 1
    assert count(lambda: [x.sum(1).sum(0), x.softmax_last_dim(), x.max(0).max(0), (x * x).sum(0).sum(0)]) == 1
    assert count(lambda: [x.softmax_last_dim(), (x * w.broadcast((64, 512))).min(1).min(0)]) == 1
    # no row kernel to ride in, another index space, or not a scalar: separate kernels as before
    assert count(lambda: [x + 1.0, x.sum(0).sum(0)]) == 2
    assert count(lambda: [x.softmax_last_dim(), z.sum(0).sum(0)]) == 2
    assert count(lambda: [x.softmax_last_dim(), x.sum(0)]) == 2
    # a reduction the row kernel itself depends on is computed first, not alongside
    s = x.sum(0).sum(0)
    y = x.softmax_last_dim() * s.broadcast((512,)).broadcast((64, 512))
    assert count(lambda: [y, s]) == 2


def test_memoisation_and_graph_growth(wgf, drydev):
    d = drydev
    x = d.tensor(np.zeros((32, 32), np.float32))
    e = x.exp()
    e.materialize()
    before = d.launch_count
    (e + 1.0).materialize()
    (e * 2.0).materialize()
    assert d.launch_count - before == 2          # e is not recomputed (the crate would re-run it)
    # nodes die with their handles: the graph does not grow without bound
    n0 = x.graph_size()
    for _ in range(50):
        t = (x + 1.0).sum(0)
        t.materialize()
        del t
    assert x.graph_size() <= n0 + 2


def test_inplace_reuse_by_liveness(wgf, drydev):
    """A tensor nobody can read any more donates its buffer (src/element_wise.rs:98-99,
    src/pair_wise.rs:95-107); a held tensor never does (tests/inplace_clone.rs)."""
    d = drydev
    x = np.zeros((64, 64), np.float32)
    cur = d.tensor(x)
    base = d.memory()[0]
    for _ in range(4):
        nxt = cur + 1.0
        cur.release()                       # `cur + 1.0` consumed cur
        nxt.materialize()
        cur = nxt
    assert d.memory()[0] == base            # no second buffer was ever needed
    held = d.tensor(x)
    before = d.memory()[0]
    y = held * 2.0
    y.materialize()
    assert d.memory()[0] > before           # held input: the result got its own buffer
    # pair-wise: the dead operand donates, whichever side it is on
    a, b = d.tensor(x), d.tensor(x)
    before = d.memory()[0]
    z = b - a
    a.release()
    z.materialize()
    assert d.memory()[0] == before
    # a cast to a narrower type cannot reuse the buffer
    c = d.tensor(x)
    before = d.memory()[0]
    h = c.cast(wgf.F16)
    c.release()
    h.materialize()
    assert d.memory()[0] > before


def test_kernel_cache_reuses_by_signature(wgf, drydev):
    d = drydev
    x = d.tensor(np.zeros((16, 128), np.float32))
    (x * 3.0 + 7.0).materialize()
    c0 = d.compile_count
    (x * 5.0 + 9.0).materialize()                # other constants: same kernel (constants are parameters)
    y = d.tensor(np.zeros((32, 128), np.float32))
    (y * 5.0 + 9.0).materialize()                # other size: same kernel
    assert d.compile_count == c0
    (x * 5.0 - 9.0).materialize()                # other op: new kernel
    assert d.compile_count == c0 + 1


def test_shape_and_dtype_errors(wgf, drydev):
    d = drydev
    a = d.tensor(np.zeros((2, 3), np.float32))
    b = d.tensor(np.zeros((3, 2), np.float32))
    h = d.tensor(np.zeros((2, 3), np.float16))
    for f, status in [(lambda: a + b, "SHAPE"), (lambda: a + h, "DTYPE"), (lambda: a.mat_mul(a), "SHAPE"),
                      (lambda: a.sum(2), "INVALID_ARGUMENT"), (lambda: a.narrow(1, 2, 5), "SHAPE"),
                      (lambda: a.reshape((7,)), "SHAPE"), (lambda: a.resize((1, 3)), "SHAPE"),
                      (lambda: a.broadcast((2, 3)), "RANK"), (lambda: a.slice([(0, 3), (0, 3)]), "SHAPE"),
                      (lambda: a.unary(wgf.OP_ADD), "INVALID_ARGUMENT"), (lambda: a.softmax(), "RANK"),
                      (lambda: wgf.Tensor.cat([a, b], 0), "SHAPE")]:
        with pytest.raises(wgf.WgfError) as e:
            f()
        assert e.value.status == status, (e.value, status)


def test_views_shapes(wgf, drydev):
    d = drydev
    a = d.tensor(np.zeros((2, 3, 4), np.float32))
    assert a.transpose(0, 2).shape == (4, 3, 2)
    assert a.slice([(0, 1), (1, 3), (0, 4)]).shape == (1, 2, 4)
    assert a.sum(1).shape == (2, 4)
    assert a.sum(0).sum(0).sum(0).shape == ()
    assert a.unsqueeze(1).shape == (2, 1, 3, 4)
    assert a.resize((3, 3, 5)).shape == (3, 3, 5)
    assert wgf.Tensor.cat([a, a], 2).shape == (2, 3, 8)
    # broadcast puts the new axis where the common prefix of the shapes ends (src/map_layout.rs:73-77)
    m = d.tensor(np.zeros((2, 2), np.float32))
    assert m.broadcast((2, 2, 3)).shape == (2, 2, 3)
    v = d.tensor(np.zeros((4,), np.float32))
    assert v.broadcast((5, 4)).shape == (5, 4)
    assert v.broadcast_axis(1, 7).shape == (4, 7)
    assert d.arange(0.0, 10.0, 2.0).shape == (5,)
    assert d.arange(5.0, 0.0, -1.0).shape == (5,)
    assert "digraph" in (a + 1.0).graphvis()


def test_shard_range(wgf):
    for n in (0, 1, 7, 8, 8192, 8193):
        for world in (1, 2, 3, 8):
            covered = []
            for r in range(world):
                b, e = wgf.shard_range(n, world, r)
                assert 0 <= b <= e <= n
                covered += list(range(b, e))
                assert (e - b) in (n // world, n // world + 1)
            assert covered == list(range(n))


def test_generated_kernels_compile_for_every_layout_class(wgf, drydev):
    """Vector / scalar / broadcast / strided operand modes, ranks 1-4, 16-bit types, long rows."""
    d = drydev
    rng = np.random.default_rng(0)
    for shape in [(7,), (1000,), (3, 5), (8, 256), (5, 7, 9), (4, 8, 16), (2, 3, 4, 5)]:
        x = d.tensor(rng.standard_normal(shape).astype(np.float32))
        ((x * 2.0).tanh() + x).materialize()
        for ax in range(len(shape)):
            (x.exp().sum(ax) + 1.0).materialize()
            x.max(ax).materialize()
        if len(shape) >= 2:
            (x.transpose(0, len(shape) - 1) * 2.0).materialize()
            x.softmax_last_dim().materialize()
        h = x.cast(wgf.F16)
        (h * 2.0 + h).sum(len(shape) - 1).materialize()
        (x.cast(wgf.BF16).cast(wgf.F32) + 1.0).materialize()
    big = d.tensor(np.zeros((2, 20000), np.float32))
    big.softmax_last_dim().materialize()
    d.tensor(np.zeros((3, 100000), np.float32)).sum(1).materialize()


def test_recorded_schedule_state_machine(wgf, drydev):
    """wgf_schedule_*: what a recording refuses, what it counts, where its memory goes."""
    d = drydev
    x = d.tensor(np.zeros((64, 512), np.float32))
    w = d.tensor(np.zeros((512,), np.float32))
    d.memory()
    with pytest.raises(wgf.WgfError):                      # nothing to end
        h = C.c_void_p()
        wgf.check(wgf.lib().wgf_schedule_end(d.h, C.byref(h)))
    in_use_before = d.memory()[1]
    before = d.launch_count
    with d.record() as s:
        with pytest.raises(wgf.WgfError):                  # one recording at a time
            wgf.check(wgf.lib().wgf_schedule_begin(d.h))
        y = x.layer_norm(w, 1e-5).softmax_last_dim()
        t = x.exp().sum(0).sum(0)
        wgf.Tensor.materialize_all([y, t])
        z = (y * 2.0 + 1.0).materialize()
        for refused in (z.as_slice, d.sync, lambda: d.tensor(np.zeros(4, np.float32)),
                        lambda: x.write(np.zeros((64, 512), np.float32))):
            with pytest.raises(wgf.WgfError) as e:
                refused()
            assert e.value.status == "UNSUPPORTED"
    assert s.kernel_count == d.launch_count - before == 2
    s.launch()
    s.launch()
    assert d.launch_count - before == 6
    # the recording's memory stays with the schedule, also once its tensors are gone ...
    y.release(), t.release(), z.release()
    held = d.memory()[1]
    assert held > in_use_before
    other = (x + 1.0).materialize()                        # must not get one of the schedule's blocks
    assert d.memory()[1] > held
    other.release()
    # ... and returns to the pool with the schedule
    s.destroy()
    assert d.memory()[1] == in_use_before


def test_recording_never_overwrites_its_inputs(wgf, drydev):
    """Outside a recording a dead input donates its buffer; inside, an input of the schedule is
    read again by every replay, so the result gets its own buffer."""
    d = drydev
    data = np.zeros((64, 64), np.float32)

    def result_ptr_equals_input_ptr(record):
        x = d.tensor(data)
        px = C.c_void_p()
        dx = x.desc()
        wgf.check(wgf.lib().wgf_buffer_device_ptr(C.c_void_p(dx.buf), C.byref(px), None))
        wgf.lib().wgf_buffer_release(C.c_void_p(dx.buf))
        y = x + 1.0
        x.release()
        if record:
            with d.record() as s:
                y.materialize()
        else:
            y.materialize()
        py = C.c_void_p()
        dy = y.desc()
        wgf.check(wgf.lib().wgf_buffer_device_ptr(C.c_void_p(dy.buf), C.byref(py), None))
        wgf.lib().wgf_buffer_release(C.c_void_p(dy.buf))
        return px.value == py.value

    assert result_ptr_equals_input_ptr(False)
    assert not result_ptr_equals_input_ptr(True)


def test_exp_form_follows_who_can_see_the_value(tmp_path):
    """Generated source: an f32 exp seen only by sums uses the two-instruction form, the exp of a
    softmax (it also reaches the output) and a plain exp keep expf, a 16-bit exp uses the short form."""
    import subprocess
    import sys
    script = tmp_path / "dump.py"
    script.write_text(
        "import sys, numpy as np\n"
        f"sys.path.insert(0, {os.path.join(ROOT, 'tests')!r})\n"
        "from conftest import load_package\n"
        "wgf = load_package(); d = wgf.Device(-1)\n"
        "x = d.tensor(np.zeros((64, 512), np.float32)); h = d.tensor(np.zeros((64, 512), np.float16))\n"
        "for name, t in (('SUMEXP', lambda: x.exp().sum(0).sum(0)), ('ROWSUMEXP', lambda: (x * 0.5).exp().sum(1)),\n"
        "                ('SOFTMAX', lambda: x.softmax_last_dim()), ('PLAIN', lambda: x.exp() * 2.0),\n"
        "                ('HALF', lambda: h.exp() * 2.0)):\n"
        "    print('@@', name, file=sys.stderr, flush=True); t().materialize()\n")
    env = dict(os.environ, WGF_KERNEL_CACHE=str(tmp_path / "cache"), WGF_JIT_VERBOSE="1", WGF_DUMP_SOURCE="1")
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    parts = {}
    for chunk in r.stderr.split("@@ ")[1:]:
        name, _, text = chunk.partition("\n")
        body = text.split('extern "C" __global__')[-1] if 'extern "C" __global__' in text else text
        calls = [c for c in ("op_exp_sfu(v", "op_exp(v", "op_exp_sfu(x", "op_exp(x") if c in text.replace("DEV float op_exp", "")]
        assert calls, f"no kernel source was generated for {name.strip()}"
        parts[name.strip()] = (body, calls)
    uses = {k: ("sfu" if any("sfu" in c for c in v[1]) else "expf") for k, v in parts.items()}
    assert uses == {"SUMEXP": "sfu", "ROWSUMEXP": "sfu", "SOFTMAX": "expf", "PLAIN": "expf", "HALF": "sfu"}, uses


def test_llama_block_kernel_count_with_and_without_matmul_epilogues(wgf, drydev, monkeypatch):
    """On the compile-only device: the decoder block resolves to 11 kernels -- RmsNorm, three
    projections, two rope kernels, fused attention, the output projection with the residual add in
    its epilogue, RmsNorm, one GEMM for silu(gate) * up, the down projection with the second residual
    add -- and to 14 when the epilogues are switched off."""
    B, S, Hd, heads, inter = 1, 256, 512, 4, 1024
    D = Hd // heads
    z = lambda *shape: np.zeros(shape, np.float16)

    def launches():
        x = drydev.tensor(z(B, S, Hd))
        W = [drydev.tensor(z(*s)) for s in [(Hd, Hd)] * 4 + [(inter, Hd), (inter, Hd), (Hd, inter)]]
        n1, n2 = drydev.tensor(z(Hd)), drydev.tensor(z(Hd))
        cos, sin = drydev.tensor(z(S, D // 2)), drydev.tensor(z(S, D // 2))
        before = drydev.launch_count
        x.llama_block(W, n1, n2, cos, sin, None, heads, 1e-5).materialize()
        return drydev.launch_count - before

    monkeypatch.delenv("WGF_NO_MATMUL_EPILOGUE", raising=False)
    assert launches() == 11
    monkeypatch.setenv("WGF_NO_MATMUL_EPILOGUE", "1")
    assert launches() == 14


def test_null_chain_with_a_length_is_an_error_not_a_crash(wgf, drydev):
    """Kernel-level launches take their op chains as (pointer, count): a NULL pointer with a non-zero
    count is refused with a status code by every one of them."""
    import ctypes as C
    x = drydev.tensor(np.zeros((4, 8), np.float32))
    d, out = x.desc(), wgf.TensorDesc()
    lib = wgf.lib()
    rc = lib.wgf_launch_elementwise(drydev.h, C.byref(d), None, C.c_uint32(2), C.c_int32(0), C.byref(out), None)
    assert wgf.STATUS[rc] == "INVALID_ARGUMENT"
    rc = lib.wgf_launch_pairwise(drydev.h, C.byref(d), C.byref(d), None, C.c_uint32(1), None, C.c_uint32(0), C.c_uint32(wgf.OP_ADD),
                                 None, C.c_uint32(0), C.byref(out), None)
    assert wgf.STATUS[rc] == "INVALID_ARGUMENT"
    rc = lib.wgf_launch_reduce(drydev.h, C.byref(d), C.c_uint32(1), None, C.c_uint32(0), C.c_uint32(wgf.OP_SUM), None, C.c_uint32(3),
                               C.byref(out), None)
    assert wgf.STATUS[rc] == "INVALID_ARGUMENT"
    lib.wgf_buffer_release(C.c_void_p(d.buf))


def test_all_reduce_over_peer_memory_costs_one_launch_per_step(wgf, drydev):
    """Host side of the scalar all-reduce over peer memory, on the compile-only device (its
    communicator needs no NCCL and compiles the same kernels).  The kernel of a step stores this
    rank's values, posts the values of the step before and settles the step six before: one launch
    per step, however many values ride along.  Results that are read before those later kernels
    have been queued are finished by one small kernel, once for all open exchanges; a
    synchronisation does the same."""
    d = drydev
    comm = wgf.Comm(d, 2, 0, bytes(128))
    x = d.tensor(np.zeros((64, 256), np.float32))

    def step():
        y = x.softmax_last_dim()
        s = x.exp().sum(0).sum(0).all_reduce(comm)
        m = x.max(0).max(0).all_reduce(comm, wgf.OP_MAX)
        before = d.launch_count
        wgf.Tensor.materialize_all([y, s, m])
        return d.launch_count - before, s, m

    def launches_of(fn):
        before = d.launch_count
        fn()
        return d.launch_count - before

    steps = [step() for _ in range(8)]
    assert [n for n, _, _ in steps] == [1] * 8
    s = [None] + [t[1] for t in steps]
    m = [None] + [t[2] for t in steps]
    assert launches_of(lambda: (s[1] * 2.0).materialize()) == 1   # settled by the kernel of step 7: a plain read
    assert launches_of(lambda: (m[2] * 2.0).materialize()) == 1   # settled by the kernel of step 8
    assert launches_of(lambda: (s[3] * 2.0).materialize()) == 2   # posted, not settled: one kernel finishes 3 .. 8
    assert launches_of(lambda: (m[8] * 2.0).materialize()) == 1   # ... so these are plain reads
    assert launches_of(lambda: (m[5] * 2.0).materialize()) == 1
    # the streaming reduction is a kernel of the same path
    alone = (x * 2.0).exp().sum(0).sum(0).all_reduce(comm)
    assert launches_of(alone.materialize) == 1
    assert launches_of(d.sync) == 1                             # a synchronisation leaves nothing open ...
    assert launches_of(d.sync) == 0                             # ... once
    assert launches_of(lambda: (alone * 2.0).materialize()) == 1
    del comm


def test_sine_and_cosine_of_bounded_values_skip_the_range_reduction(tmp_path):
    """Generated source: a sine or cosine whose argument is itself a sine, cosine or tanh (also
    through neg / abs / sqr / products of such values) uses the polynomial for [-1, 1]; any other
    argument keeps the full-range function."""
    import subprocess
    import sys
    script = tmp_path / "dump.py"
    script.write_text(
        "import sys, numpy as np\n"
        f"sys.path.insert(0, {os.path.join(ROOT, 'tests')!r})\n"
        "from conftest import load_package\n"
        "wgf = load_package(); d = wgf.Device(-1)\n"
        "x = d.tensor(np.zeros((64, 512), np.float32))\n"
        "for name, t in (('CHAIN', lambda: (x * 2.0 + 1.0).sin().cos() * 0.5 + (-(x * x)).exp()),\n"
        "                ('TANH', lambda: (-x.tanh()).sin()), ('PRODUCT', lambda: (x.sin() * x.cos()).cos()),\n"
        "                ('SCALED', lambda: (x.sin() * 2.0).cos()), ('PLAIN', lambda: x.cos())):\n"
        "    print('@@', name, file=sys.stderr, flush=True); t().materialize()\n")
    env = dict(os.environ, WGF_KERNEL_CACHE=str(tmp_path / "cache"), WGF_JIT_VERBOSE="1", WGF_DUMP_SOURCE="1")
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    uses = {}
    for chunk in r.stderr.split("@@ ")[1:]:
        name, _, text = chunk.partition("\n")
        body = text.split("DEV float prog(")[-1] if "DEV float prog(" in text else text.split("op_tan(float x)")[-1]
        uses[name.strip()] = sorted(c for c in ("op_sin_unit(", "op_cos_unit(", "op_sin(", "op_cos(") if c in body)
    assert uses["CHAIN"] == ["op_cos_unit(", "op_sin("], uses
    assert uses["TANH"] == ["op_sin_unit("], uses
    assert uses["PRODUCT"] == ["op_cos(", "op_cos_unit(", "op_sin("], uses
    assert uses["SCALED"] == ["op_cos(", "op_sin("], uses          # 2 sin(x) leaves [-1, 1]
    assert uses["PLAIN"] == ["op_cos("], uses


def test_library_runs_with_nvtx_ranges_on(tmp_path):
    """WGF_NVTX=1 wraps every materialisation and launch in an NVTX range; without a profiler attached
    the calls are no-ops, and the library must behave exactly as without them."""
    import subprocess
    import sys
    script = tmp_path / "nvtx.py"
    script.write_text(
        "import sys, numpy as np\n"
        f"sys.path.insert(0, {os.path.join(ROOT, 'tests')!r})\n"
        "from conftest import load_package\n"
        "wgf = load_package(); d = wgf.Device(-1)\n"
        "x = d.tensor(np.zeros((64, 512), np.float32))\n"
        "before = d.launch_count\n"
        "wgf.Tensor.materialize_all([x.softmax_last_dim(), x.exp().sum(0).sum(0)])\n"
        "(x * 2.0).materialize()\n"
        "print('LAUNCHES', d.launch_count - before)\n")
    env = dict(os.environ, WGF_NVTX="1", WGF_KERNEL_CACHE=str(tmp_path / "cache"))
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "LAUNCHES 2" in r.stdout


def test_f32_matmul_dispatch_between_the_two_ffma_kernels(tmp_path):
    """Which f32 products take the 128x256-tile kernel: B stored [K,N], M and N at least 512, K at least
    256 and enough tiles to fill the machine twice; everything else (a transposed view of B, small or
    few-tile problems) keeps the 128x128 kernel.  Read from the launch trace on the compile-only device."""
    import subprocess
    import sys
    script = tmp_path / "dispatch.py"
    script.write_text(
        "import sys, numpy as np\n"
        f"sys.path.insert(0, {os.path.join(ROOT, 'tests')!r})\n"
        "from conftest import load_package\n"
        "wgf = load_package(); d = wgf.Device(-1)\n"
        "z = lambda *s: d.tensor(np.zeros(s, np.float32))\n"
        "cases = {'BIG': (z(2048, 512), z(512, 4864)), 'FEWTILES': (z(1024, 512), z(512, 1024)),\n"
        "         'SHORTK': (z(2048, 128), z(128, 4864)), 'SMALL': (z(100, 100), z(100, 100)),\n"
        "         'BATCH': (z(2, 2048, 512), z(2, 512, 2560))}\n"
        "for name, (a, b) in cases.items():\n"
        "    print('@@', name, file=sys.stderr, flush=True); a.mat_mul(b).materialize()\n"
        "a, bt = z(2048, 512), z(4864, 512)\n"
        "print('@@ TRANSPOSED', file=sys.stderr, flush=True); a.mat_mul(bt.transpose(0, 1)).materialize()\n")
    env = dict(os.environ, WGF_TRACE_LAUNCHES="1", WGF_KERNEL_CACHE=str(tmp_path / "cache"))
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    seen = {}
    for chunk in r.stderr.split("@@ ")[1:]:
        name, _, text = chunk.partition("\n")
        seen[name.strip()] = [line.split("launch ", 1)[1].strip() for line in text.splitlines() if "[wgf] launch " in line]
    assert seen["BIG"] == ["sgemm_wide"], seen              # 16 x 19 = 304 tiles
    assert seen["BATCH"] == ["sgemm_wide"], seen            # 2 x 16 x 10 = 320 tiles
    assert seen["FEWTILES"] == ["sgemm"], seen              # 8 x 4 tiles: less than two per SM
    assert seen["SHORTK"] == ["sgemm"], seen
    assert seen["SMALL"] == ["sgemm"], seen
    assert seen["TRANSPOSED"] == ["sgemm"], seen            # B as an [N,K] view: the 128x128 kernel reads it in place
