"""Frozen fixtures (tests/golden/golden_v1.npz, made by tests/golden/make_golden.py).  On the CPU the
oracle must reproduce them bit for bit, and the seeded input generators must still give the frozen
inputs; on the GPU the CUDA path is compared with the frozen outputs under the tolerance each case
names: exact for moves / casts / index ops / + - * /, 2 ulp for one f32 transcendental op (4 for a
chain of several), 1 ulp for f16, 1e-5 relative for reductions, 1e-4 (f32) and 1e-2 (f16) norm-wise for matmul."""
import os
import sys
import types

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

import cases  # noqa: E402

GOLDEN = os.path.join(HERE, "golden", "golden_v1.npz")


@pytest.fixture(scope="module")
def golden():
    return dict(np.load(GOLDEN))


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view({2: np.uint16, 4: np.uint32}[a.dtype.itemsize])


def test_fixture_file_covers_every_case(golden):
    for name in cases.CASES:
        assert f"{name}/out" in golden, name
    assert len([k for k in golden if k.endswith("/out")]) == len(cases.CASES)


def test_seeded_inputs_are_stable(golden):
    for name, inputs in cases.all_inputs().items():
        for k, v in inputs.items():
            np.testing.assert_array_equal(bits(v), bits(golden[f"{name}/in/{k}"]), err_msg=f"{name}/{k}")


@pytest.mark.parametrize("name", list(cases.CASES))
def test_oracle_reproduces_golden(name, golden, orc):
    ns = types.SimpleNamespace(F32=orc.F32, F16=orc.F16, BF16=orc.BF16, cat=orc.Ref.cat)
    _, build, _ = cases.CASES[name]
    t = {k[len(name) + 4:]: orc.Ref(v) for k, v in golden.items() if k.startswith(name + "/in/")}
    got = build(t, ns).numpy()
    want = golden[f"{name}/out"]
    assert got.shape == want.shape and got.dtype == want.dtype
    np.testing.assert_array_equal(bits(got), bits(want))


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(cases.CASES))
def test_cuda_matches_golden(name, golden, wgf, dev, orc):
    ns = types.SimpleNamespace(F32=wgf.F32, F16=wgf.F16, BF16=wgf.BF16, cat=wgf.Tensor.cat)
    _, build, check = cases.CASES[name]
    t = {k[len(name) + 4:]: dev.tensor(v) for k, v in golden.items() if k.startswith(name + "/in/")}
    got = build(t, ns).as_slice()
    want = golden[f"{name}/out"]
    assert got.shape == want.shape and got.dtype == want.dtype
    if check == "exact":
        np.testing.assert_array_equal(bits(got), bits(want))
    elif check[0] == "ulp":
        diff = orc.ulp_diff_f16 if got.dtype == np.float16 else orc.ulp_diff_f32
        assert int(diff(got, want).max()) <= check[1]
    elif check[0] == "rel":
        g, w = got.astype(np.float64), want.astype(np.float64)
        assert (np.abs(g - w) / np.maximum(np.abs(w), 1e-30)).max() <= check[1]
    else:
        g, w = got.astype(np.float64), want.astype(np.float64)
        assert np.abs(g - w).max() / np.abs(w).max() <= check[1]
