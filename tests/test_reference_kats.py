"""Known answers taken from the crate's own tests, checked against BOTH the CPU oracle (always)
and the CUDA path (gpu mark).  Each case cites the test it restates.  The crate asserts exact
equality for + - * /, moves and reductions of small integers, and |err| < 1e-3 for
transcendentals; the same bounds are used here."""
import math

import numpy as np
import pytest

D23 = [[1., 2.], [3., 4.], [5., 6.]]
D322 = [[[1., 2.], [1., 2.]], [[3., 4.], [3., 4.]], [[5., 6.], [5., 6.]]]


def f32(v):
    return np.array(v, dtype=np.float32)


def fmap(fn, data=D23):
    return f32([[fn(np.float32(v)) for v in row] for row in data])


# (name, citation, build(mk, T) -> tensor, expected array, abs tolerance)
# mk(array) makes a tensor of the backend; T is the backend's tensor class (for cat).
CASES = [
    ("add_const_r3", "src/element_wise.rs:214-237", lambda mk, T: mk(f32(D322)) + 1.0, f32(D322) + 1, 0),
    ("add_const_r2", "src/element_wise.rs:239-251", lambda mk, T: mk(f32(D23)) + 1.0, f32(D23) + 1, 0),
    ("add_const_r1", "src/element_wise.rs:253-262", lambda mk, T: mk(f32([1., 2.])) + 1.0, f32([2., 3.]), 0),
    ("add_const_reversed", "src/element_wise.rs:275-324", lambda mk, T: 1.0 + mk(f32(D322)), f32(D322) + 1, 0),
    ("add_const_sliced", "src/element_wise.rs:377-396", lambda mk, T: mk(f32(D23)).slice([(0, 3), (0, 1)]) + 1.0,
     f32([[2.], [4.], [6.]]), 0),
    ("add_const_large", "src/element_wise.rs:400-418", lambda mk, T: mk(np.full((1024 * 64,), 10., np.float32)) + 1.0,
     np.full((1024 * 64,), 11., np.float32), 0),
    ("merge_add_const", "src/element_wise.rs:422-443", lambda mk, T: (mk(f32(D23)) + 1.0) + 1.0, f32(D23) + 2, 0),
    ("sub_const", "src/element_wise.rs:462-481", lambda mk, T: mk(f32(D23)) - 1.0, f32(D23) - 1, 0),
    ("sub_const_reversed", "src/element_wise.rs:502-521", lambda mk, T: 1.0 - mk(f32(D23)), 1 - f32(D23), 0),
    ("mul_const", "src/element_wise.rs:542-561", lambda mk, T: mk(f32(D23)) * 2.0, f32(D23) * 2, 0),
    ("mul_const_reversed", "src/element_wise.rs:575-594", lambda mk, T: 2.0 * mk(f32(D23)), f32(D23) * 2, 0),
    ("div_const", "src/element_wise.rs:615-634", lambda mk, T: mk(f32(D23)) / 2.0, f32(D23) / 2, 0),
    ("div_const_reversed", "src/element_wise.rs:655-674", lambda mk, T: 2.0 / mk(f32(D23)), np.float32(2) / f32(D23), 0),
    ("exp", "src/element_wise.rs:690-710", lambda mk, T: mk(f32(D23)).exp(), fmap(math.exp), 1e-3),
    ("exp2", "src/element_wise.rs:725-745", lambda mk, T: mk(f32(D23)).exp2(), fmap(lambda v: 2.0 ** v), 1e-3),
    ("log", "src/element_wise.rs:760-780", lambda mk, T: mk(f32(D23)).log(), fmap(math.log), 1e-3),
    ("log2", "src/element_wise.rs:795-815", lambda mk, T: mk(f32(D23)).log2(), fmap(math.log2), 1e-3),
    ("sqr", "src/element_wise.rs:833-856", lambda mk, T: mk(f32(D23)).sqr(), f32(D23) ** 2, 0),
    ("sqrt", "src/element_wise.rs:871-891", lambda mk, T: mk(f32(D23)).sqrt(), fmap(math.sqrt), 1e-3),
    ("sin", "src/element_wise.rs:906-926", lambda mk, T: mk(f32(D23)).sin(), fmap(math.sin), 1e-3),
    ("cos", "src/element_wise.rs:941-961", lambda mk, T: mk(f32(D23)).cos(), fmap(math.cos), 1e-3),
    ("tan", "src/element_wise.rs:976-996", lambda mk, T: mk(f32(D23)).tan(), fmap(math.tan), 1e-3),
    ("atan", "src/element_wise.rs:1089-1109", lambda mk, T: mk(f32(D23)).atan(), fmap(math.atan), 1e-3),
    ("sinh", "src/element_wise.rs:1124-1144", lambda mk, T: mk(f32(D23)).sinh(), fmap(math.sinh), 1e-3),
    ("cosh", "src/element_wise.rs:1159-1179", lambda mk, T: mk(f32(D23)).cosh(), fmap(math.cosh), 1e-3),
    ("tanh", "src/element_wise.rs:1194-1214", lambda mk, T: mk(f32(D23)).tanh(), fmap(math.tanh), 1e-3),
    ("asinh", "src/element_wise.rs:1229-1253", lambda mk, T: mk(f32(D23)).asinh(), fmap(math.asinh), 1e-3),
    ("acosh", "src/element_wise.rs:1268-1292", lambda mk, T: mk(f32(D23)).acosh(), fmap(math.acosh), 1e-3),
    ("abs", "src/element_wise.rs:1346-1366", lambda mk, T: mk(f32([[1., -2.], [-3., 4.], [5., -6.]])).abs(), f32(D23), 0),
    ("neg", "src/element_wise.rs:1384-1404", lambda mk, T: -mk(f32([[1., -2.], [-3., 4.], [5., -6.]])),
     f32([[-1., 2.], [3., -4.], [-5., 6.]]), 0),
    ("pair_add", "src/pair_wise.rs:226-251", lambda mk, T: mk(f32(D23)) + mk(f32(D23)), f32(D23) * 2, 0),
    ("pair_add_const_mul_const_fused", "src/pair_wise.rs:292-317",
     lambda mk, T: (mk(f32(D23)) + 1.0) + (mk(f32(D23)) * 2.0), (f32(D23) + 1) + f32(D23) * 2, 0),
    ("pair_add_sub_const_fused", "src/pair_wise.rs:321-346", lambda mk, T: (mk(f32(D23)) + mk(f32(D23))) - 1.0,
     f32(D23) * 2 - 1, 0),
    ("pair_add_sparse", "src/pair_wise.rs:350-374",
     lambda mk, T: mk(f32(D23)).slice([(0, 3), (0, 1)]) + mk(f32(D23)).slice([(0, 3), (0, 1)]), f32([[2.], [6.], [10.]]), 0),
    ("pair_sub", "src/pair_wise.rs:397-422", lambda mk, T: mk(f32(D23)) - mk(f32(D23)), f32(D23) * 0, 0),
    ("pair_mul", "src/pair_wise.rs:445-470", lambda mk, T: mk(f32(D23)) * mk(f32(D23)), f32(D23) ** 2, 0),
    ("pair_div", "src/pair_wise.rs:493-518", lambda mk, T: mk(f32(D23)) / mk(f32(D23)), f32(D23) / f32(D23), 0),
    ("pair_pow", "src/pair_wise.rs:532-557", lambda mk, T: mk(f32(D23)).pow(mk(f32(D23))), fmap(lambda v: v ** v), 1e-3),
    ("reduce_sum_0", "src/reduce.rs:473-500", lambda mk, T: mk(f32(D23)).sum(0), f32([9., 12.]), 0),
    ("reduce_sum_1", "src/reduce.rs:473-500", lambda mk, T: mk(f32(D23)).sum(1), f32([3., 7., 11.]), 0),
    ("reduce_sliced_sum_0", "src/reduce.rs:539-566", lambda mk, T: mk(f32(D23)).slice([(0, 3), (0, 1)]).sum(0), f32([9.]), 0),
    ("reduce_sliced_sum_1", "src/reduce.rs:539-566", lambda mk, T: mk(f32(D23)).slice([(0, 3), (0, 1)]).sum(1), f32([1., 3., 5.]), 0),
    ("reduce_add_then_sum_0", "src/reduce.rs:570-599", lambda mk, T: (mk(f32(D23)) + 1.0).sum(0), f32([12., 15.]), 0),
    ("reduce_add_then_sum_1", "src/reduce.rs:570-599", lambda mk, T: (mk(f32(D23)) + 1.0).sum(1), f32([5., 9., 13.]), 0),
    ("reduce_sum_then_add_0", "src/reduce.rs:604-631", lambda mk, T: mk(f32(D23)).sum(0) + 1.0, f32([10., 13.]), 0),
    ("reduce_sum_then_add_1", "src/reduce.rs:604-631", lambda mk, T: mk(f32(D23)).sum(1) + 1.0, f32([4., 8., 12.]), 0),
    ("reduce_max_0", "src/reduce.rs:677-704", lambda mk, T: mk(f32(D23)).max(0), f32([5., 6.]), 0),
    ("reduce_max_1", "src/reduce.rs:677-704", lambda mk, T: mk(f32(D23)).max(1), f32([2., 4., 6.]), 0),
    ("reduce_min_0", "src/reduce.rs:750-777", lambda mk, T: mk(f32(D23)).min(0), f32([1., 2.]), 0),
    ("reduce_min_1", "src/reduce.rs:750-777", lambda mk, T: mk(f32(D23)).min(1), f32([1., 3., 5.]), 0),
    ("reduce_product_0", "src/reduce.rs:819-846", lambda mk, T: mk(f32(D23)).product(0), f32([15., 48.]), 0),
    ("reduce_product_1", "src/reduce.rs:819-846", lambda mk, T: mk(f32(D23)).product(1), f32([2., 12., 30.]), 0),
    ("transpose", "src/map_layout.rs:103-124", lambda mk, T: mk(f32(D23)).transpose(0, 1), f32(D23).T, 0),
    ("broadcast", "src/map_layout.rs:128-149", lambda mk, T: mk(f32([[1., 2.], [3., 4.]])).broadcast((2, 2, 3)),
     np.repeat(f32([[1., 2.], [3., 4.]])[:, :, None], 3, axis=2), 0),
    ("matmul", "src/matmul.rs:219-239", lambda mk, T: mk(f32([[1.], [3.]])).mat_mul(mk(f32([[1., 2.]]))),
     f32([[1., 2.], [3., 6.]]), 0),
    ("resize", "src/resize.rs:149-170", lambda mk, T: mk(f32(D23)).resize((30, 20)),
     np.pad(f32(D23), ((0, 27), (0, 18))), 0),
    ("reshape_23", "src/resize.rs:174-190", lambda mk, T: mk(f32(D23)).reshape((2, 3)), f32(D23).reshape(2, 3), 0),
    ("reshape_6", "src/resize.rs:192-207", lambda mk, T: mk(f32(D23)).reshape((6,)), f32(D23).reshape(6), 0),
    ("slice_assign", "src/slice_assign.rs:84-105",
     lambda mk, T: mk(f32(D23)).slice_assign([(0, 2), (0, 2)], mk(f32([[10., 20.], [30., 40.]]))),
     f32([[10., 20.], [30., 40.], [5., 6.]]), 0),
    ("cat", "src/composite/cat.rs:45-78",
     lambda mk, T: T.cat([mk(f32([[1., -2.], [-3., 4.], [5., -6.]])), mk(f32(D23))], 1),
     f32([[1., -2., 1., 2.], [-3., 4., 3., 4.], [5., -6., 5., 6.]]), 0),
    ("narrow", "src/composite/narrow.rs:20-38", lambda mk, T: mk(f32(D23)).narrow(0, 1, 2), f32([[3., 4.], [5., 6.]]), 0),
    ("unsqueeze", "src/composite/unsqueeze.rs:57-77", lambda mk, T: mk(f32(D23)).unsqueeze(0), f32(D23)[None], 0),
    ("layer_norm", "src/composite/rms_norm.rs:20-40", lambda mk, T: mk(f32(D23)).layer_norm(mk(f32([2., 3.])), 1e-5),
     f32([[1.2649086, 3.7947257], [1.6970556, 3.3941112], [1.8107147, 3.2592864]]), 1e-3),
    ("silu", "src/composite/silu.rs:12-37", lambda mk, T: mk(f32([[1., -2.], [-3., 4.], [5., -6.]])).silu(),
     fmap(lambda v: v / (1 + math.exp(-v)), [[1., -2.], [-3., 4.], [5., -6.]]), 1e-3),
    ("softmax", "src/composite/softmax.rs:15-44", lambda mk, T: mk(f32([1., -2., -3., 4., 5., -6.])).softmax(),
     (np.exp(np.float64([1., -2., -3., 4., 5., -6.])) / np.exp(np.float64([1., -2., -3., 4., 5., -6.])).sum()).astype(np.float32),
     1e-3),
]
# unary functions whose test inputs differ from [[1,2],[3,4],[5,6]]
CASES += [
    ("asin", "src/element_wise.rs:1011-1035", lambda mk, T: mk(f32(np.sin(f32(D23)))).asin(),
     np.arcsin(np.sin(np.float64(D23))).astype(np.float32), 1e-3),
    ("acos", "src/element_wise.rs:1050-1074", lambda mk, T: mk(f32(np.cos(f32(D23)))).acos(),
     np.arccos(np.float64(np.cos(f32(D23)))).astype(np.float32), 1e-3),
    ("atanh", "src/element_wise.rs:1307-1331", lambda mk, T: mk(f32(np.tanh(f32(D23) / 4))).atanh(),
     np.arctanh(np.float64(f32(np.tanh(f32(D23) / 4)))).astype(np.float32), 1e-3),
]
IDS = [c[0] for c in CASES]


def check(got, want, tol):
    got = np.asarray(got, dtype=np.float32)
    assert got.shape == want.shape
    if tol == 0:
        np.testing.assert_array_equal(got, want)
    else:
        assert np.max(np.abs(got.astype(np.float64) - want.astype(np.float64))) < tol


@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_oracle_matches_reference_kat(case, orc):
    _, _, build, want, tol = case
    check(build(lambda a: orc.Ref(a), orc.Ref).numpy(), want, tol)


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=IDS)
def test_cuda_matches_reference_kat(case, wgf, dev):
    _, _, build, want, tol = case
    check(build(lambda a: dev.tensor(a), wgf.Tensor).as_slice(), want, tol)


# ---- f16 known answers -------------------------------------------------------------------
F16_CASES = [
    ("add_const_f16", "src/element_wise.rs:328-373", lambda mk, T: mk(np.array(D23, np.float16)) + 1.0,
     np.array(D23, np.float16) + np.float16(1)),
    ("pair_add_f16", "src/pair_wise.rs:255-288", lambda mk, T: mk(np.array(D23, np.float16)) + mk(np.array(D23, np.float16)),
     np.array(D23, np.float16) * np.float16(2)),
    ("reduce_sum_f16", "src/reduce.rs:504-535", lambda mk, T: mk(np.array(D23, np.float16)).sum(0), np.array([9., 12.], np.float16)),
    ("matmul_f16", "src/matmul.rs:243-264",
     lambda mk, T: mk(np.array([[1.], [3.]], np.float16)).mat_mul(mk(np.array([[1., 2.]], np.float16))),
     np.array([[1., 2.], [3., 6.]], np.float16)),
]


@pytest.mark.parametrize("case", F16_CASES, ids=[c[0] for c in F16_CASES])
def test_oracle_f16_kat(case, orc):
    _, _, build, want = case
    got = build(lambda a: orc.Ref(a), orc.Ref).numpy()
    assert got.dtype == np.float16
    np.testing.assert_array_equal(got, want)


@pytest.mark.gpu
@pytest.mark.parametrize("case", F16_CASES, ids=[c[0] for c in F16_CASES])
def test_cuda_f16_kat(case, wgf, dev):
    _, _, build, want = case
    got = build(lambda a: dev.tensor(a), wgf.Tensor).as_slice()
    assert got.dtype == np.float16
    np.testing.assert_array_equal(got, want)


# ---- casts: src/element_wise.rs:1440-1499 (exact vs half::f16::from_f32 / to_f32) ---------
CAST_IN = [[1., 2.], [3., 4.], [5., 6.]]


def test_oracle_casts(orc):
    h = orc.Ref(f32(CAST_IN)).cast(orc.F16).numpy()
    np.testing.assert_array_equal(h, f32(CAST_IN).astype(np.float16))
    np.testing.assert_array_equal(orc.Ref(h).cast(orc.F32).numpy(), f32(CAST_IN))


@pytest.mark.gpu
def test_cuda_casts(wgf, dev):
    h = dev.tensor(f32(CAST_IN)).cast(wgf.F16).as_slice()
    np.testing.assert_array_equal(h, f32(CAST_IN).astype(np.float16))
    np.testing.assert_array_equal(dev.tensor(h).cast(wgf.F32).as_slice(), f32(CAST_IN))


# ---- arange: src/composite/arange.rs:28-59 ------------------------------------------------
def test_oracle_arange(orc):
    np.testing.assert_array_equal(orc.arange(0., 10.).numpy(), np.arange(10, dtype=np.float32))
    np.testing.assert_array_equal(orc.arange(0., 10., 2.).numpy(), f32([0., 2., 4., 6., 8.]))


@pytest.mark.gpu
def test_cuda_arange(dev):
    np.testing.assert_array_equal(dev.arange(0., 10.).as_slice(), np.arange(10, dtype=np.float32))
    np.testing.assert_array_equal(dev.arange(0., 10., 2.).as_slice(), f32([0., 2., 4., 6., 8.]))


# ---- tests/inplace_clone.rs:6-37: in-place reuse must not change a tensor that is still held ----
@pytest.mark.gpu
def test_cuda_inplace_clone(dev):
    t = dev.tensor(f32(D322))
    for _ in range(2):
        c = t.clone()
        plus = c + 1.0
        c.release()  # `tensor.clone() + 1.0` consumes the clone
        np.testing.assert_array_equal(plus.as_slice(), f32(D322) + 1)
    np.testing.assert_array_equal(t.as_slice(), f32(D322))
