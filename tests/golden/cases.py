"""Golden cases: small seeded graphs written once against the method names that the CPU oracle
(`oracle.Ref`) and the CUDA binding (`Tensor`) share.  `make_golden.py` evaluates every case
with the oracle and freezes inputs and outputs in `golden_v1.npz`; the tests replay them.

Each case is  name -> (inputs(g) -> dict of arrays, build(t, ns) -> tensor, check)  where
  g      is numpy.random.Generator(PCG64(0x601D + index of the case)),
  t      maps input names to tensors of the implementation under test,
  ns     carries the implementation's constants and free functions (F32, F16, cat),
  check  is "exact" (moves, casts, index ops, + - * /), ("ulp", n) in units of the result type (2 for one
         f32 transcendental op, 4 for a chain of several, whose errors add; 1 for f16), or ("rel", tol)
         for reductions and ("norm", tol) for matmul.
"""
import numpy as np


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _n(g, shape, scale=1.0):
    return f32(g.standard_normal(shape) * scale)


def _u(g, shape, lo, hi):
    return f32(g.random(shape) * (hi - lo) + lo)


CASES = {}


def case(name, check):
    def deco(pair):
        inputs, build = pair()
        CASES[name] = (inputs, build, check)
        return pair
    return deco


@case("add_const_then_mul_const_3x2", "exact")
def _():
    return (lambda g: {"x": f32([[1, 2], [3, 4], [5, 6]])},
            lambda t, ns: (t["x"] + 1.0) * 2.0)


@case("fused_unary_chain_2x2", ("ulp", 4))
def _():
    return (lambda g: {"x": f32([[1, 2], [3, 4]])},
            lambda t, ns: ((t["x"] * 2.0 + 1.0).sin().cos() * 0.5).exp())


@case("binary_dag_37x129", "exact")
def _():
    return (lambda g: {"x": _n(g, (37, 129), 3), "y": _n(g, (37, 129), 3) + 5.0},
            lambda t, ns: (t["x"] + t["y"]) * (t["x"] - t["y"]) / (t["y"] + 3.0))


@case("transcendentals_1000", ("ulp", 4))
def _():
    return (lambda g: {"x": _u(g, (1000,), 0.05, 4.0)},
            lambda t, ns: (t["x"].log().sqr() + t["x"].sqrt()).tanh() + t["x"].atan() * t["x"].exp2())


@case("pow_33x17", ("ulp", 2))
def _():
    return (lambda g: {"x": _u(g, (33, 17), 0.1, 5.0), "y": _n(g, (33, 17), 1.5)},
            lambda t, ns: t["x"].pow(t["y"]))


@case("cast_f16_round_trip_4099", "exact")
def _():
    return (lambda g: {"x": np.concatenate([_n(g, (4087,), 100), f32([0, -0.0, 65504, 65519.9, 65520, 1e9, -1e9,
                                                                       np.inf, -np.inf, 6e-8, 2.9e-8, 3e-8])])},
            lambda t, ns: t["x"].cast(ns.F16).cast(ns.F32))


@case("f16_chain_64x48", ("ulp", 1))
def _():
    return (lambda g: {"x": _n(g, (64, 48)).astype(np.float16)},
            lambda t, ns: (t["x"] * 1.5 + 0.25).tanh())


@case("sum_axis0_5x7x9", ("rel", 1e-5))
def _():
    return (lambda g: {"x": _u(g, (5, 7, 9), 0.5, 2.0)}, lambda t, ns: t["x"].sum(0))


@case("sum_axis1_epilogue_5x7x9", ("rel", 1e-5))
def _():
    return (lambda g: {"x": _u(g, (5, 7, 9), 0.5, 2.0)}, lambda t, ns: (t["x"] + 1.0).sum(1) * 2.0)


@case("max_min_product_6x11", ("rel", 1e-5))
def _():
    return (lambda g: {"x": _u(g, (6, 11), 0.8, 1.25)},
            lambda t, ns: t["x"].max(1) + t["x"].min(1) + t["x"].product(1))


@case("full_sum_exp_64x96", ("rel", 1e-5))
def _():
    return (lambda g: {"x": _n(g, (64, 96))}, lambda t, ns: t["x"].exp().sum(0).sum(0))


@case("rmsnorm_softmax_16x256", ("rel", 1e-5))
def _():
    return (lambda g: {"x": _n(g, (16, 256)), "w": _u(g, (256,), 0.5, 1.5)},
            lambda t, ns: t["x"].layer_norm(t["w"], 1e-5).softmax_last_dim())


@case("softmax_rank1_117", ("rel", 1e-5))
def _():
    return (lambda g: {"x": _n(g, (117,))}, lambda t, ns: t["x"].softmax())


@case("silu_24x40", ("ulp", 6))
def _():
    return (lambda g: {"x": _n(g, (24, 40), 2)}, lambda t, ns: t["x"].silu())


@case("rope_6x8x16", "exact")
def _():
    def inputs(g):
        pos = np.arange(10)[:, None] / (10000.0 ** (np.arange(8)[None, :] / 8.0))
        return {"x": _n(g, (6, 8, 16)), "cos": f32(np.cos(pos)), "sin": f32(np.sin(pos))}
    return (inputs, lambda t, ns: t["x"].rope(t["cos"], t["sin"]))


@case("transpose_slice_add_12x20", "exact")
def _():
    return (lambda g: {"x": _n(g, (12, 20))},
            lambda t, ns: t["x"].transpose(0, 1).slice([(2, 17), (1, 11)]) + 1.0)


@case("broadcast_outer_product_7x5", "exact")
def _():
    return (lambda g: {"a": _n(g, (7,)), "b": _n(g, (5,))},
            lambda t, ns: t["a"].broadcast_axis(1, 5) * t["b"].broadcast((7, 5)))


@case("resize_grow_twice_4x6", "exact")
def _():
    return (lambda g: {"x": _n(g, (4, 6))}, lambda t, ns: (t["x"].resize((6, 9)) + 1.0).resize((6, 12)))


@case("slice_assign_6x8", "exact")
def _():
    return (lambda g: {"x": _n(g, (6, 8)), "v": _n(g, (2, 3))},
            lambda t, ns: t["x"].slice_assign([(1, 3), (4, 7)], t["v"]))


@case("cat_axis1_3x4_3x6", "exact")
def _():
    return (lambda g: {"a": _n(g, (3, 4)), "b": _n(g, (3, 6))}, lambda t, ns: ns.cat([t["a"], t["b"] * 2.0], 1))


@case("reshape_of_transposed_8x6", "exact")
def _():
    return (lambda g: {"x": _n(g, (8, 6))}, lambda t, ns: t["x"].transpose(0, 1).reshape((4, 12)))


@case("matmul_f32_37x21_21x50", ("norm", 1e-4))
def _():
    return (lambda g: {"a": _n(g, (37, 21)), "b": _n(g, (21, 50))}, lambda t, ns: t["a"].mat_mul(t["b"]))


@case("matmul_f16_batched_3x40x24_3x24x16", ("norm", 1e-2))
def _():
    return (lambda g: {"a": _n(g, (3, 40, 24)).astype(np.float16), "b": _n(g, (3, 24, 16)).astype(np.float16)},
            lambda t, ns: t["a"].mat_mul(t["b"]))


def generator(index):
    return np.random.Generator(np.random.PCG64(0x601D + index))


def all_inputs():
    """name -> dict of input arrays, in the fixed order of CASES."""
    return {name: CASES[name][0](generator(i)) for i, name in enumerate(CASES)}
