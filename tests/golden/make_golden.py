"""Regenerate tests/golden/golden_v1.npz: the inputs of every case in cases.py and the CPU oracle's
output for it.  Run from the repository root:  python tests/golden/make_golden.py

The crate these cases restate is Rust + WGSL and cannot be built or run where this file was made,
so the frozen outputs are the ORACLE's, not the crate's: they guard the oracle (and through it the
CUDA path) against drift.  The crate's own known answers are the separate literal tables in
tests/test_reference_kats.py.
"""
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, HERE)

import cases  # noqa: E402
import oracle  # noqa: E402


def oracle_outputs():
    oracle.lib()
    ns = types.SimpleNamespace(F32=oracle.F32, F16=oracle.F16, BF16=oracle.BF16, cat=oracle.Ref.cat)
    out = {}
    for name, inputs in cases.all_inputs().items():
        _, build, _ = cases.CASES[name]
        res = build({k: oracle.Ref(v) for k, v in inputs.items()}, ns).numpy()
        for k, v in inputs.items():
            out[f"{name}/in/{k}"] = v
        out[f"{name}/out"] = res
    return out


if __name__ == "__main__":
    path = os.path.join(HERE, "golden_v1.npz")
    data = oracle_outputs()
    np.savez_compressed(path, **data)
    print(f"{path}: {len(cases.CASES)} cases, {os.path.getsize(path)} bytes")
