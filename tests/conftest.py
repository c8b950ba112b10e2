"""Shared fixtures.  GPU tests carry @pytest.mark.gpu and call the CUDA path through the
C ABI (libwgf.so); everything else runs on a machine without a GPU."""
import importlib.util
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, ROOT)


def load_package():
    if "wgf_b200" in sys.modules:
        return sys.modules["wgf_b200"]
    path = os.path.join(ROOT, "wgpu-kernal-fusion_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location("wgf_b200", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["wgf_b200"] = mod
    spec.loader.exec_module(mod)
    return mod


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; runs the CUDA path through the C ABI")


@pytest.fixture(scope="session")
def wgf():
    return load_package()


@pytest.fixture(scope="session")
def orc():
    import oracle
    oracle.lib()
    return oracle


@pytest.fixture(scope="session")
def dev(wgf):
    """The GPU.  Fails (does not skip) when there is none: GPU tests must not pass silently."""
    return wgf.Device(0)


@pytest.fixture(scope="session")
def drydev(wgf):
    """Compile-only device: resolves graphs and compiles every kernel, executes nothing."""
    return wgf.Device(-1)


def seeded(config, tensor_index):
    """Input generator shared by tests, oracle and benchmarks: PCG64(0xB2000000 + 16*config + index)."""
    return np.random.Generator(np.random.PCG64(0xB2000000 + 16 * config + tensor_index))
