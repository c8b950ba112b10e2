"""The checked build (WGF_CHECKED=1): every generated kernel tests each access to tensor memory
against the extents of the buffers bound to its launch, skips an access that lies outside all of
them and reports the first one at the next synchronisation.  It stands in for a memory checker.

Two things are checked.  (1) The parity, fuzz and shape tests of the generated kernel family run
clean under it: no kernel of theirs reaches outside its buffers.  (2) The predicate itself works:
with WGF_CHECKED_SHRINK=64 the result buffer of every launch is DECLARED 64 bytes shorter than it
is, so stores that are in fact valid are refused -- nothing is ever accessed out of bounds -- and
the library must say so."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_generated_kernels_stay_inside_their_buffers(tmp_path):
    env = dict(os.environ, WGF_CHECKED="1", WGF_KERNEL_CACHE=str(tmp_path / "cache"))
    env.pop("WGF_CHECKED_SHRINK", None)
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-m", "gpu", "-p", "no:cacheprovider",
           os.path.join(HERE, "test_gpu_parity.py"), os.path.join(HERE, "test_gpu_fuzz.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500, cwd=os.path.dirname(HERE))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout


def test_an_access_outside_the_declared_extent_is_refused_and_reported(tmp_path):
    script = tmp_path / "shrunk.py"
    script.write_text(
        "import sys, numpy as np\n"
        f"sys.path.insert(0, {HERE!r})\n"
        "from conftest import load_package\n"
        "wgf = load_package(); d = wgf.Device(0)\n"
        "x = np.arange(4096, dtype=np.float32)\n"
        "t = d.tensor(x)                      # stays alive: the result gets a buffer of its own\n"
        "y = t * 2.0 + 1.0\n"
        "y.materialize()\n"
        "try:\n"
        "    d.sync()\n"
        "    print('NOT REPORTED')\n"
        "except wgf.WgfError as e:\n"
        "    print('STATUS', e.status, '|', str(e))\n"
        "r = d.tensor(np.ones((8, 512), np.float32))\n"
        "rows = r.softmax_last_dim()\n"
        "rows.materialize()\n"
        "try:\n"
        "    d.sync()\n"
        "    print('ROWS NOT REPORTED')\n"
        "except wgf.WgfError as e:\n"
        "    print('ROWS', e.status)\n")
    env = dict(os.environ, WGF_CHECKED="1", WGF_CHECKED_SHRINK="64", WGF_KERNEL_CACHE=str(tmp_path / "cache"))
    r = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "STATUS CUDA" in r.stdout and "checked build" in r.stdout and "the access was not made" in r.stdout, r.stdout
    assert "ROWS CUDA" in r.stdout, r.stdout
