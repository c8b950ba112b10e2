"""bench.py without a GPU: the reference arm (the CPU restatement timed on the host cores) prints
the contract's JSON line, the helpers of the GPU arm that need no GPU behave, and the GPU arm
refuses to run without a GPU instead of falling back to anything."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("wgf_bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_the_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "fused_chain_hbm_gbs" and line["unit"] == "GB/s"
    assert line["steps"] == 2 and line["n_gpus"] == 1 and line["higher_is_better"] is True
    assert line["value"] > 0 and abs(line["value"] - line["cpu_baseline"]["value"]) < 1e-9
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # the same bytes per step as the GPU arm counts
    assert line["config"]["bytes_per_step_per_gpu"] == 8 * 8192 * 4096 + 4 * 4096 + 4


def test_bytes_per_step_are_what_the_kernel_moves():
    b = load_bench()
    assert b.BYTES_STEP_FUSED == 8 * b.ROWS * b.H + 4 * b.H + 4          # x and w in, y and the scalar out
    assert b.BYTES_STEP_SEPARATE > b.BYTES_STEP_FUSED                     # x read a second time by the reduction


def test_clock_sampler_without_nvidia_smi(monkeypatch):
    b = load_bench()
    monkeypatch.setenv("PATH", "/nonexistent")
    out = b.ClockSampler(0).stop()
    assert out["sm_mhz"] is None and out["reasons"] == ["nvidia-smi unavailable"]


def test_barrier_of_one_rank_needs_no_process_group():
    b = load_bench()

    class Dev:
        synced = 0

        def sync(self):
            self.synced += 1

    class Torch:
        class cuda:
            @staticmethod
            def synchronize():
                pass

    dev = Dev()
    barrier = b.Barrier(dev, None, Torch, 1)
    barrier()
    barrier.start()
    assert dev.synced == 2 and barrier.started_ns > 0 and barrier.skew_us() == 0.0


def test_gpu_arm_fails_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a GPU is present")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "0", "--no-cpu", "--no-extras"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode != 0
    assert '"value"' not in r.stdout


def test_config_sweep_runs_on_the_compile_only_device():
    """bench_configs.py end to end without a GPU: the rows of the first group are built, resolved and
    recorded as schedules on the compile-only device (no times come out of it, only the structure)."""
    import sys
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from conftest import load_package
    wgf = load_package()
    spec = importlib.util.spec_from_file_location("wgf_bench_configs_under_test", os.path.join(ROOT, "bench_configs.py"))
    sweep = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(sweep)
    dev = wgf.Device(-1)
    lines = []
    rows = sweep.run(wgf, dev, 6543.4, 1668.8, iters=2, warmup=1, only="C1", emit=lines.append, peak_tflops_sustained=1376.9)
    assert len(rows) == 5 and len(lines) == 5
    names = [r["row"] for r in rows]
    assert any("wall clock per pass" in n for n in names) and any(n.startswith("C1' chain") for n in names)
    for r in rows:
        json.dumps(r)                                    # every row is a JSON object
        if "median_us" in r:
            assert "back_to_back_us" in r                # the recorded-schedule path ran too
