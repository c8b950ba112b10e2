"""Benchmark of the fused element-wise -> reduce hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (one step, per GPU): x = f32 [8192, 4096] N(0,1) resident in HBM, w = f32 [4096] N(1, 0.1);
  y = softmax_rows(rms_norm(x, w, eps 1e-5))      268 451 840 algorithmic bytes
  s = sum(exp(x)) over the whole tensor            134 217 728 algorithmic bytes
      (+ an all-reduce of the per-GPU scalar when N > 1, done by the same kernel over peer memory,
       NCCL as the fallback: rows are sharded, weak scaling)
Both results are requested together, so one fused row kernel computes y and, from the same registers,
the partial sums of s: x is read from HBM once.  --separate-kernels requests them one by one (row
kernel, then a streaming reduce), which is all the reference's one-tensor-per-call API can express.
Inputs are synthetic (seeded PCG64).  Four input buffers are rotated so that every step reads x
from HBM, not from L2.  `value` = bytes the step has to move (x and w in, y and the scalar out:
268 451 844 per GPU; with --separate-kernels x is read twice: 402 669 568) of all ranks / device time
(CUDA events on the library's stream, max over ranks).  `e2e` = the same metric through the public
C ABI with HOST buffers: upload of x from pinned memory, the kernel, download of y and s, every step.

Beside the headline the line carries
  check        the step's results against the CPU oracle, computed outside the timed regions at every
               N: y on 32 sampled rows per rank, s against the float64 sum over all ranks' shards;
               the process exits non-zero when it fails
  long_run     the same step for at least 0.25 s, with its own clock samples
  matmul       f16 4096^3 on the tensor cores (TFLOP/s, fraction of the measured bf16 burst)
  llama_block  Llama-style decoder block forward, batch 8 x seq 2048 sharded by batch over the GPUs
               of the line (strong scaling), tokens/s
(--no-extras leaves the last three out).

`--impl reference` times the CPU restatement of the reference's math (oracle/oracle.c, fast mode:
float + libm, one memory pass per kernel the reference's resolver would launch) on every host core,
whatever OMP_NUM_THREADS the launcher exported; at N > 1 a step covers N shards.
"""
import argparse
import ctypes
import datetime
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
ROWS, H = 8192, 4096
BYTES_CHAIN = ROWS * H * 4 * 2 + H * 4          # read x, read w, write y
BYTES_SUM = ROWS * H * 4                        # read x (+ 4 bytes out)
BYTES_STEP_SEPARATE = BYTES_CHAIN + BYTES_SUM    # two kernels, x read by each
BYTES_STEP_FUSED = BYTES_CHAIN + 4              # one kernel: x, w in; y and the scalar out
NBUF = 4


def load(name, path):
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs.
    nvidia-smi writes to a file that is read when the sampling stops: no thread of this process
    wakes up while a timed region runs (a reader thread would take the interpreter lock from the
    thread that queues the steps every time a line arrives).  The timed region of the headline is
    about a millisecond long, so its sampler runs at a slow rate from the warm-up on (each sample is a
    driver query on a machine whose other GPUs are busy too); the 0.25 s long run is sampled densely."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index, period_ms=20):
        self.proc = None
        self.out = None
        try:
            import tempfile
            self.out = tempfile.NamedTemporaryFile(mode="w+", prefix="wgf_clocks_", suffix=".csv")
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", str(period_ms)],
                                         stdout=self.out, stderr=subprocess.DEVNULL)
            self.period_ms = period_ms
        except OSError:
            self.proc = None

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15 + self.period_ms / 1000.0)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.flush()
        self.out.seek(0)
        lines = [line.strip() for line in self.out.read().splitlines()]
        self.out.close()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def make_inputs(rank, k):
    g = np.random.Generator(np.random.PCG64(0xB2000000 + 16 * 2 + 64 * rank + k))
    return g.standard_normal((ROWS, H), dtype=np.float32)


def make_weight():
    g = np.random.Generator(np.random.PCG64(0xB2000000 + 16 * 2 + 1))
    return (1.0 + 0.1 * g.standard_normal(H)).astype(np.float32)


# --------------------------------------------------------------------------------------------
# CPU arm: the oracle's fast mode
# --------------------------------------------------------------------------------------------
class CpuWorkload:
    """The workload (or its first `rows` rows) on the host cores."""

    def __init__(self, rows=ROWS):
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import oracle
        self.lib = oracle.lib()
        # every host core this process may run on, whatever OMP_NUM_THREADS says (torch.distributed.run
        # exports OMP_NUM_THREADS=1 to its children)
        try:
            avail = len(os.sched_getaffinity(0))
        except AttributeError:
            avail = os.cpu_count() or 1
        self.cores = int(self.lib.orc_set_threads(avail))
        self.rows = rows
        self.x = make_inputs(0, 0)[:rows].copy()
        self.w = make_weight()
        f = np.float32
        self.norm, self.m, self.s = np.empty(rows, f), np.empty(rows, f), np.empty(rows, f)
        self.tmp, self.normed = np.empty((rows, H), f), np.empty((rows, H), f)
        self.t1, self.t2, self.out = np.empty((rows, H), f), np.empty((rows, H), f), np.empty((rows, H), f)
        self.col = np.empty(H, f)
        self.bytes_step = rows * H * 4 * 2 + H * 4 + 4      # the same unit of work as the GPU arm's value

    def step(self):
        p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        L, R = self.lib, ctypes.c_int64(self.rows)
        L.orc_fast_rms_norm(p(self.x), p(self.w), ctypes.c_float(1e-5), p(self.norm), p(self.tmp), p(self.normed),
                            R, ctypes.c_int64(H))
        L.orc_fast_softmax_rows(p(self.normed), p(self.m), p(self.t1), p(self.t2), p(self.s), p(self.out),
                                R, ctypes.c_int64(H))
        return float(L.orc_fast_sum_exp(p(self.x), p(self.col), R, ctypes.c_int64(H)))

    def time(self, steps, warmup, shards=1):
        """One step = `shards` passes over the sample (the N shards of an N-GPU line, one after the other)."""
        for _ in range(warmup):
            self.step()
        t0 = time.perf_counter()
        for _ in range(steps * shards):
            self.step()
        dt = time.perf_counter() - t0
        return self.bytes_step * shards * steps / dt / 1e9, dt / steps * 1e3


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # Each step is a bounded sample of the workload: as many leading rows as keep the whole
    # run near one minute (never fewer than 256 rows = 4 MiB per array, beyond the core caches).
    shards = max(args.gpus, 1)
    probe = CpuWorkload(256)
    _, probe_ms = probe.time(2, 1)
    budget_ms = 60e3 / max((args.steps + args.warmup) * shards, 1)
    rows = int(min(ROWS, max(256, 256 * budget_ms / max(probe_ms, 1e-3))))
    rows -= rows % 256
    cpu = CpuWorkload(rows)
    gbs, ms = cpu.time(args.steps, args.warmup, shards)
    sample = (f"first {rows} of {ROWS} rows ({rows}x{H} f32) of each of {shards} shard(s) per step, "
              f"{args.steps} steps after {args.warmup} warm-up")
    print(json.dumps({
        "impl": "reference", "metric": "fused_chain_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "rmsnorm->softmax rows + sum(exp(x)), f32 [8192,4096] per GPU", "device": "host cpu",
                   "bytes_per_step_per_gpu": BYTES_STEP_FUSED, "shards_per_step": shards},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cpu.cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# --------------------------------------------------------------------------------------------
# Secondary workloads of the metric: f16 matmul on the tensor cores, Llama-style decoder block
# --------------------------------------------------------------------------------------------
def bf16_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f).get("bf16_tflops", 1590.0)), "measured"
    return 1590.0, "fallback"


def all_host_threads():
    """Context manager: numpy's BLAS on every host core (launchers export OMP_NUM_THREADS=1)."""
    try:
        from threadpoolctl import threadpool_limits
        try:
            n = len(os.sched_getaffinity(0))
        except AttributeError:
            n = os.cpu_count() or 1
        return threadpool_limits(limits=n)
    except ImportError:
        import contextlib
        return contextlib.nullcontext()


class LlamaBlock:
    """Llama-style decoder block forward, f16, random init: hidden 4096, 32 heads x 128, MLP 11008,
    global batch 8 x seq, sharded by batch over the ranks (strong scaling), causal attention."""
    Hd, heads, inter, Bg = 4096, 32, 11008, 8

    def __init__(self, wgf, dev, world, rank, seq, masked):
        self.wgf, self.dev, self.seq = wgf, dev, seq
        Hd, heads, inter = self.Hd, self.heads, self.inter
        D = Hd // heads
        self.b0, self.b1 = wgf.shard_range(self.Bg, world, rank)
        g = np.random.Generator(np.random.PCG64(0xB2000000 + 16 * 5))
        h16 = lambda a: a.astype(np.float16)
        shapes = [(Hd, Hd)] * 4 + [(inter, Hd), (inter, Hd), (Hd, inter)]
        self.W_host = [h16(g.standard_normal(s, dtype=np.float32) * 0.02) for s in shapes]
        self.W = [dev.tensor(w) for w in self.W_host]
        self.n_host = np.ones(Hd, np.float16)
        self.n1, self.n2 = dev.tensor(self.n_host), dev.tensor(self.n_host)
        pos = np.arange(seq, dtype=np.float32)[:, None]
        inv = (1.0 / (10000.0 ** (np.arange(0, D, 2, dtype=np.float32) / D)))[None, :]
        self.cos_host, self.sin_host = h16(np.cos(pos * inv)), h16(np.sin(pos * inv))
        self.cos, self.sin = dev.tensor(self.cos_host), dev.tensor(self.sin_host)
        # causal attention: the fused tensor-core kernel (no mask tensor), or batched matmul + masked
        # softmax + batched matmul through an additive mask
        self.mask = None
        if masked:
            self.mask = dev.tensor(np.where(np.arange(seq)[None, :] <= np.arange(seq)[:, None], 0.0, -np.inf).astype(np.float16))
        xg = np.random.Generator(np.random.PCG64(0xB2000000 + 16 * 5 + 1))
        x_all = h16(xg.standard_normal((self.Bg, seq, Hd), dtype=np.float32))
        self.x_host = x_all[self.b0:self.b1]
        self.x = dev.tensor(self.x_host) if self.b1 > self.b0 else None

    def request(self):
        return self.x.llama_block(self.W, self.n1, self.n2, self.cos, self.sin, self.mask, self.heads, 1e-5)

    def step(self):
        if self.x is not None:
            self.request().materialize()

    def check(self):
        """Output rows of sampled tokens of this rank's first batch element against float64
        (oracle/dense_ref.py): norm-wise error, bound 2e-2 for the f16 block."""
        if self.x is None:
            return 0.0
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import dense_ref
        tokens = np.array([0, 127, 128, self.seq // 2, self.seq - 1])
        out = self.request().as_slice()
        with all_host_threads():
            ref = dense_ref.llama_block_tokens(self.x_host[0], self.W_host, self.n_host, self.n_host, self.cos_host,
                                               self.sin_host, self.heads, 1e-5, tokens)
        if not np.isfinite(out.astype(np.float32)).all():
            return float("inf")
        return float(np.max(np.abs(out[0, tokens].astype(np.float64) - ref)) / np.max(np.abs(ref)))

    def flop(self):
        tokens = self.Bg * self.seq      # attention counted in full (masked half included)
        return tokens * (4 * 2 * self.Hd * self.Hd + 3 * 2 * self.Hd * self.inter + 4 * self.seq * self.Hd)


class Barrier:
    """barrier(): device sync of the library, dist.barrier(), torch.cuda.synchronize().
    barrier.start() is the barrier that opens a timed region.  Ranks leave a barrier tens of
    microseconds apart (every host thread wakes up by itself), and a rank that starts early spends
    that time inside its region waiting for the others' first all-reduce: the maximum over ranks
    would contain the barrier's own jitter.  The ranks of one node read the same monotonic clock, so
    after the barrier rank 0 names an instant 2 ms ahead and every rank spins until then; the spread
    of the instants at which the ranks really started is kept in skew_us()."""

    def __init__(self, dev, dist, torch, world):
        self.dev, self.dist, self.torch, self.world = dev, dist, torch, world
        self.started_ns = 0

    def __call__(self):
        self.dev.sync()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def start(self):
        self()
        if self.world > 1:
            t = self.torch.tensor([time.monotonic_ns() + 2_000_000], dtype=self.torch.int64, device="cuda")
            self.dist.broadcast(t, 0)
            deadline = int(t.item())
            self.torch.cuda.synchronize()
            while time.monotonic_ns() < deadline:
                pass
        self.started_ns = time.monotonic_ns()

    def skew_us(self):
        """Spread of the ranks' last start() instants (a collective: call outside timed regions)."""
        if self.world == 1:
            return 0.0
        t = self.torch.tensor([self.started_ns, -self.started_ns], dtype=self.torch.int64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(int(t[0]) + int(t[1])) / 1e3


class NoCollections:
    """The interpreter's cyclic garbage collector stays off inside a timed region (as `timeit` keeps
    it): a collection that falls into a millisecond-long region of one rank holds up every rank."""

    def __enter__(self):
        import gc
        self.was_on = gc.isenabled()
        gc.disable()          # (no collection here: a full one right before the region leaves the caches cold)

    def __exit__(self, *exc):
        import gc
        if self.was_on:
            gc.enable()
        return False


def time_region(torch, stream, barrier, fn, steps, close=None):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with NoCollections():
        barrier.start()
        e0.record(stream)
        last = None
        for i in range(steps):
            last = fn(i)
        if close is not None:
            close(last)
        del last
        e1.record(stream)
        barrier()
    return e0.elapsed_time(e1) / steps


def matmul_record(wgf, dev, torch, stream, barrier, launches=60):
    """f16 [4096,4096] x [4096,4096] -> f16, fp32 accumulation in tensor memory: three operand pairs
    rotated (192 MiB of operands, more than L2), `launches` timed launches after 20 warm-up ones.
    Checked through projections: for every block of 256 columns C[:, blk] v against A (B[:, blk] v) in
    float64 (every tile of the schedule takes part; oracle/dense_ref.py)."""
    n = 4096
    g = np.random.Generator(np.random.PCG64(0xB2000000 + 16 * 4))
    host = [((g.random((n, n), dtype=np.float32) * 2 - 1).astype(np.float16),
             (g.random((n, n), dtype=np.float32) * 2 - 1).astype(np.float16)) for _ in range(3)]
    ops = [(dev.tensor(a), dev.tensor(b)) for a, b in host]
    fn = lambda i: ops[i % 3][0].mat_mul(ops[i % 3][1]).materialize()
    for i in range(20):
        fn(i)
    # Device time per launch from the event pair the library keeps around every kernel (the analogue
    # of the crate's timestamp queries): what the host does between launches is not in it.  The same
    # launches bracketed by one event pair give the time per launch as the stream saw it.
    dev.set_timing(True)
    seen = [len(o[0].all_timing_information()) for o in ops]
    sampler = ClockSampler(torch.cuda.current_device())
    before = dev.launch_count
    stream_ms = time_region(torch, stream, barrier, fn, launches)
    count = dev.launch_count - before
    clocks = sampler.stop()
    per_launch_ns = []
    for o, already in zip(ops, seen):
        per_launch_ns += o[0].all_timing_information()[already:]
    dev.set_timing(False)
    ms = float(np.mean(per_launch_ns)) / 1e6
    c = ops[0][0].mat_mul(ops[0][1]).as_slice().astype(np.float64)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import dense_ref
    with all_host_threads():
        err = dense_ref.matmul_projection_error(c, host[0][0], host[0][1], vectors=2)
    peak, kind = bf16_peak()
    tf = 2.0 * n ** 3 / (ms * 1e-3) / 1e12
    return {"workload": "f16 4096^3 -> f16, fp32 accumulate", "tflops": tf, "kernel_ms": ms,
            "kernel_ms_median": float(np.median(per_launch_ns)) / 1e6, "stream_ms_per_launch": stream_ms, "launches": launches,
            "gpu_launches": count, "frac_bf16_burst": tf / peak, "peak_bf16_tflops": peak, "peak_kind": kind,
            "frac_nominal_2250": tf / 2250.0, "l2": "three operand pairs rotated: 192 MiB of operands",
            "check": {"projection_rel": err, "bound": 1e-3, "ok": bool(err <= 1e-3)}, "clocks": clocks}


def llama_record(wgf, dev, torch, dist, stream, barrier, world, rank, seq=2048, masked=False, steps=10, warmup=3,
                 check=True, breakdown=False):
    blk = LlamaBlock(wgf, dev, world, rank, seq, masked)
    for _ in range(warmup):
        blk.step()
    sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 else None
    before = dev.launch_count
    ms = time_region(torch, stream, barrier, lambda i: blk.step(), steps)
    launches = dev.launch_count - before
    clocks = sampler.stop() if sampler else None
    err = blk.check() if check else None
    # device time of every kernel of one step (event pair around each launch), after the timed region
    kernels = None
    if breakdown and blk.x is not None:
        dev.set_timing(True)
        for _ in range(2):
            seen = len(blk.x.all_timing_information())
            out = blk.request().materialize()
            dev.sync()
            ns, labels = blk.x.all_timing_information()[seen:], blk.x.timing_labels()[seen:]
            del out
        dev.set_timing(False)
        kernels = [{"kernel": name, "us": round(t / 1e3, 1)} for name, t in zip(labels, ns)]
    vals = torch.tensor([ms, float(launches), err if err is not None else 0.0], dtype=torch.float64, device="cuda")
    if world > 1:
        mx, sm = vals.clone(), vals.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, launches, err = float(mx[0]), int(sm[1]), (float(mx[2]) if err is not None else None)
    tokens = blk.Bg * seq
    rec = {"workload": "llama-style decoder block forward, f16", "tokens_per_s": tokens / (ms * 1e-3), "ms_per_step": ms,
           "steps": steps, "global_batch": blk.Bg, "seq_len": seq, "hidden": blk.Hd, "heads": blk.heads, "mlp": blk.inter,
           "sharding": f"batch/{world}", "scaling": "strong", "gpu_launches": launches,
           "kernels_per_step": launches // max(steps * min(world, blk.Bg), 1),
           "tflops_nominal": blk.flop() / (ms * 1e-3) / 1e12,
           "attention": "matmul + masked softmax + matmul" if masked else "fused tcgen05 kernel", "clocks": clocks}
    if err is not None:
        rec["check"] = {"sampled_tokens_rel": err, "ok": bool(err <= 2e-2)}
    if kernels is not None:
        rec["kernels_of_one_step"] = kernels
    return rec


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    # Libraries (NCCL) print to stdout; keep stdout for the one JSON line.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        # a rank that fails must not leave the others waiting for the default 10 minutes
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))

    wgf = load("wgf_b200", os.path.join(ROOT, "wgpu-kernal-fusion_b200", "__init__.py"))
    dev = wgf.Device(local)
    sm_count, stream_ptr = dev.info()
    stream = torch.cuda.ExternalStream(stream_ptr, device=torch.device("cuda", local))

    comm = None
    if world > 1:
        ids = [wgf.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = wgf.Comm(dev, world, rank, ids[0])

    w_host = make_weight()
    w = dev.tensor(w_host)
    xs = [dev.tensor(make_inputs(rank, k)) for k in range(NBUF)]

    fused = not args.separate_kernels

    def request(y, s):
        # One request for both results: sum(exp(x)) rides along in the row kernel, which has every
        # element of x in registers anyway (x is read from HBM once per step instead of twice).
        if fused:
            wgf.Tensor.materialize_all([y, s])
        else:
            y.materialize()
            s.materialize()

    def step(i):
        x = xs[i % NBUF]
        y = x.layer_norm(w, 1e-5).softmax_last_dim()
        s = x.exp().sum(0).sum(0)
        if comm is not None:
            s = s.all_reduce(comm)
        request(y, s)
        return s

    def close_region(s):
        # At N > 1 the kernel of a step stores this rank's scalar, posts the scalar of the step
        # before to the other ranks and combines the ranks' scalars of the step six before; the
        # last six steps' exchanges are still open when the loop ends.  The last result is consumed
        # here, inside the timed region (the library finishes them with one small kernel, then a
        # one-element multiply reads it): the region contains every step's all-reduce in full.
        if comm is not None and s is not None:
            (s * 1.0).materialize()

    barrier = Barrier(dev, dist, torch, world)

    # ---- device-resident timing --------------------------------------------------------------
    sampler = ClockSampler(local, period_ms=100) if rank == 0 else None   # sampled from the warm-up on: the timed region is short
    last = None
    for i in range(max(args.warmup, 3)):
        last = step(i)
    close_region(last)      # also compiles the small kernel that closes a region at N > 1, outside the timed regions
    del last
    # The first step a process queues right after a collective of torch's costs the host about 0.1 ms
    # more than any later one (one-time set-up): the opening of a region is rehearsed here, so that
    # the timed regions see the steady host path, like every other part of the warm-up.
    for _ in range(2):
        barrier.start()
        close_region(step(0))
    barrier()
    # Region A (the reported value): K steps bracketed by one event pair, per-kernel events off
    # (an event pair around every launch costs the stream ~2.5 us per kernel).
    dev.set_timing(False)
    launches_before = dev.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    no_collections = NoCollections()
    no_collections.__enter__()
    barrier.start()
    e0.record(stream)
    host_t0 = time.perf_counter()
    last = None
    host_marks = []
    for i in range(args.steps):
        last = step(i)
        host_marks.append(time.perf_counter())
    host_ms = (host_marks[-1] - host_t0) * 1e3 / args.steps   # time the host needs to queue one step
    host_first_us = [round((b - a) * 1e6, 1) for a, b in zip([host_t0] + host_marks[:5], host_marks[:6])]
    e_loop = torch.cuda.Event(enable_timing=True)
    e_loop.record(stream)
    close_region(last)
    del last
    e1.record(stream)
    barrier()
    no_collections.__exit__(None, None, None)
    ms_total = e0.elapsed_time(e1)
    start_skew_us = barrier.skew_us()    # how far apart the ranks opened the region
    close_ms = e_loop.elapsed_time(e1)   # what consuming the last step's all-reduced scalar adds to the region
    launches = dev.launch_count - launches_before

    # Region B (the roofline): the same K steps again with an event pair around every launch.
    # All inputs share one graph through w, so the records are in launch order:
    # rows, stream_reduce[, all_reduce] per step.
    dev.set_timing(True)
    n_timing_before = len(xs[0].all_timing_information())
    for i in range(args.steps):
        step(i)
    barrier()
    clocks = sampler.stop() if sampler else None
    kernels_per_step = 1 if fused else 2
    recs = xs[0].all_timing_information()[n_timing_before:]
    # one more record per step when the all-reduce is a launch of its own (NCCL) rather than part of
    # the reduction kernel (peer memory)
    per_step = max(kernels_per_step, len(recs) // max(args.steps, 1))
    row_ns = recs[0::per_step]
    row_ms = float(np.mean(row_ns)) / 1e6 if row_ns else float("nan")
    sum_ms = None
    if not fused:
        sum_ns = recs[1::per_step]
        sum_ms = float(np.mean(sum_ns)) / 1e6 if sum_ns else float("nan")
    # what the all-reduce costs the device stream (the collective itself runs beside it)
    ar_ms = float(np.mean(recs[kernels_per_step::per_step])) / 1e6 if per_step > kernels_per_step else None

    # ---- end to end through the C ABI with host buffers ---------------------------------------
    # Every step uploads its own input from pinned host memory and downloads its results.  The
    # upload of step i+1 is issued (asynchronously, on the library's upload stream) before the
    # download of step i is waited for, so the two PCIe directions work at the same time -- the
    # double buffering any host application of the library would do.
    pin_x = [wgf.PinnedArray((ROWS, H), np.float32) for _ in range(2)]
    pin_y = wgf.PinnedArray((ROWS, H), np.float32)
    pin_s = wgf.PinnedArray((), np.float32)
    for k in range(2):
        pin_x[k].array[...] = make_inputs(rank, k)
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_loop(n):
        x_next = dev.tensor_pinned(pin_x[0])                         # H2D of step 0
        for i in range(n):
            x = x_next
            y = x.layer_norm(w, 1e-5).softmax_last_dim()
            s = x.exp().sum(0).sum(0)
            if comm is not None:
                s = s.all_reduce(comm)
            request(y, s)
            if i + 1 < n:
                x_next = dev.tensor_pinned(pin_x[(i + 1) % 2])       # H2D of step i+1 ...
            y.download_into(pin_y.array)                             # ... beside the D2H of step i
            s.download_into(pin_s.array)

    e2e_loop(2)
    barrier()
    t0 = time.perf_counter()
    e2e_loop(e2e_steps)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps

    # ---- correctness of the step, outside the timed regions, at every N -------------------------
    # y on 32 sampled rows of this rank's shard against the CPU oracle (relative, the bound of the
    # row-chain parity tests), s against the float64 sum of exp over ALL ranks' shards (1e-5).
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    x_host = make_inputs(rank, 0)
    rows = np.unique(np.concatenate([[0, 1, ROWS // 2, ROWS - 2, ROWS - 1],
                                     np.random.Generator(np.random.PCG64(7 + rank)).integers(0, ROWS, 27)]))
    y = xs[0].layer_norm(w, 1e-5).softmax_last_dim()
    s = xs[0].exp().sum(0).sum(0)
    if comm is not None:
        s = s.all_reduce(comm)
    request(y, s)
    y_rows = y.as_slice()[rows]
    s_got = float(s.as_slice())
    del y, s
    y_ref = oracle.Ref(x_host[rows]).layer_norm(oracle.Ref(w_host), 1e-5).softmax_last_dim().numpy()
    y_err = float(np.max(np.abs(y_rows.astype(np.float64) - y_ref) / np.maximum(np.abs(y_ref.astype(np.float64)), 1e-30)))
    part = torch.tensor([np.exp(x_host.astype(np.float64)).sum()], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(part, op=dist.ReduceOp.SUM)
    s_ref = float(part[0])
    s_err = abs(s_got - s_ref) / s_ref
    del x_host

    # ---- the same step for at least 0.25 s, with its own clock samples -----------------------------
    long_run = None
    if not args.no_extras:
        # every rank must run the same number of steps (each step is an all-reduce): agree on the slowest rank's time
        agreed = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(agreed, op=dist.ReduceOp.MAX)
        n_long = max(args.steps, int(0.25 / max(float(agreed[0]) / args.steps * 1e-3, 1e-6)))
        long_sampler = ClockSampler(local) if rank == 0 else None
        dev.set_timing(False)      # as in region A: no event pair around each launch
        long_ms = time_region(torch, stream, barrier, step, n_long, close_region)
        long_run = {"steps": n_long, "ms_per_step": long_ms, "clocks": long_sampler.stop() if long_sampler else None}

    # ---- max over ranks ---------------------------------------------------------------------
    vals = torch.tensor([ms_total, e2e_ms, float(launches), y_err, s_err, long_run["ms_per_step"] if long_run else 0.0],
                        dtype=torch.float64, device="cuda")
    if world > 1:
        mx = vals.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = vals.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms_total, e2e_ms, launches = float(mx[0]), float(mx[1]), int(sm[2])
        y_err, s_err = float(mx[3]), float(mx[4])
        if long_run:
            long_run["ms_per_step"] = float(mx[5])
    check = {"y_rows_max_rel": y_err, "y_rows_per_rank": int(len(rows)), "y_bound": 1e-4, "sum_rel": s_err,
             "sum_bound": 1e-5, "sum": s_got, "sum_float64": s_ref, "ok": bool(y_err <= 1e-4 and s_err <= 1e-5)}

    # ---- the other two parts of the metric: f16 matmul and the decoder block ------------------------
    matmul = llama = None
    if not args.no_extras:
        xs.clear()
        dev.set_timing(False)
        if rank == 0:
            matmul = matmul_record(wgf, dev, torch, stream, Barrier(dev, None, torch, 1))   # this rank alone
        llama = llama_record(wgf, dev, torch, dist, stream, barrier, world, rank)

    if rank == 0:
        peak, peak_kind = measured_peak()
        ms_step = ms_total / args.steps
        bytes_step = BYTES_STEP_FUSED if fused else BYTES_STEP_SEPARATE
        value = bytes_step * world / (ms_step * 1e-3) / 1e9
        if long_run:
            long_run["value"] = bytes_step * world / (long_run["ms_per_step"] * 1e-3) / 1e9
        # bytes the dominant kernel has to move per launch: x, w in, y out (+ the 4-byte scalar when
        # the reduction rides along)
        kernel_bytes = BYTES_CHAIN + (4 if fused else 0)
        # Average duration of a launch: with one kernel per step the timed region IS K launches of that
        # kernel between one event pair, so its average is region A's; an event pair around every
        # single launch (region B) adds about 2.5 us of event handling to each and is reported beside it
        # (ncu's gpu__time_duration of the same launches, serialised and cold: 46.3 us).  With two kernels
        # per step only the event pairs can tell them apart.
        launch_ms = ms_step if fused and world == 1 else row_ms
        achieved = kernel_bytes / (launch_ms * 1e-3) / 1e9
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on this workload, from
        # the ncu captures summarised under profiles/ (134.26 MB read + 85.19 MB written with the
        # reduction riding along; 134.25 + 84.19 without); the rest of the 134 MB output is still
        # dirty in L2 when the kernel ends
        traffic = 219_449_088 if fused else 218_444_800
        sum_exp = None
        if not fused:
            sum_exp = {"achieved": BYTES_SUM / (sum_ms * 1e-3) / 1e9, "launch_ms": sum_ms,
                       "frac": BYTES_SUM / (sum_ms * 1e-3) / 1e9 / peak}
        # CPU baseline on rank 0, N=1 only: the oracle's fast mode on the full workload
        cpu_baseline = None
        if world == 1 and not args.no_cpu:
            cpu = CpuWorkload()
            reps = 8
            gbs, _ = cpu.time(reps, 1)
            cpu_baseline = {"value": gbs, "unit": "GB/s", "cores": cpu.cores, "kind": "port",
                            "sample": f"full workload ({ROWS}x{H} f32), {reps} repetitions after 1 warm-up"}
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps({
            "metric": "fused_chain_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "rmsnorm->softmax rows + sum(exp(x)), f32 [8192,4096] per GPU",
                       "rows_per_gpu": ROWS, "row_len": H, "sharding": "rows" if world > 1 else "none",
                       "l2": f"{NBUF} input buffers of 128 MiB rotated: inputs larger than L2",
                       "bytes_per_step_per_gpu": bytes_step,
                       "algorithmic_bytes_if_separate": BYTES_STEP_SEPARATE,
                       "kernels_per_step": kernels_per_step,
                       "note": ("one kernel per step reads x and w once and writes y and the scalar: value counts those "
                                "bytes; the reference's resolver runs the step as 11 kernels"
                                if fused else "two kernels per step: row kernel, then streaming reduce; each reads x")},
            "roofline": {"bound": "hbm",
                         "kernel": "fused rmsnorm->softmax row kernel" + (" with sum(exp(x)) riding along" if fused else ""),
                         "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "launch_ms": launch_ms,
                         "launch_ms_with_event_pair_per_launch": row_ms,
                         "bytes_per_launch": kernel_bytes, "sum_exp_kernel": sum_exp},
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": bytes_step * world / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
                    "steps": e2e_steps, "h2d_bytes_per_step": ROWS * H * 4, "d2h_bytes_per_step": ROWS * H * 4 + 4},
            "gpu_launches": launches,
            "check": check,
            "long_run": long_run,
            "matmul": matmul,
            "llama_block": llama,
            "host_queue_ms_per_step": host_ms,
            "region_close_ms": close_ms,
            "host_queue_first_steps_us": host_first_us,
            "row_kernel_first_launches_us": [round(t / 1e3, 1) for t in row_ns[:6]],
            "row_kernel_median_us": (round(float(np.median(row_ns)) / 1e3, 1) if row_ns else None),
            "region_start_skew_us": start_skew_us,
            "all_reduce": (None if comm is None else
                           "over peer memory, inside the steps' own kernels: the kernel of step k stores this rank's value, posts the value of step k-1 and combines the ranks' values of step k-6"
                           if per_step == kernels_per_step else "NCCL launch"),
            "all_reduce_on_device_stream_ms": ar_ms,
            "clocks": clocks,
        }))
        sys.stdout.flush()
    ok = check["ok"] and (matmul is None or matmul["check"]["ok"]) and (llama is None or llama.get("check", {}).get("ok", True))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        print("bench: a correctness check failed (see the check keys of the line)", file=sys.stderr)
        sys.exit(1)


# --------------------------------------------------------------------------------------------
# Secondary workload as the headline (--workload llama_block): tokens/s of the decoder block, batch 8
# sharded by batch over the GPUs (strong scaling: the global batch stays 8).  No collective.
# --------------------------------------------------------------------------------------------
def run_llama(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    wgf = load("wgf_b200", os.path.join(ROOT, "wgpu-kernal-fusion_b200", "__init__.py"))
    dev = wgf.Device(local)
    _, stream_ptr = dev.info()
    stream = torch.cuda.ExternalStream(stream_ptr, device=torch.device("cuda", local))
    dev.set_timing(False)

    barrier = Barrier(dev, dist, torch, world)
    rec = llama_record(wgf, dev, torch, dist, stream, barrier, world, rank, seq=args.seq, masked=args.separate_kernels,
                       steps=args.steps, warmup=max(args.warmup, 3), check=not args.no_cpu, breakdown=args.breakdown)
    if rank == 0:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps({
            "metric": "llama_block_tokens_per_s", "value": rec["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "llama-style decoder block forward", "hidden": rec["hidden"], "heads": rec["heads"],
                       "head_dim": rec["hidden"] // rec["heads"], "mlp": rec["mlp"], "global_batch": rec["global_batch"],
                       "seq_len": rec["seq_len"], "sharding": rec["sharding"], "attention": rec["attention"]},
            "tflops_nominal": rec["tflops_nominal"], "gpu_launches": rec["gpu_launches"], "check": rec.get("check"),
            "kernels_of_one_step": rec.get("kernels_of_one_step"), "clocks": rec["clocks"],
        }))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_configs(args):
    """--workload configs: every benchmark configuration on one GPU, one JSON object per row
    (the sweep itself is bench_configs.py)."""
    wgf = load("wgf_b200", os.path.join(ROOT, "wgpu-kernal-fusion_b200", "__init__.py"))
    sweep = load("wgf_b200_bench_configs", os.path.join(ROOT, "bench_configs.py"))
    peak_gbs, which = measured_peak()
    peak_tf, peak_tf_sustained = 1590.0, 1400.0
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peaks = json.load(f)
        peak_tf = float(peaks.get("bf16_tflops", peak_tf))
        peak_tf_sustained = float(peaks.get("bf16_tflops_sustained", peak_tf_sustained))
    dev = wgf.Device(int(os.environ.get("LOCAL_RANK", "0")))
    sampler = ClockSampler(0)
    rows = sweep.run(wgf, dev, peak_gbs, peak_tf, iters=args.steps, warmup=max(args.warmup, 3), only=args.rows,
                     peak_tflops_sustained=peak_tf_sustained)
    print(json.dumps({"workload": "configs", "rows": len(rows), "peak_hbm_gbs": peak_gbs, "peak_bf16_tflops": peak_tf,
                      "peak_bf16_tflops_sustained": peak_tf_sustained,
                      "peaks": which, "clocks": sampler.stop()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="wgf", choices=["wgf", "reference"])
    ap.add_argument("--workload", default="fused_chain", choices=["fused_chain", "llama_block", "configs"])
    ap.add_argument("--seq", type=int, default=2048, help="sequence length of the llama_block workload")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (llama_block: the float64 check)")
    ap.add_argument("--breakdown", action="store_true", help="llama_block: also list the device time of every kernel of one step")
    ap.add_argument("--no-extras", action="store_true",
                    help="fused_chain: leave out the long_run, matmul and llama_block records")
    ap.add_argument("--rows", default=None, help="configs workload: only the rows whose name contains this text")
    ap.add_argument("--separate-kernels", action="store_true",
                    help="fused_chain: request the two results one by one (row kernel, then streaming reduce); "
                         "llama_block: attention as matmul + masked softmax + matmul instead of the fused kernel")
    args = ap.parse_args()
    llama = args.workload == "llama_block"
    configs = args.workload == "configs"
    if args.steps is None:
        args.steps = 10 if llama else 30 if configs else 2000
    if args.warmup is None:
        args.warmup = 3 if llama else 5 if configs else 200
    try:
        if args.impl == "reference":
            run_reference(args)
        elif configs:
            run_configs(args)
        elif llama:
            run_llama(args)
        else:
            run_gpu(args)
    except SystemExit:
        raise
    except BaseException:
        # Under a multi-process launcher a rank that dies in a Python exception can sit in the teardown
        # of its libraries while the other ranks wait for it: report and leave at once, so that the
        # launcher ends the job.
        import traceback
        traceback.print_exc()
        sys.stderr.flush()
        if int(os.environ.get("WORLD_SIZE", "1")) > 1:
            os._exit(1)
        raise


if __name__ == "__main__":
    main()
