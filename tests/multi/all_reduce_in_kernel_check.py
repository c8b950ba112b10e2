"""Run under torch.distributed.run with one rank per GPU (tests/test_gpu_multi.py starts it).

Each rank owns a shard x_r of f32 [1024,512].  One request asks for the softmax rows of the shard and
three all-reduced whole-tensor reductions of it (sum of exp, max, sum of squares): one kernel per rank
computes all four and posts the three scalars to the other ranks over peer memory (no NCCL launch);
the kernel of the next such step posts them, the kernel six steps on combines what the ranks posted, and one
small kernel does both when a result is read first.  Checked against float64 numpy over all shards, for 40 steps of two exchanges each
(sequence numbers wrap the mailbox slots five times), and that every rank holds identical bits.  With
WGF_NO_PEER_ALLREDUCE=1 the same script checks the NCCL path (four launches per step)."""
import datetime
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from conftest import load_package  # noqa: E402

rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=90))
wgf = load_package()
dev = wgf.Device(local)
ids = [wgf.Comm.unique_id() if rank == 0 else None]
dist.broadcast_object_list(ids, src=0)
comm = wgf.Comm(dev, world, rank, ids[0])
expected_launches = 4 if os.environ.get("WGF_NO_PEER_ALLREDUCE") else 1
alone_expected = 2 if os.environ.get("WGF_NO_PEER_ALLREDUCE") else 1


def data(r, step):
    return np.random.default_rng(1000 * step + r).standard_normal((1024, 512), dtype=np.float32)


bad = 0
for step in range(40):
    xs = [data(r, step) for r in range(world)]
    x = dev.tensor(xs[rank])
    y = x.softmax_last_dim()
    s = x.exp().sum(0).sum(0).all_reduce(comm)
    m = x.max(0).max(0).all_reduce(comm, wgf.OP_MAX)
    q = (x * x).sum(1).sum(0).all_reduce(comm)
    before = dev.launch_count
    wgf.Tensor.materialize_all([y, s, m, q])
    launches = dev.launch_count - before
    es = sum(np.exp(a.astype(np.float64)).sum() for a in xs)
    em = max(a.max() for a in xs)
    eq = sum((a.astype(np.float64) ** 2).sum() for a in xs)
    gs, gm, gq = float(s.as_slice()), float(m.as_slice()), float(q.as_slice())
    rows = y.as_slice().sum(1)
    # the same all-reduced sum requested on its own: a streaming reduction that does the exchange itself
    before = dev.launch_count
    alone = (x * 2.0).exp().sum(0).sum(0).all_reduce(comm)
    alone.materialize()
    alone_launches = dev.launch_count - before
    ea = sum(np.exp(2.0 * a.astype(np.float64)).sum() for a in xs)
    ga = float(alone.as_slice())
    if abs(ga - ea) / ea > 1e-5 or alone_launches != alone_expected:
        print(f"rank {rank} step {step}: stand-alone all-reduce: {alone_launches} launches, got {ga}, expected {ea}", flush=True)
        bad += 1
    ok = (abs(gs - es) / es < 1e-5 and gm == em and abs(gq - eq) / eq < 1e-5 and launches == expected_launches
          and np.abs(rows - 1).max() < 1e-5)
    if not ok:
        print(f"rank {rank} step {step}: launches {launches}, got {gs} {gm} {gq}, expected {es} {em} {eq}", flush=True)
        bad += 1
    t = torch.tensor([gs, gm, gq], dtype=torch.float64, device="cuda")
    t2 = t.clone()
    dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    if not torch.equal(t, t2):
        print(f"rank {rank} step {step}: the ranks hold different bits", flush=True)
        bad += 1
# Second phase: 100 exchanges queued without reading anything back, rank 1 starting late: the kernel
# of exchange k settles exchange k - 6, so the other ranks' streams stop six exchanges ahead of rank 1
# until it arrives (well inside the wait limit); then every result is read, the last six through a
# kernel of their own.
import time  # noqa: E402

x = dev.tensor(data(rank, 0))
xs = [data(r, 0).astype(np.float64) for r in range(world)]
dev.sync()
dist.barrier()
if rank == 1:
    time.sleep(0.3)
kept = []
for k in range(100):
    c = 0.5 + 0.01 * k
    y = (x * c).softmax_last_dim()
    s = (x * c).exp().sum(0).sum(0).all_reduce(comm)
    wgf.Tensor.materialize_all([y, s])
    kept.append((c, s))
for c, s in kept:
    c32 = float(np.float32(c))
    expect = sum(np.exp((a.astype(np.float32) * np.float32(c32)).astype(np.float64)).sum() for a in xs)
    got = float(s.as_slice())
    if abs(got - expect) / expect > 1e-5:
        print(f"rank {rank}: run-ahead exchange with factor {c}: got {got}, expected {expect}", flush=True)
        bad += 1
print(f"rank {rank}: {'PASS' if bad == 0 else 'FAIL'}", flush=True)
dist.barrier()
dist.destroy_process_group()
sys.exit(1 if bad else 0)
