"""Run under torch.distributed.run with two ranks (tests/test_gpu_multi.py starts it with
WGF_PEER_WAIT_MS=50 and NVLS off).

Both ranks do one all-reduce over peer memory; then rank 1 sits one exchange out (it is idle, between
steps, with nothing in flight).  Rank 0's settling kernel (queued by the synchronisation) must give up after its 50 ms
limit and return, rank 0's next synchronisation must raise WGF_ERR_TIMEOUT, further all-reduces on that device
must be refused, and both ranks must be able to release the communicator and leave cleanly.  No GPU
is faulted: the wait is a bounded poll of a word that nobody writes."""
import datetime
import os
import sys
import time

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from conftest import load_package  # noqa: E402

rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
assert world == 2
torch.cuda.set_device(local)
dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=60))
wgf = load_package()
dev = wgf.Device(local)
ids = [wgf.Comm.unique_id() if rank == 0 else None]
dist.broadcast_object_list(ids, src=0)
comm = wgf.Comm(dev, world, rank, ids[0])
x = np.random.default_rng(rank).standard_normal((256, 512), dtype=np.float32)
t = dev.tensor(x)
ok = True

# exchange 1: both ranks take part
s = t.exp().sum(0).sum(0).all_reduce(comm)
got = float(s.as_slice())
expect = sum(np.exp(np.random.default_rng(r).standard_normal((256, 512), dtype=np.float32).astype(np.float64)).sum() for r in range(2))
ok = ok and abs(got - expect) / expect < 1e-5
dev.sync()
dist.barrier()

# exchange 2: rank 0 alone
if rank == 0:
    t0 = time.perf_counter()
    s2 = t.exp().sum(0).sum(0).all_reduce(comm)
    s2.materialize()
    try:
        dev.sync()
        print("rank 0: the sync after a one-sided exchange did not fail", flush=True)
        ok = False
    except wgf.WgfError as e:
        waited = time.perf_counter() - t0
        ok = ok and e.status == "TIMEOUT" and waited < 2.0
        if e.status != "TIMEOUT" or waited >= 2.0:
            print(f"rank 0: status {e.status} after {waited:.3f} s", flush=True)
    dev.sync()                                  # the error word was cleared: the device is usable
    ok = ok and float((t * 2.0).sum(0).sum(0).as_slice()) == float((dev.tensor(x) * 2.0).sum(0).sum(0).as_slice())
    try:                                        # the ranks are out of step: further all-reduces are refused
        t.exp().sum(0).sum(0).all_reduce(comm).materialize()
        print("rank 0: an all-reduce after the timeout was not refused", flush=True)
        ok = False
    except wgf.WgfError as e:
        ok = ok and e.status == "TIMEOUT"
dist.barrier()
# ncclCommDestroy is a collective among the ranks of a node: every rank has to let go of its
# communicator, and a tensor of an all-reduce node holds a reference to it
s2 = None
del s, comm
dev.sync()
print(f"rank {rank}: {'PASS' if ok else 'FAIL'}", flush=True)
dist.barrier()
dist.destroy_process_group()
sys.exit(0 if ok else 1)
