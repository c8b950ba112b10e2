"""Multi-process path on CPU (gloo, world size 2 and 3): rows are sharded with wgf_shard_range, every
rank works on its own rows only, and the one exchange of the path -- the all-reduce that closes a
full-tensor reduction -- combines the partials.  The per-rank math is the CPU oracle here (no GPU);
what is under test is the partition, the independence of the shards and the combine step."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ROWS, H = 37, 64   # 37 rows: the shards are uneven


def _inputs():
    g = np.random.Generator(np.random.PCG64(0xB2000000 + 16 * 2))
    return g.standard_normal((ROWS, H)).astype(np.float32), (1 + 0.1 * g.standard_normal(H)).astype(np.float32)


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import conftest
    import oracle
    wgf = conftest.load_package()
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, w = _inputs()
    b, e = wgf.shard_range(ROWS, world, rank)
    mine = oracle.Ref(x[b:e])
    rows = mine.layer_norm(oracle.Ref(w), 1e-5).softmax_last_dim().numpy()
    partial = np.exp(x[b:e].astype(np.float64)).sum()
    t = torch.tensor([partial], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)           # the path's only collective
    np.save(os.path.join(out_dir, f"rows_{rank}.npy"), rows)
    np.save(os.path.join(out_dir, f"sum_{rank}.npy"), t.numpy())
    np.save(os.path.join(out_dir, f"range_{rank}.npy"), np.array([b, e]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_row_sharding_and_allreduce(world, tmp_path, orc):
    port = 29500 + os.getpid() % 2000 + world
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    x, w = _inputs()
    full_rows = orc.Ref(x).layer_norm(orc.Ref(w), 1e-5).softmax_last_dim().numpy()
    full_sum = np.exp(x.astype(np.float64)).sum()
    got, prev_end = [], 0
    for r in range(world):
        b, e = np.load(tmp_path / f"range_{r}.npy")
        assert b == prev_end
        prev_end = e
        got.append(np.load(tmp_path / f"rows_{r}.npy"))
        s = np.load(tmp_path / f"sum_{r}.npy")[0]
        assert abs(s - full_sum) <= 1e-12 * full_sum      # every rank holds the combined value
    assert prev_end == ROWS
    np.testing.assert_array_equal(np.concatenate(got, 0), full_rows)   # shards are independent: bit-identical
