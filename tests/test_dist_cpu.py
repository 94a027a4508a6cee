"""world_size-2 gloo test of the batch-sharded path (host logic; the math runs on the CPU oracle)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from mamba2d_b200 import shard
    from oracle import cpu, inputs
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        inp = inputs.make_inputs(5, 6, 7, 8, 4, seed=3)
        mine = shard.shard_inputs(inp, world, rank)
        lo, hi = shard.shard_bounds(5, world, rank)
        y = cpu.forward(mine, "f64")
        g = cpu.backward(mine, mode="f64")
        pg = [torch.from_numpy(g[k].copy()) for k in ("d_AT", "d_AL", "d_D")]
        shard.sum_param_grads(pg)
        slow = shard.max_over_ranks(1.0 + rank)
        ret[rank] = dict(lo=lo, hi=hi, y=y, d_x=g["d_x"], d_BT=g["d_BT"], pg=[t.numpy() for t in pg], slow=slow)
    finally:
        dist.destroy_process_group()


def test_two_rank_batch_sharding_equals_single_rank():
    from oracle import cpu, inputs
    world, port = 2, 29000 + os.getpid() % 2000
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    inp = inputs.make_inputs(5, 6, 7, 8, 4, seed=3)
    y = cpu.forward(inp, "f64")
    g = cpu.backward(inp, mode="f64")
    assert (ret[0]["lo"], ret[0]["hi"], ret[1]["lo"], ret[1]["hi"]) == (0, 3, 3, 5)
    np.testing.assert_allclose(np.concatenate([ret[0]["y"], ret[1]["y"]]), y, rtol=1e-13, atol=1e-13)
    np.testing.assert_allclose(np.concatenate([ret[0]["d_x"], ret[1]["d_x"]]), g["d_x"], rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(np.concatenate([ret[0]["d_BT"], ret[1]["d_BT"]]), g["d_BT"], rtol=1e-12, atol=1e-13)
    for r in (0, 1):   # parameter gradients are batch sums: equal on both ranks after the all-reduce
        for got, k in zip(ret[r]["pg"], ("d_AT", "d_AL", "d_D")):
            np.testing.assert_allclose(got, g[k], rtol=1e-11, atol=1e-12)
        assert ret[r]["slow"] == 2.0


def test_shard_bounds_tile_the_batch():
    from mamba2d_b200.shard import shard_bounds
    for B in (0, 1, 5, 8, 128, 1024):
        for world in (1, 2, 3, 4, 8):
            cuts = [shard_bounds(B, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == B
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            sizes = [hi - lo for lo, hi in cuts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)
