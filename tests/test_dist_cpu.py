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


def _ddp_worker(rank, world, port, ret):
    """Two ranks, each with half of the global batch, one optimiser step under DistributedDataParallel."""
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        model, x, labels = _tiny_classifier()
        ddp = torch.nn.parallel.DistributedDataParallel(model)
        from mamba2d_b200 import refmodel
        opt = refmodel.make_optimizer(ddp, lr=1e-3)
        n = x.shape[0] // world
        loss = refmodel.train_step(ddp, opt, x[rank * n:(rank + 1) * n], labels[rank * n:(rank + 1) * n], micro_batch=1,
                                   autocast_dtype=None)
        ret[rank] = dict(loss=float(loss), params=[p.detach().clone().numpy() for p in model.parameters()])
    finally:
        dist.destroy_process_group()


def _tiny_classifier():
    """A four-stage classifier built from the reference's own classes (small widths, one block per
    stage) with a naive PyTorch scan standing in for the kernels, and a seeded batch of 4 images."""
    from mamba2d_b200 import refmodel
    from oracle import torch_ref

    def naive(x, *w, recomp="partial", scan_start="TL"):
        if len(w) == 9:
            *w, recomp = w
        if scan_start == "BR":
            return torch_ref.scan_from_weights(x.flip(1, 2), *w).flip(1, 2)
        return torch_ref.scan_from_weights(x, *w)

    m, u = refmodel.import_reference_models()
    m.wavefront_scan_cuda = naive
    torch.manual_seed(0)
    backbone = m.Mamba2DBackbone(n_blocks=[2, 1, 1, 1], embed_dim=[16, 16, 32, 32], drop_path_rate=0.0,
                                 res_scale_init_values=[1.0] * 4, inter_flip=True,
                                 token_mixer=["2D_local", "2D_local", "RopeAttention", "RopeAttention"])
    model = refmodel.Classifier(backbone, u.MlpHead(dim=32, n_classes=10)).double()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(4, 3, 32, 32, generator=g, dtype=torch.float64)
    labels = torch.randint(0, 10, (4,), generator=g)
    return model, x, labels


@pytest.mark.skipif(__import__("mamba2d_b200.refmodel", fromlist=["x"]).reference_root() is None,
                    reason="no copy of the reference's models/ package")
def test_ddp_training_step_equals_single_rank_step():
    """The training configuration's step (forward + backward + AdamW with the reference's parameter
    groups) on two gloo ranks with micro-batches and gradient accumulation gives the same updated
    weights as one rank on the whole batch: the weight-gradient all-reduce averages what it should."""
    from mamba2d_b200 import refmodel
    world, port = 2, 31000 + os.getpid() % 2000
    ret = mp.Manager().dict()
    mp.spawn(_ddp_worker, args=(world, port, ret), nprocs=world, join=True)
    model, x, labels = _tiny_classifier()
    opt = refmodel.make_optimizer(model, lr=1e-3)
    groups = refmodel.param_groups(model)
    assert groups[1]["weight_decay"] == 0.0 and any(getattr(p, "_no_weight_decay", False) for p in groups[1]["params"])
    assert all(p.dim() >= 2 for p in groups[0]["params"])
    loss = refmodel.train_step(model, opt, x, labels, micro_batch=4, autocast_dtype=None)
    want = [p.detach().numpy() for p in model.parameters()]
    assert abs(0.5 * (ret[0]["loss"] + ret[1]["loss"]) - float(loss)) < 1e-9      # each rank reports its share's mean
    refmodel.purge_models_modules()      # the model module imported here has the naive scan patched in
    for r in (0, 1):
        for a, b in zip(ret[r]["params"], want):
            np.testing.assert_allclose(a, b, rtol=1e-7, atol=1e-9)
