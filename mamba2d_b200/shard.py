"""Batch sharding for multi-GPU runs: every (image, channel, state) recurrence is independent, so
the scan shards over the batch with no collective on the data path.  One process per GPU."""
import torch


def shard_bounds(batch, world_size, rank):
    """Contiguous, balanced [lo, hi) slice of the batch owned by ``rank`` (first ranks take the
    remainder).  Slices tile [0, batch) exactly; a rank may own an empty slice when batch < world."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    base, rem = divmod(batch, world_size)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_inputs(tensors, world_size, rank, batched=("x", "dT", "dL", "BT", "BL", "C", "gy")):
    """Slice the batched tensors of an input dict; per-channel parameters are replicated."""
    out = {}
    for k, v in tensors.items():
        if k in batched:
            lo, hi = shard_bounds(v.shape[0], world_size, rank)
            out[k] = v[lo:hi]
        else:
            out[k] = v
    return out


def max_over_ranks(value, device=None):
    """Max of a Python float over all ranks (identity without an initialised process group)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_param_grads(grads, device=None):
    """All-reduce (sum) the per-channel parameter gradients d_AT, d_AL, d_D of a batch-sharded
    backward -- the only quantities of the scan that couple ranks (they are sums over the batch)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return grads
    for g in grads:
        dist.all_reduce(g, op=dist.ReduceOp.SUM)
    return grads
