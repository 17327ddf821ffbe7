"""Batch sharding of the CNN workloads across the GPUs of one node.

Images are independent units: every rank (one process per GPU) runs the same program with the same
seeded weights on its own slice of the batch; there is no collective on the data path. The process
group is used only to line ranks up (barrier) and to combine device-measured times (max over
ranks) and counters (sum). The reference has no multi-device runtime (its interpreter runs one
function on one host thread, src/Native/src/runtime/interpreter.cpp:214-248).
"""
import torch
import torch.distributed as dist


def shard_range(total, world, rank):
    """Contiguous slice [start, start + count) of `total` units owned by `rank`: sizes differ by at
    most one, earlier ranks take the remainder, every unit belongs to exactly one rank."""
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError("bad sharding arguments")
    base, rem = divmod(total, world)
    count = base + (1 if rank < rem else 0)
    start = rank * base + min(rank, rem)
    return start, count


def max_over_ranks(values, device="cpu"):
    """Element-wise maximum of a list of floats over all ranks (identity without a process group)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(values)
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def sum_over_ranks(values, device="cpu"):
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return list(values)
    t = torch.tensor(list(values), dtype=torch.int64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return [int(x) for x in t]


def gather_outputs(local, counts, device="cpu"):
    """Host-side gather of per-rank result rows (e.g. logits) onto every rank, in rank order."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local
    width = tuple(local.shape[1:])
    most = max(counts)
    padded = torch.zeros((most,) + width, dtype=local.dtype, device=device)  # all_gather wants equal shapes
    padded[: local.shape[0]] = local.to(device)
    bufs = [torch.empty_like(padded) for _ in counts]
    dist.all_gather(bufs, padded)
    return torch.cat([b[:c] for b, c in zip(bufs, counts)], 0)
