"""Batch sharding of the path over ranks: every image is independent, so rank r of R owns a
contiguous slice of the global batch, weights are replicated and no collective touches the
data path.  The only exchange is the reduction of the timing (max over ranks) and of the
image counts for the throughput line."""


def shard_slice(global_batch, rank, world):
    """Contiguous [start, stop) of the global batch owned by `rank`; remainders go to the
    first ranks."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank %d outside world of %d" % (rank, world))
    base, rem = divmod(global_batch, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def aggregate_throughput(local_images, local_ms, group=None):
    """Whole-job images/s = (sum of images over ranks) / (max of the ranks' times)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return local_images / (local_ms / 1e3), local_ms
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([local_ms], dtype=torch.float64, device=dev)
    n = torch.tensor([float(local_images)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    dist.all_reduce(n, op=dist.ReduceOp.SUM, group=group)
    return float(n.item()) / (float(t.item()) / 1e3), float(t.item())
