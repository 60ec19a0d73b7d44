"""Multi-GPU host logic: one process per GPU, independent replicas, images sharded by index.

The forward of one image depends on nothing but the (read-only) weights, so the path shards with
no collective on the data path: every rank builds the same plan on its own device and runs its own
contiguous slice of the job. torch.distributed is used only for the start/stop barrier of a timed
region, the max-over-ranks of the device time and the gather of per-rank results (works with the
`gloo` backend on CPU, which is how the tests run it).
"""
import os


def env_rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def shard_range(n_items, rank, world):
    """Contiguous [lo, hi) of rank's items; the first n_items % world ranks get one extra."""
    if world < 1 or not (0 <= rank < world) or n_items < 0:
        raise ValueError("bad shard arguments")
    base, extra = divmod(n_items, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def weak_job(per_gpu_batch, rank, world):
    """Weak scaling: every rank owns per_gpu_batch images; image ids are global and disjoint."""
    return rank * per_gpu_batch, (rank + 1) * per_gpu_batch


def reduce_max(value, dist=None):
    """Max over ranks of a python float (no-op without an initialised process group)."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    import torch
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def reduce_sum(value, dist=None):
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    import torch
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def gather_in_image_order(local_results, lo, dist=None):
    """local_results: list of per-image results of this rank, first image id `lo`. Returns on every
    rank the list over all ranks in global image order."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return list(local_results)
    bucket = [None] * dist.get_world_size()
    dist.all_gather_object(bucket, (lo, list(local_results)))
    out = []
    for start, items in sorted(bucket, key=lambda t: t[0]):
        out.extend(items)
    return out
