"""Batch sharding of detector inference over the GPUs of one box.

Images are independent (no cross-image operation exists in the detector forward or in NMS, which loops over
images: KAD-CNet/utils/general.py:925 of the reference project), so the batch is split contiguously by rank, each
rank holds a full replica of the ~7 M-parameter model, and the only exchange is the final gather of the
variable-length detection lists to rank 0 through host memory. No collective runs on the data path.
"""
import torch


def shard_range(n_items, rank, world):
    """Contiguous [start, stop) of `n_items` for `rank`; the first n_items % world ranks get one extra item."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f'bad rank {rank} of {world}')
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def gather_detections(local, rank, world, group=None):
    """`local`: this rank's list of [n_i,6] tensors (any device). Returns the concatenated list in image order on
    rank 0 (CPU tensors) and None elsewhere. Uses gather_object on a CPU (gloo) group: host memory only."""
    local = [t.detach().cpu() for t in local]
    if world == 1:
        return local
    import torch.distributed as dist
    out = [None] * world if rank == 0 else None
    dist.gather_object(local, out, dst=0, group=group)
    if rank != 0:
        return None
    return [t for part in out for t in part]
