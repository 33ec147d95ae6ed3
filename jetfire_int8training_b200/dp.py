"""Data-parallel exchange of the INT8 linear layer's weight gradients.

The path shards by data parallelism only (INT8_GPT2/train.py:94-107, 227 of the reference wraps the model in DDP): every rank
runs the layer on its own batch and the single exchange step is the sum (then mean) of the weight gradients.  This helper
packs the gradients of one step into one flat buffer per dtype, issues one all-reduce per buffer on the given process group
(NCCL over NVLink on GPUs, gloo in the CPU tests) and scatters the averaged values back in place.
"""
import torch
import torch.distributed as dist


def allreduce_mean_(tensors, group=None, bucket_bytes=None):
    """In-place mean of `tensors` over the ranks of `group`.  Tensors are grouped by dtype into flat buckets of at most
    `bucket_bytes` (None = one bucket per dtype) so that small gradients do not pay one collective each."""
    if not dist.is_available() or not dist.is_initialized():
        return tensors
    world = dist.get_world_size(group)
    if world == 1:
        return tensors
    by_dtype = {}
    for t in tensors:
        by_dtype.setdefault((t.dtype, t.device), []).append(t)
    for (dtype, device), ts in by_dtype.items():
        bucket, size = [], 0
        limit = bucket_bytes if bucket_bytes else float("inf")

        def flush(bucket):
            if not bucket:
                return
            if len(bucket) == 1 and bucket[0].is_contiguous():
                flat = bucket[0].view(-1)
                dist.all_reduce(flat, group=group)
                flat.div_(world)
                return
            flat = torch.cat([b.reshape(-1) for b in bucket])
            dist.all_reduce(flat, group=group)
            flat.div_(world)
            off = 0
            for b in bucket:
                n = b.numel()
                b.copy_(flat[off:off + n].view_as(b))
                off += n
        for t in ts:
            nbytes = t.numel() * t.element_size()
            if bucket and size + nbytes > limit:
                flush(bucket)
                bucket, size = [], 0
            bucket.append(t)
            size += nbytes
        flush(bucket)
    return tensors


def shard_range(total, rank, world):
    """Contiguous [begin, end) share of `total` items for `rank` (the first total % world ranks get one more)."""
    base, rem = divmod(total, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)
