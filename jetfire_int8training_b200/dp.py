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


class MeanReducer:
    """Mean of the weight gradients across ranks: submit() issues the collective, wait() orders the current stream after it.

    On NCCL the division by the world size is folded into the collective (ReduceOp.AVG); gloo (the CPU tests) has no AVG, there
    the sum is divided afterwards.  With one rank (or no process group) both calls do nothing.

    overlap=False (default): the collective runs on the current stream, right behind the kernel that produced the gradients.
    overlap=True: it runs on a side stream that waits for the gradients, so that later kernels on the current stream (the next
    step's forward and input-gradient GEMMs, which do not need the reduced gradient) may run beside it.  Measured on two B200s
    with the 8192^3 layer this is SLOWER (5.93 ms per step against 5.70 ms): the GEMMs are persistent kernels with one CTA of
    608 threads x 96 registers per SM, so no SM has room for the collective's CTAs until a GEMM kernel drains, and the two
    then alternate at kernel granularity with a tail on each switch.  It is kept for callers whose kernels leave SMs free.
    """

    def __init__(self, group=None, device=None, overlap=False):
        self.group = group
        self.active = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if self.active else 1
        self.cuda = bool(self.active and overlap and device is not None and torch.device(device).type == "cuda")
        self.stream = torch.cuda.Stream(device) if self.cuda else None
        self.avg = self.active and dist.get_backend(group) == "nccl"
        self.pending = []        # (tensors, done event or None)

    def submit(self, tensors):
        if not self.active:
            return
        tensors = [t for t in tensors]
        if self.cuda:
            ready = torch.cuda.Event()
            ready.record()                                   # the gradients are complete at this point of the current stream
            with torch.cuda.stream(self.stream):
                self.stream.wait_event(ready)
                self._reduce(tensors)
                done = torch.cuda.Event()
                done.record(self.stream)
            for t in tensors:
                t.record_stream(self.stream)                 # the caching allocator must not reuse them before the collective ran
            self.pending.append((tensors, done))
        else:
            self._reduce(tensors)
            self.pending.append((tensors, None))

    def _reduce(self, tensors):
        for t in tensors:
            flat = t if t.is_contiguous() else None
            assert flat is not None, "gradients are reduced in place and must be contiguous"
            if self.avg:
                dist.all_reduce(t, op=dist.ReduceOp.AVG, group=self.group)
            else:
                dist.all_reduce(t, group=self.group)
                t.div_(self.world)

    def wait(self):
        """Order the current stream after every submitted collective; returns the reduced tensors in submission order."""
        out = []
        for tensors, done in self.pending:
            if done is not None:
                torch.cuda.current_stream().wait_event(done)
            out.extend(tensors)
        self.pending = []
        return out


def shard_range(total, rank, world):
    """Contiguous [begin, end) share of `total` items for `rank` (the first total % world ranks get one more)."""
    base, rem = divmod(total, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)
