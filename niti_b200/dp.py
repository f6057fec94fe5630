"""Data-parallel plumbing for the integer training step: batch sharding and the flat int32
gradient bucket that is summed across ranks.

The only exchange of a data-parallel NITI step is the sum of the int32 weight-gradient
accumulators (integer addition is associative, so the result does not depend on the reduction
order); every rank then applies the identical integer update and replicas stay bit-identical.
Nothing in this module touches CUDA: it works on whatever device its tensors live on, which is
how the multi-rank logic is tested with the gloo backend on CPU.
"""
import torch
import torch.distributed as dist


def shard_range(global_batch, rank, world):
    """Contiguous shard [lo, hi) of the batch owned by ``rank``; sizes differ by at most one."""
    base, rem = divmod(global_batch, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


class GradBucket:
    """One flat int32 buffer with a 16-byte-aligned view per weight tensor."""

    def __init__(self, shapes, device, flat=None):
        """``flat``: an int32 tensor to adopt as the bucket (a region of peer-visible memory, say) instead of a new one."""
        self.shapes = [tuple(s) for s in shapes]
        self.offsets = []
        off = 0
        for s in self.shapes:
            self.offsets.append(off)
            n = 1
            for d in s:
                n *= d
            off += (n + 3) // 4 * 4
        if flat is None:
            flat = torch.zeros(off, dtype=torch.int32, device=device)
        assert flat.dtype == torch.int32 and flat.numel() == off and flat.is_contiguous()
        self.flat = flat
        self.views = []
        for s, o in zip(self.shapes, self.offsets):
            n = 1
            for d in s:
                n *= d
            self.views.append(self.flat[o:o + n].view(s))

    @staticmethod
    def numel_for(shapes):
        """Length of the flat buffer that __init__ lays out for `shapes`."""
        off = 0
        for s in shapes:
            n = 1
            for d in s:
                n *= d
            off += (n + 3) // 4 * 4
        return off

    def nbytes(self):
        return self.flat.numel() * 4

    def allreduce_(self, group=None):
        """Sum over ranks, in place (NCCL over NVLink on GPUs, gloo on CPU)."""
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
        return self.flat

    def comm_groups(self, min_bytes=4 << 20):
        """Contiguous runs of layers to all-reduce together, in the order their gradients become ready in the
        backward pass (last layer first); small neighbours are merged so no message is tiny.  Returns
        [(first_layer, last_layer, flat_start, flat_end)] with first_layer the one that is ready LAST."""
        groups, hi = [], len(self.shapes) - 1
        while hi >= 0:
            lo = hi
            end = self.flat.numel() if hi == len(self.shapes) - 1 else self.offsets[hi + 1]
            while lo > 0 and (end - self.offsets[lo]) * 4 < min_bytes:
                lo -= 1
            groups.append((lo, hi, self.offsets[lo], end))
            hi = lo - 1
        return groups

    def checksum(self):
        """Order-independent digest used to assert that replicas hold identical values."""
        f = self.flat.to(torch.int64)
        return int(f.sum().item()), int((f * (torch.arange(f.numel(), device=f.device) % 8191 + 1)).sum().item())
