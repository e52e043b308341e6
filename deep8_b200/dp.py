"""Batch sharding of the path over the GPUs of one box (one process per GPU, torch.distributed).

The path shards on the batch (row) dimension: forward outputs and the gradients of per-sample operands stay on the rank
that owns the samples; operands shared by every sample (a batch-1 MatrixMultiply operand, a Conv2d/DeConv2d filter) are
replicated and their gradients - sums over the batch - are completed with one all-reduce (sum) per gradient tensor.
The reference has no multi-device support (its Executor pins device 0, deep8/src/model/Executor.cu:6-8); this is the
only exchange step the path needs.  NCCL on GPUs; the same code runs on gloo for the CPU tests.
"""
import torch.distributed as dist


def shard_range(total, world, rank):
    """Rows [lo, hi) of `total` owned by `rank`: contiguous, sizes differing by at most one."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank %d outside world of %d" % (rank, world))
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class GradientSync:
    """All-reduce (sum) of replicated-operand gradients, started as soon as each is complete so that the transfer
    overlaps the rest of the backward pass; wait() before the gradients are read."""

    def __init__(self, group=None):
        self.group = group
        self.pending = []

    def start(self, grad):
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            self.pending.append(dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        return grad

    def wait(self):
        for w in self.pending:
            w.wait()
        self.pending = []
