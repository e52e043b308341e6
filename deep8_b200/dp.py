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


# ---------------------------------------------------------------------------------------------- exchange over peer memory
def gradient_shards(numel, world, align=128):
    """[lo, hi) element ranges, one per rank, that partition a gradient of `numel` elements; every boundary but the last
    is a multiple of `align` elements so that each shard starts on a 16-byte boundary for any element type."""
    per = -(-numel // world)
    per = -(-per // align) * align
    return [(min(k * per, numel), min((k + 1) * per, numel)) for k in range(world)]


def row_block_shards(rows, cols, world, align_rows=128):
    """(block_rows, shards): the gradient as a rows x cols matrix cut into `world` blocks of block_rows rows (a multiple of
    `align_rows`, which is what the contraction's scattered epilogue needs); shards are the blocks' [lo, hi) element
    ranges, empty for trailing ranks when there are fewer blocks than ranks."""
    per = -(-rows // world)
    block_rows = -(-per // align_rows) * align_rows
    shards = [(min(k * block_rows, rows) * cols, min((k + 1) * block_rows, rows) * cols) for k in range(world)]
    return block_rows, shards


def peer_rotation(world, rank):
    """Order in which `rank` visits its peers: rank+1, rank+2, ...  At visit k every rank talks to a different peer, so
    the transfers of one round never meet at one GPU."""
    return [(rank + k) % world for k in range(1, world)]


def sgd_coefficients(learning_rate, weight_decay):
    """(alpha, beta) with which SGDTrainer::update calls Math::AXPBY (deep8/src/trainer/SGDTrainer.cpp:13-14):
    alpha = -1 * lr and beta = 1.0 - lr * decay, the product in float, the difference in double, both stored as float."""
    import struct

    def f32(v):
        return struct.unpack("f", struct.pack("f", v))[0]

    lr, wd = f32(learning_rate), f32(weight_decay)
    return f32(-1.0 * lr), f32(1.0 - f32(lr * wd))


class CudaRuntime:
    """The pieces of torch.cuda that PeerAllReduce needs - events, stream ordering, tensors over raw addresses - behind
    one small interface, so that the protocol itself can be exercised on host memory by the CPU tests."""

    def __init__(self):
        import torch
        self.torch = torch

    def event(self):
        return self.torch.cuda.Event()

    def record_current(self, event):
        event.record(self.torch.cuda.current_stream())

    def record(self, event, stream):
        event.record(stream)

    def stream_wait(self, stream, event):
        stream.wait_event(event)

    def current_wait(self, event):
        self.torch.cuda.current_stream().wait_event(event)

    def view(self, ptr, shape, dtype, device):
        from .ops import tensor_view
        return tensor_view(ptr, shape, dtype, device)

    def element_size(self, dtype):
        return self.torch.empty((), dtype=dtype).element_size()

    def synchronize(self):
        self.torch.cuda.synchronize()


class PeerAllReduce:
    """Sum of one replicated-operand gradient over the GPUs of a box without a collective kernel.

    Each rank's contraction writes its partial gradient into `partial` (memory the peers map).  Then, on a side stream:
    the rank tells its peers the partial is ready, pulls its own shard of every peer's partial with the copy engines, adds
    the shards in rank order (fp32, one rounding - every rank would get the same bits for the same shard), pushes the
    finished shard into every peer's `result`, and waits until the other shards have arrived.  No SM moves data between
    GPUs and the three small kernels involved share SMs with whatever contraction is running, so the exchange hides
    behind the rest of the backward pass instead of competing with it.

    Waits between ranks are kernels with a time limit: a peer that never arrives sets the context's status word (read it
    with Context.status()) and the stream carries on.

        ar = PeerAllReduce(ctx_main, ctx_side, side_stream, numel, torch.float16, device)
        ar.before_write()                 # main stream: peers are done reading the previous partial
        ...contraction writes ar.partial...
        ar.start()                        # exchange runs on the side stream
        ...more work on the main stream...
        ar.finish()                       # main stream waits; ar.result holds the sum
    """

    FLAG_WORDS = 64  # per kind: one word per peer, padded

    def __init__(self, ctx_main, ctx_side, side_stream, numel, dtype, device, group=None, timeout_ms=2000.0, rows=None,
                 runtime=None, with_weights=False, gather="copy"):
        """rows: the gradient is a rows x (numel / rows) matrix to be cut into row blocks - needed for scatter_grad_y,
        where the contraction's epilogue stores each block straight into its owner's staging memory.
        runtime: CudaRuntime unless a test substitutes host memory.
        with_weights: also keep the operand itself in peer memory (`weights`), so that start(sgd=...) can apply the
        trainer's step to the shard this rank sums and send updated weights instead of gradients.
        gather: "copy" - the finished shard reaches the peers by copy-engine transfers; "kernel" - the sum kernel itself
        stores every finished 16 bytes into the peers' buffers (sum and all-gather in one kernel, no copy engine)."""
        if gather not in ("copy", "kernel"):
            raise ValueError("gather is 'copy' or 'kernel'")
        self.gather = gather
        self.rt = runtime if runtime is not None else CudaRuntime()
        self.ctx_main, self.ctx_side, self.side = ctx_main, ctx_side, side_stream
        self.numel, self.dtype, self.device, self.group, self.timeout_ms = numel, dtype, device, group, timeout_ms
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        if self.world > 16:
            raise ValueError("at most 16 GPUs exchange through peer memory")
        self.esize = self.rt.element_size(dtype)
        self.rows, self.cols, self.block_rows = rows, None, None
        if rows is None:
            self.shards = gradient_shards(numel, self.world)
        else:
            if numel % rows:
                raise ValueError("numel is not a multiple of rows")
            self.cols = numel // rows
            self.block_rows, self.shards = row_block_shards(rows, self.cols, self.world)
        self.step = 0
        lo, hi = self.shards[self.rank]
        self.shard_elems = self.shards[0][1] - self.shards[0][0] if rows is None else self.block_rows * self.cols
        grad_bytes = -(-numel * self.esize // 256) * 256
        stage_bytes = -(-self.shard_elems * self.esize // 256) * 256
        # one allocation: partial | result | staging slot per rank | flags (ready, pulled, gathered)
        self.off_partial, self.off_result = 0, grad_bytes
        self.off_stage = 2 * grad_bytes
        self.off_weights = self.off_stage + self.world * stage_bytes
        self.off_flags = self.off_weights + (grad_bytes if with_weights else 0)
        self.stage_bytes = stage_bytes
        total = self.off_flags + 3 * self.FLAG_WORDS * 4
        self.base, handle = ctx_main.peer_alloc(total)
        self.peers = [None] * self.world
        self.peers[self.rank] = self.base
        if self.world > 1:
            handles = [None] * self.world
            dist.all_gather_object(handles, handle, group=group)
            for q in range(self.world):
                if q != self.rank:
                    self.peers[q] = ctx_main.peer_open(handles[q])
        self.partial = self.rt.view(self.base + self.off_partial, (numel,), dtype, device)
        self.result = self.rt.view(self.base + self.off_result, (numel,), dtype, device) if self.world > 1 else self.partial
        self.weights = self.rt.view(self.base + self.off_weights, (numel,), dtype, device) if with_weights else None
        self.order = peer_rotation(self.world, self.rank)
        self.adam_m = self.adam_v = None  # optimiser state of the owned shard, created by the first start(adam=...)
        self.e_written = self.rt.event()
        self.e_done = self.rt.event()
        if self.world > 1:
            dist.barrier(group=group)  # every rank has mapped every buffer before the first signal

    def _flag(self, owner, kind, writer):
        return self.peers[owner] + self.off_flags + (kind * self.FLAG_WORDS + writer) * 4

    def scatter_grad_y(self, x, dz):
        """The contraction and the reduce-scatter's transfer in one kernel: dy = x^T * dz (replicated y, x [b, r, rows],
        dz [b, r, cols]) with every row block stored by the epilogue into its owner's staging slot for this rank, over
        NVLink where the owner is a peer.  Replaces `contraction writes partial` + the pull phase; call before_write()
        first and start() after, as usual.  `partial` is not written in this mode."""
        if self.rows is None:
            raise ValueError("PeerAllReduce was built without rows")
        if x.shape[2] != self.rows or dz.shape[2] != self.cols:
            raise ValueError("the shape is error")
        nblocks = -(-self.rows // self.block_rows)
        if self.world == 1:
            bases = [self.base + self.off_partial]  # one block, nobody to exchange with: the result in place
        else:
            bases = [self.peers[k] + self.off_stage + self.rank * self.stage_bytes for k in range(nblocks)]
        self.ctx_main.matmul_grad_y_scatter(x, self.cols, dz, bases, self.block_rows)
        self.scattered = True

    def before_write(self):
        """Main stream: hold the next write of `partial` (or of the peers' staging slots) until every peer has consumed
        the previous step's data."""
        if self.world > 1 and self.step > 0:
            self.ctx_main.peer_wait([self._flag(self.rank, 1, q) for q in self.order], self.step, self.timeout_ms)

    def start(self, sgd=None, adam=None):
        """Call after the contraction that writes `partial` has been enqueued on the main stream.
        adam = (beta1, beta2, epsilon, learning_rate, weight_decay, steps): Math::AdamUpdate (AdamTrainer::update,
        deep8/src/trainer/AdamTrainer.cpp:9-31) runs inside the sum on the shard this rank owns, with this rank's m and v for
        that shard (`adam_m`, `adam_v`, zero at first: 1 / world of the optimiser's state per GPU), and the all-gather
        carries the updated `weights`.  Same rules as sgd.
        sgd = (learning_rate, weight_decay): the reference's SGD step (SGDTrainer::update) runs inside the sum on the shard
        this rank owns, and the all-gather carries the updated `weights`; `result` then holds only this rank's shard of
        the summed gradient.  Every rank must pass the same values; `weights` must hold the same data on every rank.
        From start(sgd=...) until finish() `weights` is being rewritten - this rank's shard by the sum kernel, the rest by
        the peers' transfers - so nothing on any stream may read it in between: enqueue start(sgd=...) only after the last
        contraction of the backward pass that reads the operand (the reference runs the whole backward pass before
        SGDTrainer::update, deep8/src/trainer/Trainer.cpp:12-32), and finish() before the next forward pass."""
        coeff = None
        if sgd is not None and adam is not None:
            raise ValueError("one trainer step per exchange: sgd or adam")
        if sgd is not None or adam is not None:
            if self.weights is None:
                raise ValueError("PeerAllReduce was built without weights")
        if sgd is not None:
            coeff = sgd_coefficients(*sgd)
        lo, hi = self.shards[self.rank]
        if adam is not None and self.adam_m is None:
            import torch
            n_own = max(hi - lo, 1)
            self.adam_m = torch.zeros(n_own, dtype=self.dtype, device=self.device)
            self.adam_v = torch.zeros(n_own, dtype=self.dtype, device=self.device)

        def adam_args(weights_addr):
            return (weights_addr, self.adam_m.data_ptr(), self.adam_v.data_ptr()) + tuple(adam)

        if self.world == 1:
            self.scattered = False
            if coeff is not None:
                self.ctx_main.sum_shards(self.dtype, None, [self.base + self.off_partial], self.numel,
                                         sgd=(self.base + self.off_weights, coeff[0], coeff[1]))
            elif adam is not None:
                self.ctx_main.sum_shards(self.dtype, None, [self.base + self.off_partial], self.numel, adam=adam_args(self.base + self.off_weights))
            return
        c, r = self.ctx_side, self.rank
        self.step += 1
        s = self.step
        self.rt.record_current(self.e_written)
        self.rt.stream_wait(self.side, self.e_written)
        lo, hi = self.shards[r]
        n = hi - lo
        c.peer_signal([self._flag(q, 0, r) for q in self.order], s)                       # my partial is ready
        c.peer_wait([self._flag(r, 0, q) for q in self.order], s, self.timeout_ms)        # so are theirs
        scattered, self.scattered = getattr(self, "scattered", False), False
        mine = self.base + self.off_result + lo * self.esize
        step = None if coeff is None else (self.base + self.off_weights + lo * self.esize, coeff[0], coeff[1])
        astep = None if adam is None else adam_args(self.base + self.off_weights + lo * self.esize)
        trained = step is not None or astep is not None
        off = (self.off_weights if trained else self.off_result) + lo * self.esize  # what the all-gather carries
        copies = [self.peers[q] + off for q in self.order] if self.gather == "kernel" else None
        if scattered:
            # every rank's epilogue has already put its block of partial sums into my staging slots
            if n > 0:
                c.sum_shards(self.dtype, mine, [self.base + self.off_stage + q * self.stage_bytes for q in range(self.world)], n, sgd=step,
                             copies=copies, adam=astep)
            c.peer_signal([self._flag(q, 1, r) for q in self.order], s)                   # my staging slots may be rewritten
        else:
            if n > 0:
                for q in self.order:                                                       # reduce-scatter: pull my shard
                    c.peer_copy(self.base + self.off_stage + q * self.stage_bytes,
                                self.peers[q] + self.off_partial + lo * self.esize, n * self.esize)
            c.peer_signal([self._flag(q, 1, r) for q in self.order], s)                   # their partials may be rewritten
            if n > 0:
                srcs = [self.base + self.off_partial + lo * self.esize if q == r else self.base + self.off_stage + q * self.stage_bytes
                        for q in range(self.world)]
                c.sum_shards(self.dtype, mine, srcs, n, sgd=step, copies=copies, adam=astep)
        if n > 0 and copies is None:
            for q in self.order:                                                           # all-gather: push the finished shard
                c.peer_copy(self.peers[q] + off, self.base + off, n * self.esize)
        c.peer_signal([self._flag(q, 2, r) for q in self.order], s)                       # my shard has been delivered
        c.peer_wait([self._flag(r, 2, q) for q in self.order], s, self.timeout_ms)        # and so have theirs
        self.rt.record(self.e_done, self.side)

    def finish(self):
        """Main stream waits for the exchange; `result` then holds the sum on every rank."""
        if self.world > 1:
            self.rt.current_wait(self.e_done)

    def close(self):
        if getattr(self, "base", None) is None:
            return
        self.rt.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)  # nobody unmaps or frees while a peer may still copy
        for q, p in enumerate(self.peers):
            if q != self.rank and p is not None:
                self.ctx_main.peer_close(p)
        if self.world > 1:
            dist.barrier(group=self.group)
        self.ctx_main.peer_free(self.base)
        self.base = None
