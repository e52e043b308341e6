"""The gradient exchange over peer memory (include/d8k.h d8k_peer_* / d8k_sum_shards, deep8_b200.dp.PeerAllReduce).

CPU: the shard and rotation plans.  GPU, one device: the fixed-order sum kernel against numpy, flags (a signal that
arrives, and a wait on a flag nothing sets, which must end by itself with the status word set), copies.  GPU, two
devices (skipped on a one-GPU box): two processes exchange a gradient and each compares the result with the sum
computed from both partials on the host.
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


# ------------------------------------------------------------------------------------------------ CPU: plans
def test_gradient_shards_partition_and_alignment():
    from deep8_b200.dp import gradient_shards
    for numel in (1, 100, 1000, 4096 * 16384, 12345679):
        for world in (1, 2, 3, 8, 16):
            spans = gradient_shards(numel, world)
            assert len(spans) == world and spans[0][0] == 0 and spans[-1][1] == numel
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(lo % 128 == 0 or lo == numel for lo, _ in spans)
            assert all(hi - lo <= spans[0][1] - spans[0][0] for lo, hi in spans)  # slot 0 is the largest: staging size


def test_peer_rotation_is_a_permutation_every_round():
    from deep8_b200.dp import peer_rotation
    for world in (2, 3, 4, 8):
        orders = [peer_rotation(world, r) for r in range(world)]
        for r, o in enumerate(orders):
            assert sorted(o) == [q for q in range(world) if q != r]
        for k in range(world - 1):
            assert sorted(o[k] for o in orders) == list(range(world))  # no GPU is visited twice in one round


# ------------------------------------------------------------------------------------------------ CPU: the protocol on host memory
class _HostContext:
    """Stands in for deep8_b200.Context in the protocol test: "device memory" is POSIX shared memory that the other
    rank maps, flags are words in it, and every call runs at once on the calling process - so the order of signals,
    waits, copies and sums that PeerAllReduce issues is executed for real by two processes, only not on GPUs."""

    def __init__(self):
        self.blocks = {}
        self.timeouts = 0

    def peer_alloc(self, nbytes):
        import ctypes
        from multiprocessing import shared_memory
        shm = shared_memory.SharedMemory(create=True, size=nbytes)
        shm.buf[:nbytes] = bytes(nbytes)
        addr = ctypes.addressof(ctypes.c_char.from_buffer(shm.buf))
        self.blocks[addr] = shm
        return addr, shm.name.encode().ljust(64, b"\0")

    def peer_open(self, handle):
        import ctypes
        from multiprocessing import shared_memory
        shm = shared_memory.SharedMemory(name=handle.rstrip(b"\0").decode())
        addr = ctypes.addressof(ctypes.c_char.from_buffer(shm.buf))
        self.blocks[addr] = shm
        return addr

    def peer_close(self, ptr):
        self.blocks.pop(ptr)  # the mapping lives until the process exits: ctypes views pin the buffer

    def peer_free(self, ptr):
        self.blocks.pop(ptr).unlink()

    def peer_signal(self, flags, value):
        import ctypes
        for f in flags:
            ctypes.c_uint32.from_address(f).value = value

    def peer_wait(self, flags, value, timeout_ms):
        import ctypes
        import time
        t0 = time.time()
        for f in flags:
            while ctypes.c_int32(ctypes.c_uint32.from_address(f).value - value).value < 0:
                if (time.time() - t0) * 1e3 > timeout_ms:
                    self.timeouts += 1
                    return
                time.sleep(0.0005)

    def peer_copy(self, dst, src, nbytes):
        import ctypes
        ctypes.memmove(dst, src, nbytes)

    @staticmethod
    def _f16(addr, count):
        import ctypes
        return np.ctypeslib.as_array((ctypes.c_uint16 * count).from_address(addr)).view(np.float16)

    def sum_shards(self, dtype, out, srcs, count, sgd=None, copies=None, adam=None):
        assert adam is None, "the host stand-in covers the plain sum and the SGD step"
        acc = np.zeros(count, dtype=np.float32)
        for a in srcs:
            acc = acc + self._f16(a, count).astype(np.float32)
        g = acc.astype(np.float16)
        if out:
            self._f16(out, count)[:] = g
        if sgd is not None:
            w, alpha, beta = sgd
            wv = self._f16(w, count)
            wv[:] = (g.astype(np.float32) * np.float32(alpha) + wv.astype(np.float32) * np.float32(beta)).astype(np.float16)
            g = wv.copy()
        for a in copies or []:
            self._f16(a, count)[:] = g

    def matmul_grad_y_scatter(self, x, yc, dz, row_blocks, block_rows):
        dy = (x[0].numpy().astype(np.float32).T @ dz[0].numpy().astype(np.float32)).astype(np.float16)
        for k, addr in enumerate(row_blocks):
            rows = dy[k * block_rows:(k + 1) * block_rows]
            self._f16(addr, rows.size)[:] = rows.reshape(-1)


class _HostRuntime:
    def event(self):
        return None

    def record_current(self, event):
        pass

    def record(self, event, stream):
        pass

    def stream_wait(self, stream, event):
        pass

    def current_wait(self, event):
        pass

    def view(self, ptr, shape, dtype, device):
        n = int(np.prod(shape))
        return torch.from_numpy(_HostContext._f16(ptr, n)).view(*shape)

    def element_size(self, dtype):
        return 2

    def synchronize(self):
        pass


def _protocol_worker(rank, world, port, out_dir, gather="copy"):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    from deep8_b200.dp import PeerAllReduce
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = _HostContext()
    ok = True
    # copy-engine variant: partial -> pull -> sum -> push
    numel = 5000
    ar = PeerAllReduce(ctx, ctx, None, numel, torch.float16, "cpu", runtime=_HostRuntime(), timeout_ms=5000.0, gather=gather)
    for s in range(3):
        parts = [torch.from_numpy(np.random.default_rng(10 * s + q).standard_normal(numel).astype(np.float16)) for q in range(world)]
        ar.before_write()
        ar.partial.copy_(parts[rank])
        ar.start()
        ar.finish()
        acc = np.zeros(numel, dtype=np.float32)
        for q in range(world):
            acc = acc + parts[q].numpy().astype(np.float32)
        ok = ok and np.array_equal(ar.result.numpy(), acc.astype(np.float16))
    ar.close()
    # scattered variant: each rank's contraction writes row blocks into the owners' staging slots
    r, rows, cols = 24, 300, 40
    ar = PeerAllReduce(ctx, ctx, None, rows * cols, torch.float16, "cpu", runtime=_HostRuntime(), timeout_ms=5000.0, rows=rows, gather=gather)
    for s in range(3):
        xs = [torch.from_numpy(np.random.default_rng(100 * s + q).standard_normal((1, r, rows)).astype(np.float16)) for q in range(world)]
        dzs = [torch.from_numpy(np.random.default_rng(100 * s + 50 + q).standard_normal((1, r, cols)).astype(np.float16)) for q in range(world)]
        ar.before_write()
        ar.scatter_grad_y(xs[rank], dzs[rank])
        ar.start()
        ar.finish()
        acc = np.zeros((rows, cols), dtype=np.float32)
        for q in range(world):
            acc = acc + (xs[q][0].numpy().astype(np.float32).T @ dzs[q][0].numpy().astype(np.float32)).astype(np.float16).astype(np.float32)
        ok = ok and np.array_equal(ar.result.numpy().reshape(rows, cols), acc.astype(np.float16))
    ar.close()
    # the trainer's step inside the sum: every rank ends with the same updated weights
    ar = PeerAllReduce(ctx, ctx, None, numel, torch.float16, "cpu", runtime=_HostRuntime(), timeout_ms=5000.0, with_weights=True,
                       gather=gather)
    w0 = np.random.default_rng(7).standard_normal(numel).astype(np.float16)
    ar.weights.copy_(torch.from_numpy(w0))
    want = w0.copy()
    from deep8_b200.dp import sgd_coefficients
    alpha, beta = sgd_coefficients(0.05, 0.001)
    for s in range(3):
        parts = [np.random.default_rng(20 * s + q).standard_normal(numel).astype(np.float16) for q in range(world)]
        ar.before_write()
        ar.partial.copy_(torch.from_numpy(parts[rank]))
        ar.start(sgd=(0.05, 0.001))
        ar.finish()
        acc = np.zeros(numel, dtype=np.float32)
        for q in range(world):
            acc = acc + parts[q].astype(np.float32)
        g = acc.astype(np.float16).astype(np.float32)
        want = (g * np.float32(alpha) + want.astype(np.float32) * np.float32(beta)).astype(np.float16)
        ok = ok and np.array_equal(ar.weights.numpy(), want)
    ar.close()
    with open(os.path.join(out_dir, "rank%d.txt" % rank), "w") as f:
        f.write("%d %d" % (int(ok), ctx.timeouts))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,gather", [(2, "copy"), (3, "copy"), (2, "kernel"), (3, "kernel")])
def test_exchange_protocol_on_host_memory(tmp_path, world, gather):
    """Two and three gloo ranks run PeerAllReduce's own sequence of signals, bounded waits, copies and sums against shared
    host memory: every rank ends with the rank-ordered sum, no wait runs out, for both the copy variant and the
    scattered-contraction variant, three steps each (so the reuse hazards of staging and partial buffers are exercised)."""
    import torch.multiprocessing as mp
    mp.spawn(_protocol_worker, args=(world, _free_port(), str(tmp_path), gather), nprocs=world, join=True)
    for r in range(world):
        assert open(os.path.join(str(tmp_path), "rank%d.txt" % r)).read() == "1 0"


# ------------------------------------------------------------------------------------------------ GPU: one device
def _sum_reference(parts, dtype):
    acc = np.zeros(parts[0].shape, dtype=np.float32)
    for p in parts:  # same order, fp32 accumulation, one rounding
        acc = acc + p.astype(np.float32)
    return acc.astype(dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("nsrc,count", [(1, 1000), (2, 4096 * 33), (3, 77), (8, 1 << 20), (5, 8 * 1024 + 3)])
def test_sum_shards_matches_ordered_fp32_sum(ctx, dtype, nsrc, count):
    g = torch.Generator(device="cuda").manual_seed(nsrc * 1000 + count % 997)
    parts = [(torch.randn(count, device="cuda", generator=g) * (1 + i)).to(dtype) for i in range(nsrc)]
    out = torch.empty(count, device="cuda", dtype=dtype)
    ctx.sum_shards(dtype, out.data_ptr(), [p.data_ptr() for p in parts], count)
    torch.cuda.synchronize()
    want = _sum_reference([p.cpu().numpy() for p in parts], out.cpu().numpy().dtype)
    assert np.array_equal(out.cpu().numpy(), want)  # bit-exact: the order and the rounding are part of the contract
    assert ctx.status() == 0


@pytest.mark.gpu
def test_sum_shards_unaligned_and_in_place(ctx):
    a = torch.arange(0, 1001, device="cuda", dtype=torch.float32)
    b = torch.ones(1001, device="cuda", dtype=torch.float32)
    ctx.sum_shards(torch.float32, a[1:].data_ptr(), [a[1:].data_ptr(), b[1:].data_ptr()], 1000)  # 4-byte aligned only; out is a source
    torch.cuda.synchronize()
    assert torch.equal(a[1:], torch.arange(1, 1001, device="cuda", dtype=torch.float32) + 1)
    assert a[0].item() == 0


@pytest.mark.gpu
def test_signal_wait_copy_on_one_device(ctx):
    from deep8_b200.ops import tensor_view
    ptr, handle = ctx.peer_alloc(4096)
    assert len(handle) == 64
    try:
        words = tensor_view(ptr, (1024,), torch.int32, torch.device("cuda", 0))
        assert int(words.abs().sum().item()) == 0  # zero-filled
        ctx.peer_signal([ptr, ptr + 4, ptr + 8], 7)
        ctx.peer_wait([ptr, ptr + 4, ptr + 8], 7, 500.0)
        ctx.peer_wait([ptr], 5, 500.0)  # a flag already past the value
        assert ctx.status() == 0
        assert words[:4].tolist() == [7, 7, 7, 0]
        src = torch.arange(256, device="cuda", dtype=torch.int32)
        ctx.peer_copy(ptr + 1024, src.data_ptr(), 1024)
        torch.cuda.synchronize()
        assert torch.equal(words[256:512], src)
    finally:
        ctx.peer_free(ptr)


@pytest.mark.gpu
def test_wait_on_a_flag_nothing_sets_gives_up_and_reports(ctx):
    """The failure path without a fault: the wait runs out after its limit, the kernel returns, the status word says
    which flag was behind, the context keeps working."""
    import time
    ptr, _ = ctx.peer_alloc(256)
    try:
        ctx.peer_signal([ptr], 1)
        t0 = time.perf_counter()
        ctx.peer_wait([ptr, ptr + 4], 1, 30.0)  # flag 1 is never written
        with pytest.raises(Exception) as info:
            ctx.status()
        waited = time.perf_counter() - t0
        assert "status %d" % ((5 << 8) | 1) in str(info.value)
        assert 0.02 < waited < 5.0
        assert ctx.status() == 0  # reading the status cleared it
        x = torch.ones(64, device="cuda")
        ctx.sum_shards(torch.float32, x.data_ptr(), [x.data_ptr(), x.data_ptr()], 64)
        torch.cuda.synchronize()
        assert x.sum().item() == 128
    finally:
        ctx.peer_free(ptr)


@pytest.mark.gpu
def test_exchange_arguments_are_checked(ctx):
    from deep8_b200 import D8kError
    with pytest.raises(D8kError):
        ctx.peer_wait([0], 1, 10.0)
    ptr, _ = ctx.peer_alloc(256)
    try:
        with pytest.raises(D8kError):
            ctx.peer_wait([ptr], 1, 0.0)
        with pytest.raises(D8kError):
            ctx.peer_signal([ptr + 2], 1)
        with pytest.raises(D8kError):
            ctx.peer_signal([ptr] * 17, 1)
        with pytest.raises(TypeError):
            ctx.sum_shards(torch.int32, ptr, [ptr], 4)
    finally:
        ctx.peer_free(ptr)


@pytest.mark.gpu
def test_single_rank_exchange_is_the_identity(ctx):
    from deep8_b200.dp import PeerAllReduce
    side = torch.cuda.Stream()
    ar = PeerAllReduce(ctx, ctx, side, 1000, torch.float16, torch.device("cuda", 0))
    ar.before_write()
    ar.partial.copy_(torch.arange(1000, device="cuda").to(torch.float16))
    ar.start()
    ar.finish()
    torch.cuda.synchronize()
    assert ar.result.data_ptr() == ar.partial.data_ptr()
    assert ar.result[999].item() == 999
    ar.close()


@pytest.mark.gpu
@pytest.mark.parametrize("r,rows,cols", [(256, 512, 384), (1024, 4096, 4096), (64, 200, 72)])
def test_scattered_grad_y_equals_grad_y(ctx, r, rows, cols):
    """One GPU: the scattered epilogue with the row blocks laid end to end (or shuffled) gives matmul_grad_y's bits."""
    g = torch.Generator(device="cuda").manual_seed(rows + cols)
    x = torch.randn((1, r, rows), device="cuda", generator=g).to(torch.float16)
    dz = torch.randn((1, r, cols), device="cuda", generator=g).to(torch.float16)
    want = torch.zeros((1, rows, cols), device="cuda", dtype=torch.float16)
    ctx.matmul_grad_y(x, want, want, dz, accumulate=False)
    block = 128
    n = -(-rows // block)
    if n > 16:
        block = -(-rows // 16 // 128) * 128
        n = -(-rows // block)
    pool = torch.full((n, block, cols), 7.0, device="cuda", dtype=torch.float16)
    perm = list(reversed(range(n)))  # block k lands in slot perm[k]
    ctx.matmul_grad_y_scatter(x, cols, dz, [pool[perm[k]].data_ptr() for k in range(n)], block)
    torch.cuda.synchronize()
    assert ctx.status() == 0
    for k in range(n):
        lo, hi = k * block, min(rows, (k + 1) * block)
        assert torch.equal(pool[perm[k]][: hi - lo], want[0, lo:hi])
        assert bool((pool[perm[k]][hi - lo:] == 7.0).all())  # rows past the matrix are left alone


@pytest.mark.gpu
def test_scattered_grad_y_arguments_are_checked(ctx):
    from deep8_b200 import D8kError
    x = torch.zeros((1, 64, 256), device="cuda", dtype=torch.float16)
    dz = torch.zeros((1, 64, 128), device="cuda", dtype=torch.float16)
    out = torch.zeros((256, 128), device="cuda", dtype=torch.float16)
    # the front-end refuses bad block plans before anything is launched; the library has the same checks behind it
    with pytest.raises(ValueError):
        ctx.matmul_grad_y_scatter(x, 128, dz, [out.data_ptr()], 100)       # not a multiple of 128
    with pytest.raises(ValueError):
        ctx.matmul_grad_y_scatter(x, 128, dz, [out.data_ptr()], 128)       # one block of 128 rows does not cover 256
    import ctypes
    blocks = (ctypes.c_void_p * 1)(out.data_ptr())
    rc = ctx.lib.d8k_matmul_grad_y_scatter(ctx.h, 0, ctypes.c_void_p(x.data_ptr()), 1, 64, 256, 128, ctypes.c_void_p(dz.data_ptr()), blocks, 1, 100)
    assert rc == 1 and b"128" in ctx.lib.d8k_last_error()
    rc = ctx.lib.d8k_matmul_grad_y_scatter(ctx.h, 0, ctypes.c_void_p(x.data_ptr()), 1, 64, 256, 128, ctypes.c_void_p(dz.data_ptr()), blocks, 1, 128)
    assert rc == 1
    with pytest.raises(D8kError):
        ctx.matmul_grad_y_scatter(x, 128, dz, [out.data_ptr(), 0], 128)    # null block
    ctx.matmul_grad_y_scatter(x, 128, dz, [out.data_ptr(), out[128:].data_ptr()], 128)
    torch.cuda.synchronize()


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1000, 4096 * 33 + 5])
def test_axpby_is_the_reference_sgd_step(ctx, restated, n):
    """fp32: bit for bit the reference's x * alpha + y * beta (two roundings, no fused multiply-add); fp16 within 2e-2."""
    from oracle import pyoracle
    alpha, beta = pyoracle.sgd_coefficients(0.01, 0.0005)
    from deep8_b200.dp import sgd_coefficients
    assert sgd_coefficients(0.01, 0.0005) == (alpha, beta)
    rng = np.random.default_rng(n)
    g, w = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    want = restated.axpby(g, alpha, w, beta)
    W = torch.from_numpy(w).cuda()
    ctx.axpby(torch.from_numpy(g).cuda(), alpha, W, beta)
    torch.cuda.synchronize()
    assert np.array_equal(W.cpu().numpy(), want)
    if pyoracle.Reference.available():
        assert np.array_equal(pyoracle.Reference().axpby(g, alpha, w, beta), want)
    gh, wh = g.astype(np.float16), w.astype(np.float16)
    Wh = torch.from_numpy(wh).cuda()
    ctx.axpby(torch.from_numpy(gh).cuda(), alpha, Wh, beta)
    torch.cuda.synchronize()
    want16 = restated.axpby(gh.astype(np.float32), alpha, wh.astype(np.float32), beta)
    assert np.abs(Wh.cpu().numpy().astype(np.float32) - want16).max() <= 2e-2 * np.abs(want16).max()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_sum_shards_sgd_equals_sum_then_axpby(ctx, dtype):
    n = 8 * 1024 + 3
    g = torch.Generator(device="cuda").manual_seed(5)
    parts = [torch.randn(n, device="cuda", generator=g).to(dtype) for _ in range(4)]
    w = torch.randn(n, device="cuda", generator=g).to(dtype)
    grad = torch.empty(n, device="cuda", dtype=dtype)
    ctx.sum_shards(dtype, grad.data_ptr(), [p.data_ptr() for p in parts], n)
    w_two = ctx.axpby(grad, -0.05, w.clone(), 0.999)
    w_one, grad_one = w.clone(), torch.empty_like(grad)
    ctx.sum_shards(dtype, grad_one.data_ptr(), [p.data_ptr() for p in parts], n, sgd=(w_one.data_ptr(), -0.05, 0.999))
    torch.cuda.synchronize()
    assert torch.equal(grad_one, grad) and torch.equal(w_one, w_two)
    w_none = w.clone()
    ctx.sum_shards(dtype, None, [p.data_ptr() for p in parts], n, sgd=(w_none.data_ptr(), -0.05, 0.999))
    torch.cuda.synchronize()
    assert torch.equal(w_none, w_two)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_sum_shards_gather_writes_every_copy(ctx, dtype):
    """Sum and all-gather in one kernel: the copies (here on the same GPU) receive the sum, or the updated weights."""
    n = 8 * 1024 + 5
    g = torch.Generator(device="cuda").manual_seed(9)
    parts = [torch.randn(n, device="cuda", generator=g).to(dtype) for _ in range(3)]
    want = torch.empty(n, device="cuda", dtype=dtype)
    ctx.sum_shards(dtype, want.data_ptr(), [p.data_ptr() for p in parts], n)
    out = torch.empty_like(want)
    copies = [torch.zeros_like(want) for _ in range(3)]
    ctx.sum_shards(dtype, out.data_ptr(), [p.data_ptr() for p in parts], n, copies=[c.data_ptr() for c in copies])
    torch.cuda.synchronize()
    assert torch.equal(out, want) and all(torch.equal(c, want) for c in copies)
    w = torch.randn(n, device="cuda", generator=g).to(dtype)
    w_want = ctx.axpby(want, -0.05, w.clone(), 0.999)
    w_got = w.clone()
    ctx.sum_shards(dtype, out.data_ptr(), [p.data_ptr() for p in parts], n, sgd=(w_got.data_ptr(), -0.05, 0.999),
                   copies=[c.data_ptr() for c in copies])
    torch.cuda.synchronize()
    assert torch.equal(w_got, w_want) and all(torch.equal(c, w_want) for c in copies)
    assert ctx.status() == 0


# ------------------------------------------------------------------------------------------------ GPU: two devices
def _exchange_worker(rank, world, port, numel, steps, out_dir, gather="copy"):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    import deep8_b200
    from deep8_b200.dp import PeerAllReduce
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)  # host plumbing only: handles and barriers
    main = torch.cuda.Stream(device=dev)
    side = torch.cuda.Stream(device=dev)
    c_main, c_side = deep8_b200.Context(rank, 1 << 20), deep8_b200.Context(rank, 1 << 20)
    c_main.use_stream(main)
    c_side.use_stream(side)
    ar = PeerAllReduce(c_main, c_side, side, numel, torch.float16, dev, gather=gather)
    ok = True
    with torch.cuda.stream(main):
        for s in range(steps):
            g = torch.Generator(device=dev).manual_seed(100 * s + rank)
            mine = torch.randn(numel, device=dev, generator=g).to(torch.float16)
            ar.before_write()
            ar.partial.copy_(mine)
            ar.start()
            ar.finish()
            got = ar.result.clone()
            main.synchronize()
            acc = np.zeros(numel, dtype=np.float32)
            for q in range(world):  # rebuild every rank's partial from its seed, sum in rank order
                gq = torch.Generator(device=dev).manual_seed(100 * s + q)
                acc = acc + torch.randn(numel, device=dev, generator=gq).to(torch.float16).cpu().numpy().astype(np.float32)
            ok = ok and np.array_equal(got.cpu().numpy(), acc.astype(np.float16))
    ar.close()
    # the SGD step inside the sum: both ranks end with the same weights, equal to sum -> round -> axpby on the host
    from deep8_b200.dp import sgd_coefficients
    ar = PeerAllReduce(c_main, c_side, side, numel, torch.float16, dev, with_weights=True, gather=gather)
    alpha, beta = sgd_coefficients(0.05, 0.001)
    with torch.cuda.stream(main):
        w0 = torch.randn(numel, device=dev, generator=torch.Generator(device=dev).manual_seed(77)).to(torch.float16)
        ar.weights.copy_(w0)
        want = w0.cpu().numpy()
        for s in range(2):
            g = torch.Generator(device=dev).manual_seed(300 * s + rank)
            ar.before_write()
            ar.partial.copy_(torch.randn(numel, device=dev, generator=g).to(torch.float16))
            ar.start(sgd=(0.05, 0.001))
            ar.finish()
            main.synchronize()
            acc = np.zeros(numel, dtype=np.float32)
            for q in range(world):
                gq = torch.Generator(device=dev).manual_seed(300 * s + q)
                acc = acc + torch.randn(numel, device=dev, generator=gq).to(torch.float16).cpu().numpy().astype(np.float32)
            gsum = acc.astype(np.float16).astype(np.float32)
            want = (gsum * np.float32(alpha) + want.astype(np.float32) * np.float32(beta)).astype(np.float16)
            ok = ok and np.array_equal(ar.weights.cpu().numpy(), want)
    status = (c_main.status(), c_side.status())
    ar.close()
    # Adam inside the sum: every rank ends with the same weights, equal to sum -> round -> AdamUpdate on one GPU
    ar = PeerAllReduce(c_main, c_side, side, numel, torch.float16, dev, with_weights=True, gather=gather)
    args = (0.875, 0.9990234375, 2.0 ** -20, 0.0078125, 0.00048828125)
    with torch.cuda.stream(main):
        ar.weights.copy_(w0)
        w_ref, m_ref, v_ref = w0.clone(), torch.zeros_like(w0), torch.zeros_like(w0)
        for s in range(2):
            g = torch.Generator(device=dev).manual_seed(500 * s + rank)
            ar.before_write()
            ar.partial.copy_(torch.randn(numel, device=dev, generator=g).to(torch.float16))
            ar.start(adam=args + (s,))
            ar.finish()
            main.synchronize()
            parts = [torch.randn(numel, device=dev, generator=torch.Generator(device=dev).manual_seed(500 * s + q)).to(torch.float16)
                     for q in range(world)]
            gsum = torch.empty_like(w0)
            c_main.sum_shards(torch.float16, gsum.data_ptr(), [p.data_ptr() for p in parts], numel)
            c_main.adam_update(w_ref, gsum, m_ref, v_ref, *args, s)
            main.synchronize()
            ok = ok and torch.equal(ar.weights, w_ref)
    status = (c_main.status() | status[0], c_side.status() | status[1])
    ar.close()
    with open(os.path.join(out_dir, "rank%d.txt" % rank), "w") as f:
        f.write("%d %d %d" % (int(ok), status[0], status[1]))
    dist.destroy_process_group()


def _fused_worker(rank, world, port, r, rows, cols, steps, out_dir, gather="copy"):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    import deep8_b200
    from deep8_b200.dp import PeerAllReduce
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    main = torch.cuda.Stream(device=dev)
    side = torch.cuda.Stream(device=dev)
    c_main, c_side = deep8_b200.Context(rank), deep8_b200.Context(rank, 1 << 20)
    c_main.use_stream(main)
    c_side.use_stream(side)
    ar = PeerAllReduce(c_main, c_side, side, rows * cols, torch.float16, dev, rows=rows, gather=gather)
    ok = True

    def inputs(s, q):
        g = torch.Generator(device=dev).manual_seed(1000 * s + q)
        return (torch.randn((1, r, rows), device=dev, generator=g).to(torch.float16),
                torch.randn((1, r, cols), device=dev, generator=g).to(torch.float16))

    with torch.cuda.stream(main):
        for s in range(steps):
            x, dz = inputs(s, rank)
            ar.before_write()
            ar.scatter_grad_y(x, dz)
            ar.start()
            ar.finish()
            got = ar.result.clone().view(rows, cols)
            main.synchronize()
            acc = np.zeros((rows, cols), dtype=np.float32)
            part = torch.empty((1, rows, cols), device=dev, dtype=torch.float16)
            for q in range(world):  # every rank's partial, by the same kernel on the same inputs, summed in rank order
                xq, dzq = inputs(s, q)
                c_main.matmul_grad_y(xq, part, part, dzq, accumulate=False)
                main.synchronize()
                acc = acc + part[0].cpu().numpy().astype(np.float32)
            ok = ok and np.array_equal(got.cpu().numpy(), acc.astype(np.float16))
    status = (c_main.status(), c_side.status())
    ar.close()
    with open(os.path.join(out_dir, "rank%d.txt" % rank), "w") as f:
        f.write("%d %d %d" % (int(ok), status[0], status[1]))
    dist.destroy_process_group()


def _sgd_order_worker(rank, world, port, r, rows, cols, steps, out_dir):
    """A backward pass with the trainer's step inside the exchange, in the order the exchange requires: the gradient of x,
    which reads the weights, is enqueued BEFORE start(sgd=...).  It must equal the product with the weights as they were,
    and the weights must end as sum -> round -> x * alpha + y * beta on every rank."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch.distributed as dist
    import deep8_b200
    from deep8_b200.dp import PeerAllReduce, sgd_coefficients
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    main = torch.cuda.Stream(device=dev)
    side = torch.cuda.Stream(device=dev)
    c_main, c_side = deep8_b200.Context(rank), deep8_b200.Context(rank, 1 << 20)
    c_main.use_stream(main)
    c_side.use_stream(side)
    ar = PeerAllReduce(c_main, c_side, side, rows * cols, torch.float16, dev, rows=rows, with_weights=True)
    lr, wd = 0.05, 0.001
    alpha, beta = sgd_coefficients(lr, wd)
    ok = True

    def inputs(s, q):
        g = torch.Generator(device=dev).manual_seed(1000 * s + q)
        return (torch.randn((1, r, rows), device=dev, generator=g).to(torch.float16),
                torch.randn((1, r, cols), device=dev, generator=g).to(torch.float16))

    with torch.cuda.stream(main):
        w0 = (torch.randn(rows * cols, device=dev, generator=torch.Generator(device=dev).manual_seed(5)) * 0.1).to(torch.float16)
        ar.weights.copy_(w0)
        W = ar.weights.view(1, rows, cols)
        for s in range(steps):
            x, dz = inputs(s, rank)
            w_before = W.clone()
            ar.before_write()
            ar.scatter_grad_y(x, dz)
            dx = torch.empty_like(x)
            c_main.matmul_grad_x(x, dx, W, dz, accumulate=False)   # the last reader of the weights in this backward pass
            ar.start(sgd=(lr, wd))
            ar.finish()
            main.synchronize()
            dx_want = torch.empty_like(x)
            c_main.matmul_grad_x(x, dx_want, w_before, dz, accumulate=False)
            main.synchronize()
            ok = ok and torch.equal(dx, dx_want)
            acc = np.zeros((rows, cols), dtype=np.float32)
            part = torch.empty((1, rows, cols), device=dev, dtype=torch.float16)
            for q in range(world):
                xq, dzq = inputs(s, q)
                c_main.matmul_grad_y(xq, part, part, dzq, accumulate=False)
                main.synchronize()
                acc = acc + part[0].cpu().numpy().astype(np.float32)
            gsum = acc.astype(np.float16).astype(np.float32)
            want = (gsum * np.float32(alpha) + w_before[0].cpu().numpy().astype(np.float32) * np.float32(beta)).astype(np.float16)
            ok = ok and np.array_equal(W[0].cpu().numpy(), want)
    status = (c_main.status(), c_side.status())
    ar.close()
    with open(os.path.join(out_dir, "rank%d.txt" % rank), "w") as f:
        f.write("%d %d %d" % (int(ok), status[0], status[1]))
    dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpu_sgd_inside_exchange_after_the_last_reader_of_the_weights(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_sgd_order_worker, args=(world, _free_port(), 256, 512, 384, 3, str(tmp_path)), nprocs=world, join=True)
    for q in range(world):
        assert open(os.path.join(str(tmp_path), "rank%d.txt" % q)).read() == "1 0 0"


@pytest.mark.gpu
@pytest.mark.parametrize("gather", ["copy", "kernel"])
@pytest.mark.parametrize("r,rows,cols", [(512, 4096, 4096), (96, 200, 72)])
def test_two_gpu_fused_scatter_exchange_is_bit_exact(tmp_path, r, rows, cols, gather):
    """The contraction whose epilogue stores each row block into its owner's memory, then sum + all-gather: equal, bit
    for bit, to summing the ranks' ordinary matmul_grad_y results in rank order."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_fused_worker, args=(world, _free_port(), r, rows, cols, 3, str(tmp_path), gather), nprocs=world, join=True)
    for q in range(world):
        assert open(os.path.join(str(tmp_path), "rank%d.txt" % q)).read() == "1 0 0"


@pytest.mark.gpu
@pytest.mark.parametrize("gather", ["copy", "kernel"])
@pytest.mark.parametrize("numel", [1 << 20, 100003])
def test_two_gpu_exchange_sums_partials_bit_exactly(tmp_path, numel, gather):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_exchange_worker, args=(world, _free_port(), numel, 3, str(tmp_path), gather), nprocs=world, join=True)
    for r in range(world):
        assert open(os.path.join(str(tmp_path), "rank%d.txt" % r)).read() == "1 0 0"


@pytest.mark.gpu
def test_two_gpu_cpp_host_sums_gradients_and_trains(tmp_path):
    """The C++ host side of the multi-GPU path (Deep8::FileRendezvous, Deep8::PeerGradientSum, SGDTrainer): two processes, one
    GPU each, run tests/cpp/test_deep8_dp and compare with the CPU oracle for equality."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import subprocess
    exe = os.path.join(ROOT, "tests", "cpp", "bin", "test_deep8_dp")
    assert os.path.exists(exe), "tests/cpp/bin/test_deep8_dp is missing: run __graft_entry__.build()"
    procs = [subprocess.Popen([exe, str(tmp_path), str(r), "2"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180)[0] for p in procs]
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and ("rank %d: OK" % r) in out, out


@pytest.mark.gpu
def test_cpp_host_gradient_sum_with_one_rank(tmp_path):
    """The same program with a world of one: rendezvous, the trainer step and the oracle comparison without a peer."""
    import subprocess
    exe = os.path.join(ROOT, "tests", "cpp", "bin", "test_deep8_dp")
    assert os.path.exists(exe), "tests/cpp/bin/test_deep8_dp is missing: run __graft_entry__.build()"
    r = subprocess.run([exe, str(tmp_path), "0", "1"], capture_output=True, text=True, timeout=180)
    assert r.returncode == 0 and "rank 0: OK" in r.stdout, r.stdout + r.stderr
