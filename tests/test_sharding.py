"""CPU tests of the multi-rank host logic on the gloo backend (world size 2): a batch-sharded MatrixMultiply /
Conv2d step whose replicated-operand gradients are all-reduced equals the single-rank step on the whole batch.
The per-rank arithmetic here is the CPU oracle: these tests cover sharding and the exchange step, not the kernels."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_partitions():
    from deep8_b200.dp import shard_range
    for total in (0, 1, 7, 64, 65536):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from deep8_b200.dp import GradientSync, shard_range
    from oracle import pyoracle
    o = pyoracle.Restated()
    # MatrixMultiply with a broadcast weight: x [8, 16, 12] sharded on the batch, y [1, 12, 10] replicated
    x, y = cases.uniform(1, (8, 16, 12)), cases.uniform(2, (1, 12, 10))
    dz = cases.normal(3, (8, 16, 10))
    lo, hi = shard_range(8, world, rank)
    xs, dzs = np.ascontiguousarray(x[lo:hi]), np.ascontiguousarray(dz[lo:hi])
    z = o.matmul_forward(xs, y)
    dx = o.matmul_grad_x(xs, y, dzs)
    dy = torch.from_numpy(o.matmul_grad_y(xs, y, dzs))
    # Conv2d filter gradient, images sharded on the batch
    cx, cw = cases.uniform(4, (4, 6, 6, 3)), cases.normal(5, (2, 3, 3, 3), 0.3)
    cz = o.conv2d_forward(cx, cw, True, (1, 1), (1, 1))
    cdz = cases.normal(6, cz.shape)
    clo, chi = shard_range(4, world, rank)
    cdw = torch.from_numpy(o.conv2d_grad_y(np.ascontiguousarray(cx[clo:chi]), cw, np.ascontiguousarray(cdz[clo:chi]), True, (1, 1), (1, 1)))
    sync = GradientSync()
    sync.start(dy)
    sync.start(cdw)
    sync.wait()
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), z=z, dx=dx, dy=dy.numpy(), cdw=cdw.numpy(), lo=lo, hi=hi)
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_step_equals_whole_batch(tmp_path, restated):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    x, y = cases.uniform(1, (8, 16, 12)), cases.uniform(2, (1, 12, 10))
    dz = cases.normal(3, (8, 16, 10))
    z, dx, dy = restated.matmul_forward(x, y), restated.matmul_grad_x(x, y, dz), restated.matmul_grad_y(x, y, dz)
    cx, cw = cases.uniform(4, (4, 6, 6, 3)), cases.normal(5, (2, 3, 3, 3), 0.3)
    cdz = cases.normal(6, restated.conv2d_forward(cx, cw, True, (1, 1), (1, 1)).shape)
    cdw = restated.conv2d_grad_y(cx, cw, cdz, True, (1, 1), (1, 1))
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    assert np.array_equal(np.concatenate([p["z"] for p in parts]), z)        # per-sample outputs need no exchange
    assert np.array_equal(np.concatenate([p["dx"] for p in parts]), dx)
    for p in parts:                                                          # every rank holds the full sums
        assert cases.rel_max(p["dy"], dy) < 1e-6
        assert cases.rel_max(p["cdw"], cdw) < 1e-6


def test_batch_shares_follow_the_measured_speeds():
    """bench.py's split of the global batch over GPUs of unequal speed: shares sum to the batch, are multiples of 256 rows,
    give a faster rank at least as many rows as a slower one, and never predict a slower step than the equal split."""
    sys.path.insert(0, ROOT)
    import bench
    for ms in ([5.0, 5.0], [4.46, 5.48], [4.7, 4.9, 5.0, 5.1], [4.7, 4.9, 5.0, 5.1, 5.2, 4.8, 5.3, 4.95], [5.0] * 8):
        world = len(ms)
        rows = bench.balance_rows(ms, 8192 * world)
        assert sum(rows) == 8192 * world and all(r % 256 == 0 and r > 0 for r in rows)
        for a in range(world):
            for b in range(world):
                if ms[a] < ms[b]:
                    assert rows[a] >= rows[b]
        predict = lambda r, k: ms[k] * bench.step_cost(r) / bench.step_cost(8192)
        assert max(predict(rows[k], k) for k in range(world)) <= max(ms) + 1e-9
    assert bench.balance_rows([5.0, 5.0, 5.0], 8192 * 3) == [8192] * 3
