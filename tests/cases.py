"""Shapes and seeded inputs shared by the CPU and GPU tests.

Shape lists follow the reference's own unit tests (test/MatrixMultiplyTest.h, test/Conv2dTest.h, test/DeConv2dTest.h) and
the five benchmark configurations; the rest are edge cases (ragged extents, one channel, one pixel, broadcast batches).
Inputs come from numpy's counter-based Philox generator, so a (seed, shape) pair names one array everywhere.
"""
import numpy as np


def rng(seed):
    return np.random.Generator(np.random.Philox(seed))


def uniform(seed, shape, lo=-1.0, hi=1.0, dtype=np.float32):
    return rng(seed).uniform(lo, hi, size=shape).astype(dtype)


def normal(seed, shape, std=1.0, dtype=np.float32):
    return (rng(seed).standard_normal(size=shape) * std).astype(dtype)


def small_ints(seed, shape, hi=50, dtype=np.float32):
    """The reference's test data: rand() % 50 stored as float (test/TestUtils.h:13-40)."""
    return rng(seed).integers(0, hi, size=shape).astype(dtype)


# (x shape, y shape): [batch, rows, cols]
MATMUL_REFERENCE_TESTS = [
    ((10, 400, 200), (1, 200, 300)),   # test/MatrixMultiplyTest.h:8-43  (y broadcast: batch folds into rows)
    ((1, 300, 100), (10, 100, 1)),     # test/MatrixMultiplyTest.h:45-86 (x broadcast, matrix-vector branch)
]
MATMUL_EDGE = [
    ((3, 17, 5), (3, 5, 9)),           # general per-batch branch
    ((1, 40, 24), (4, 24, 56)),        # x broadcast, gradient of x sums over the batch
    ((1, 1, 1), (1, 1, 1)),
    ((2, 129, 65), (1, 65, 33)),       # one past the tile edges
    ((1, 128, 64), (1, 64, 128)),      # exactly one tile
    ((3, 50, 72), (1, 72, 1)),         # y is one column, batch 1: the matrix-vector kernels (16-byte rows)
    ((1, 257, 1001), (1, 1001, 1)),    # the same with rows that are not 16-byte multiples
    ((2, 37, 4096), (1, 4096, 1)),     # rows of 8 KB and more take a CTA each
    ((1, 64, 128), (6, 128, 1)),       # x broadcast, y a batch of columns: one contraction Y * X^T through TMA
]
MATMUL_CFG1 = ((1, 256, 512), (1, 512, 128))
MATMUL_CFG2 = ((64, 128, 256), (1, 256, 256))

# (x shape, w shape, covered, stride, dilation)
CONV_REFERENCE_TESTS = [
    ((2, 32, 32, 64), (32, 4, 4, 64), True, (2, 2), (2, 2)),    # test/Conv2dTest.h:8-90
    ((2, 32, 32, 64), (32, 5, 5, 64), True, (1, 1), (1, 1)),    # test/Conv2dTest.h:92-246
    ((2, 32, 32, 64), (32, 4, 4, 64), False, (2, 2), (2, 2)),   # test/Conv2dTest.h:250-334
]
CONV_EDGE = [
    ((1, 9, 9, 3), (5, 3, 3, 3), True, (1, 1), (1, 1)),         # 3 channels: taps are not 16-byte multiples
    ((2, 7, 10, 8), (4, 3, 2, 8), False, (1, 2), (1, 1)),       # non-square everything, not covered
    ((1, 1, 1, 16), (8, 1, 1, 16), True, (1, 1), (1, 1)),       # one pixel, 1x1 filter
    ((3, 11, 11, 20), (70, 3, 3, 20), True, (2, 2), (1, 1)),    # 70 output channels: ragged N
    # channel counts the TMA im2col producer takes (multiples of 32 / 64), with nothing square or symmetric
    ((2, 9, 13, 32), (32, 3, 2, 32), False, (1, 2), (2, 1)),
    ((1, 10, 7, 64), (64, 2, 3, 64), True, (2, 1), (1, 2)),
    ((3, 6, 5, 64), (96, 3, 3, 64), True, (1, 1), (1, 1)),      # 96 filters: the last tile of N is half empty
]
CONV_CFG3 = ((32, 56, 56, 64), (64, 3, 3, 64), True, (1, 1), (1, 1))

# (x shape, w shape, covered, stride)
DECONV_REFERENCE_TESTS = [
    ((2, 32, 32, 64), (32, 4, 4, 64), False, (3, 3)),           # test/DeConv2dTest.h:8-93
    ((2, 32, 32, 64), (32, 4, 4, 64), True, (3, 3)),            # test/DeConv2dTest.h:95-267
]
DECONV_EDGE = [
    ((2, 7, 7, 16), (8, 4, 4, 16), True, (2, 2)),
    ((2, 7, 7, 16), (8, 3, 3, 16), False, (2, 2)),
    ((2, 7, 7, 16), (8, 3, 3, 16), True, (1, 1)),
    ((1, 5, 6, 3), (2, 2, 3, 3), False, (2, 1)),
    ((2, 6, 9, 64), (64, 3, 2, 64), False, (1, 1)),             # stride 1: every contraction goes through TMA im2col
    ((2, 5, 8, 32), (32, 2, 3, 32), True, (2, 3)),              # unequal strides
    ((1, 4, 4, 32), (32, 2, 2, 32), False, (3, 3)),             # stride beyond the filter: every third output row and column is zero
    ((2, 6, 6, 64), (64, 5, 5, 64), True, (2, 2)),              # 3 + 2 taps per axis in the two residue classes
]
DECONV_CFG4 = ((16, 14, 14, 256), (128, 4, 4, 256), True, (2, 2))   # output 27x27, what the reference's shape rule yields


def rel_max(got, want):
    """max |got - want| / max |want| : the tolerance measure of the parity tests."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    denom = max(np.abs(want).max(), 1e-30)
    return float(np.abs(got - want).max() / denom)


def rel_fro(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm((got - want).ravel()) / max(np.linalg.norm(want.ravel()), 1e-30))
