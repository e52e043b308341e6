"""Argument checks of the Python front-end (deep8_b200/ops.py) that must fire before anything is launched: a
caller-supplied output of the wrong shape, dtype or layout would otherwise become an out-of-bounds device write.
CPU only: the contexts here carry a library stub whose compute entry points fail the test when reached."""
import pytest
import torch

from deep8_b200 import ops


class _NoLaunchLib:
    """Answers the two shape helpers (host arithmetic, deep8/src/nodes/Conv2d.cpp:47-63, DeConv2d.cpp:36-52) and refuses
    everything else."""

    @staticmethod
    def d8k_conv2d_out_dim(size, f, stride, dilation, covered):
        real = f + (f - 1) * (dilation - 1)
        return (size - 1) // stride + 1 if covered else (size - real) // stride + 1

    @staticmethod
    def d8k_deconv2d_out_dim(size, f, stride, covered):
        return (size - 1) * stride + 1 if covered else (size - 1) * stride + f

    def __getattr__(self, name):
        def refuse(*a, **k):
            raise AssertionError("%s was reached: the argument check did not fire" % name)
        return refuse


@pytest.fixture
def c():
    ctx = ops.Context.__new__(ops.Context)
    ctx.lib, ctx.h = _NoLaunchLib(), None
    return ctx


def test_out_accepts_the_computed_shape_only():
    like = torch.zeros((2, 3, 4), dtype=torch.float16)
    assert ops._out(None, (2, 3, 5), like).shape == (2, 3, 5)
    ok = torch.empty((2, 3, 5), dtype=torch.float16)
    assert ops._out(ok, (2, 3, 5), like) is ok
    with pytest.raises(ValueError):
        ops._out(torch.empty((2, 3, 4), dtype=torch.float16), (2, 3, 5), like)
    with pytest.raises(ValueError):
        ops._out(torch.empty((2, 3, 5), dtype=torch.float32), (2, 3, 5), like)
    with pytest.raises(ValueError):
        ops._out(torch.empty((2, 5, 3), dtype=torch.float16).transpose(1, 2), (2, 3, 5), like)


def test_matmul_outputs_are_checked(c):
    x, y = torch.zeros((2, 8, 4)), torch.zeros((1, 4, 6))
    with pytest.raises(ValueError):
        c.matmul_forward(x, y, out=torch.zeros((2, 8, 5)))
    with pytest.raises(ValueError):
        c.matmul_forward(x, y, out=torch.zeros((2, 8, 6), dtype=torch.float16))
    with pytest.raises(ValueError):
        c.matmul_forward_bias(x, y, torch.zeros(6), out=torch.zeros((1, 8, 6)))
    with pytest.raises(ValueError):
        c.add_bias(x, torch.zeros(4), out=torch.zeros((2, 8, 3)))
    with pytest.raises(ValueError):
        c.relu_forward(x, out=torch.zeros((2, 8, 5)))


def test_conv_outputs_are_checked(c):
    x, w = torch.zeros((2, 9, 9, 8)), torch.zeros((4, 3, 3, 8))
    with pytest.raises(ValueError):
        c.conv2d_forward(x, w, True, (1, 1), (1, 1), out=torch.zeros((2, 9, 9, 5)))
    with pytest.raises(ValueError):
        c.conv2d_forward(x, w, False, (1, 1), (1, 1), out=torch.zeros((2, 9, 9, 4)))   # not covered: 7 x 7
    with pytest.raises(ValueError):
        c.deconv2d_forward(x, w, True, (2, 2), out=torch.zeros((2, 18, 18, 4)))         # covered: 17 x 17


def test_scattered_gradient_arguments_are_checked(c):
    x, dz = torch.zeros((1, 64, 256), dtype=torch.float16), torch.zeros((1, 64, 32), dtype=torch.float16)
    blocks = [1 << 20, 2 << 20]
    with pytest.raises(ValueError):
        c.matmul_grad_y_scatter(x, 48, dz, blocks, 128)          # dz has 32 columns, not 48
    with pytest.raises(ValueError):
        c.matmul_grad_y_scatter(x, 32, dz, blocks, 100)          # row blocks are multiples of 128
    with pytest.raises(ValueError):
        c.matmul_grad_y_scatter(x, 32, dz, blocks[:1], 128)      # one block of 128 rows cannot hold 256
    with pytest.raises(ValueError):
        c.matmul_grad_y_scatter(x, 32, torch.zeros((1, 63, 32), dtype=torch.float16), blocks, 128)
