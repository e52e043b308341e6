"""Writes tests/golden/*.npz from the reference's own CPU code (oracle/_ref/libd8ref.so, built by oracle/Makefile from the
unmodified reference sources with the reference's flags).  Run where the reference tree is present:

    python tests/golden/make_golden.py

Only square geometries (equal strides, dilations, filter sides and image sides) are recorded: the reference's CPU path
hands its height padding to Eigen's width argument (deep8/src/math/Conv2d.cpp:352-353) and returns garbage for
non-square gradients, so for those the index rule of its GPU kernels (restated in oracle/d8_oracle.c) is the specification.

Each file holds the seeded inputs' seeds/shapes and the reference's outputs (float32): forward, gradient of x and
gradient of y with zero-initialised gradients.  Inputs are regenerated from the seeds by tests/cases.py.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import cases  # noqa: E402
from oracle import pyoracle  # noqa: E402

GOLDEN_MATMUL = [((3, 17, 5), (3, 5, 9)), ((1, 40, 24), (4, 24, 56)), ((2, 129, 65), (1, 65, 33)), ((1, 30, 20), (5, 20, 1))]
GOLDEN_CONV = [((1, 9, 9, 3), (5, 3, 3, 3), True, (1, 1), (1, 1)), ((2, 10, 10, 8), (4, 3, 3, 8), False, (2, 2), (1, 1)),
               ((2, 12, 12, 16), (8, 4, 4, 16), True, (2, 2), (2, 2))]
GOLDEN_DECONV = [((2, 7, 7, 16), (8, 4, 4, 16), True, (2, 2)), ((1, 6, 6, 3), (2, 3, 3, 3), False, (2, 2)),
                 ((2, 6, 6, 8), (4, 4, 4, 8), False, (3, 3))]


def main():
    pyoracle.build(ref=True)
    ref = pyoracle.Reference()
    out = {}
    for i, (xs, ys) in enumerate(GOLDEN_MATMUL):
        x, y = cases.uniform(100 + i, xs), cases.uniform(200 + i, ys)
        z = ref.matmul_forward(x, y)
        dz = cases.normal(300 + i, z.shape)
        out["matmul%d" % i] = dict(xs=xs, ys=ys, seeds=(100 + i, 200 + i, 300 + i), z=z, dx=ref.matmul_grad_x(x, y, dz),
                                   dy=ref.matmul_grad_y(x, y, dz))
    for i, (xs, ws, cov, st, dil) in enumerate(GOLDEN_CONV):
        x, w = cases.uniform(400 + i, xs), cases.normal(500 + i, ws, 0.2)
        z = ref.conv2d_forward(x, w, cov, st, dil)
        dz = cases.normal(600 + i, z.shape)
        out["conv%d" % i] = dict(xs=xs, ys=ws, covered=cov, stride=st, dilation=dil, seeds=(400 + i, 500 + i, 600 + i), z=z,
                                 dx=ref.conv2d_grad_x(x, w, dz, cov, st, dil), dy=ref.conv2d_grad_y(x, w, dz, cov, st, dil))
    for i, (xs, ws, cov, st) in enumerate(GOLDEN_DECONV):
        x, w = cases.uniform(700 + i, xs), cases.normal(800 + i, ws, 0.2)
        z = ref.deconv2d_forward(x, w, cov, st)
        dz = cases.normal(900 + i, z.shape)
        out["deconv%d" % i] = dict(xs=xs, ys=ws, covered=cov, stride=st, seeds=(700 + i, 800 + i, 900 + i), z=z,
                                   dx=ref.deconv2d_grad_x(x, w, dz, cov, st), dy=ref.deconv2d_grad_y(x, w, dz, cov, st))
    for name, d in out.items():
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **{k: np.asarray(v) for k, v in d.items()})
        print(name, {k: np.asarray(v).shape for k, v in d.items() if k in ("z", "dx", "dy")})


if __name__ == "__main__":
    main()
