"""CPU tests: the restated oracle against the reference's golden vectors and (where built) the reference's own CPU code;
the shape rules; and that the C-ABI library loads and exports every symbol include/d8k.h declares."""
import glob
import os
import re

import numpy as np
import pytest

import cases

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))
# float32 golden outputs come from Eigen's float accumulation; the oracle is the correctly rounded sum.
F32_GOLDEN_TOL = 2e-6


def run_all(impl, kind, x, w, dz_seed, meta):
    """(z, dx, dy) of one operator on one implementation; dz is drawn after z's shape is known."""
    if kind == "matmul":
        z = impl.matmul_forward(x, w)
        dz = cases.normal(dz_seed, z.shape, dtype=x.dtype)
        return z, impl.matmul_grad_x(x, w, dz), impl.matmul_grad_y(x, w, dz)
    if kind == "conv":
        cov, st, dil = meta
        z = impl.conv2d_forward(x, w, cov, st, dil)
        dz = cases.normal(dz_seed, z.shape, dtype=x.dtype)
        return z, impl.conv2d_grad_x(x, w, dz, cov, st, dil), impl.conv2d_grad_y(x, w, dz, cov, st, dil)
    cov, st = meta
    z = impl.deconv2d_forward(x, w, cov, st)
    dz = cases.normal(dz_seed, z.shape, dtype=x.dtype)
    return z, impl.deconv2d_grad_x(x, w, dz, cov, st), impl.deconv2d_grad_y(x, w, dz, cov, st)


def load_golden(path):
    g = np.load(path)
    name = os.path.basename(path)[:-4]
    kind = re.match(r"[a-z]+", name).group(0)
    xs, ys = tuple(int(v) for v in g["xs"]), tuple(int(v) for v in g["ys"])
    s0, s1, s2 = (int(v) for v in g["seeds"])
    x = cases.uniform(s0, xs)
    w = cases.uniform(s1, ys) if kind == "matmul" else cases.normal(s1, ys, 0.2)
    if kind == "matmul":
        meta = None
    elif kind == "conv":
        meta = (bool(g["covered"]), tuple(int(v) for v in g["stride"]), tuple(int(v) for v in g["dilation"]))
    else:
        meta = (bool(g["covered"]), tuple(int(v) for v in g["stride"]))
    return kind, x, w, s2, meta, (g["z"], g["dx"], g["dy"])


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_restated_matches_golden(restated, path):
    kind, x, w, dz_seed, meta, want = load_golden(path)
    got = run_all(restated, kind, x, w, dz_seed, meta)
    for name, g, r in zip(("z", "dx", "dy"), got, want):
        assert g.shape == r.shape
        assert cases.rel_max(g, r) <= F32_GOLDEN_TOL, name


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_golden_regenerates_from_reference(reference, path):
    """Where the reference library is built, the committed vectors are what it produces today."""
    kind, x, w, dz_seed, meta, want = load_golden(path)
    got = run_all(reference, kind, x, w, dz_seed, meta)
    for g, r in zip(got, want):
        assert cases.rel_max(g, r) <= 1e-6


def _exact(restated, reference, kind, xs, ws, meta, hi=50):
    x, w = cases.small_ints(1, xs, hi), cases.small_ints(2, ws, hi)
    if kind == "matmul":
        zshape = restated.matmul_forward(x, w).shape
    elif kind == "conv":
        zshape = restated.conv2d_forward(x, w, *meta).shape
    else:
        zshape = restated.deconv2d_forward(x, w, *meta).shape
    dz = cases.small_ints(3, zshape, hi)

    def all3(impl):
        if kind == "matmul":
            return impl.matmul_forward(x, w), impl.matmul_grad_x(x, w, dz), impl.matmul_grad_y(x, w, dz)
        if kind == "conv":
            return impl.conv2d_forward(x, w, *meta), impl.conv2d_grad_x(x, w, dz, *meta), impl.conv2d_grad_y(x, w, dz, *meta)
        return impl.deconv2d_forward(x, w, *meta), impl.deconv2d_grad_x(x, w, dz, *meta), impl.deconv2d_grad_y(x, w, dz, *meta)

    for a, b in zip(all3(restated), all3(reference)):
        assert np.array_equal(a, b)  # the reference's tests assert equality on integer-valued data


@pytest.mark.parametrize("xs,ys", cases.MATMUL_REFERENCE_TESTS + cases.MATMUL_EDGE)
def test_matmul_restated_equals_reference_on_integers(restated, reference, xs, ys):
    _exact(restated, reference, "matmul", xs, ys, None)


def _square(xs, ws, st, dil=(1, 1)):
    """The reference's CPU path is only self-consistent for square geometries: it hands its height padding to Eigen's
    width argument (deep8/src/math/Conv2d.cpp:352-353) and its gradients return garbage otherwise.  For the rest the
    index rule of its GPU kernels, which the restatement follows, is the specification."""
    return xs[1] == xs[2] and ws[1] == ws[2] and st[0] == st[1] and dil[0] == dil[1]


@pytest.mark.parametrize("xs,ws,cov,st,dil", [c for c in cases.CONV_REFERENCE_TESTS + cases.CONV_EDGE if _square(c[0], c[1], c[3], c[4])])
def test_conv_restated_equals_reference_on_integers(restated, reference, xs, ws, cov, st, dil):
    _exact(restated, reference, "conv", xs, ws, (cov, st, dil), hi=20)


@pytest.mark.parametrize("xs,ws,cov,st", [c for c in cases.DECONV_REFERENCE_TESTS + cases.DECONV_EDGE if _square(c[0], c[1], c[3])])
def test_deconv_restated_equals_reference_on_integers(restated, reference, xs, ws, cov, st):
    _exact(restated, reference, "deconv", xs, ws, (cov, st), hi=20)


def test_float64_path_agrees(restated, reference):
    """The reference's double CPU path (MatrixMultiply.cpp:123-125) against the restatement, to 1e-13."""
    x = cases.uniform(5, (2, 31, 17), dtype=np.float64)
    y = cases.uniform(6, (1, 17, 23), dtype=np.float64)
    assert cases.rel_max(restated.matmul_forward(x, y), reference.matmul_forward(x, y)) < 1e-13


def test_shape_rules(restated):
    lib = restated.lib
    # deep8/src/nodes/Conv2d.cpp:47-63
    assert lib.d8o_conv2d_out_dim(56, 3, 1, 1, 1) == 56
    assert lib.d8o_conv2d_out_dim(32, 4, 2, 2, 1) == 16
    assert lib.d8o_conv2d_out_dim(32, 4, 2, 2, 0) == 13
    # deep8/src/nodes/DeConv2d.cpp:36-52: 14x14, 4x4 filter, stride 2 gives 27 (covered) or 30, never 28
    assert lib.d8o_deconv2d_out_dim(14, 4, 2, 1) == 27
    assert lib.d8o_deconv2d_out_dim(14, 4, 2, 0) == 30
    assert lib.d8o_conv2d_pad_before(56, 56, 3, 1, 1) == -1
    assert lib.d8o_deconv2d_pad_before(14, 27, 4, 2) == -1


def test_reference_rejects_28x28_deconv(reference):
    """A 16x28x28x128 DeConv2d output (as benchmark configuration 4 was first stated) is not producible: the reference throws on it (deep8/src/math/DeConv2d.cpp:68)."""
    x = np.zeros((1, 14, 14, 4), np.float32)
    w = np.zeros((2, 4, 4, 4), np.float32)
    z = np.zeros((1, 28, 28, 2), np.float32)
    with pytest.raises(RuntimeError):
        reference._deconv(0, x, None, w, None, z, None, True, (2, 2))


def test_library_exports_every_declared_symbol():
    """No compute: only that libdeep8_b200.so loads and has each function include/d8k.h declares."""
    from deep8_b200 import _lib
    header = open(os.path.join(os.path.dirname(os.path.dirname(__file__)), "include", "d8k.h")).read()
    declared = set(re.findall(r"D8K_API[^;(]*?\b(d8k_\w+)\s*\(", header))
    assert len(declared) >= 20
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), name
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_axpby_restated_equals_reference_bit_for_bit(restated, reference, dtype):
    """Math::AXPBY as SGDTrainer::update calls it: the plain-C restatement and the reference's Eigen expression round the two
    products and the sum the same way, so the results are identical, not merely close."""
    from oracle import pyoracle
    rng = np.random.default_rng(3)
    g, w = rng.standard_normal(100003).astype(dtype), rng.standard_normal(100003).astype(dtype)
    for lr, decay in ((0.01, 0.0005), (0.5, 0.0), (1e-3, 0.1)):
        alpha, beta = pyoracle.sgd_coefficients(lr, decay)
        assert alpha == float(np.float32(-lr)) and abs(beta - (1 - lr * decay)) < 1e-6
        assert np.array_equal(restated.axpby(g, alpha, w, beta), reference.axpby(g, alpha, w, beta))


def test_sgd_coefficients_host_side_agrees_with_the_oracle():
    from deep8_b200.dp import sgd_coefficients
    from oracle import pyoracle
    for lr, decay in ((0.01, 0.0005), (0.5, 0.0), (1e-3, 0.1), (0.3, 0.7)):
        assert sgd_coefficients(lr, decay) == pyoracle.sgd_coefficients(lr, decay)


def test_bias_add_and_its_gradient_restated_equal_reference(restated, reference):
    """Math::Add / Math::AddGradY with a bias (1, {cols}) broadcast over batch and rows."""
    rng = np.random.default_rng(5)
    for shape in ((3, 50, 33), (1, 7, 128), (2, 1, 1)):
        x = rng.standard_normal(shape).astype(np.float32)
        b = rng.standard_normal((1, shape[2])).astype(np.float32)
        assert np.array_equal(restated.add_bias(x, b), reference.add_bias(x, b))
        xi = rng.integers(0, 50, shape).astype(np.float32)  # integer data: any summation order gives the same bits
        assert np.array_equal(restated.add_bias_grad(xi, b * 0 + 3), reference.add_bias_grad(xi, b * 0 + 3))
        got, want = restated.add_bias_grad(x, b), reference.add_bias_grad(x, b)
        assert np.abs(got - want).max() <= 1e-5 * max(np.abs(want).max(), 1e-30)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_relu_and_linear_restated_equal_reference_bit_for_bit(restated, reference, dtype):
    """Math::ReLu / ReLuGrad (deep8/src/math/ReLu.cpp) and Math::Linear / LinearGrad (deep8/src/math/Linear.cpp): the
    restatement rounds where the reference's Eigen expressions round, so the arrays are identical.  a and b are floats in
    the reference's interface: values a float holds exactly make the float64 case comparable too."""
    rng = np.random.default_rng(11)
    n = 100003
    x, dy, d0 = (rng.standard_normal(n).astype(dtype) for _ in range(3))
    x[::17] = 0  # the boundary of x > 0
    assert np.array_equal(restated.relu(x), reference.relu(x))
    assert np.array_equal(restated.relu_grad(x, dy, d0), reference.relu_grad(x, dy, d0))
    for a, b in ((0.375, -1.25), (-3.0, 0.0), (1.0, 2.0 ** -10)):
        assert np.array_equal(restated.linear(x, a, b), reference.linear(x, a, b))
        assert np.array_equal(restated.linear_grad(dy, a, d0), reference.linear_grad(dy, a, d0))


@pytest.mark.parametrize("steps", [0, 1, 7, 1000])
def test_adam_update_restated_against_reference(restated, reference, steps):
    """Math::AdamUpdate (deep8/src/math/AdamUpdate.cpp:24-41): gradient, m and v come out identical; value goes through the
    reference's sqrt, which under EIGEN_FAST_MATH is Eigen's reciprocal-square-root approximation with one Newton step,
    so it is compared to a few units in the last place instead."""
    rng = np.random.default_rng(13)
    n = 50001
    w, g = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    m, v = (rng.standard_normal(n) * 0.1).astype(np.float32), (rng.random(n) * 0.01).astype(np.float32)
    args = (0.875, 0.9990234375, 2.0 ** -20, 0.0078125, 0.00048828125, steps)   # exactly representable floats
    got, want = restated.adam_update(w, g, m, v, *args), reference.adam_update(w, g, m, v, *args)
    for k in (1, 2, 3):
        assert np.array_equal(got[k], want[k])
    assert np.abs(got[0] - want[0]).max() <= 4 * np.finfo(np.float32).eps * np.abs(want[0]).max()
    assert not np.array_equal(got[0], w)
