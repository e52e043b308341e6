"""TEST INFRASTRUCTURE: numpy front-ends to the two CPU checkers.

``Restated``  -> oracle/libd8oracle.so, the plain-C restatement (d8_oracle.c).
``Reference`` -> oracle/_ref/libd8ref.so, the reference's own CPU sources compiled unmodified (ref_wrap.cpp).

Both expose the same methods so a test can run either.  Array conventions:
  matmul : x [xb, xr, xc], y [yb, xc, yc], z [max(xb, yb), xr, yc]   (a batch of 1 is broadcast)
  conv   : x [b, ih, iw, ic], w [oc, fh, fw, ic], z [b, oh, ow, oc]  (the reference's NHWC / OHWI layout)
Gradient methods return ``d0 + gradient`` (the reference accumulates into the gradient tensor); ``d0`` defaults to zeros.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
RESTATED_LIB = os.path.join(_HERE, "libd8oracle.so")
REFERENCE_LIB = os.path.join(_HERE, "_ref", "libd8ref.so")


def reference_root():
    """Where the reference project's source tree is: $DEEP8_REFERENCE, else a directory named `reference` beside this
    repository.  None when neither exists (then a prebuilt oracle/_ref is used as it is)."""
    for cand in (os.environ.get("DEEP8_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")):
        if cand and os.path.exists(os.path.join(cand, "deep8", "src", "math", "MatrixMultiply.cpp")):
            return cand
    return None


def build(ref=True):
    """Run oracle/Makefile (the restatement always; the reference library when its source tree is present)."""
    targets = ["oracle"] + (["ref"] if ref else [])
    root = reference_root()
    subprocess.run(["make", "-s", "-C", _HERE] + (["REF=" + root] if root else []) + targets, check=True)


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def _suffix(dtype):
    if dtype == np.float32:
        return "f32"
    if dtype == np.float64:
        return "f64"
    raise TypeError("the CPU path of the reference supports float32 and float64 only, got %s" % dtype)


def conv2d_out_dim(size, f, stride, dilation, covered):
    """deep8/src/nodes/Conv2d.cpp:47-63."""
    real = f + (f - 1) * (dilation - 1)
    return (size - 1) // stride + 1 if covered else (size - real) // stride + 1


def deconv2d_out_dim(size, f, stride, covered):
    """deep8/src/nodes/DeConv2d.cpp:36-52."""
    return (size - 1) * stride + 1 if covered else (size - 1) * stride + f


class _Base:
    def _check(self, *arrays):
        dt = arrays[0].dtype
        for a in arrays:
            assert a.dtype == dt and a.flags.c_contiguous, "arrays must share a dtype and be C-contiguous"
        return dt

    @staticmethod
    def _grad0(d0, shape, dtype):
        return np.zeros(shape, dtype) if d0 is None else np.array(d0, dtype=dtype, order="C", copy=True)

    # shared shape logic ------------------------------------------------------------------------------------------
    def conv2d_forward(self, x, w, covered, stride, dilation):
        b, ih, iw, ic = x.shape
        oc, fh, fw, _ = w.shape
        oh = conv2d_out_dim(ih, fh, stride[0], dilation[0], covered)
        ow = conv2d_out_dim(iw, fw, stride[1], dilation[1], covered)
        z = np.zeros((b, oh, ow, oc), x.dtype)
        self._conv(0, x, None, w, None, z, None, covered, stride, dilation)
        return z

    def conv2d_grad_x(self, x, w, dz, covered, stride, dilation, d0=None):
        dx = self._grad0(d0, x.shape, x.dtype)
        self._conv(1, x, dx, w, None, np.zeros_like(dz), dz, covered, stride, dilation)
        return dx

    def conv2d_grad_y(self, x, w, dz, covered, stride, dilation, d0=None):
        dw = self._grad0(d0, w.shape, x.dtype)
        self._conv(2, x, None, w, dw, np.zeros_like(dz), dz, covered, stride, dilation)
        return dw

    def deconv2d_forward(self, x, w, covered, stride):
        b, ih, iw, ic = x.shape
        oc, fh, fw, _ = w.shape
        oh = deconv2d_out_dim(ih, fh, stride[0], covered)
        ow = deconv2d_out_dim(iw, fw, stride[1], covered)
        z = np.zeros((b, oh, ow, oc), x.dtype)
        self._deconv(0, x, None, w, None, z, None, covered, stride)
        return z

    def deconv2d_grad_x(self, x, w, dz, covered, stride, d0=None):
        dx = self._grad0(d0, x.shape, x.dtype)
        self._deconv(1, x, dx, w, None, np.zeros_like(dz), dz, covered, stride)
        return dx

    def deconv2d_grad_y(self, x, w, dz, covered, stride, d0=None):
        dw = self._grad0(d0, w.shape, x.dtype)
        self._deconv(2, x, None, w, dw, np.zeros_like(dz), dz, covered, stride)
        return dw

    def matmul_forward(self, x, y):
        zb = max(x.shape[0], y.shape[0])
        z = np.zeros((zb, x.shape[1], y.shape[2]), x.dtype)
        self._matmul(0, x, None, y, None, z, None)
        return z

    def matmul_grad_x(self, x, y, dz, d0=None):
        dx = self._grad0(d0, x.shape, x.dtype)
        self._matmul(1, x, dx, y, None, np.zeros_like(dz), dz)
        return dx

    def matmul_grad_y(self, x, y, dz, d0=None):
        dy = self._grad0(d0, y.shape, x.dtype)
        self._matmul(2, x, None, y, dy, np.zeros_like(dz), dz)
        return dy


def sgd_coefficients(learning_rate, weight_decay):
    """alpha, beta of SGDTrainer::update (deep8/src/trainer/SGDTrainer.cpp:13-14) with its float/double mix:
    alpha = -1 * lr in float; beta = (1.0 - lr * decay) with the product in float and the difference in double,
    stored to float."""
    lr, wd = np.float32(learning_rate), np.float32(weight_decay)
    alpha = np.float32(-1) * lr
    beta = np.float32(1.0 - float(np.float32(lr * wd)))
    return float(alpha), float(beta)


def adam_ratio(learning_rate, beta1, beta2, steps, dtype=np.float32):
    """learningRate * sqrt(1 - beta2^steps) / (1 - beta1^steps) in the tensor's element type, steps <= 0 taken as 1
    (deep8/src/math/AdamUpdate.cpp:11-14, 38)."""
    t = np.float32 if dtype == np.float32 else np.float64
    steps = max(int(steps), 1)
    lr, b1, b2 = t(learning_rate), t(beta1), t(beta2)
    return float(t(t(lr * np.sqrt(t(t(1) - np.power(b2, t(steps))))) / t(t(1) - np.power(b1, t(steps)))))


class Restated(_Base):
    kind = "port"

    def __init__(self):
        if not os.path.exists(RESTATED_LIB):
            build(ref=False)
        self.lib = ctypes.CDLL(RESTATED_LIB)

    def threads(self):
        return os.cpu_count() or 1

    def add_bias(self, x, bias):
        """x [batch, rows, cols] + bias [1, cols] (Math::Add with the bias broadcast), a new array."""
        dt = self._check(x, bias)
        z = np.empty_like(x)
        rows, cols = x.shape[0] * x.shape[1], x.shape[2]
        getattr(self.lib, "d8o_add_bias_" + _suffix(dt))(_ptr(x), _ptr(bias), _ptr(z), ctypes.c_size_t(rows), ctypes.c_size_t(cols))
        return z

    def add_bias_grad(self, dz, d0):
        """d0 [1, cols] + sum of dz [batch, rows, cols] over batch and rows (Math::AddGradY), a new array."""
        dt = self._check(dz, d0)
        out = d0.copy()
        rows, cols = dz.shape[0] * dz.shape[1], dz.shape[2]
        getattr(self.lib, "d8o_add_bias_grad_" + _suffix(dt))(_ptr(out), _ptr(dz), ctypes.c_size_t(rows), ctypes.c_size_t(cols))
        return out

    def axpby(self, x, alpha, y, beta):
        """x * alpha + y * beta (Math::AXPBY), a new array."""
        dt = self._check(x, y)
        z = np.empty_like(x)
        ct = ctypes.c_float if dt == np.float32 else ctypes.c_double
        getattr(self.lib, "d8o_axpby_" + _suffix(dt))(_ptr(x), ct(alpha), _ptr(y), ct(beta), _ptr(z), ctypes.c_size_t(x.size))
        return z

    def relu(self, x):
        """max(x, 0) (Math::ReLu), a new array."""
        dt = self._check(x)
        y = np.empty_like(x)
        getattr(self.lib, "d8o_relu_" + _suffix(dt))(_ptr(x), _ptr(y), ctypes.c_size_t(x.size))
        return y

    def relu_grad(self, x, dy, d0=None):
        """d0 + (x > 0 ? dy : 0) (Math::ReLuGrad), a new array."""
        dt = self._check(x, dy)
        dx = self._grad0(d0, x.shape, dt)
        getattr(self.lib, "d8o_relu_grad_" + _suffix(dt))(_ptr(x), _ptr(dx), _ptr(dy), ctypes.c_size_t(x.size))
        return dx

    def linear(self, x, a, b):
        """x * a + b (Math::Linear), a new array."""
        dt = self._check(x)
        y = np.empty_like(x)
        ct = ctypes.c_float if dt == np.float32 else ctypes.c_double
        getattr(self.lib, "d8o_linear_" + _suffix(dt))(_ptr(x), ct(a), ct(b), _ptr(y), ctypes.c_size_t(x.size))
        return y

    def linear_grad(self, dy, a, d0=None):
        """d0 + dy * a (Math::LinearGrad), a new array."""
        dt = self._check(dy)
        dx = self._grad0(d0, dy.shape, dt)
        ct = ctypes.c_float if dt == np.float32 else ctypes.c_double
        getattr(self.lib, "d8o_linear_grad_" + _suffix(dt))(_ptr(dx), ct(a), _ptr(dy), ctypes.c_size_t(dy.size))
        return dx

    def adam_update(self, value, gradient, m, v, beta1, beta2, epsilon, learning_rate, weight_decay, steps):
        """Math::AdamUpdate: returns new (value, gradient, m, v); the inputs are left alone."""
        dt = self._check(value, gradient, m, v)
        out = [np.array(a, copy=True, order="C") for a in (value, gradient, m, v)]
        ratio = adam_ratio(learning_rate, beta1, beta2, steps, dt)
        ct = ctypes.c_float if dt == np.float32 else ctypes.c_double
        getattr(self.lib, "d8o_adam_update_" + _suffix(dt))(_ptr(out[0]), _ptr(out[1]), _ptr(out[2]), _ptr(out[3]), ct(beta1), ct(beta2),
                                                            ct(epsilon), ct(weight_decay), ct(ratio), ctypes.c_size_t(value.size))
        return tuple(out)

    def _matmul(self, which, x, dx, y, dy, z, dz):
        dt = self._check(x, y)
        s = _suffix(dt)
        xb, xr, xc = x.shape
        yb, yr, yc = y.shape
        assert yr == xc
        sz = ctypes.c_size_t
        if which == 0:
            getattr(self.lib, "d8o_matmul_forward_" + s)(_ptr(x), sz(xb), sz(xr), sz(xc), _ptr(y), sz(yb), sz(yc), _ptr(z))
        elif which == 1:
            getattr(self.lib, "d8o_matmul_grad_x_" + s)(_ptr(dx), sz(xb), sz(xr), sz(xc), _ptr(y), sz(yb), sz(yc), _ptr(dz))
        else:
            getattr(self.lib, "d8o_matmul_grad_y_" + s)(_ptr(x), sz(xb), sz(xr), sz(xc), _ptr(dy), sz(yb), sz(yc), _ptr(dz))

    def _conv(self, which, x, dx, w, dw, z, dz, covered, stride, dilation):
        dt = self._check(x, w)
        s = _suffix(dt)
        b, ih, iw, ic = x.shape
        oc, fh, fw, _ = w.shape
        _, oh, ow, _ = z.shape
        tail = (oh, ow, stride[0], stride[1], dilation[0], dilation[1])
        if which == 0:
            getattr(self.lib, "d8o_conv2d_forward_" + s)(_ptr(x), b, ih, iw, ic, _ptr(w), oc, fh, fw, _ptr(z), *tail)
        elif which == 1:
            getattr(self.lib, "d8o_conv2d_grad_x_" + s)(_ptr(dx), b, ih, iw, ic, _ptr(w), oc, fh, fw, _ptr(dz), *tail)
        else:
            getattr(self.lib, "d8o_conv2d_grad_y_" + s)(_ptr(x), b, ih, iw, ic, _ptr(dw), oc, fh, fw, _ptr(dz), *tail)

    def _deconv(self, which, x, dx, w, dw, z, dz, covered, stride):
        dt = self._check(x, w)
        s = _suffix(dt)
        b, ih, iw, ic = x.shape
        oc, fh, fw, _ = w.shape
        _, oh, ow, _ = z.shape
        tail = (oh, ow, stride[0], stride[1])
        if which == 0:
            getattr(self.lib, "d8o_deconv2d_forward_" + s)(_ptr(x), b, ih, iw, ic, _ptr(w), oc, fh, fw, _ptr(z), *tail)
        elif which == 1:
            getattr(self.lib, "d8o_deconv2d_grad_x_" + s)(_ptr(dx), b, ih, iw, ic, _ptr(w), oc, fh, fw, _ptr(dz), *tail)
        else:
            getattr(self.lib, "d8o_deconv2d_grad_y_" + s)(_ptr(x), b, ih, iw, ic, _ptr(dw), oc, fh, fw, _ptr(dz), *tail)


class Reference(_Base):
    kind = "reference"

    @staticmethod
    def available():
        return os.path.exists(REFERENCE_LIB)

    def __init__(self, path=REFERENCE_LIB):
        self.lib = ctypes.CDLL(path)
        self.lib.d8ref_last_error.restype = ctypes.c_char_p

    def threads(self):
        return int(self.lib.d8ref_threads())

    def _ok(self, rc):
        if rc != 0:
            raise RuntimeError(self.lib.d8ref_last_error().decode())

    def add_bias(self, x, bias):
        dt = self._check(x, bias)
        z = np.empty_like(x)
        b, r, c = x.shape
        sz = ctypes.c_size_t
        self._ok(self.lib.d8ref_add_bias(0, 0 if dt == np.float32 else 1, _ptr(x), sz(b), sz(r), sz(c), _ptr(bias), None, _ptr(z), None))
        return z

    def add_bias_grad(self, dz, d0):
        dt = self._check(dz, d0)
        out = d0.copy()
        b, r, c = dz.shape
        sz = ctypes.c_size_t
        x = np.zeros_like(dz)
        self._ok(self.lib.d8ref_add_bias(2, 0 if dt == np.float32 else 1, _ptr(x), sz(b), sz(r), sz(c), _ptr(d0), _ptr(out), _ptr(x),
                                         _ptr(dz)))
        return out

    def axpby(self, x, alpha, y, beta):
        dt = self._check(x, y)
        z = np.empty_like(x)
        self._ok(self.lib.d8ref_axpby(0 if dt == np.float32 else 1, _ptr(x), ctypes.c_float(alpha), _ptr(y), ctypes.c_float(beta),
                                      _ptr(z), ctypes.c_size_t(x.size)))
        return z

    def relu(self, x):
        dt = self._check(x)
        y = np.empty_like(x)
        self._ok(self.lib.d8ref_relu(0, 0 if dt == np.float32 else 1, _ptr(x), None, _ptr(y), None, ctypes.c_size_t(x.size)))
        return y

    def relu_grad(self, x, dy, d0=None):
        dt = self._check(x, dy)
        dx = self._grad0(d0, x.shape, dt)
        y = np.zeros_like(x)
        self._ok(self.lib.d8ref_relu(1, 0 if dt == np.float32 else 1, _ptr(x), _ptr(dx), _ptr(y), _ptr(dy), ctypes.c_size_t(x.size)))
        return dx

    def linear(self, x, a, b):
        dt = self._check(x)
        y = np.empty_like(x)
        self._ok(self.lib.d8ref_linear(0, 0 if dt == np.float32 else 1, _ptr(x), None, ctypes.c_float(a), ctypes.c_float(b), _ptr(y), None,
                                       ctypes.c_size_t(x.size)))
        return y

    def linear_grad(self, dy, a, d0=None):
        dt = self._check(dy)
        dx = self._grad0(d0, dy.shape, dt)
        x = np.zeros_like(dy)
        self._ok(self.lib.d8ref_linear(1, 0 if dt == np.float32 else 1, _ptr(x), _ptr(dx), ctypes.c_float(a), ctypes.c_float(0.0), _ptr(x),
                                       _ptr(dy), ctypes.c_size_t(dy.size)))
        return dx

    def adam_update(self, value, gradient, m, v, beta1, beta2, epsilon, learning_rate, weight_decay, steps):
        dt = self._check(value, gradient, m, v)
        out = [np.array(a, copy=True, order="C") for a in (value, gradient, m, v)]
        f = ctypes.c_float
        self._ok(self.lib.d8ref_adam_update(0 if dt == np.float32 else 1, _ptr(out[0]), _ptr(out[1]), _ptr(out[2]), _ptr(out[3]), f(beta1),
                                            f(beta2), f(epsilon), f(learning_rate), f(weight_decay), ctypes.c_longlong(steps),
                                            ctypes.c_size_t(value.size)))
        return tuple(out)

    def _matmul(self, which, x, dx, y, dy, z, dz):
        dt = self._check(x, y)
        code = 0 if dt == np.float32 else 1
        _suffix(dt)
        xb, xr, xc = x.shape
        yb, yr, yc = y.shape
        sz = ctypes.c_size_t
        self._ok(self.lib.d8ref_matmul(which, code, _ptr(x), _ptr(dx), sz(xb), 2, sz(xr), sz(xc),
                                       _ptr(y), _ptr(dy), sz(yb), 1 if yc == 1 else 2, sz(yr), sz(yc), _ptr(z), _ptr(dz)))

    def _conv(self, which, x, dx, w, dw, z, dz, covered, stride, dilation):
        dt = self._check(x, w)
        code = 0 if dt == np.float32 else 1
        _suffix(dt)
        sz = ctypes.c_size_t
        b, ih, iw, ic = x.shape
        oc, fh, fw, _ = w.shape
        _, oh, ow, _ = z.shape
        self._ok(self.lib.d8ref_conv2d(which, code, _ptr(x), _ptr(dx), sz(b), sz(ih), sz(iw), sz(ic), _ptr(w), _ptr(dw),
                                       sz(oc), sz(fh), sz(fw), _ptr(z), _ptr(dz), sz(oh), sz(ow), int(bool(covered)),
                                       stride[0], stride[1], dilation[0], dilation[1]))

    def _deconv(self, which, x, dx, w, dw, z, dz, covered, stride):
        dt = self._check(x, w)
        code = 0 if dt == np.float32 else 1
        _suffix(dt)
        sz = ctypes.c_size_t
        b, ih, iw, ic = x.shape
        oc, fh, fw, _ = w.shape
        _, oh, ow, _ = z.shape
        self._ok(self.lib.d8ref_deconv2d(which, code, _ptr(x), _ptr(dx), sz(b), sz(ih), sz(iw), sz(ic), _ptr(w), _ptr(dw),
                                         sz(oc), sz(fh), sz(fw), _ptr(z), _ptr(dz), sz(oh), sz(ow), int(bool(covered)),
                                         stride[0], stride[1]))
