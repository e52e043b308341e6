"""Operator front-end over the C ABI, with torch tensors as device buffers.

Mirrors the reference's operator interface for the path: forward returns a new tensor, gradient calls ACCUMULATE into
the gradient tensor passed in (deep8/src/nodes/MatrixMultiply.cpp:36-52, Conv2d.cpp:74-152, DeConv2d.cpp:63-126).
Layouts are the reference's: matrices [batch, rows, cols]; images [batch, height, width, channel]; filters
[outChannel, filterHeight, filterWidth, inChannel].
"""
import ctypes

import torch

from . import _lib
from ._lib import F16, F32, check


def _dtype_code(t):
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.float32:
        return F32
    raise TypeError("type %s is not support" % t.dtype)  # the reference's message for an unsupported element type


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _out(out, shape, like):
    """A caller-supplied output: same device, dtype and layout rules as the inputs and exactly the computed shape - a wrong
    size here would otherwise become an out-of-bounds device write.  None allocates."""
    if out is None:
        return torch.empty(shape, dtype=like.dtype, device=like.device)
    _same(like, out)
    if tuple(out.shape) != tuple(shape):
        raise ValueError("the shape is error")
    return out


def _same(*ts):
    d0 = ts[0]
    for t in ts:
        if t.device != d0.device:
            raise ValueError("the device type must be same")
        if t.dtype != d0.dtype:
            raise ValueError("the data type must be same")
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous")
    return _dtype_code(d0)


class Context:
    """One d8k context: a device, a stream and the split-K scratch memory.  Not for concurrent use."""

    def __init__(self, device=0, scratch_bytes=0):
        self.lib = _lib.load()
        self.device = device
        h = ctypes.c_void_p()
        check(self.lib.d8k_ctx_create(device, scratch_bytes, ctypes.byref(h)))
        self.h = h
        self.num_sms = self.lib.d8k_ctx_num_sms(h)

    def close(self):
        if getattr(self, "h", None):
            self.lib.d8k_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def use_stream(self, stream):
        """Enqueue on a torch.cuda.Stream (or None for the legacy default stream)."""
        check(self.lib.d8k_ctx_set_stream(self.h, ctypes.c_void_p(stream.cuda_stream if stream is not None else 0)))

    def status(self):
        s = ctypes.c_int(0)
        check(self.lib.d8k_ctx_status(self.h, ctypes.byref(s)))
        return s.value

    def launch_count(self):
        return int(self.lib.d8k_launch_count())

    def last_kernel(self):
        """Text describing the contraction kernel of this thread's last launch (d8k_last_kernel)."""
        return self.lib.d8k_last_kernel().decode()

    # ------------------------------------------------------------------------------------------------ gemm
    def gemm(self, A, B, C, transA=False, transB=False, beta=0, reduce_batch=False):
        """C[b] (+)= op(A[b % batchA]) op(B[b % batchB]); A, B, C are [batch, rows, cols] tensors."""
        dt = _same(A, B, C)
        batchA, ar, ac = A.shape
        batchB, br, bc = B.shape
        M, K = (ac, ar) if transA else (ar, ac)
        K2, N = (bc, br) if transB else (br, bc)
        if K != K2:
            raise ValueError("the shape is error")
        batch = max(batchA, batchB)
        if reduce_batch:
            assert C.shape == (1, M, N)
        else:
            assert C.shape == (batch, M, N)
        check(self.lib.d8k_gemm(self.h, dt, int(transA), int(transB), M, N, K, _p(A), ac, batchA, ar * ac, _p(B), bc, batchB, br * bc,
                                _p(C), N, M * N, batch, int(beta), int(reduce_batch)))
        return C

    # ------------------------------------------------------------------------------------------------ MatrixMultiply
    @staticmethod
    def _mm_dims(x, y):
        xb, xr, xc = x.shape
        yb, yr, yc = y.shape
        if yr != xc or (xb != yb and xb != 1 and yb != 1):
            raise ValueError("the shape is error")
        return xb, xr, xc, yb, yc

    def matmul_forward(self, x, y, out=None):
        dt = _same(x, y)
        xb, xr, xc, yb, yc = self._mm_dims(x, y)
        z = _out(out, (max(xb, yb), xr, yc), x)
        check(self.lib.d8k_matmul_forward(self.h, dt, _p(x), xb, xr, xc, _p(y), yb, yc, _p(z)))
        return z

    def matmul_grad_x(self, x, dx, y, dz, accumulate=True):
        """dx (+)= dz y^T.  accumulate=False overwrites (first contribution, no zeroGradient needed)."""
        dt = _same(x, dx, y, dz)
        xb, xr, xc, yb, yc = self._mm_dims(x, y)
        if dx.shape != x.shape or tuple(dz.shape) != (max(xb, yb), xr, yc):
            raise ValueError("the shape is error")
        check(self.lib.d8k_matmul_grad_x_into(self.h, dt, _p(dx), xb, xr, xc, _p(y), yb, yc, _p(dz), int(accumulate)))
        return dx

    def matmul_grad_y(self, x, y, dy, dz, accumulate=True):
        dt = _same(x, y, dy, dz)
        xb, xr, xc, yb, yc = self._mm_dims(x, y)
        if dy.shape != y.shape or tuple(dz.shape) != (max(xb, yb), xr, yc):
            raise ValueError("the shape is error")
        check(self.lib.d8k_matmul_grad_y_into(self.h, dt, _p(x), xb, xr, xc, _p(dy), yb, yc, _p(dz), int(accumulate)))
        return dy

    def matmul_forward_relu(self, x, y, z, a):
        """z = x y and a = relu(z) in one launch (MatrixMultiply node followed by ReLu node)."""
        dt = _same(x, y, z, a)
        xb, xr, xc, yb, yc = self._mm_dims(x, y)
        if tuple(z.shape) != (max(xb, yb), xr, yc) or a.shape != z.shape:
            raise ValueError("the shape is error")
        check(self.lib.d8k_matmul_forward_relu(self.h, dt, _p(x), xb, xr, xc, _p(y), yb, yc, _p(z), _p(a)))
        return z, a

    def matmul_forward_linear(self, x, y, z, l, a, b):
        """z = x y and l = z * a + b in one launch (MatrixMultiply node followed by Linear node)."""
        dt = _same(x, y, z, l)
        xb, xr, xc, yb, yc = self._mm_dims(x, y)
        if tuple(z.shape) != (max(xb, yb), xr, yc) or l.shape != z.shape:
            raise ValueError("the shape is error")
        check(self.lib.d8k_matmul_forward_linear(self.h, dt, _p(x), xb, xr, xc, _p(y), yb, yc, _p(z), float(a), float(b), _p(l)))
        return z, l

    def matmul_forward_bias(self, x, y, bias, out=None):
        """z = x * y + bias, bias [1, yc] added to every row (MatrixMultiply followed by Add, one launch)."""
        dt = _same(x, y, bias)
        xb, xr, xc, yb, yc = self._mm_dims(x, y)
        if bias.numel() != yc:
            raise ValueError("the shape is error")
        z = _out(out, (max(xb, yb), xr, yc), x)
        check(self.lib.d8k_matmul_forward_bias(self.h, dt, _p(x), xb, xr, xc, _p(y), yb, yc, _p(bias), _p(z)))
        return z

    def add_bias(self, x, bias, out=None):
        """x [..., cols] + bias [cols] broadcast over the leading dimensions (Math::Add for a bias)."""
        dt = _same(x, bias)
        cols = x.shape[-1]
        if bias.numel() != cols:
            raise ValueError("the shape is error")
        z = _out(out, tuple(x.shape), x)
        check(self.lib.d8k_add_bias(self.h, dt, _p(x), _p(bias), _p(z), x.numel() // cols, cols))
        return z

    def add_bias_grad(self, dbias, dz):
        """dbias [cols] += sum of dz [..., cols] over the leading dimensions (Math::AddGradY for a bias)."""
        dt = _same(dbias, dz)
        cols = dz.shape[-1]
        if dbias.numel() != cols:
            raise ValueError("the shape is error")
        check(self.lib.d8k_add_bias_grad(self.h, dt, _p(dbias), _p(dz), dz.numel() // cols, cols))
        return dbias

    def matmul_grad_x_relu(self, x, dx, y, dz, h, dh, accumulate_dx=True, accumulate_dh=True):
        """For x = relu(h): dx (+)= dz y^T, then dh (+)= (h > 0 ? dx : 0), in one launch."""
        dt = _same(x, dx, y, dz, h, dh)
        xb, xr, xc, yb, yc = self._mm_dims(x, y)
        if dx.shape != x.shape or tuple(dz.shape) != (max(xb, yb), xr, yc) or h.shape != x.shape or dh.shape != x.shape:
            raise ValueError("the shape is error")
        check(self.lib.d8k_matmul_grad_x_relu(self.h, dt, _p(dx), xb, xr, xc, _p(y), yb, yc, _p(dz), int(accumulate_dx), _p(h), _p(dh),
                                              int(accumulate_dh)))
        return dx, dh

    # ------------------------------------------------------------------------------------------------ Conv2d
    def conv2d_out_shape(self, x, w, covered, stride, dilation):
        b, ih, iw, ic = x.shape
        oc, fh, fw, wc = w.shape
        if wc != ic:
            raise ValueError("the shape is error")
        oh = self.lib.d8k_conv2d_out_dim(ih, fh, stride[0], dilation[0], int(covered))
        ow = self.lib.d8k_conv2d_out_dim(iw, fw, stride[1], dilation[1], int(covered))
        return (b, oh, ow, oc)

    def conv2d_forward(self, x, w, covered=False, stride=(1, 1), dilation=(1, 1), out=None):
        dt = _same(x, w)
        b, oh, ow, oc = self.conv2d_out_shape(x, w, covered, stride, dilation)
        z = _out(out, (b, oh, ow, oc), x)
        _, ih, iw, ic = x.shape
        _, fh, fw, _ = w.shape
        check(self.lib.d8k_conv2d_forward(self.h, dt, _p(x), b, ih, iw, ic, _p(w), oc, fh, fw, _p(z), oh, ow, stride[0], stride[1],
                                          dilation[0], dilation[1], None, 0))
        return z

    def conv2d_grad_x(self, x, dx, w, dz, covered=False, stride=(1, 1), dilation=(1, 1), accumulate=True):
        dt = _same(x, dx, w, dz)
        b, oh, ow, oc = self.conv2d_out_shape(x, w, covered, stride, dilation)
        if tuple(dz.shape) != (b, oh, ow, oc) or dx.shape != x.shape:
            raise ValueError("the shape is error")
        _, ih, iw, ic = x.shape
        _, fh, fw, _ = w.shape
        check(self.lib.d8k_conv2d_grad_x_into(self.h, dt, _p(dx), b, ih, iw, ic, _p(w), oc, fh, fw, _p(dz), oh, ow, stride[0], stride[1],
                                              dilation[0], dilation[1], None, 0, int(accumulate)))
        return dx

    def conv2d_grad_y(self, x, w, dw, dz, covered=False, stride=(1, 1), dilation=(1, 1), accumulate=True):
        dt = _same(x, w, dw, dz)
        b, oh, ow, oc = self.conv2d_out_shape(x, w, covered, stride, dilation)
        if tuple(dz.shape) != (b, oh, ow, oc) or dw.shape != w.shape:
            raise ValueError("the shape is error")
        _, ih, iw, ic = x.shape
        _, fh, fw, _ = w.shape
        check(self.lib.d8k_conv2d_grad_y_into(self.h, dt, _p(x), b, ih, iw, ic, _p(dw), oc, fh, fw, _p(dz), oh, ow, stride[0], stride[1],
                                              dilation[0], dilation[1], None, 0, int(accumulate)))
        return dw

    # ------------------------------------------------------------------------------------------------ DeConv2d
    def deconv2d_out_shape(self, x, w, covered, stride):
        b, ih, iw, ic = x.shape
        oc, fh, fw, wc = w.shape
        if wc != ic:
            raise ValueError("the shape is error")
        oh = self.lib.d8k_deconv2d_out_dim(ih, fh, stride[0], int(covered))
        ow = self.lib.d8k_deconv2d_out_dim(iw, fw, stride[1], int(covered))
        return (b, oh, ow, oc)

    def deconv2d_forward(self, x, w, covered=False, stride=(1, 1), out=None):
        dt = _same(x, w)
        b, oh, ow, oc = self.deconv2d_out_shape(x, w, covered, stride)
        z = _out(out, (b, oh, ow, oc), x)
        _, ih, iw, ic = x.shape
        _, fh, fw, _ = w.shape
        check(self.lib.d8k_deconv2d_forward(self.h, dt, _p(x), b, ih, iw, ic, _p(w), oc, fh, fw, _p(z), oh, ow, stride[0], stride[1], None, 0))
        return z

    def deconv2d_grad_x(self, x, dx, w, dz, covered=False, stride=(1, 1), accumulate=True):
        dt = _same(x, dx, w, dz)
        b, oh, ow, oc = self.deconv2d_out_shape(x, w, covered, stride)
        if tuple(dz.shape) != (b, oh, ow, oc) or dx.shape != x.shape:
            raise ValueError("the shape is error")
        _, ih, iw, ic = x.shape
        _, fh, fw, _ = w.shape
        check(self.lib.d8k_deconv2d_grad_x_into(self.h, dt, _p(dx), b, ih, iw, ic, _p(w), oc, fh, fw, _p(dz), oh, ow, stride[0], stride[1], None, 0,
                                                int(accumulate)))
        return dx

    def deconv2d_grad_y(self, x, w, dw, dz, covered=False, stride=(1, 1), accumulate=True):
        dt = _same(x, w, dw, dz)
        b, oh, ow, oc = self.deconv2d_out_shape(x, w, covered, stride)
        if tuple(dz.shape) != (b, oh, ow, oc) or dw.shape != w.shape:
            raise ValueError("the shape is error")
        _, ih, iw, ic = x.shape
        _, fh, fw, _ = w.shape
        check(self.lib.d8k_deconv2d_grad_y_into(self.h, dt, _p(x), b, ih, iw, ic, _p(dw), oc, fh, fw, _p(dz), oh, ow, stride[0], stride[1], None, 0,
                                                int(accumulate)))
        return dw

    # ------------------------------------------------------------------------------------------------ neighbours
    def relu_forward(self, x, out=None):
        dt = _same(x)
        y = _out(out, tuple(x.shape), x)
        check(self.lib.d8k_relu_forward(self.h, dt, _p(x), _p(y), x.numel()))
        return y

    def relu_backward(self, x, dx, dy):
        dt = _same(x, dx, dy)
        check(self.lib.d8k_relu_backward(self.h, dt, _p(x), _p(dx), _p(dy), x.numel()))
        return dx

    def linear_forward(self, x, a, b, out=None):
        """x * a + b (Math::Linear)."""
        dt = _same(x)
        y = _out(out, tuple(x.shape), x)
        check(self.lib.d8k_linear_forward(self.h, dt, _p(x), float(a), float(b), _p(y), x.numel()))
        return y

    def linear_grad(self, dx, a, dy):
        """dx += dy * a (Math::LinearGrad)."""
        dt = _same(dx, dy)
        if dx.shape != dy.shape:
            raise ValueError("the shape is error")
        check(self.lib.d8k_linear_grad(self.h, dt, _p(dx), float(a), _p(dy), dx.numel()))
        return dx

    def adam_update(self, value, gradient, m, v, beta1, beta2, epsilon, learning_rate, weight_decay, steps):
        """Math::AdamUpdate on all four tensors in place (AdamTrainer::update)."""
        dt = _same(value, gradient, m, v)
        if not (value.numel() == gradient.numel() == m.numel() == v.numel()):
            raise ValueError("the param shape size must be same")
        check(self.lib.d8k_adam_update(self.h, dt, _p(value), _p(gradient), _p(m), _p(v), float(beta1), float(beta2), float(epsilon),
                                       float(learning_rate), float(weight_decay), int(steps), value.numel()))
        return value

    def zero(self, t):
        check(self.lib.d8k_zero(self.h, _p(t), t.numel() * t.element_size()))
        return t

    # ------------------------------------------------------------------------------------------------ exchange between GPUs
    # Raw device addresses (ints): the memory belongs to the library (d8k_peer_alloc) or to a peer process.
    def peer_alloc(self, nbytes):
        """(address, handle): zero-filled device memory that peer processes can map; `handle` is 64 bytes to send them."""
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(_lib.IPC_HANDLE_BYTES)
        check(self.lib.d8k_peer_alloc(self.h, nbytes, ctypes.byref(ptr), handle))
        return ptr.value, handle.raw

    def peer_free(self, ptr):
        check(self.lib.d8k_peer_free(self.h, ctypes.c_void_p(ptr)))

    def peer_open(self, handle):
        ptr = ctypes.c_void_p()
        check(self.lib.d8k_peer_open(self.h, ctypes.create_string_buffer(bytes(handle), _lib.IPC_HANDLE_BYTES), ctypes.byref(ptr)))
        return ptr.value

    def peer_close(self, ptr):
        check(self.lib.d8k_peer_close(self.h, ctypes.c_void_p(ptr)))

    @staticmethod
    def _ptr_array(ptrs):
        return (ctypes.c_void_p * len(ptrs))(*ptrs)

    def peer_signal(self, flags, value):
        check(self.lib.d8k_peer_signal(self.h, self._ptr_array(flags), len(flags), value & 0xFFFFFFFF))

    def peer_wait(self, flags, value, timeout_ms=2000.0):
        check(self.lib.d8k_peer_wait(self.h, self._ptr_array(flags), len(flags), value & 0xFFFFFFFF, float(timeout_ms)))

    def peer_copy(self, dst, src, nbytes):
        check(self.lib.d8k_peer_copy(self.h, ctypes.c_void_p(dst), ctypes.c_void_p(src), nbytes))

    def matmul_grad_y_scatter(self, x, yc, dz, row_blocks, block_rows):
        """dy = x^T * dz for a replicated y ([1, xc, yc]), rows [k * block_rows, ...) written to address row_blocks[k]."""
        dt = _same(x, dz)
        xb, xr, xc = x.shape
        if tuple(dz.shape) != (xb, xr, yc) or block_rows < 128 or block_rows % 128 or not 1 <= len(row_blocks) <= 16 or \
                len(row_blocks) * block_rows < xc:
            raise ValueError("the shape is error")
        check(self.lib.d8k_matmul_grad_y_scatter(self.h, dt, _p(x), xb, xr, xc, yc, _p(dz), self._ptr_array(row_blocks),
                                                 len(row_blocks), block_rows))

    @staticmethod
    def _code(dtype):
        code = F16 if dtype == torch.float16 else F32 if dtype == torch.float32 else None
        if code is None:
            raise TypeError("type %s is not support" % dtype)
        return code

    def sum_shards(self, dtype, out, srcs, count, sgd=None, copies=None, adam=None):
        """out[i] = srcs[0][i] + ... + srcs[-1][i] in that order (fp32 accumulation); dtype is a torch dtype.
        sgd = (weights address, alpha, beta): also weights = sum * alpha + weights * beta (out may then be None).
        adam = (weights, m, v addresses, beta1, beta2, epsilon, learning_rate, weight_decay, steps): Math::AdamUpdate on the summed
        shard instead; out (may be None) receives the gradient after the decay term.
        copies: addresses (peers' buffers) that also receive the result - the updated weights with sgd or adam, else the sum."""
        code = self._code(dtype)
        if adam is not None:
            w, m, v, b1, b2, eps, lr, wd, steps = adam
            cp = self._ptr_array(copies) if copies else None
            check(self.lib.d8k_sum_shards_adam(self.h, code, ctypes.c_void_p(out) if out else None, self._ptr_array(srcs), len(srcs), count,
                                               ctypes.c_void_p(w), ctypes.c_void_p(m), ctypes.c_void_p(v), b1, b2, eps, lr, wd, int(steps), cp,
                                               len(copies) if copies else 0))
            return
        if copies:
            w, alpha, beta = sgd if sgd is not None else (None, 0.0, 0.0)
            check(self.lib.d8k_sum_shards_gather(self.h, code, ctypes.c_void_p(out) if out else None, self._ptr_array(srcs), len(srcs),
                                                 count, ctypes.c_void_p(w) if w else None, alpha, beta, self._ptr_array(copies), len(copies)))
        elif sgd is None:
            check(self.lib.d8k_sum_shards(self.h, code, ctypes.c_void_p(out), self._ptr_array(srcs), len(srcs), count))
        else:
            w, alpha, beta = sgd
            check(self.lib.d8k_sum_shards_sgd(self.h, code, ctypes.c_void_p(out) if out else None, self._ptr_array(srcs), len(srcs), count,
                                              ctypes.c_void_p(w), alpha, beta))

    def axpby(self, x, alpha, y, beta):
        """y = x * alpha + y * beta (Math::AXPBY as the trainers call it); returns y."""
        dt = _same(x, y)
        check(self.lib.d8k_axpby(self.h, dt, _p(x), alpha, _p(y), beta, x.numel()))
        return y


class _RawCuda:
    """Array-interface shim so that torch can view device memory it did not allocate."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"data": (ptr, False), "shape": tuple(shape), "typestr": typestr, "version": 2, "strides": None}


def tensor_view(ptr, shape, dtype, device):
    """A torch tensor over `ptr` (library or peer memory); the caller keeps the memory alive."""
    typestr = {torch.float16: "<f2", torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1"}[dtype]
    return torch.as_tensor(_RawCuda(ptr, shape, typestr), device=device)
