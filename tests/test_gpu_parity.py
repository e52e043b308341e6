"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle on the same seeded inputs.

Tolerances (per output tensor, max |got - want| / max |want|):
  fp32 (3xTF32)              1e-5   against the oracle (the exact contraction, correctly rounded)
  fp16 in, fp32 accumulate   2e-2   against the fp32 oracle on the fp16-rounded inputs (the reference has no CPU half)
  integer-valued data        exact  (what the reference's own unit tests assert)
"""
import glob
import os

import numpy as np
import pytest
import torch

import cases
from test_oracle import load_golden, GOLDEN

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
F16_TOL = 2e-2
DEV = "cuda:0"


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    return t if dtype is None else t.to(dtype)


def host(t):
    return t.float().cpu().numpy()


def check(ctx, got, want, tol, what=""):
    assert ctx.status() == 0
    got = host(got)
    assert got.shape == want.shape, what
    err = cases.rel_max(got, want)
    assert err <= tol, "%s: rel_max %.3e > %.1e" % (what, err, tol)
    return err


class Runner:
    """Runs forward and both gradients of one operator on the GPU and on an oracle, gradients starting from d0."""

    def __init__(self, ctx, oracle, kind, meta):
        self.ctx, self.oracle, self.kind, self.meta = ctx, oracle, kind, meta

    def gpu(self, x, w, dz, dx0, dw0, tdtype):
        c = self.ctx
        X, W = dev(x, tdtype), dev(w, tdtype)
        if self.kind == "matmul":
            z = c.matmul_forward(X, W)
        elif self.kind == "conv":
            cov, st, dil = self.meta
            z = c.conv2d_forward(X, W, cov, st, dil)
        else:
            cov, st = self.meta
            z = c.deconv2d_forward(X, W, cov, st)
        if dz is None:
            return z, None, None
        DZ, DX, DW = dev(dz, tdtype), dev(dx0, tdtype), dev(dw0, tdtype)
        if self.kind == "matmul":
            c.matmul_grad_x(X, DX, W, DZ)
            c.matmul_grad_y(X, W, DW, DZ)
        elif self.kind == "conv":
            c.conv2d_grad_x(X, DX, W, DZ, cov, st, dil)
            c.conv2d_grad_y(X, W, DW, DZ, cov, st, dil)
        else:
            c.deconv2d_grad_x(X, DX, W, DZ, cov, st)
            c.deconv2d_grad_y(X, W, DW, DZ, cov, st)
        return z, DX, DW

    def cpu(self, x, w, dz, dx0, dw0):
        o = self.oracle
        if self.kind == "matmul":
            z = o.matmul_forward(x, w)
            if dz is None:
                return z, None, None
            return z, o.matmul_grad_x(x, w, dz, dx0), o.matmul_grad_y(x, w, dz, dw0)
        if self.kind == "conv":
            z = o.conv2d_forward(x, w, *self.meta)
            if dz is None:
                return z, None, None
            return z, o.conv2d_grad_x(x, w, dz, *self.meta, d0=dx0), o.conv2d_grad_y(x, w, dz, *self.meta, d0=dw0)
        z = o.deconv2d_forward(x, w, *self.meta)
        if dz is None:
            return z, None, None
        return z, o.deconv2d_grad_x(x, w, dz, *self.meta, d0=dx0), o.deconv2d_grad_y(x, w, dz, *self.meta, d0=dw0)

    def zshape(self, x, w):
        return self.cpu(x, w, None, None, None)[0].shape


def parity(ctx, oracle, kind, xs, ws, meta, tdtype, tol, seed=0, gen="float"):
    r = Runner(ctx, oracle, kind, meta)
    if gen == "float":
        x, w = cases.uniform(seed, xs), cases.normal(seed + 1, ws, 0.25)
    else:
        hi = 4 if tdtype == torch.float16 else 20
        x, w = cases.small_ints(seed, xs, hi), cases.small_ints(seed + 1, ws, hi)
    if tdtype == torch.float16:  # the oracle sees exactly the values the GPU sees
        x, w = x.astype(np.float16).astype(np.float32), w.astype(np.float16).astype(np.float32)
    zs = r.zshape(x, w)
    if gen == "float":
        dz, dx0, dw0 = cases.normal(seed + 2, zs), cases.normal(seed + 3, xs), cases.normal(seed + 4, ws)
    else:
        dz, dx0, dw0 = cases.small_ints(seed + 2, zs, hi), cases.small_ints(seed + 3, xs, hi), cases.small_ints(seed + 4, ws, hi)
    if tdtype == torch.float16:
        dz, dx0, dw0 = (a.astype(np.float16).astype(np.float32) for a in (dz, dx0, dw0))
    got = r.gpu(x, w, dz, dx0, dw0, tdtype)
    want = r.cpu(x, w, dz, dx0, dw0)
    errs = [check(ctx, g, wnt, tol, name) for name, g, wnt in zip(("z", "dx", "dy"), got, want)]
    return errs


# ------------------------------------------------------------------------------------------------ MatrixMultiply
@pytest.mark.parametrize("xs,ys", cases.MATMUL_REFERENCE_TESTS + cases.MATMUL_EDGE + [cases.MATMUL_CFG1, cases.MATMUL_CFG2])
def test_matmul_f32(ctx, restated, xs, ys):
    parity(ctx, restated, "matmul", xs, ys, None, torch.float32, F32_TOL)


@pytest.mark.parametrize("xs,ys", cases.MATMUL_REFERENCE_TESTS + cases.MATMUL_EDGE + [cases.MATMUL_CFG1, cases.MATMUL_CFG2])
def test_matmul_f16(ctx, restated, xs, ys):
    parity(ctx, restated, "matmul", xs, ys, None, torch.float16, F16_TOL)


@pytest.mark.parametrize("xs,ys", cases.MATMUL_REFERENCE_TESTS + cases.MATMUL_EDGE)
def test_matmul_integers_exact_f32(ctx, restated, xs, ys):
    """test/MatrixMultiplyTest.h asserts equality on rand() % 50 data; so do we."""
    parity(ctx, restated, "matmul", xs, ys, None, torch.float32, 0.0, gen="int")


def test_matmul_integers_exact_f16(ctx, restated):
    parity(ctx, restated, "matmul", (3, 40, 24), (1, 24, 56), None, torch.float16, 0.0, gen="int")
    parity(ctx, restated, "matmul", (1, 129, 17), (2, 17, 31), None, torch.float16, 0.0, gen="int")


# ------------------------------------------------------------------------------------------------ Conv2d
@pytest.mark.parametrize("xs,ws,cov,st,dil", cases.CONV_REFERENCE_TESTS + cases.CONV_EDGE)
def test_conv_f32(ctx, restated, xs, ws, cov, st, dil):
    parity(ctx, restated, "conv", xs, ws, (cov, st, dil), torch.float32, F32_TOL)


@pytest.mark.parametrize("xs,ws,cov,st,dil", cases.CONV_REFERENCE_TESTS + cases.CONV_EDGE)
def test_conv_f16(ctx, restated, xs, ws, cov, st, dil):
    parity(ctx, restated, "conv", xs, ws, (cov, st, dil), torch.float16, F16_TOL)


@pytest.mark.parametrize("xs,ws,cov,st,dil", cases.CONV_REFERENCE_TESTS + cases.CONV_EDGE)
def test_conv_integers_exact(ctx, restated, xs, ws, cov, st, dil):
    parity(ctx, restated, "conv", xs, ws, (cov, st, dil), torch.float32, 0.0, gen="int")


def test_conv_cfg3_full_size(ctx, restated):
    xs, ws, cov, st, dil = cases.CONV_CFG3
    parity(ctx, restated, "conv", xs, ws, (cov, st, dil), torch.float32, F32_TOL, seed=4)


# ------------------------------------------------------------------------------------------------ DeConv2d
@pytest.mark.parametrize("xs,ws,cov,st", cases.DECONV_REFERENCE_TESTS + cases.DECONV_EDGE)
def test_deconv_f32(ctx, restated, xs, ws, cov, st):
    parity(ctx, restated, "deconv", xs, ws, (cov, st), torch.float32, F32_TOL)


@pytest.mark.parametrize("xs,ws,cov,st", cases.DECONV_REFERENCE_TESTS + cases.DECONV_EDGE)
def test_deconv_f16(ctx, restated, xs, ws, cov, st):
    parity(ctx, restated, "deconv", xs, ws, (cov, st), torch.float16, F16_TOL)


@pytest.mark.parametrize("xs,ws,cov,st", cases.DECONV_REFERENCE_TESTS + cases.DECONV_EDGE)
def test_deconv_integers_exact(ctx, restated, xs, ws, cov, st):
    parity(ctx, restated, "deconv", xs, ws, (cov, st), torch.float32, 0.0, gen="int")


def test_deconv_cfg4_full_size(ctx, restated):
    xs, ws, cov, st = cases.DECONV_CFG4
    parity(ctx, restated, "deconv", xs, ws, (cov, st), torch.float32, F32_TOL, seed=7)


# ------------------------------------------------------------------------------------------------ golden vectors
@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_gpu_matches_reference_golden(ctx, path):
    """Against the committed outputs of the reference's own CPU code (float accumulation: 1e-5 covers both sides)."""
    kind, x, w, dz_seed, meta, want = load_golden(path)
    r = Runner(ctx, None, kind, meta)
    dz = cases.normal(dz_seed, want[0].shape)
    got = r.gpu(x, w, dz, np.zeros_like(x), np.zeros_like(w), torch.float32)
    for name, g, wnt in zip(("z", "dx", "dy"), got, want):
        check(ctx, g, wnt, F32_TOL, name)


def test_gpu_matches_reference_library(ctx, reference):
    """Where the reference's CPU library travelled with the repo, compare with it directly on config 1."""
    xs, ys = cases.MATMUL_CFG1
    x, y = cases.uniform(0, xs), cases.uniform(10, ys)
    dz = cases.uniform(1, (1, xs[1], ys[2]))
    r = Runner(ctx, reference, "matmul", None)
    got = r.gpu(x, y, dz, np.zeros_like(x), np.zeros_like(y), torch.float32)
    want = r.cpu(x, y, dz, None, None)
    for g, wnt in zip(got, want):
        check(ctx, g, wnt, F32_TOL)


# ------------------------------------------------------------------------------------------------ full-size properties
def test_cfg5_mlp_layer_sampled_rows(ctx, restated):
    """Config 5 sizes do not fit the oracle; check rows sampled from the full-size product against it, and linearity."""
    torch.manual_seed(10)
    M, K, N = 8192, 4096, 16384
    X = torch.randn(1, M, K, device=DEV, dtype=torch.float16)
    W = (torch.randn(1, K, N, device=DEV) * 0.02).to(torch.float16)
    H = ctx.matmul_forward(X, W)
    assert ctx.status() == 0
    rows = [0, 1, 127, 128, 4095, 8191]
    want = restated.matmul_forward(np.ascontiguousarray(host(X[:, rows, :])), host(W))
    assert cases.rel_max(host(H[:, rows, :]), want) <= F16_TOL
    # gradient of the weights over the full batch: sampled columns against the oracle (K of this product = 8192 rows)
    dH = (torch.randn(1, M, N, device=DEV) * 0.01).to(torch.float16)
    dW = torch.zeros_like(W)
    ctx.matmul_grad_y(X, W, dW, dH)
    assert ctx.status() == 0
    cols = [0, 255, 256, 16383]
    want = restated.matmul_grad_y(host(X), np.zeros((1, K, len(cols)), np.float32), np.ascontiguousarray(host(dH[:, :, cols])))
    assert cases.rel_max(host(dW[:, :, cols]), want) <= F16_TOL
    # dx = dH W^T on sampled rows
    dX = torch.zeros_like(X)
    ctx.matmul_grad_x(X, dX, W, dH)
    assert ctx.status() == 0
    want = restated.matmul_grad_x(np.zeros((1, len(rows), K), np.float32), host(W), np.ascontiguousarray(host(dH[:, rows, :])))
    assert cases.rel_max(host(dX[:, rows, :]), want) <= F16_TOL


@pytest.mark.parametrize("tA,tB", [(False, False), (False, True), (True, False), (True, True)])
def test_paired_cta_kernel(ctx, restated, tA, tB):
    """Large aligned fp16 problems run on CTA pairs (256 x 256 tiles, cta_group::2): ragged edges, every operand layout, beta = 1."""
    M, N, K = 2240, 2112, 192   # ragged against the 256-tiles, an odd number of k-blocks
    a = cases.uniform(11, (1, K, M) if tA else (1, M, K)).astype(np.float16).astype(np.float32)
    b = cases.normal(12, (1, N, K) if tB else (1, K, N), 0.25).astype(np.float16).astype(np.float32)
    c0 = cases.normal(13, (1, M, N)).astype(np.float16).astype(np.float32)
    C = dev(c0, torch.float16)
    ctx.gemm(dev(a, torch.float16), dev(b, torch.float16), C, transA=tA, transB=tB, beta=1)
    a_eff = np.ascontiguousarray(a.transpose(0, 2, 1)) if tA else a
    b_eff = np.ascontiguousarray(b.transpose(0, 2, 1)) if tB else b
    want = restated.matmul_forward(a_eff, b_eff) + c0
    check(ctx, C, want, F16_TOL)


@pytest.mark.parametrize("tdtype,rows,din,dhid", [(torch.float16, 2304, 256, 2304), (torch.float16, 200, 72, 136),
                                                   (torch.float32, 200, 72, 136), (torch.float16, 130, 33, 50)])
def test_fused_step_equals_unfused(ctx, tdtype, rows, din, dhid):
    """ReLU inside the contraction epilogues and first-touch gradients give the tensors of the reference's call sequence
    (zero fill, MatrixMultiply, ReLu, ..., ReLuGrad, +=) bit for bit: paired kernel, single-CTA TMA kernel, loader kernels."""
    X = dev(cases.normal(21, (1, rows, din)), tdtype)
    W1 = dev(cases.normal(22, (1, din, dhid), 0.1), tdtype)
    W2 = dev(cases.normal(23, (1, dhid, din), 0.1), tdtype)
    dY = dev(cases.normal(24, (1, rows, din), 0.1), tdtype)
    z = lambda t: torch.zeros_like(t)
    # reference sequence
    H = ctx.matmul_forward(X, W1)
    A = ctx.relu_forward(H)
    Y = ctx.matmul_forward(A, W2)
    dA, dH, dX, dW1, dW2 = z(A), z(H), z(X), z(W1), z(W2)
    ctx.matmul_grad_x(A, dA, W2, dY)
    ctx.matmul_grad_y(A, W2, dW2, dY)
    ctx.relu_backward(H, dH, dA)
    ctx.matmul_grad_x(X, dX, W1, dH)
    ctx.matmul_grad_y(X, W1, dW1, dH)
    # fused sequence into buffers full of garbage
    g = lambda t: torch.full_like(t, 7.0)
    H2, A2, Y2, dA2, dH2, dX2, dW12, dW22 = g(H), g(A), g(Y), g(dA), g(dH), g(dX), g(dW1), g(dW2)
    ctx.matmul_forward_relu(X, W1, H2, A2)
    ctx.matmul_forward(A2, W2, out=Y2)
    ctx.matmul_grad_x_relu(A2, dA2, W2, dY, H2, dH2, accumulate_dx=False, accumulate_dh=False)
    ctx.matmul_grad_y(A2, W2, dW22, dY, accumulate=False)
    ctx.matmul_grad_x(X, dX2, W1, dH2, accumulate=False)
    ctx.matmul_grad_y(X, W1, dW12, dH2, accumulate=False)
    assert ctx.status() == 0
    for name, a, b in (("H", H, H2), ("A", A, A2), ("Y", Y, Y2), ("dA", dA, dA2), ("dH", dH, dH2), ("dX", dX, dX2), ("dW1", dW1, dW12),
                       ("dW2", dW2, dW22)):
        assert torch.equal(a, b), name
    # accumulating variants: run the fused backward once more on top
    ctx.matmul_grad_x_relu(A2, dA2, W2, dY, H2, dH2, accumulate_dx=True, accumulate_dh=True)
    ctx.matmul_grad_x(A, dA, W2, dY)
    dH_ref = dH.clone()
    ctx.relu_backward(H, dH_ref, dA)
    assert ctx.status() == 0
    assert torch.equal(dA, dA2) and torch.equal(dH_ref, dH2)


def test_gradients_accumulate(ctx):
    """Calling a gradient twice adds twice (beta = 1 in the reference's gemm calls, MatrixMultiply.cu:203, 391)."""
    x = dev(cases.small_ints(1, (2, 64, 32), 4))
    y = dev(cases.small_ints(2, (1, 32, 48), 4))
    dz = dev(cases.small_ints(3, (2, 64, 48), 4))
    dx = torch.zeros_like(x)
    ctx.matmul_grad_x(x, dx, y, dz)
    once = dx.clone()
    ctx.matmul_grad_x(x, dx, y, dz)
    assert ctx.status() == 0
    assert torch.equal(dx, 2 * once)


def test_empty_and_bad_arguments(ctx):
    import deep8_b200
    x = torch.zeros(1, 4, 8, device=DEV)
    y = torch.zeros(3, 9, 2, device=DEV)
    with pytest.raises(ValueError):
        ctx.matmul_forward(x, y)                       # inner extents differ
    with pytest.raises(ValueError):
        ctx.matmul_forward(torch.zeros(2, 4, 8, device=DEV), torch.zeros(3, 8, 2, device=DEV))  # batches 2 and 3
    with pytest.raises(TypeError):
        ctx.matmul_forward(x.double(), torch.zeros(1, 8, 2, device=DEV).double())   # "type ... is not support"
    with pytest.raises(deep8_b200.D8kError):
        deep8_b200._lib.check(ctx.lib.d8k_matmul_forward(ctx.h, 0, None, 1, 4, 8, None, 1, 2, None))  # null pointers
    # K = 0 through the general entry point: an empty contraction overwrites C with zeros
    C = torch.ones(1, 4, 6, device=DEV)
    ctx.gemm(torch.zeros(1, 4, 0, device=DEV), torch.zeros(1, 0, 6, device=DEV), C)
    assert ctx.status() == 0 and float(C.abs().sum()) == 0.0


def test_relu_matches_reference_rule(ctx):
    for dt in (torch.float32, torch.float16):
        x = torch.randn(1000003, device=DEV).to(dt)
        y = ctx.relu_forward(x)
        assert torch.equal(y, torch.where(x > 0, x, torch.zeros_like(x)))
        dy = torch.randn_like(x)
        dx0 = torch.randn_like(x)
        dx = dx0.clone()
        ctx.relu_backward(x, dx, dy)
        want = torch.where(x > 0, (dx0.float() + dy.float()).to(dt), dx0)
        assert torch.equal(dx, want)
    assert ctx.status() == 0


def test_split_k_is_deterministic(ctx):
    """The split-K reduction sums partial tiles in split order: two runs give identical bits."""
    x = dev(cases.normal(2, (64, 128, 256), 0.05))
    dz = dev(cases.normal(3, (64, 128, 256)))
    y = dev(cases.normal(4, (1, 256, 256), 0.05))
    a, b = torch.zeros_like(y), torch.zeros_like(y)
    ctx.matmul_grad_y(x, y, a, dz)
    ctx.matmul_grad_y(x, y, b, dz)
    assert ctx.status() == 0
    assert torch.equal(a, b)


def test_cpp_host_interface():
    """The C++ Deep8:: interface (include/deep8/Deep8.h) over the C ABI: node, executor, pool and error-behaviour tests in
    the style of the reference's gtest headers, compiled by deep8_b200.build.build_cpp_tests() (tests/cpp/)."""
    import subprocess
    exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cpp", "bin", "test_deep8_host")
    assert os.path.exists(exe), "tests/cpp/bin/test_deep8_host is missing: run __graft_entry__.build()"
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    print(r.stdout)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "0 failed" in r.stdout


@pytest.mark.gpu
def test_conv_contractions_take_the_tma_paths(ctx):
    """Channel counts that are multiples of 32: the virtual im2col operand arrives through im2col tensor maps and the
    filter-by-tap operand through its 4-D map, not through the loader warps."""
    x = torch.zeros((2, 8, 8, 64), device="cuda")
    w = torch.zeros((64, 3, 3, 64), device="cuda")
    dz = torch.zeros((2, 8, 8, 64), device="cuda")
    ctx.conv2d_forward(x, w, True, (1, 1), (1, 1))
    assert "tma a=im2col b=tiled" in ctx.last_kernel()
    ctx.conv2d_grad_x(x, torch.zeros_like(x), w, dz, True, (1, 1), (1, 1))
    assert "tma a=im2col b=filter-tap" in ctx.last_kernel()
    ctx.conv2d_grad_y(x, w, torch.zeros_like(w), dz, True, (1, 1), (1, 1))
    assert "tma a=tiled b=im2col-mn" in ctx.last_kernel()
    ctx.conv2d_forward(x.half(), w.half(), True, (1, 1), (1, 1))
    assert "f16 tma a=im2col" in ctx.last_kernel()
    x3 = torch.zeros((1, 9, 9, 3), device="cuda")
    ctx.conv2d_forward(x3, torch.zeros((5, 3, 3, 3), device="cuda"), True, (1, 1), (1, 1))
    assert "gather" in ctx.last_kernel()  # 3 channels: no 128-byte channel slices
    # stride 2: one launch per residue class of output pixels, each over its own sub-grid of taps
    xd, wd = torch.zeros((2, 6, 6, 64), device="cuda"), torch.zeros((64, 4, 4, 64), device="cuda")
    zd = ctx.deconv2d_forward(xd, wd, True, (2, 2))
    assert "tma a=im2col b=filter-sub" in ctx.last_kernel()
    ctx.deconv2d_grad_y(xd, wd, torch.zeros_like(wd), torch.zeros_like(zd), True, (2, 2))
    assert "tma a=im2col-mn b=im2col-mn" in ctx.last_kernel()
    ctx.conv2d_grad_x(x, torch.zeros_like(x), w, torch.zeros((2, 4, 4, 64), device="cuda"), True, (2, 2), (1, 1))
    assert "tma a=im2col b=filter-tap-sub" in ctx.last_kernel()
    a = torch.zeros((1, 256, 512), device="cuda")
    ctx.matmul_forward(a, torch.zeros((1, 512, 128), device="cuda"))
    assert "f32 tma a=tiled b=tiled" in ctx.last_kernel()
    torch.cuda.synchronize()
    assert ctx.status() == 0


def _random_conv_cases(n, seed):
    """Seeded random geometries with channel counts the TMA producer takes: everything else is drawn freely, so strides,
    dilations, paddings, filter shapes and residue classes meet in combinations no hand-written list covers."""
    r = np.random.Generator(np.random.Philox(seed))
    out = []
    while len(out) < n:
        ic, oc = int(r.choice([32, 64, 96])), int(r.choice([32, 64, 96, 128]))
        fh, fw = int(r.integers(1, 5)), int(r.integers(1, 5))
        sy, sx = int(r.integers(1, 4)), int(r.integers(1, 4))
        dy, dx = int(r.integers(1, 3)), int(r.integers(1, 3))
        h, w = int(r.integers(fh * dy + 1, 13)), int(r.integers(fw * dx + 1, 13))
        out.append(((int(r.integers(1, 4)), h, w, ic), (oc, fh, fw, ic), bool(r.integers(0, 2)), (sy, sx), (dy, dx)))
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("xs,ws,cov,st,dil", _random_conv_cases(16, 2024))
def test_conv_random_geometries_f32(ctx, restated, xs, ws, cov, st, dil):
    parity(ctx, restated, "conv", xs, ws, (cov, st, dil), torch.float32, F32_TOL, seed=11)


@pytest.mark.gpu
@pytest.mark.parametrize("xs,ws,cov,st,dil", _random_conv_cases(6, 2025))
def test_conv_random_geometries_integers_exact_and_f16(ctx, restated, xs, ws, cov, st, dil):
    parity(ctx, restated, "conv", xs, ws, (cov, st, dil), torch.float32, 0.0, gen="int")
    parity(ctx, restated, "conv", xs, ws, (cov, st, dil), torch.float16, F16_TOL)  # fp16 outputs round: sums pass 2048


@pytest.mark.gpu
@pytest.mark.parametrize("xs,ws,cov,st,dil", _random_conv_cases(16, 2026))
def test_deconv_random_geometries_f32(ctx, restated, xs, ws, cov, st, dil):
    parity(ctx, restated, "deconv", xs, ws, (cov, st), torch.float32, F32_TOL, seed=12)


@pytest.mark.gpu
@pytest.mark.parametrize("xs,ws,cov,st,dil", _random_conv_cases(6, 2027))
def test_deconv_random_geometries_integers_exact_and_f16(ctx, restated, xs, ws, cov, st, dil):
    parity(ctx, restated, "deconv", xs, ws, (cov, st), torch.float32, 0.0, gen="int")
    parity(ctx, restated, "deconv", xs, ws, (cov, st), torch.float16, F16_TOL)


# ------------------------------------------------------------------------------------------------ bias (Add after MatrixMultiply)
@pytest.mark.gpu
@pytest.mark.parametrize("tdtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("xs,ys", [((2, 129, 65), (1, 65, 33)), ((1, 512, 256), (1, 256, 384)), ((3, 40, 24), (3, 24, 56)),
                                   ((1, 2048, 512), (1, 512, 1024))])
def test_matmul_forward_bias(ctx, restated, tdtype, xs, ys):
    """One launch equals MatrixMultiply followed by Add bit for bit, and both follow the oracle."""
    x, y, b = cases.uniform(21, xs), cases.normal(22, ys, 0.25), cases.uniform(23, (1, ys[2]))
    if tdtype == torch.float16:
        x, y, b = (a.astype(np.float16).astype(np.float32) for a in (x, y, b))
    X, Y, B = dev(x, tdtype), dev(y, tdtype), dev(b, tdtype)
    fused = ctx.matmul_forward_bias(X, Y, B)
    two = ctx.add_bias(ctx.matmul_forward(X, Y), B)
    torch.cuda.synchronize()
    assert torch.equal(fused, two)
    want = restated.add_bias(restated.matmul_forward(x, y), b)
    check(ctx, fused, want, F32_TOL if tdtype == torch.float32 else F16_TOL, "z")


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(3, 50, 33), (1, 8192, 4096), (2, 1, 7), (1, 100, 1)])
def test_bias_gradient(ctx, restated, shape):
    dz, d0 = cases.normal(31, shape), cases.normal(32, (1, shape[2]))
    want = restated.add_bias_grad(dz, d0)
    DB = dev(d0)
    ctx.add_bias_grad(DB, dev(dz))
    check(ctx, DB, want, F32_TOL, "dbias")
    DB2 = dev(d0)
    ctx.add_bias_grad(DB2, dev(dz))
    torch.cuda.synchronize()
    assert torch.equal(DB, DB2)  # fixed order of addition: the same bits every run
    dzi, d0i = cases.small_ints(33, shape), cases.small_ints(34, (1, shape[2]))
    DBi = dev(d0i)
    ctx.add_bias_grad(DBi, dev(dzi))
    check(ctx, DBi, restated.add_bias_grad(dzi, d0i), 0.0, "dbias on integers")
    dzh = dz.astype(np.float16).astype(np.float32)
    DBh = dev(d0, torch.float16)
    ctx.add_bias_grad(DBh, dev(dzh, torch.float16))
    check(ctx, DBh, restated.add_bias_grad(dzh, d0.astype(np.float16).astype(np.float32)), F16_TOL, "dbias f16")


# ------------------------------------------------------------------------------------------------ the benchmark configurations as stated
def _config_inputs(n):
    """Inputs of benchmark configuration n exactly as it words them (distributions, scales, seeds; the second operand of
    configurations 1 and 2 takes seed + 10)."""
    if n == 1:
        return "matmul", None, cases.uniform(0, (1, 256, 512)), cases.uniform(10, (1, 512, 128)), cases.uniform(1, (1, 256, 128))
    if n == 2:
        return "matmul", None, cases.normal(2, (64, 128, 256), 0.05), cases.normal(12, (1, 256, 256), 0.05), cases.normal(3, (64, 128, 256))
    if n == 3:
        return ("conv", (True, (1, 1), (1, 1)), cases.uniform(4, (32, 56, 56, 64)), cases.normal(5, (64, 3, 3, 64), (2.0 / 576) ** 0.5),
                cases.normal(6, (32, 56, 56, 64)))
    return ("deconv", (True, (2, 2)), cases.uniform(7, (16, 14, 14, 256)), cases.normal(8, (128, 4, 4, 256), 1.0 / 64),
            cases.normal(9, (16, 27, 27, 128)))


@pytest.mark.parametrize("n", [1, 2, 3, 4])
def test_benchmark_configuration_with_its_own_inputs(ctx, restated, n):
    """Configurations 1-4 at full size with the value distributions and seeds they name (He-normal filter for 3, N(0, 1/64) for 4,
    the 0.05 scale for 2), gradients from zero: fp32 within 1e-5 of the oracle."""
    kind, meta, x, w, dz = _config_inputs(n)
    r = Runner(ctx, restated, kind, meta)
    got = r.gpu(x, w, dz, np.zeros_like(x), np.zeros_like(w), torch.float32)
    want = r.cpu(x, w, dz, None, None)
    for name, g, wnt in zip(("z", "dx", "dy"), got, want):
        check(ctx, g, wnt, F32_TOL, "config %d %s" % (n, name))


@pytest.mark.parametrize("n", [3, 4])
def test_benchmark_configuration_on_fp16_storage(ctx, restated, n):
    kind, meta, x, w, dz = _config_inputs(n)
    x, w, dz = (a.astype(np.float16).astype(np.float32) for a in (x, w, dz))
    r = Runner(ctx, restated, kind, meta)
    got = r.gpu(x, w, dz, np.zeros_like(x), np.zeros_like(w), torch.float16)
    want = r.cpu(x, w, dz, None, None)
    for name, g, wnt in zip(("z", "dx", "dy"), got, want):
        check(ctx, g, wnt, F16_TOL, "config %d %s" % (n, name))


def test_cfg5_second_layer_and_fused_tails_sampled(ctx, restated):
    """Config 5 at full size, the half of the step the first-layer test leaves out: Y = A W2 (K = 16384), dA = dY W2^T,
    dW2 = A^T dY, and the fused calls - forward + ReLU, gradient of x + ReLU gradient - over 8192 x 16384, on sampled rows and
    columns against the oracle."""
    torch.manual_seed(10)
    M, K, N = 8192, 16384, 4096    # second layer: A [M x K], W2 [K x N]
    g = torch.Generator(device=DEV).manual_seed(10)
    X = torch.randn(1, M, N, device=DEV, generator=g).to(torch.float16)
    W1 = (torch.randn(1, N, K, device=DEV, generator=g) * 0.02).to(torch.float16)
    W2 = (torch.randn(1, K, N, device=DEV, generator=g) * 0.02).to(torch.float16)
    dY = (torch.randn(1, M, N, device=DEV, generator=g) * 0.01).to(torch.float16)
    H, A = torch.empty(1, M, K, device=DEV, dtype=torch.float16), torch.empty(1, M, K, device=DEV, dtype=torch.float16)
    ctx.matmul_forward_relu(X, W1, H, A)            # fused forward + ReLU at 8192 x 16384
    rows = [0, 127, 128, 4097, 8191]
    h_want = restated.matmul_forward(np.ascontiguousarray(host(X[:, rows, :])), host(W1))
    assert cases.rel_max(host(H[:, rows, :]), h_want) <= F16_TOL
    assert np.array_equal(host(A[:, rows, :]), restated.relu(host(H[:, rows, :])))      # ReLU of the stored H, exactly
    Y = ctx.matmul_forward(A, W2)
    want = restated.matmul_forward(np.ascontiguousarray(host(A[:, rows, :])), host(W2))
    assert cases.rel_max(host(Y[:, rows, :]), want) <= F16_TOL
    dA, dH = torch.empty_like(A), torch.empty_like(H)
    ctx.matmul_grad_x_relu(A, dA, W2, dY, H, dH, accumulate_dx=False, accumulate_dh=False)   # fused at 8192 x 16384
    want = restated.matmul_grad_x(np.zeros((1, len(rows), K), np.float32), host(W2), np.ascontiguousarray(host(dY[:, rows, :])))
    assert cases.rel_max(host(dA[:, rows, :]), want) <= F16_TOL
    dh_want = restated.relu_grad(host(H[:, rows, :]), host(dA[:, rows, :]))                   # from the stored dA, exactly
    assert np.array_equal(host(dH[:, rows, :]), dh_want)
    dW2 = torch.empty_like(W2)
    ctx.matmul_grad_y(A, W2, dW2, dY, accumulate=False)
    cols = [0, 255, 256, 4095]
    want = restated.matmul_grad_y(host(A), np.zeros((1, K, len(cols)), np.float32), np.ascontiguousarray(host(dY[:, :, cols])))
    assert cases.rel_max(host(dW2[:, :, cols]), want) <= F16_TOL
    assert ctx.status() == 0


# ------------------------------------------------------------------------------------------------ element-wise neighbours
@pytest.mark.parametrize("n", [1000, 4096 * 33 + 5])
def test_relu_against_the_oracles(ctx, restated, n):
    """ReLu / ReLuGrad against the oracle (pinned to deep8/src/math/ReLu.cpp): identical in fp32 and in fp16."""
    rng = np.random.default_rng(n)
    x, dy, d0 = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    x[::13] = 0
    for tdtype in (torch.float32, torch.float16):
        xs, dys, d0s = (a.astype(np.float16).astype(np.float32) for a in (x, dy, d0)) if tdtype == torch.float16 else (x, dy, d0)
        X, DY, DX = dev(xs, tdtype), dev(dys, tdtype), dev(d0s, tdtype)
        assert np.array_equal(host(ctx.relu_forward(X)), restated.relu(xs))
        ctx.relu_backward(X, DX, DY)
        want = restated.relu_grad(xs, dys, d0s)
        if tdtype == torch.float16:
            want = want.astype(np.float16).astype(np.float32)   # one fp32 sum of two fp16 values, rounded to fp16
        assert np.array_equal(host(DX), want)


@pytest.mark.parametrize("n", [1000, 4096 * 33 + 5])
def test_linear_against_the_oracles(ctx, restated, n):
    """Linear / LinearGrad: fp32 bit for bit the reference's CPU arithmetic; fp16 (half arithmetic, as the reference's half
    kernel) within 2e-2 of it."""
    rng = np.random.default_rng(n + 1)
    x, dy, d0 = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    a, b = 0.375, -1.25
    X, DY, DX = dev(x), dev(dy), dev(d0)
    assert np.array_equal(host(ctx.linear_forward(X, a, b)), restated.linear(x, a, b))
    ctx.linear_grad(DX, a, DY)
    assert np.array_equal(host(DX), restated.linear_grad(dy, a, d0))
    xh, dyh, d0h = (v.astype(np.float16).astype(np.float32) for v in (x, dy, d0))
    Xh, DYh, DXh = dev(xh, torch.float16), dev(dyh, torch.float16), dev(d0h, torch.float16)
    check(ctx, ctx.linear_forward(Xh, a, b), restated.linear(xh, a, b), F16_TOL)
    ctx.linear_grad(DXh, a, DYh)
    check(ctx, DXh, restated.linear_grad(dyh, a, d0h), F16_TOL)


@pytest.mark.parametrize("tdtype,xs,ys", [(torch.float32, (2, 70, 40), (1, 40, 96)), (torch.float16, (1, 2304, 256), (1, 256, 2304)),
                                          (torch.float16, (1, 130, 33), (1, 33, 50))])
def test_matmul_forward_linear_equals_the_two_calls(ctx, tdtype, xs, ys):
    """The Linear tail of the epilogue (paired kernel, single-CTA kernels, ragged path) stores what MatrixMultiply followed by
    Linear stores."""
    X, Y = dev(cases.normal(31, xs), tdtype), dev(cases.normal(32, ys, 0.1), tdtype)
    Z = ctx.matmul_forward(X, Y)
    L = ctx.linear_forward(Z, 0.375, -1.25)
    Z2, L2 = torch.full_like(Z, 3.0), torch.full_like(Z, 3.0)
    ctx.matmul_forward_linear(X, Y, Z2, L2, 0.375, -1.25)
    assert ctx.status() == 0
    assert torch.equal(Z, Z2) and torch.equal(L, L2)


@pytest.mark.parametrize("steps", [0, 1, 25])
def test_adam_update_against_the_oracle(ctx, restated, steps):
    """AdamUpdate: fp32 equal to the restated reference arithmetic bit for bit (gradient, m, v and value); fp16 within 2e-2."""
    rng = np.random.default_rng(40 + steps)
    n = 4096 * 9 + 3
    w, g = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    m, v = (rng.standard_normal(n) * 0.1).astype(np.float32), (rng.random(n) * 0.01).astype(np.float32)
    args = (0.875, 0.9990234375, 2.0 ** -20, 0.0078125, 0.00048828125, steps)
    want = restated.adam_update(w, g, m, v, *args)
    W, G, M, V = dev(w), dev(g), dev(m), dev(v)
    ctx.adam_update(W, G, M, V, *args)
    assert ctx.status() == 0
    for name, got, wnt in zip(("value", "gradient", "m", "v"), (W, G, M, V), want):
        assert np.array_equal(host(got), wnt), name
    h = lambda a: a.astype(np.float16).astype(np.float32)
    wh, gh, mh, vh = h(w), h(g), h(m), h(v)
    want = restated.adam_update(wh, gh, mh, vh, *args)
    Wh, Gh, Mh, Vh = (dev(a, torch.float16) for a in (wh, gh, mh, vh))
    ctx.adam_update(Wh, Gh, Mh, Vh, *args)
    for got, wnt in zip((Wh, Gh, Mh, Vh), want):
        check(ctx, got, wnt, F16_TOL)


def test_sum_shards_adam_equals_sum_then_adam(ctx):
    for dtype in (torch.float16, torch.float32):
        n = 8 * 1024 + 3
        gen = torch.Generator(device="cuda").manual_seed(6)
        parts = [torch.randn(n, device="cuda", generator=gen).to(dtype) for _ in range(3)]
        w = torch.randn(n, device="cuda", generator=gen).to(dtype)
        m = (torch.randn(n, device="cuda", generator=gen) * 0.1).to(dtype)
        v = (torch.rand(n, device="cuda", generator=gen) * 0.01).to(dtype)
        args = (0.875, 0.9990234375, 2.0 ** -20, 0.0078125, 0.00048828125, 3)
        grad = torch.empty(n, device="cuda", dtype=dtype)
        ctx.sum_shards(dtype, grad.data_ptr(), [p.data_ptr() for p in parts], n)
        w2, m2, v2 = w.clone(), m.clone(), v.clone()
        ctx.adam_update(w2, grad, m2, v2, *args)
        w1, m1, v1, g1 = w.clone(), m.clone(), v.clone(), torch.empty_like(grad)
        copies = [torch.zeros_like(w) for _ in range(2)]
        ctx.sum_shards(dtype, g1.data_ptr(), [p.data_ptr() for p in parts], n, adam=(w1.data_ptr(), m1.data_ptr(), v1.data_ptr()) + args,
                       copies=[c.data_ptr() for c in copies])
        torch.cuda.synchronize()
        assert torch.equal(w1, w2) and torch.equal(m1, m2) and torch.equal(v1, v2) and torch.equal(g1, grad)
        assert all(torch.equal(c, w2) for c in copies)
    assert ctx.status() == 0


# ------------------------------------------------------------------------------------------------ first-touch convolution gradients
@pytest.mark.parametrize("case", [("conv",) + cases.CONV_REFERENCE_TESTS[0], ("conv",) + cases.CONV_EDGE[3], ("conv",) + cases.CONV_EDGE[6],
                                  ("deconv",) + cases.DECONV_REFERENCE_TESTS[1], ("deconv",) + cases.DECONV_EDGE[6], ("deconv",) + cases.DECONV_EDGE[3]])
def test_convolution_gradients_overwrite_without_zero_fill(ctx, case):
    """accumulate=False into buffers full of garbage gives the bits of zero fill followed by +=, stride beyond the filter and
    residue classes included."""
    kind, xs, ws, cov, st = case[:5]
    meta = (cov, st) + ((case[5],) if kind == "conv" else ())
    X, W = dev(cases.uniform(51, xs)), dev(cases.normal(52, ws, 0.25))
    fwd = ctx.conv2d_forward if kind == "conv" else ctx.deconv2d_forward
    gx = ctx.conv2d_grad_x if kind == "conv" else ctx.deconv2d_grad_x
    gy = ctx.conv2d_grad_y if kind == "conv" else ctx.deconv2d_grad_y
    Z = fwd(X, W, *meta)
    DZ = dev(cases.normal(53, tuple(Z.shape)))
    dx_ref, dw_ref = torch.zeros_like(X), torch.zeros_like(W)
    gx(X, dx_ref, W, DZ, *meta)
    gy(X, W, dw_ref, DZ, *meta)
    dx, dw = torch.full_like(X, 7.0), torch.full_like(W, 7.0)
    gx(X, dx, W, DZ, *meta, accumulate=False)
    gy(X, W, dw, DZ, *meta, accumulate=False)
    assert ctx.status() == 0
    assert torch.equal(dx, dx_ref) and torch.equal(dw, dw_ref)


def test_matrix_vector_kernels_take_the_single_column_case(ctx):
    X, Y = dev(cases.uniform(61, (2, 64, 256))), dev(cases.uniform(62, (1, 256, 1)))
    ctx.matmul_forward(X, Y)
    assert "matvec rows" in ctx.last_kernel()
    dz, dx, dy = dev(cases.uniform(63, (2, 64, 1))), torch.zeros_like(X), torch.zeros_like(Y)
    ctx.matmul_grad_x(X, dx, Y, dz)
    assert "outer product" in ctx.last_kernel()
    ctx.matmul_grad_y(X, Y, dy, dz)
    assert "matvec columns" in ctx.last_kernel()
    Yb = dev(cases.uniform(64, (6, 256, 1)))
    Xb = dev(cases.uniform(65, (1, 64, 256)))
    ctx.matmul_forward(Xb, Yb)
    assert "tma" in ctx.last_kernel()       # the batch of vectors as one contraction through the TMA producer
    assert ctx.status() == 0


# ------------------------------------------------------------------------------------------------ the halo form (off by default)
@pytest.mark.parametrize("case", [("conv", (16, 28, 28, 32), (64, 3, 3, 32), True, (1, 1), (1, 1)), ("conv",) + cases.CONV_REFERENCE_TESTS[1],
                                  ("conv", (3, 6, 5, 64), (96, 3, 3, 64), True, (1, 1), (1, 1)),
                                  ("conv", (2, 20, 17, 32), (64, 3, 2, 32), False, (1, 1), (2, 1)),
                                  ("deconv", (2, 6, 9, 64), (64, 3, 2, 64), False, (1, 1)), ("deconv", (2, 6, 6, 64), (64, 5, 5, 64), True, (2, 2))])
def test_halo_patches_give_the_same_results(ctx, restated, monkeypatch, case):
    """D8K_HALO=1: a stride-1 fp32 image operand is fetched once per tile and 32-channel slice as a patch (rows of the padded
    raster, taps as row shifts) instead of once per filter tap.  Same tolerance against the oracle as the default path."""
    monkeypatch.setenv("D8K_HALO", "1")
    kind, xs, ws, cov, st = case[:5]
    meta = (cov, st) + ((case[5],) if kind == "conv" else ())
    x, w = cases.uniform(71, xs), cases.normal(72, ws, 0.25)
    r = Runner(ctx, restated, kind, meta)
    dz = cases.normal(73, r.zshape(x, w))
    dx0, dw0 = cases.normal(74, xs), cases.normal(75, ws)
    X, W = dev(x), dev(w)
    fwd = ctx.conv2d_forward if kind == "conv" else ctx.deconv2d_forward
    fwd(X, W, *meta)
    used = ctx.last_kernel()
    got = r.gpu(x, w, dz, dx0, dw0, torch.float32)
    want = r.cpu(x, w, dz, dx0, dw0)
    for name, g, wnt in zip(("z", "dx", "dy"), got, want):
        check(ctx, g, wnt, F32_TOL, name)
    if xs[0] == 16:  # enough tiles for every SM: the halo form is what ran (smaller problems keep the split contraction)
        assert "halo" in used, used


@pytest.mark.gpu
@pytest.mark.parametrize("case", [("conv", (8, 56, 56, 64), (64, 3, 3, 64), True, (1, 1), (1, 1)), ("conv", (16, 40, 40, 32), (128, 1, 1, 32), True, (1, 1), (1, 1)),
                                  ("matmul", (1, 4096, 512), (1, 512, 512)), ("matmul", (48, 256, 96), (1, 96, 128))])
def test_two_ctas_per_sm_give_the_same_bits(ctx, restated, monkeypatch, case):
    """fp32 launches with more tiles than SMs and no split run two CTAs per SM (half the stages, one accumulator buffer and one
    converter group each).  The accumulation order does not change, so every result equals the single-CTA kernel's bit for bit -
    both forms of the paired kernel (A entirely in tensor memory; only its lo image there) - and the oracle within the fp32 bar."""
    kind = case[0]
    if kind == "matmul":
        x, y = cases.normal(81, case[1], 0.5), cases.normal(82, case[2], 0.5)
        X, Y = dev(x), dev(y)
        dz = cases.normal(83, (max(case[1][0], case[2][0]), case[1][1], case[2][2]))
        DZ = dev(dz)

        def run():
            DX, DY = torch.zeros_like(X), torch.zeros_like(Y)
            Z = ctx.matmul_forward(X, Y)
            used = ctx.last_kernel()
            ctx.matmul_grad_x(X, DX, Y, DZ)
            ctx.matmul_grad_y(X, Y, DY, DZ)
            return used, (Z, DX, DY)
        oracle_args, runner = (x, y, dz, np.zeros(case[1], np.float32), np.zeros(case[2], np.float32)), Runner(ctx, restated, "matmul", None)
    else:
        xs, ws, cov, st, dil = case[1:]
        x, w = cases.uniform(84, xs), cases.normal(85, ws, 0.25)
        X, W = dev(x), dev(w)
        meta = (cov, st, dil)
        shp = ctx.conv2d_out_shape(X, W, *meta)
        dz = cases.normal(86, tuple(shp))
        DZ = dev(dz)

        def run():
            DX, DW = torch.zeros_like(X), torch.zeros_like(W)
            Z = ctx.conv2d_forward(X, W, *meta)
            used = ctx.last_kernel()
            ctx.conv2d_grad_x(X, DX, W, DZ, *meta)
            ctx.conv2d_grad_y(X, W, DW, DZ, *meta)
            return used, (Z, DX, DW)
        oracle_args, runner = (x, w, dz, np.zeros(xs, np.float32), np.zeros(ws, np.float32)), Runner(ctx, restated, "conv", meta)
    monkeypatch.setenv("D8K_F32_DUAL", "0")
    used0, single = run()
    assert "dual" not in used0, used0
    monkeypatch.delenv("D8K_F32_DUAL")
    used, auto = run()
    assert "dual" in used, used
    for mode in ("1", "2"):
        monkeypatch.setenv("D8K_F32_DUAL", mode)
        usedm, forced = run()
        assert "dual" in usedm, usedm
        for name, a, b in zip(("z", "dx", "dy"), forced, single):
            assert torch.equal(a, b), (mode, name)
    for name, a, b in zip(("z", "dx", "dy"), auto, single):
        assert torch.equal(a, b), name
    for name, g, wnt in zip(("z", "dx", "dy"), auto, runner.cpu(*oracle_args)):
        check(ctx, g, wnt, F32_TOL, name)
    assert ctx.status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("case", [("conv", (2, 20, 17, 64), (64, 3, 3, 64), True, (1, 1), (1, 1)), ("conv", (4, 14, 14, 96), (32, 4, 4, 96), False, (2, 2), (1, 1)),
                                  ("deconv", (2, 6, 6, 64), (64, 5, 5, 64), True, (2, 2)), ("matmul", (1, 384, 1056), (1, 1056, 192)),
                                  ("matmul", (3, 130, 64), (3, 64, 70))])
def test_twin_issuing_threads_give_the_same_bits(ctx, restated, monkeypatch, case):
    """fp32 launches that keep one CTA per SM (a split contraction, or fewer tiles than SMs) run with two TMA-issuing and two
    MMA-issuing threads; a token orders the MMA threads, so the sums are formed in the same order as with one thread each and
    every result equals that kernel's bit for bit."""
    kind = case[0]
    monkeypatch.setenv("D8K_GROUP", "0")  # one launch per residue class in both runs: the same split plans, so the same partial sums
    meta = None if kind == "matmul" else ((case[3], case[4], case[5]) if kind == "conv" else (case[3], case[4]))
    x, w = cases.normal(91, case[1], 0.5), cases.normal(92, case[2], 0.25)
    r = Runner(ctx, restated, kind, meta)
    dz = cases.normal(93, r.zshape(x, w))
    dx0, dw0 = cases.normal(94, case[1]), cases.normal(95, case[2])
    monkeypatch.setenv("D8K_F32_DUAL", "0")
    single = r.gpu(x, w, dz, dx0, dw0, torch.float32)
    used0 = ctx.last_kernel()
    monkeypatch.delenv("D8K_F32_DUAL")
    auto = r.gpu(x, w, dz, dx0, dw0, torch.float32)
    used = ctx.last_kernel()
    assert "twin" not in used0 and "dual" not in used0, used0
    if "tma" in used:  # shapes TMA cannot describe stay on the loader warps, which have no twin form
        assert "twin" in used, used
    for name, a, b in zip(("z", "dx", "dy"), auto, single):
        assert torch.equal(a, b), name
    for name, g, wnt in zip(("z", "dx", "dy"), auto, r.cpu(x, w, dz, dx0, dw0)):
        check(ctx, g, wnt, F32_TOL, name)
    assert ctx.status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("case", [("conv", (4, 28, 28, 64), (128, 3, 3, 64), True, (1, 1), (1, 1)), ("matmul", (1, 1024, 512), (1, 512, 384)),
                                  ("matmul", (5, 128, 192), (1, 192, 256))])
def test_twin_issuing_threads_fp16_same_bits(ctx, restated, monkeypatch, case):
    """The fp16 single-CTA kernels run with twin TMA-issuing and MMA-issuing threads too; D8K_F16_TWIN=0 is the form with one
    thread each, and both give the same bits."""
    kind = case[0]
    meta = None if kind == "matmul" else (case[3], case[4], case[5])
    h = lambda a: a.astype(np.float16).astype(np.float32)
    x, w = h(cases.normal(96, case[1], 0.5)), h(cases.normal(97, case[2], 0.25))
    r = Runner(ctx, restated, kind, meta)
    dz = h(cases.normal(98, r.zshape(x, w)))
    dx0, dw0 = h(cases.normal(99, case[1])), h(cases.normal(100, case[2]))
    monkeypatch.setenv("D8K_F16_TWIN", "0")
    single = r.gpu(x, w, dz, dx0, dw0, torch.float16)
    assert "twin" not in ctx.last_kernel(), ctx.last_kernel()
    monkeypatch.delenv("D8K_F16_TWIN")
    twin = r.gpu(x, w, dz, dx0, dw0, torch.float16)
    used = ctx.last_kernel()
    if " tma " in used:
        assert "twin" in used, used
    for name, a, b in zip(("z", "dx", "dy"), twin, single):
        assert torch.equal(a, b), name
    for name, g, wnt in zip(("z", "dx", "dy"), twin, r.cpu(x, w, dz, dx0, dw0)):
        check(ctx, g, wnt, F16_TOL, name)
    assert ctx.status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("case", [("deconv", (4, 14, 14, 64), (32, 4, 4, 64), True, (2, 2)), ("deconv", (2, 9, 7, 32), (64, 3, 3, 32), False, (3, 2)),
                                  ("conv", (2, 33, 29, 64), (64, 3, 3, 64), True, (2, 2), (1, 1)), ("conv", (3, 24, 24, 32), (96, 5, 4, 32), False, (2, 3), (1, 1))])
@pytest.mark.parametrize("tdtype", [torch.float32, torch.float16])
def test_residue_classes_in_one_launch(ctx, restated, monkeypatch, case, tdtype):
    """A strided rule runs one contraction per residue class of pixels (or of taps).  By default their work items share ONE
    launch (every class with its own parameters, tensor maps, scratch region and tickets in device memory); D8K_GROUP=0
    launches them one after the other.  Both within the bar of the oracle and of each other (the grouped launch chooses its
    split count for all classes together, so the partial sums differ)."""
    kind = case[0]
    meta = (case[3], case[4], case[5]) if kind == "conv" else (case[3], case[4])
    h = (lambda a: a.astype(np.float16).astype(np.float32)) if tdtype == torch.float16 else (lambda a: a)
    x, w = h(cases.uniform(101, case[1])), h(cases.normal(102, case[2], 0.25))
    r = Runner(ctx, restated, kind, meta)
    dz = h(cases.normal(103, r.zshape(x, w)))
    dx0, dw0 = h(cases.normal(104, case[1])), h(cases.normal(105, case[2]))
    monkeypatch.setenv("D8K_GROUP", "0")
    before = ctx.launch_count()
    apart = r.gpu(x, w, dz, dx0, dw0, tdtype)
    launches_apart = ctx.launch_count() - before
    assert "grouped" not in ctx.last_kernel(), ctx.last_kernel()
    monkeypatch.delenv("D8K_GROUP")
    before = ctx.launch_count()
    together = r.gpu(x, w, dz, dx0, dw0, tdtype)
    launches_together = ctx.launch_count() - before
    if " tma " in ctx.last_kernel():  # which of the three contractions has the divisor depends on the operator: count launches
        assert launches_together < launches_apart, (launches_together, launches_apart)
    tol = F32_TOL if tdtype == torch.float32 else F16_TOL
    for name, a, b in zip(("z", "dx", "dy"), together, apart):  # the group plans its splits as a whole: other partial sums, same values
        assert cases.rel_max(host(a), host(b)) <= tol, name
    for name, g, wnt in zip(("z", "dx", "dy"), together, r.cpu(x, w, dz, dx0, dw0)):
        check(ctx, g, wnt, tol, name)
    assert ctx.status() == 0
