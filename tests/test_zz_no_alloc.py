"""d8k_gemm_static, the entry point for callers that may not allocate device memory (a framework that has given the
whole GPU to its own pool, a latency-critical loop, a plug-in that cannot create a context): its split-K scratch is a
static device array inside the library.  Checked through the C ABI against d8k_gemm, the entry point with a context, on
two calls in a row (the second call finds the array as the first left it).  Collected last on purpose."""
import ctypes

import numpy as np
import pytest
import torch

import cases

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F32_TOL = 1e-5
F16_TOL = 2e-2


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, F32_TOL), (torch.float16, F16_TOL)])
def test_static_scratch_matches_context_entry_point(ctx, dtype, tol):
    from deep8_b200 import _lib
    lib = _lib.load()
    code = _lib.F32 if dtype == torch.float32 else _lib.F16
    # the broadcast-weight gradient of benchmark config 2: dB[256 x 256] += A^T[256 x 8192] dC[8192 x 256], split over K
    M, N, K = 256, 256, 8192
    A = torch.from_numpy(cases.normal(2, (1, K, M), 0.05)).to(DEV).to(dtype)
    B = torch.from_numpy(cases.normal(3, (1, K, N))).to(DEV).to(dtype)
    C0 = torch.from_numpy(cases.normal(4, (1, M, N), 0.5)).to(DEV).to(dtype)
    for call in range(2):
        want = C0.clone()
        ctx.gemm(A, B, want, transA=True, transB=False, beta=1)
        assert ctx.status() == 0
        got = C0.clone()
        torch.cuda.synchronize()
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.d8k_gemm_static(code, 1, 0, M, N, K, _ptr(A), M, _ptr(B), N, _ptr(got), N, 1, ctypes.c_void_p(stream))
        assert rc == 0, lib.d8k_last_error().decode()
        torch.cuda.synchronize()
        err = cases.rel_max(got.float().cpu().numpy(), want.float().cpu().numpy())
        assert err <= tol, "call %d: rel_max %.3e" % (call, err)
        # and against the exact contraction, so that two wrong answers cannot agree
        exact = (C0.double() + A.double().transpose(1, 2) @ B.double()).cpu().numpy()
        assert cases.rel_max(got.float().cpu().numpy(), exact) <= tol


def test_static_scratch_rejects_oversize(monkeypatch):
    from deep8_b200 import _lib
    lib = _lib.load()
    # The launcher's own split choice never needs more than 148 partial tiles (9.25 MiB).  D8K_SPLITS asks for more:
    # 144 tiles of 128x128 in 4 splits are 36 MiB of partial tiles, over the 16 MiB array.
    monkeypatch.setenv("D8K_SPLITS", "4")
    M, N, K = 1152, 2048, 8192
    A = torch.zeros(M, K, device=DEV, dtype=torch.float16)
    B = torch.zeros(N, K, device=DEV, dtype=torch.float16)
    C = torch.zeros(M, N, device=DEV, dtype=torch.float16)
    rc = lib.d8k_gemm_static(_lib.F16, 0, 1, M, N, K, _ptr(A), K, _ptr(B), K, _ptr(C), N, 0, None)
    assert rc == 1
    assert "static maximum" in lib.d8k_last_error().decode()
    monkeypatch.delenv("D8K_SPLITS")
    rc = lib.d8k_gemm_static(_lib.F16, 0, 1, M, N, K, _ptr(A), K, _ptr(B), K, _ptr(C), N, 0, None)  # unsplit: fits
    assert rc == 0, lib.d8k_last_error().decode()
    torch.cuda.synchronize()
