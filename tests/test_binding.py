"""The reference-side binding (deep8_b200/csrc/reference_binding/d8k_binding.cpp: the nine `...GPU` functions and the six
`...InterimSize` GPU branches a maintainer of the reference would compile in) is compiled against the reference's own
headers, unmodified.  No GPU is needed: this is a compile check.  Skipped where the reference tree is absent."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINDING = os.path.join(ROOT, "deep8_b200", "csrc", "reference_binding", "d8k_binding.cpp")


def _reference_root():
    from oracle import pyoracle
    root = pyoracle.reference_root()
    if root is None:
        pytest.skip("the reference's source tree is not present")
    return root


def _compile(source, ref, out):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    inc = ["third_party", "third_party/eigen", "deep8/include", "deep8/include/basic", "deep8/include/math", "deep8/include/model",
           "deep8/include/nodes"]
    # the reference's GPU headers include CUDA device headers (deep8/include/basic/GPUBasic.h:8-15): compiled as CUDA source
    cmd = [nvcc, "-std=c++11", "-x", "cu", "-w", "-DHAVE_CUDA", "-DHAVE_HALF", "-gencode", "arch=compute_100a,code=sm_100a"]
    cmd += ["-I" + os.path.join(ref, d) for d in inc] + ["-I" + os.path.join(ROOT, "include"), "-c", source, "-o", out]
    return subprocess.run(cmd, capture_output=True, text=True)


def test_binding_compiles_against_the_reference_headers(tmp_path):
    ref = _reference_root()
    r = _compile(BINDING, ref, str(tmp_path / "binding.o"))
    assert r.returncode == 0, r.stderr[-3000:]
    # every seam function is defined in the object
    nm = subprocess.run(["nm", "-C", "--defined-only", str(tmp_path / "binding.o")], capture_output=True, text=True).stdout
    for name in ("MatrixMultiplyGPU", "MatrixMultiplyGradXGPU", "MatrixMultiplyGradYGPU", "Conv2dGPU", "Conv2dGradXGPU", "Conv2dGradYGPU",
                 "DeConv2dGPU", "DeConv2dGradXGPU", "DeConv2dGradYGPU"):
        assert "Deep8::Math::%s(" % name in nm, name


@pytest.mark.parametrize("old,new", [
    ("void MatrixMultiplyGPU(const Tensor& x, const Tensor& y, Tensor& z) {", "void MatrixMultiplyGPU(const Tensor& x, const Tensor& y, Tensor& z, int extra) {"),
    ("int dilationY, int dilationX, void* xcol) {\n    Geometry g = geometry(x, y, z);\n    d8kCheck(d8k_conv2d_forward(",
     "int dilationY, void* xcol, int dilationX) {\n    Geometry g = geometry(x, y, z);\n    d8kCheck(d8k_conv2d_forward("),
    ("size_t d8kDeConv2dGradYInterimSize(const Tensor& x, const Tensor& y, Tensor&, const Tensor& z, const Tensor&, bool, int, int) {",
     "size_t d8kDeConv2dGradYInterimSize(const Tensor& x, const Tensor& y, Tensor&, const Tensor& z, const Tensor&, bool, int) {"),
])
def test_a_stub_that_disagrees_with_the_reference_signature_does_not_compile(tmp_path, old, new):
    ref = _reference_root()
    text = open(BINDING).read()
    assert old in text
    mutated = tmp_path / "mutated.cpp"
    mutated.write_text(text.replace(old, new, 1))
    r = _compile(str(mutated), ref, str(tmp_path / "mutated.o"))
    assert r.returncode != 0
