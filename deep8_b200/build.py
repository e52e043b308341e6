"""Builds libdeep8_b200.so (the CUDA kernels + the C ABI of include/d8k.h) in-tree with nvcc for sm_100a.

    python -m deep8_b200.build [--force]

Each .cu under csrc/ is compiled to an object in csrc/build/ (in parallel, skipped when up to date) and linked into
deep8_b200/libdeep8_b200.so.  No GPU is needed to build.
"""
import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "libdeep8_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-I", INCLUDE, "-I", CSRC,
]


def _nvcc():
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is needed to build deep8_b200")
    return exe


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "host", "*.cu")))


def headers():
    pats = ["*.cuh", "*.h", os.path.join("host", "*.h")]
    out = [os.path.join(INCLUDE, "d8k.h")]
    for p in pats:
        out += glob.glob(os.path.join(CSRC, p))
    out += glob.glob(os.path.join(INCLUDE, "*.h")) + glob.glob(os.path.join(INCLUDE, "deep8", "*.h"))
    return sorted(set(out))


def _compile(nvcc, src, obj, verbose):
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return r.stderr


def build(force=False, verbose=False):
    nvcc = _nvcc()
    os.makedirs(OBJ, exist_ok=True)
    srcs = sources()
    hdr_time = _newest(headers() + [os.path.abspath(__file__)])
    jobs, objs = [], []
    for src in srcs:
        obj = os.path.join(OBJ, os.path.relpath(src, CSRC).replace(os.sep, "_")[:-3] + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time)
        if stale:
            jobs.append((src, obj))
    logs = []
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            futs = [pool.submit(_compile, nvcc, s, o, verbose) for s, o in jobs]
            for f in futs:
                logs.append(f.result())
    if jobs or not os.path.exists(LIB) or os.path.getmtime(LIB) < _newest(objs):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return LIB, "\n".join(logs)


def build_cpp_tests():
    """Compile tests/cpp/*.cu into tests/cpp/bin/ against libdeep8_b200.so and the CPU oracle (a checker, linked by the tests only)."""
    nvcc = _nvcc()
    root = os.path.dirname(HERE)
    src_dir = os.path.join(root, "tests", "cpp")
    out_dir = os.path.join(src_dir, "bin")
    os.makedirs(out_dir, exist_ok=True)
    built = []
    for src in sorted(glob.glob(os.path.join(src_dir, "*.cu"))):
        exe = os.path.join(out_dir, os.path.basename(src)[:-3])
        deps = [src, LIB, os.path.join(INCLUDE, "deep8", "Deep8.h"), os.path.join(root, "oracle", "libd8oracle.so")]
        if os.path.exists(exe) and os.path.getmtime(exe) >= _newest([d for d in deps if os.path.exists(d)]):
            built.append(exe)
            continue
        cmd = [nvcc, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-I", INCLUDE, src, "-o", exe,
               "-L", HERE, "-ldeep8_b200", "-L", os.path.join(root, "oracle"), "-ld8oracle",
               "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../deep8_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../oracle"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
        built.append(exe)
    return built


if __name__ == "__main__":
    lib, log = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    if log.strip():
        print(log)
    print(lib)
