"""Build libfp8gmm_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

Usage: python fp8_gmm_b200/csrc/build.py [--force] [--verbose]   (run as a script: it must not import the
package, whose import needs the library this script produces)

The library has no Python, torch or pybind dependency: it is plain CUDA C++ linked against the static
CUDA runtime, and is loaded from Python with ctypes (fp8_gmm_b200/_lib.py).  nvcc cross-compiles
without a GPU present.
"""
import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
OUT = os.path.join(PKG, "libfp8gmm_b200.so")
BUILD = os.path.join(HERE, "_build")

# (source, extra flags).  The elementwise and GEMM kernels use fast-math like the reference build
# (reference setup.py:21), which fixes flush-to-zero and the tanh/exp approximations they share with it.
SOURCES = [
    ("runtime.cu", []),
    ("peer.cu", []),
    ("routing.cu", []),
    ("pointwise.cu", ["--use_fast_math"]),
    ("pad_fusion.cu", ["--use_fast_math"]),
    ("gemm_sm100.cu", ["--use_fast_math"]),
]
COMMON = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
HEADERS = ["common.cuh", os.path.join("..", "..", "include", "fp8_gmm_b200.h")]


def _nvcc():
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _digest(paths, flags):
    h = hashlib.sha256()
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def build(force=False, verbose=False):
    os.makedirs(BUILD, exist_ok=True)
    nvcc = _nvcc()
    hdrs = [os.path.join(HERE, h) for h in HEADERS]
    sources = [(s, f) for s, f in SOURCES if os.path.exists(os.path.join(HERE, s))]
    jobs, objs = [], []
    for src, extra in sources:
        path = os.path.join(HERE, src)
        obj = os.path.join(BUILD, src.replace(".cu", ".o"))
        stamp = obj + ".sha"
        flags = COMMON + extra + (["-Xptxas", "-v"] if verbose else [])
        dig = _digest([path] + hdrs, flags)
        objs.append(obj)
        if not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
            continue
        jobs.append((path, obj, stamp, dig, flags))

    def compile_one(job):
        path, obj, stamp, dig, flags = job
        cmd = [nvcc] + flags + ["-c", path, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {path}")
        with open(stamp, "w") as f:
            f.write(dig)

    with ThreadPoolExecutor(max(1, min(4, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    if jobs or force or not os.path.exists(OUT):
        cmd = [nvcc, "-shared", "-o", OUT] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link failed")
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
