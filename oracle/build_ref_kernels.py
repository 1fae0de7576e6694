"""Compile the reference's elementwise CUDA kernels for sm_100a into oracle/_ref/ (test infrastructure).

Sources are compiled in place from the reference checkout (nothing is copied into this repository);
the flags mirror the reference's setup.py:9-24 except for the architecture, which that file pins to
sm_90a.  The result, ``oracle/_ref/ref_fp8_gmm_kernels*.so``, is git-ignored but travels with the
working tree to a GPU machine, where tests/test_gpu_vs_reference_kernels.py loads it as a byte-exact
GPU-side oracle.  Takes several minutes (each translation unit includes torch/extension.h).

Usage: python oracle/build_ref_kernels.py /path/to/reference     (or FP8GMM_REFERENCE_DIR=/path/to/reference)
"""
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FP8GMM_REFERENCE_DIR")
    if not ref:
        print("usage: python oracle/build_ref_kernels.py /path/to/reference   (or set FP8GMM_REFERENCE_DIR); nothing built")
        return 0
    csrc = os.path.join(ref, "csrc")
    if not os.path.isdir(csrc):
        print(f"reference checkout not found at {ref}; nothing built")
        return 0
    import torch
    from torch.utils import cpp_extension as ce

    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    name = "ref_fp8_gmm_kernels"
    incs = ce.include_paths("cuda") + [sysconfig.get_paths()["include"], csrc]
    common = [
        "nvcc", "-std=c++17", "-gencode=arch=compute_100a,code=sm_100a", "-O3", "--use_fast_math",
        "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
        "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
        "-U__CUDA_NO_BFLOAT162_OPERATORS__", "-U__CUDA_NO_BFLOAT162_CONVERSIONS__",
        "--expt-relaxed-constexpr", "--expt-extended-lambda", "-Xcompiler", "-fPIC",
        f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
    ] + [f"-I{p}" for p in incs]
    srcs = [
        (os.path.join(csrc, "multi_pointwise.cu"), "multi_pointwise.o"),
        (os.path.join(csrc, "multi_pad_fusion.cu"), "multi_pad_fusion.o"),
        (os.path.join(HERE, "ref_kernels_binding.cpp"), "binding.o"),
    ]

    def compile_one(item):
        src, obj = item
        cmd = common + (["-x", "cu"] if src.endswith(".cpp") else []) + ["-c", src, "-o", os.path.join(out_dir, obj)]
        subprocess.run(cmd, check=True)

    with ThreadPoolExecutor(3) as ex:
        list(ex.map(compile_one, srcs))
    so = os.path.join(out_dir, name + sysconfig.get_config_var("EXT_SUFFIX"))
    libdirs = ce.library_paths("cuda")
    link = ["g++", "-shared", "-o", so] + [os.path.join(out_dir, o) for _, o in srcs]
    link += [f"-L{d}" for d in libdirs] + [f"-Wl,-rpath,{libdirs[0]}"]
    link += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
    subprocess.run(link, check=True)
    for _, o in srcs:
        os.remove(os.path.join(out_dir, o))
    print("built", so)
    return 0


if __name__ == "__main__":
    sys.exit(main())
