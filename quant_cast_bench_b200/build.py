"""Build the CUDA library in-tree:  python -m quant_cast_bench_b200.build [--force] [--torch]

Compiles csrc/*.cu for sm_100a with nvcc (no fast-math: IEEE division, no flush-to-zero, no
contraction across statements matter for bit-exact results) and links
quant_cast_bench_b200/lib/libquant_cast_cuda.so.  Needs no GPU.
"""
import concurrent.futures
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libquant_cast_cuda.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--ftz=false", "--prec-div=true", "--prec-sqrt=true", "--fmad=false",
    "-Xcompiler", "-fPIC",
]


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps():
    return _sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + [
        os.path.join(os.path.dirname(HERE), "include", "quant_cast_cuda.h")]


def _compile(src, verbose):
    obj = os.path.join(LIB_DIR, os.path.basename(src)[:-3] + ".o")
    extra = os.environ.get("QCC_NVCC_EXTRA", "").split()  # e.g. -DQCC_MX_GROUP_M=8 when tuning
    cmd = [NVCC] + FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    if not force and os.path.exists(LIB) and all(os.path.getmtime(LIB) >= os.path.getmtime(d) for d in _deps()):
        return LIB
    with concurrent.futures.ThreadPoolExecutor(max_workers=4) as ex:
        results = list(ex.map(lambda s: _compile(s, verbose), _sources()))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    objs = [o for o, _ in results]
    cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


TORCH_LIB = os.path.join(LIB_DIR, "libquant_cast_torch.so")
TORCH_SRC = os.path.join(CSRC, "torch_binding.cpp")


def build_torch_binding(force: bool = False) -> str:
    """lib/libquant_cast_torch.so: the native PyTorch operators (csrc/torch_binding.cpp, TORCH_LIBRARY) over the C ABI.
    Compiled with g++ against the installed torch's headers and linked to libquant_cast_cuda.so beside it; needs no GPU.
    The ctypes route does not depend on it."""
    import torch
    from torch.utils import cpp_extension as ext
    lib = build(force=force)
    deps = [TORCH_SRC, lib, os.path.join(os.path.dirname(HERE), "include", "quant_cast_cuda.h")]
    if not force and os.path.exists(TORCH_LIB) and all(os.path.getmtime(TORCH_LIB) >= os.path.getmtime(d) for d in deps):
        return TORCH_LIB
    cxx = os.environ.get("CXX", "g++")
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", TORCH_SRC, "-o", TORCH_LIB,
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{p}" for p in ext.include_paths("cuda")]
    cmd += [f"-L{p}" for p in ext.library_paths("cuda")] + [f"-L{LIB_DIR}"]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lquant_cast_cuda", "-lcudart",
            "-Wl,-rpath,$ORIGIN", "-Wl,--no-as-needed"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building the torch binding failed:\n{r.stdout}\n{r.stderr[-4000:]}")
    return TORCH_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--torch" in sys.argv:
        print(build_torch_binding(force="--force" in sys.argv))
